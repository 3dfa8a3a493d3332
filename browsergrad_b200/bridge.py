"""``CudaBridge``: the realizer-bridge object for ``bg.register_webgpu_bridge``.

Same method surface as the reference's ``createWebGpuRealizerBridge`` object
(packages/browsergrad-kernels/src/realizer.ts:77-280, :902-1006) seen through the Python
Protocol the realizers call (packages/browsergrad-jit/src/python/_bridge.py:61-289):
``upload / materialize / release / matmul / fused_elementwise / cast / flash_attention /
run_tensor_plan[_resident][_semantic]`` plus the diagnostics ``aliveHandleCount /
resourceSnapshot / flushProfiles``.  Every method forwards to the C ABI in ``include/bgcuda.h``;
convolutions and user WGSL kernels raise (outside the forward path / not executable on CUDA).

Differences from the WebGPU bridge, all widening: every IR dtype is accepted (the reference
asserts float32, realizer.ts:310-317); elementwise operands may broadcast; MATMUL may be
batched; REDUCE has max/min/argmax/any/all; CONST, WHERE, INDEX, CROSS_ENTROPY are executable.
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib, wire
from .errors import KernelError


def _shape_arr(shape: Sequence[int]) -> Any:
    return (C.c_int64 * max(len(shape), 1))(*[int(d) for d in shape])


def _as_buffer(data: Any) -> Tuple[Any, int, Any]:
    """Return (pointer, nbytes, keepalive) for bytes / bytearray / memoryview / ndarray."""
    if isinstance(data, np.ndarray):
        arr = np.ascontiguousarray(data)
        return arr.ctypes.data_as(C.c_void_p), arr.nbytes, arr
    if isinstance(data, (bytes, bytearray, memoryview)):
        arr = np.frombuffer(data, dtype=np.uint8)
        return arr.ctypes.data_as(C.c_void_p), arr.nbytes, (arr, data)
    raise KernelError(f"CUDA bridge: upload: unsupported data type {type(data).__name__}", 1)


class CudaBridge:
    """One bridge = one ``bg_context`` on one GPU; single-threaded like the reference's."""

    def __init__(self, device: int = 0, profiling: bool = False) -> None:
        self._lib = _lib.load()
        ctx = C.c_void_p()
        rc = self._lib.bg_create(int(device), C.byref(ctx))
        if rc != 0 or not ctx.value:
            raise KernelError(
                f"CUDA bridge: cannot create a context on device {device} "
                f"({_lib.STATUS_NAMES.get(rc, rc)}); an sm_100 GPU is required and there is no CPU fallback", rc)
        self._ctx = ctx
        self.device = int(device)
        self._plan_cache: Dict[int, Tuple[Any, wire.EncodedPlan]] = {}
        if profiling:
            self.set_option("profiling", 1)

    # -- plumbing -----------------------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc != 0:
            msg = self._lib.bg_last_error(self._ctx)
            raise KernelError(msg.decode("utf-8", "replace") if msg else f"CUDA bridge: status {rc}", rc)

    def close(self) -> None:
        if getattr(self, "_ctx", None) is not None and self._ctx.value:
            self._lib.bg_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self) -> None:  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, key: str, value: int) -> None:
        self._check(self._lib.bg_set_option(self._ctx, key.encode(), int(value)))

    @staticmethod
    def _dt(dtype: str) -> int:
        if dtype not in _lib.DTYPE_CODE:
            raise KernelError(f"CUDA bridge: unknown dtype {dtype!r}", 1)
        return _lib.DTYPE_CODE[dtype]

    # -- buffer lifecycle (_bridge.py:65-71) ---------------------------------------------
    def upload(self, data: Any, shape: Sequence[int], dtype: str) -> int:
        ptr, nbytes, keep = _as_buffer(data)
        h = C.c_int64()
        self._check(self._lib.bg_upload(self._ctx, ptr, nbytes, _shape_arr(shape), len(shape), self._dt(dtype),
                                        C.byref(h)))
        del keep
        return int(h.value)

    def selftest_wait_timeout(self, limit_cycles: int = 2_000_000) -> None:
        """Runs the bounded device wait until it gives up; raises ``KernelError`` with status 6 (device-side wait timed
        out).  The bridge stays usable."""
        self._check(self._lib.bg_selftest_wait_timeout(self._ctx, int(limit_cycles)))

    def alloc(self, shape: Sequence[int], dtype: str) -> int:
        """A device buffer the caller fills itself through ``device_pointer`` on ``stream()`` (the destination of a
        device-side collective); released like any other handle."""
        h = C.c_int64()
        self._check(self._lib.bg_alloc(self._ctx, _shape_arr(shape), len(shape), self._dt(dtype), C.byref(h)))
        return int(h.value)

    def materialize(self, handle: int, shape: Sequence[int], dtype: str) -> bytes:
        n = C.c_int64()
        self._check(self._lib.bg_handle_nbytes(self._ctx, int(handle), C.byref(n)))
        out = np.empty(int(n.value), dtype=np.uint8)
        self._check(self._lib.bg_materialize(self._ctx, int(handle), out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out.tobytes()

    def materialize_array(self, handle: int, shape: Sequence[int], dtype: str) -> np.ndarray:
        """``materialize`` without the intermediate ``bytes`` copy."""
        np_dtype = np.float32 if dtype == "bfloat16" else np.dtype(dtype)
        if dtype == "bfloat16":
            raw = np.empty(tuple(shape), dtype=np.uint16)
            self._check(self._lib.bg_materialize(self._ctx, int(handle), raw.ctypes.data_as(C.c_void_p), raw.nbytes))
            return (raw.astype(np.uint32) << 16).view(np.float32)
        out = np.empty(tuple(shape), dtype=np_dtype)
        self._check(self._lib.bg_materialize(self._ctx, int(handle), out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def release(self, handle: int) -> None:
        self._check(self._lib.bg_release(self._ctx, int(handle)))

    # -- compute ops (_bridge.py:74-105) --------------------------------------------------
    def matmul(self, a: int, b: int, m: int, k: int, n: int, dtype: str) -> int:
        h = C.c_int64()
        self._check(self._lib.bg_matmul(self._ctx, int(a), int(b), int(m), int(k), int(n), self._dt(dtype), C.byref(h)))
        return int(h.value)

    def fused_elementwise(self, inputs: Sequence[int], ops: Sequence[Sequence[Any]], shape: Sequence[int],
                          dtype: str) -> int:
        flat: List[int] = []
        for opcode, lhs, rhs in ops:
            if opcode not in _lib.OP_CODE:
                raise KernelError(f"CUDA bridge: fused_elementwise: unknown opcode {opcode!r}", 1)
            unary = opcode in ("NEG", "EXP", "LOG")
            # Python passes None for unary ops, the TypeScript fixtures a dummy int: accept both
            flat.extend((_lib.OP_CODE[opcode], int(lhs), _lib.REF_NONE if (rhs is None or unary) else int(rhs)))
        ins = (C.c_int64 * max(len(inputs), 1))(*[int(h) for h in inputs])
        trip = (C.c_int32 * max(len(flat), 1))(*flat)
        h = C.c_int64()
        self._check(self._lib.bg_fused_elementwise(self._ctx, ins, len(inputs), trip, len(ops), _shape_arr(shape),
                                                   len(shape), self._dt(dtype), C.byref(h)))
        return int(h.value)

    def cast(self, handle: int, src_dtype: str, dst_dtype: str, shape: Sequence[int]) -> int:
        h = C.c_int64()
        self._check(self._lib.bg_cast(self._ctx, int(handle), self._dt(src_dtype), self._dt(dst_dtype),
                                      _shape_arr(shape), len(shape), C.byref(h)))
        return int(h.value)

    def flash_attention(self, q: int, k: int, v: int, mask: Optional[int], b: int, h: int, sq: int, sk: int, d: int,
                        scale: float, dtype: str, mask_shape: Optional[Sequence[int]] = None) -> int:
        out = C.c_int64()
        ms = None
        if mask is not None:
            if mask_shape is None:
                n = C.c_int64()
                self._check(self._lib.bg_handle_nbytes(self._ctx, int(mask), C.byref(n)))
                per = int(sq) * int(sk) * _lib.DTYPE_SIZE[dtype]
                lead = int(n.value) // per if per else 0
                if lead == 1:
                    mask_shape = (1, 1, sq, sk)
                elif lead == b * h:
                    mask_shape = (b, h, sq, sk)
                else:
                    raise KernelError("CUDA bridge: flash_attention: pass mask_shape for a [B,1,..] or [1,H,..] mask", 1)
            ms = _shape_arr(mask_shape)
        self._check(self._lib.bg_flash_attention(self._ctx, int(q), int(k), int(v), int(mask or 0), ms, int(b), int(h),
                                                 int(sq), int(sk), int(d), float(scale), self._dt(dtype), C.byref(out)))
        return int(out.value)

    # -- outside the forward path ----------------------------------------------------------
    def _unsupported(self, name: str) -> Any:
        raise KernelError(f"CUDA bridge: {name} is unsupported on the CUDA bridge (outside the forward hot path)", 2)

    def conv1d(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv1d")

    def conv2d(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv2d")

    def conv1d_backward_input(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv1d_backward_input")

    def conv1d_backward_weight(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv1d_backward_weight")

    def conv1d_backward_bias(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv1d_backward_bias")

    def conv2d_backward_input(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv2d_backward_input")

    def conv2d_backward_weight(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv2d_backward_weight")

    def conv2d_backward_bias(self, *a: Any, **k: Any) -> Any:
        return self._unsupported("conv2d_backward_bias")

    def run_user_kernel(self, *a: Any, **k: Any) -> Any:
        raise KernelError("CUDA bridge: run_user_kernel: WGSL source cannot execute on the CUDA bridge", 2)

    # -- whole-plan methods (_bridge.py:262-289) ---------------------------------------------
    def _encode(self, plan: Dict[str, Any], requests_json: Optional[str]) -> wire.EncodedPlan:
        """The flat encoding of ``plan``, remembered per plan object: a plan dict must not be edited in place after
        its first run (build a new dict instead), or the remembered encoding goes stale."""
        key = id(plan)
        hit = self._plan_cache.get(key)
        if hit is not None and hit[0] is plan and requests_json is None:
            return hit[1]
        axes = wire.validate_semantic_requests(plan, requests_json) if requests_json is not None else None
        ep = wire.encode_plan(plan, axes)
        if requests_json is None:
            if len(self._plan_cache) > 64:
                self._plan_cache.clear()
            self._plan_cache[key] = (plan, ep)
        return ep

    def _bind(self, ep: wire.EncodedPlan, inputs: Sequence[Dict[str, Any]]) -> Tuple[Any, int, List[Any]]:
        arr = (_lib.PlanInput * max(len(inputs), 1))()
        keep: List[Any] = []
        for i, item in enumerate(inputs):
            arr[i].value_id = int(item.get("value_id", item.get("valueId")))
            if item.get("handle") is not None:
                arr[i].handle = int(item["handle"])
            else:
                ptr, nbytes, k = _as_buffer(item["data"])
                arr[i].data = ptr
                arr[i].nbytes = nbytes
                keep.append(k)
        return arr, len(inputs), keep

    def run_tensor_plan(self, plan: Dict[str, Any], inputs: Sequence[Dict[str, Any]], dtype: str) -> bytes:
        return self.run_tensor_plan_array(plan, inputs, dtype).tobytes()

    def run_tensor_plan_array(self, plan: Dict[str, Any], inputs: Sequence[Dict[str, Any]], dtype: str,
                              requests_json: Optional[str] = None, out: Optional[np.ndarray] = None) -> np.ndarray:
        """``run_tensor_plan`` returning an ndarray (no ``bytes`` round trip).  ``out`` may name a
        caller-owned destination of the root's shape and dtype (page-locked memory is filled by one DMA)."""
        ep = self._encode(plan, requests_json)
        if dtype != ep.root_dtype:
            raise KernelError(f"CUDA bridge: run_tensor_plan: dtype {dtype!r} does not match the root's {ep.root_dtype!r}", 1)
        arr, n, keep = self._bind(ep, inputs)
        if out is not None:
            want_dtype = np.uint16 if ep.root_dtype == "bfloat16" else np.dtype(ep.root_dtype)
            if tuple(out.shape) != tuple(ep.root_shape) or out.dtype != want_dtype or not out.flags["C_CONTIGUOUS"]:
                raise KernelError(f"CUDA bridge: run_tensor_plan: `out` must be a C-contiguous {want_dtype} array of shape {ep.root_shape}", 1)
        elif ep.root_dtype == "bfloat16":
            out = np.empty(ep.root_shape, dtype=np.uint16)
        else:
            out = np.empty(ep.root_shape, dtype=np.dtype(ep.root_dtype))
        self._check(self._lib.bg_run_tensor_plan(self._ctx, C.byref(ep.plan), arr, n, out.ctypes.data_as(C.c_void_p),
                                                 out.nbytes))
        del keep
        if ep.root_dtype == "bfloat16":
            return (out.astype(np.uint32) << 16).view(np.float32)
        return out

    def run_tensor_plan_semantic(self, plan: Dict[str, Any], semantic_requests_json: str,
                                 inputs: Sequence[Dict[str, Any]], dtype: str) -> bytes:
        return self.run_tensor_plan_array(plan, inputs, dtype, semantic_requests_json).tobytes()

    def run_tensor_plan_resident(self, plan: Dict[str, Any], inputs: Sequence[Dict[str, Any]], dtype: str,
                                 requests_json: Optional[str] = None) -> int:
        ep = self._encode(plan, requests_json)
        if dtype != ep.root_dtype:
            raise KernelError(f"CUDA bridge: run_tensor_plan_resident: dtype {dtype!r} does not match the root's {ep.root_dtype!r}", 1)
        arr, n, keep = self._bind(ep, inputs)
        h = C.c_int64()
        self._check(self._lib.bg_run_tensor_plan_resident(self._ctx, C.byref(ep.plan), arr, n, C.byref(h)))
        del keep
        return int(h.value)

    def run_tensor_plan_resident_semantic(self, plan: Dict[str, Any], semantic_requests_json: str,
                                          inputs: Sequence[Dict[str, Any]], dtype: str) -> int:
        return self.run_tensor_plan_resident(plan, inputs, dtype, semantic_requests_json)

    # -- diagnostics (realizer.ts:273-298, :945-993) ---------------------------------------------
    def aliveHandleCount(self) -> int:
        n = C.c_int64()
        self._check(self._lib.bg_alive_handle_count(self._ctx, C.byref(n)))
        return int(n.value)

    alive_handle_count = aliveHandleCount

    def resourceSnapshot(self) -> Dict[str, int]:
        st = _lib.ResourceStats()
        self._check(self._lib.bg_resource_snapshot(self._ctx, C.byref(st)))
        return {
            "currentBytes": st.current_bytes, "peakBytes": st.peak_bytes,
            "totalAllocatedBytes": st.total_allocated_bytes, "totalReleasedBytes": st.total_released_bytes,
            "aliveHandles": st.alive_handles, "logicalTensorPlanPeakBytes": st.logical_tensor_plan_peak_bytes,
            "kernelLaunches": st.kernel_launches, "planCacheHits": st.plan_cache_hits,
            "planCacheMisses": st.plan_cache_misses,
        }

    resource_snapshot = resourceSnapshot

    def flushProfiles(self) -> List[Dict[str, Any]]:
        n = C.c_int()
        self._check(self._lib.bg_flush_profiles(self._ctx, None, 0, C.byref(n)))
        cap = max(int(n.value), 1)
        buf = (_lib.ProfileEntry * cap)()
        self._check(self._lib.bg_flush_profiles(self._ctx, buf, cap, C.byref(n)))
        return [{"name": buf[i].name.decode(), "ms": float(buf[i].ms), "launches": int(buf[i].launches)}
                for i in range(min(cap, int(n.value)))]

    flush_profiles = flushProfiles

    def last_plan_trace(self) -> List[str]:
        buf = C.create_string_buffer(1 << 16)
        self._check(self._lib.bg_last_plan_trace(self._ctx, buf, len(buf)))
        return [ln for ln in buf.value.decode().split("\n") if ln]

    def semanticTensorPlanExecutionTrace(self, handle: int) -> List[str]:
        return self.last_plan_trace()

    def device_pointer(self, handle: int) -> int:
        p = C.c_void_p()
        self._check(self._lib.bg_device_pointer(self._ctx, int(handle), C.byref(p)))
        return int(p.value or 0)

    def stream(self) -> int:
        return int(self._lib.bg_stream(self._ctx) or 0)

    def synchronize(self) -> None:
        n = C.c_int()
        self._check(self._lib.bg_flush_profiles(self._ctx, None, 0, C.byref(n)))


def create_cuda_realizer_bridge(device: int = 0, profiling: bool = False) -> CudaBridge:
    """Python spelling of ``createCudaRealizerBridge()``."""
    return CudaBridge(device, profiling)
