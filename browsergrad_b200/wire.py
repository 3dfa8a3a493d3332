"""Tensor-plan wire format: the reference's plan dictionary -> the C structs of ``bgcuda.h``.

The dictionary is ``GpuExecutionPlan.summary()`` (packages/browsergrad-jit/src/python/
_gpu_plan.py:176-209); the TypeScript side accepts snake_case and camelCase keys
(packages/browsergrad-kernels/src/tensor_plan.ts:141-179) and so does this module.  ``arg`` is
a live Python object on the reference's wire (dicts with tuple values, contract-id strings);
``encode_plan`` flattens it into ``iarg`` / ``farg`` / ``ext`` as ``bgcuda.h`` documents, and
refuses the opcode variants the CUDA bridge does not implement.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Any, Dict, List, Optional, Sequence, Tuple

from . import _lib
from .errors import JitNotImplementedError, KernelError

SEMANTIC_SCHEMA = "browsergrad.jit.tensor-plan-semantic-requests"
VIEW_COPY_KIND = "dense-permutation-view-copy"


def _get(d: Dict[str, Any], snake: str, camel: Optional[str] = None, default: Any = None) -> Any:
    if snake in d:
        return d[snake]
    if camel is None:
        parts = snake.split("_")
        camel = parts[0] + "".join(p.title() for p in parts[1:])
    return d.get(camel, default)


def normalize_axis_mask(axis: Any, rank: int) -> int:
    if axis is None:
        return (1 << rank) - 1
    axes = (axis,) if isinstance(axis, int) else tuple(axis)
    mask = 0
    for a in axes:
        a = int(a)
        if a < -rank or a >= max(rank, 1):
            raise KernelError(f"CUDA bridge: REDUCE axis {a} out of range for rank {rank}", 1)
        mask |= 1 << (a % rank if rank else 0)
    return mask


class EncodedPlan:
    """Owns the ctypes arrays a ``bg_plan`` points into."""

    def __init__(self, steps: Any, ext: Any, n_steps: int, root_id: int, buffer_steps: List[Tuple[int, Any]],
                 root_shape: Tuple[int, ...], root_dtype: str) -> None:
        self.steps = steps
        self.ext = ext
        self.plan = _lib.Plan(steps, n_steps, root_id, ext, len(ext))
        self.buffer_steps = buffer_steps      # (value_id, BUFFER arg)
        self.root_shape = root_shape
        self.root_dtype = root_dtype


def validate_semantic_requests(plan: Dict[str, Any], requests_json: str) -> Dict[int, Tuple[int, ...]]:
    """Check the dense-permutation-view-copy side table against the plan's PERMUTE steps
    (request construction: _gpu_plan.py:668-734; wire: :225-260) and return ``value_id -> axes``."""
    try:
        doc = json.loads(requests_json)
    except (TypeError, ValueError) as exc:
        raise KernelError(f"CUDA bridge: run_tensor_plan_semantic requests are not valid JSON: {exc}", 1)
    if not isinstance(doc, dict) or doc.get("schema") != SEMANTIC_SCHEMA:
        raise KernelError("CUDA bridge: run_tensor_plan_semantic: unknown request schema", 1)
    ver = doc.get("version") or {}
    if ver.get("major") != 1:
        raise KernelError("CUDA bridge: run_tensor_plan_semantic: unsupported request version", 1)
    steps = {int(_get(s, "value_id")): s for s in plan["steps"]}
    out: Dict[int, Tuple[int, ...]] = {}
    for req in doc.get("requests", []):
        if req.get("kind") != VIEW_COPY_KIND:
            raise KernelError(f"CUDA bridge: run_tensor_plan_semantic: unknown request kind {req.get('kind')!r}", 1)
        vid = int(req["valueId"])
        step = steps.get(vid)
        if step is None or step["op"] != "PERMUTE":
            raise KernelError(f"CUDA bridge: semantic request names value {vid}, which is not a PERMUTE step", 1)
        in_shape = tuple(int(x) for x in req["inputShape"])
        axes = tuple(int(a) for a in req["axes"])
        if sorted(axes) != list(range(len(in_shape))):
            raise KernelError(f"CUDA bridge: semantic request for value {vid}: axes are not a permutation", 1)
        src = steps[int(_get(step, "input_ids")[0])]
        if tuple(int(x) for x in src["shape"]) != in_shape:
            raise KernelError(f"CUDA bridge: semantic request for value {vid}: input shape does not match the plan", 1)
        if tuple(in_shape[a] for a in axes) != tuple(int(x) for x in step["shape"]):
            raise KernelError(f"CUDA bridge: semantic request for value {vid}: permuted shape does not match the plan", 1)
        if vid in out:
            raise KernelError(f"CUDA bridge: duplicate semantic request for value {vid}", 1)
        out[vid] = axes
    for vid, step in steps.items():
        if step["op"] == "PERMUTE" and vid not in out and not (isinstance(step.get("arg"), dict) and "axes" in step["arg"]):
            raise KernelError(f"CUDA bridge: PERMUTE value {vid} has neither axes nor a semantic request", 1)
    return out


def encode_plan(plan: Dict[str, Any], permute_axes: Optional[Dict[int, Tuple[int, ...]]] = None) -> EncodedPlan:
    steps_in: Sequence[Dict[str, Any]] = plan["steps"]
    n = len(steps_in)
    declared = _get(plan, "step_count")
    if declared is not None and int(declared) != n:
        raise KernelError("CUDA bridge: run_tensor_plan: step_count does not match steps", 1)
    steps = (_lib.PlanStep * max(n, 1))()
    ext: List[int] = []
    buffers: List[Tuple[int, Any]] = []
    for i, s in enumerate(steps_in):
        vid = int(_get(s, "value_id"))
        if vid != i:
            raise KernelError(f"CUDA bridge: run_tensor_plan: value_id {vid} at step {i} (must equal the step index)", 1)
        op = s["op"]
        if op not in _lib.OP_CODE:
            raise JitNotImplementedError(
                f"CUDA bridge: opcode {op!r} is not supported. Supported set: {sorted(_lib.OP_CODE)}. "
                "Fall back to bg.realize() (NumPy).")
        dtype = s["dtype"]
        if dtype not in _lib.DTYPE_CODE:
            raise KernelError(f"CUDA bridge: unknown dtype {dtype!r}", 1)
        shape = tuple(int(d) for d in s["shape"])
        if len(shape) > _lib.MAX_RANK:
            raise KernelError(f"CUDA bridge: rank {len(shape)} exceeds {_lib.MAX_RANK}", 2)
        ins = [int(x) for x in _get(s, "input_ids")]
        if len(ins) > _lib.MAX_STEP_INPUTS:
            raise KernelError(f"CUDA bridge: {op} with {len(ins)} inputs exceeds {_lib.MAX_STEP_INPUTS}", 2)
        st = steps[i]
        st.op = _lib.OP_CODE[op]
        st.dtype = _lib.DTYPE_CODE[dtype]
        st.rank = len(shape)
        st.n_inputs = len(ins)
        for d, v in enumerate(shape):
            st.shape[d] = v
        for d, v in enumerate(ins):
            st.input_ids[d] = v
        arg = s.get("arg")
        if op == "BUFFER":
            buffers.append((vid, arg))
        elif op == "CONST":
            value = arg["value"]
            st.farg[0] = float(value)
            if dtype.startswith("float") or dtype == "bfloat16":
                st.iarg[0] = 0
            else:
                st.iarg[0] = int(value)
        elif op == "CMP":
            st.iarg[0] = _lib.CMP_CODE[arg["op"]]
        elif op == "REDUCE":
            rop = arg["op"]
            if rop not in _lib.REDUCE_CODE:
                raise KernelError(f"CUDA bridge: REDUCE: unknown op {rop!r}", 1)
            in_rank = len(steps_in[ins[0]]["shape"])
            st.iarg[0] = _lib.REDUCE_CODE[rop]
            st.iarg[1] = normalize_axis_mask(arg.get("axis"), in_rank)
            st.iarg[2] = 1 if arg.get("keepdims") else 0
        elif op == "PERMUTE":
            axes = None
            if permute_axes and vid in permute_axes:
                axes = permute_axes[vid]
            elif isinstance(arg, dict) and "axes" in arg:
                axes = tuple(int(a) for a in arg["axes"])
            if axes is None:
                raise KernelError(f"CUDA bridge: PERMUTE value {vid} carries no axes", 1)
            for d, a in enumerate(axes):
                st.iarg[d] = a % max(len(axes), 1)
        elif op == "FUSED_SOFTMAX":
            rank = len(shape)
            st.iarg[0] = int(arg["axis"]) % max(rank, 1)
        elif op == "LAYER_NORM":
            st.iarg[0] = int(arg["rows"])
            st.iarg[1] = int(arg["cols"])
            st.farg[0] = float(arg.get("eps", 1e-5))
        elif op in ("INDEX", "SCATTER"):
            st.iarg[0] = int(arg["dim"])
        elif op in ("TRIL", "TRIU"):
            st.iarg[0] = int(arg["diagonal"])
        elif op in ("FLIP", "CONCAT"):
            st.iarg[0] = int(arg["axis"])
        elif op == "CUMSUM":
            st.iarg[0] = int(arg["axis"])
            st.iarg[1] = 1 if arg.get("reverse") else 0
        elif op == "SORT_INDICES":
            st.iarg[0] = int(arg["axis"])
            st.iarg[1] = 1 if arg.get("descending") else 0
        elif op == "TOPK_INDICES":
            st.iarg[0] = int(arg["axis"])
            st.iarg[1] = int(arg["k"])
            st.iarg[2] = 1 if arg.get("largest", True) else 0
            st.iarg[3] = 1 if arg.get("sorted", True) else 0
        elif op == "SLICE":
            src_shape = tuple(int(d) for d in steps_in[ins[0]]["shape"])
            slices = tuple(arg["slices"])
            if len(slices) > len(src_shape) or any(not isinstance(sl, slice) for sl in slices):
                raise JitNotImplementedError("CUDA bridge: SLICE takes one slice object per leading axis (no integers, "
                                             "ellipsis or new axes). Fall back to bg.realize() (NumPy).")
            slices = slices + (slice(None),) * (len(src_shape) - len(slices))
            for d, (sl, extent) in enumerate(zip(slices, src_shape)):
                start, stop, step = sl.indices(extent)
                if step < 1:
                    raise JitNotImplementedError("CUDA bridge: SLICE with a negative step is not supported. "
                                                 "Fall back to bg.realize() (NumPy).")
                length = max(0, (stop - start + step - 1) // step)
                if d >= len(shape) or shape[d] != length:
                    raise KernelError(f"CUDA bridge: SLICE: declared shape {shape} does not match the slices", 1)
                st.iarg[d] = (start if length else 0) + (step << 40)
        elif op == "CROSS_ENTROPY":
            mode = arg.get("target_mode", "indices")
            if mode not in ("indices", "probabilities"):
                raise KernelError(f"CUDA bridge: CROSS_ENTROPY: unknown target_mode {mode!r}", 1)
            has_weight = bool(arg.get("has_weight"))
            if len(ins) != (3 if has_weight else 2):
                raise KernelError("CUDA bridge: CROSS_ENTROPY: inputs are (logits, targets[, class weights])", 1)
            st.iarg[0] = {"none": 0, "mean": 1, "sum": 2}[arg["reduction"]]
            st.iarg[1] = int(arg["ignore_index"])
            st.iarg[2] = int(arg.get("batch_rank", 0))
            st.iarg[3] = (1 if mode == "probabilities" else 0) | (2 if has_weight else 0)
            st.farg[0] = float(arg.get("label_smoothing", 0.0) or 0.0)
        elif op == "ATTENTION_FORWARD":
            st.farg[0] = float(arg["scale"])
        elif op == "FUSED_ELEMENTWISE":
            st.ext_offset = len(ext)
            ops = arg["ops"]
            st.ext_count = len(ops)
            for opcode, lhs, rhs in ops:
                if opcode not in _lib.OP_CODE:
                    raise KernelError(f"CUDA bridge: FUSED_ELEMENTWISE: unknown inner opcode {opcode!r}", 1)
                unary = opcode in ("NEG", "EXP", "LOG")
                ext.extend((_lib.OP_CODE[opcode], int(lhs), _lib.REF_NONE if (rhs is None or unary) else int(rhs)))
        elif op == "WHERE":
            pass  # arg is None or the masked-fill contract id; semantics are the same select
    ext_arr = (C.c_int32 * max(len(ext), 1))(*ext) if ext else (C.c_int32 * 1)()
    root_id = int(_get(plan, "root_id"))
    if not (0 <= root_id < n):
        raise KernelError("CUDA bridge: run_tensor_plan: root_id out of range", 1)
    ep = EncodedPlan(steps, ext_arr, n, root_id, buffers,
                     tuple(int(d) for d in steps_in[root_id]["shape"]), steps_in[root_id]["dtype"])
    ep.plan.n_ext = len(ext)
    return ep
