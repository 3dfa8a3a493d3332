"""``realize_cuda``: the realizer front for the CUDA bridge.

The reference has two GPU entry points and both refuse most forward graphs on the Python side:
``bg.realize_webgpu`` skips fusion and whitelists 16 opcodes (packages/browsergrad-jit/src/python/
_realize_webgpu.py:347-364, :374-473) and ``bg.realize_tensor_plan_webgpu`` raises on WHERE,
CROSS_ENTROPY, INDEX, ... while building its plan (_gpu_plan.py:350-591).  This front keeps their
protocol -- same pass order as ``_realize.realize`` (cast pass -> fuse -> toposort,
_realize.py:1890-1902), same plan dictionary (``GpuExecutionPlan.summary()``, _gpu_plan.py:176-209),
same input binding (``{value_id, handle}`` | ``{value_id, data}``, _realize_webgpu.py:490-519), one
``bridge.run_tensor_plan`` call per realization -- without the refusals.  It accepts the
reference's ``TensorProxy`` / ``UOp`` and this package's ``graph.Tensor`` / ``graph.Node``.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from . import _lib, graph, passes
from .bridge import CudaBridge
from .errors import BufferTableError, JitNotImplementedError, RealizationError

_DTYPE_BYTES = _lib.DTYPE_SIZE


class DeviceBufferTable:
    """``buffer id -> device handle`` with the methods of ``GpuBufferTable``
    (packages/browsergrad-jit/src/python/_gpu_buffer_table.py:35-131): ``register`` / ``get`` / ``has`` / ``detach`` /
    ``replace`` / ``release`` / ``release_all``, plus ``upload``, which is idempotent per id.  Handles live until they
    are released or detached."""

    def __init__(self, bridge: CudaBridge) -> None:
        self.bridge = bridge
        self._handles: Dict[str, int] = {}
        self._uploads = 0

    def get(self, buffer_id: str) -> Optional[int]:
        return self._handles.get(buffer_id)

    def has(self, buffer_id: str) -> bool:
        return buffer_id in self._handles

    def upload(self, buffer_id: str, array: np.ndarray) -> int:
        h = self._handles.get(buffer_id)
        if h is None:
            h = self.bridge.upload(array, array.shape, array.dtype.name)
            self._handles[buffer_id] = h
            self._uploads += 1
        return h

    def register(self, buffer_id: str, handle: int) -> None:
        """Bind ``buffer_id`` to ``handle``; an id that is already bound raises (_gpu_buffer_table.py:63-74:
        registering twice would hide a double upload).  ``replace`` rebinds."""
        if buffer_id in self._handles:
            raise BufferTableError(f"DeviceBufferTable: buffer_id {buffer_id!r} is already registered with a handle; "
                                   "consult get() before uploading again, or use replace()")
        self._handles[buffer_id] = handle

    def detach(self, buffer_id: str) -> int:
        """Remove a handle without releasing it: the caller owns it from here (_gpu_buffer_table.py:82-90)."""
        if buffer_id not in self._handles:
            raise BufferTableError(f"DeviceBufferTable: cannot detach unknown buffer_id {buffer_id!r}")
        return self._handles.pop(buffer_id)

    def replace(self, buffer_id: str, handle: int) -> None:
        """Bind ``buffer_id`` to ``handle`` and release the handle it had (_gpu_buffer_table.py:92-99): the next
        realization that names the id reads the new buffer, e.g. a key / value cache that grew."""
        old = self._handles.pop(buffer_id, None)
        if old is not None and old != handle:
            self.bridge.release(old)
        self._handles[buffer_id] = handle

    def release(self, buffer_id: str) -> None:
        h = self._handles.pop(buffer_id, None)
        if h is not None:
            self.bridge.release(h)

    def release_all(self) -> None:
        for h in self._handles.values():
            self.bridge.release(h)
        self._handles.clear()

    def stats(self) -> Dict[str, int]:
        return {"resident": len(self._handles), "uploads": self._uploads}


_REGISTERED: Optional[CudaBridge] = None
_REGISTERED_TABLE: Optional[DeviceBufferTable] = None


def register_cuda_bridge(bridge: Optional[CudaBridge]) -> None:
    """Counterpart of ``register_webgpu_bridge`` (_realize_webgpu.py:628-636) for this front."""
    global _REGISTERED, _REGISTERED_TABLE
    if _REGISTERED_TABLE is not None and bridge is not _REGISTERED:
        _REGISTERED_TABLE.release_all()
    _REGISTERED = bridge
    _REGISTERED_TABLE = DeviceBufferTable(bridge) if bridge is not None else None


def unregister_cuda_bridge() -> None:
    register_cuda_bridge(None)


def registered() -> Tuple[Optional[CudaBridge], Optional[DeviceBufferTable]]:
    return _REGISTERED, _REGISTERED_TABLE


def _numel(shape: Tuple[int, ...]) -> int:
    n = 1
    for d in shape:
        n *= max(int(d), 1)
    return n


def build_plan(root: Any) -> Dict[str, Any]:
    """The plan dictionary of ``build_gpu_execution_plan(...).summary()`` for an already
    prepared graph (_gpu_plan.py:595-638), with liveness computed in one sweep."""
    order = graph.toposort(root)
    index = {id(n): i for i, n in enumerate(order)}
    last = {id(n): i for i, n in enumerate(order)}
    for i, n in enumerate(order):
        for inp in n.inputs:
            last[id(inp)] = i
    steps: List[Dict[str, Any]] = []
    buffers: List[Dict[str, Any]] = []
    delta = [0] * (len(order) + 1)
    for i, n in enumerate(order):
        shape = [int(d) for d in n.shape]
        steps.append({"step": i, "value_id": i, "op": n.op, "input_ids": [index[id(x)] for x in n.inputs],
                      "shape": shape, "dtype": n.dtype, "arg": n.arg})
        nbytes = _numel(tuple(shape)) * _DTYPE_BYTES.get(n.dtype, 4)
        buffers.append({"value_id": i, "op": n.op, "shape": shape, "dtype": n.dtype, "bytes": nbytes,
                        "first_step": i, "last_step": last[id(n)], "materialize": n is root})
        delta[i] += nbytes
        delta[last[id(n)] + 1] -= nbytes
    peak = live = 0
    for d in delta[:-1]:
        live += d
        peak = max(peak, live)
    return {"step_count": len(steps), "root_id": index[id(root)], "materialization_boundary": "root",
            "peak_live_bytes": peak, "has_custom_ops": False, "ops": [s["op"] for s in steps],
            "steps": steps, "buffers": buffers}


def _unwrap(tensor: Any) -> Tuple[Any, Any]:
    """Return (root node, buffer table) for a Tensor / TensorProxy / bare node."""
    node = getattr(tensor, "_uop", tensor)
    store = getattr(tensor, "_store", None)
    if store is None and hasattr(tensor, "_get_session"):
        store = tensor._get_session().buffer_table
    if store is None:
        store = graph.default_store()
    return node, store


_PLAN_MEMO: Dict[Tuple[int, bool], Tuple[Any, Any, Dict[str, Any]]] = {}


def plan_for(node: Any, fusion: bool = True) -> Tuple[Any, Dict[str, Any]]:
    """Prepared root and plan for a graph, memoised on the root object so that repeated
    realizations of one graph skip the passes (the reference memoises whole traces,
    packages/browsergrad-jit/src/python/_trace_cache.py:183-265)."""
    key = (id(node), bool(fusion))
    hit = _PLAN_MEMO.get(key)
    if hit is not None and hit[0] is node:
        return hit[1], hit[2]
    prepared = passes.lower_composites(passes.prepare(node, fusion=fusion))
    plan = build_plan(prepared)
    for s in plan["steps"]:
        if s["op"] not in _lib.OP_CODE:
            raise JitNotImplementedError(
                f"CUDA realizer: opcode {s['op']!r} is not supported. Supported set: {sorted(_lib.OP_CODE)}. "
                "Fall back to bg.realize() (NumPy).")
    if len(_PLAN_MEMO) > 128:
        _PLAN_MEMO.clear()
    _PLAN_MEMO[key] = (node, prepared, plan)
    return prepared, plan


def _bind_inputs(plan: Dict[str, Any], store: Any, table: Optional[DeviceBufferTable], resident_leaves: bool) -> List[Dict[str, Any]]:
    inputs: List[Dict[str, Any]] = []
    for step in plan["steps"]:
        if step["op"] != "BUFFER":
            continue
        bid = step["arg"]
        handle = table.get(bid) if table is not None else None
        if handle is None and resident_leaves and table is not None:
            handle = table.upload(bid, store.get(bid))
        if handle is not None:
            inputs.append({"value_id": step["value_id"], "handle": handle})
            continue
        arr = store.get(bid)
        if arr.dtype.name != step["dtype"]:
            raise RealizationError(f"CUDA tensor plan: buffer {step['value_id']} dtype mismatch: "
                                   f"plan={step['dtype']} table={arr.dtype.name}")
        inputs.append({"value_id": step["value_id"], "data": arr})
    return inputs


def realize_cuda(tensor: Any, bridge: Optional[CudaBridge] = None, *, resident_leaves: bool = False,
                 fusion: bool = True, out: Optional[np.ndarray] = None) -> np.ndarray:
    """Realize ``tensor`` on the GPU and return the ndarray ``tensor.numpy()`` would return.

    With ``resident_leaves`` leaf buffers are uploaded once and kept on the device across calls
    (what ``GpuBufferTable.upload`` does for ``bg.realize_webgpu``); otherwise each call uploads
    its leaves and frees them, as ``realize_tensor_plan_webgpu`` does for unregistered buffers.
    ``out`` optionally names the destination array (e.g. page-locked memory).
    """
    table = None
    if bridge is None:
        bridge, table = registered()
        if bridge is None:
            raise RealizationError("CUDA realizer: no bridge registered; call register_cuda_bridge(CudaBridge())")
    elif _REGISTERED is bridge:
        table = _REGISTERED_TABLE
    elif resident_leaves:
        table = getattr(bridge, "_front_table", None)
        if table is None:
            table = DeviceBufferTable(bridge)
            bridge._front_table = table
    node, store = _unwrap(tensor)
    prepared, plan = plan_for(node, fusion)
    inputs = _bind_inputs(plan, store, table, resident_leaves)
    return bridge.run_tensor_plan_array(plan, inputs, prepared.dtype, out=out)


def resident_table(bridge: CudaBridge) -> Optional[DeviceBufferTable]:
    """The table of leaves ``realize_cuda(..., resident_leaves=True)`` keeps on the device for ``bridge``."""
    return _REGISTERED_TABLE if _REGISTERED is bridge else getattr(bridge, "_front_table", None)


def release_resident_leaves(bridge: CudaBridge) -> None:
    """Drop the leaves ``realize_cuda(..., resident_leaves=True)`` kept on the device for ``bridge``."""
    table = resident_table(bridge)
    if table is not None:
        table.release_all()


def realize_cuda_resident(tensor: Any, bridge: Optional[CudaBridge] = None) -> "graph.Tensor":
    """Realize and keep the root on the device: returns a leaf ``graph.Tensor`` whose buffer id is
    registered with the bridge's device table (``realize_tensor_plan_webgpu_resident``,
    _realize_webgpu.py:557-596).  Use ``materialize_resident`` to fetch it."""
    if bridge is None:
        bridge, table = registered()
        if bridge is None:
            raise RealizationError("CUDA realizer: no bridge registered; call register_cuda_bridge(CudaBridge())")
    else:
        table = _REGISTERED_TABLE if _REGISTERED is bridge else getattr(bridge, "_front_table", None)
        if table is None:
            table = DeviceBufferTable(bridge)
            bridge._front_table = table
    node, store = _unwrap(tensor)
    prepared, plan = plan_for(node)
    inputs = _bind_inputs(plan, store, table, True)
    handle = bridge.run_tensor_plan_resident(plan, inputs, prepared.dtype)
    bid = f"resident_{handle}"
    table.register(bid, handle)
    buf = graph.Node("BUFFER", (), tuple(prepared.shape), prepared.dtype, bid)
    leaf = graph.Tensor(graph.Node("LOAD", (buf,), buf.shape, buf.dtype, None), _ResidentStore(store, table, bridge))
    return leaf


class _ResidentStore:
    """Buffer table view that fetches device-resident buffers on demand."""

    def __init__(self, base: Any, table: DeviceBufferTable, bridge: CudaBridge) -> None:
        self._base, self._table, self._bridge = base, table, bridge
        self._meta: Dict[str, Tuple[Tuple[int, ...], str]] = {}

    def new_buffer(self, array: np.ndarray) -> str:
        return self._base.new_buffer(array)

    def is_materialized(self, bid: str) -> bool:
        return self._table.get(bid) is None

    def get(self, bid: str) -> np.ndarray:
        h = self._table.get(bid)
        if h is None or not bid.startswith("resident_"):
            return self._base.get(bid)
        raise RealizationError(f"buffer {bid!r} is device-resident; use materialize_resident()")


def materialize_resident(tensor: "graph.Tensor") -> np.ndarray:
    store = tensor._store
    buf = tensor._uop.inputs[0] if tensor._uop.op == "LOAD" else tensor._uop
    h = store._table.get(buf.arg)
    if h is None:
        raise RealizationError(f"CUDA buffer {buf.arg!r} is not registered")
    return store._bridge.materialize_array(h, buf.shape, buf.dtype)
