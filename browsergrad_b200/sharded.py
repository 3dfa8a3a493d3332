"""Batch-sharded realization across the GPUs of one node (one process per GPU).

Every forward configuration is independent along its leading batch / row axis, so a plan shards
without any exchange inside the forward: each rank realizes the same graph on its contiguous block
of the batch-carrying inputs while weights, biases, masks and tables are replicated.  The only
collective is the optional all-gather of the root output over ``torch.distributed`` (NCCL over
NVLink for CUDA tensors; gloo in the CPU tests).  A mean-reduced scalar root (cross entropy) is
combined from per-rank (sum, count) pairs with one all-reduce.

The reference has no counterpart: its only "collective" is a single-device simulation
(packages/browsergrad-kernels/src/semantic_host_graph_wgsl.ts:143-160).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np


def shard_bounds(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block [start, stop) of ``n`` rows for ``rank``; the first ``n % world`` ranks get
    one extra row."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_inputs(arrays: Dict[str, np.ndarray], sharded_keys: Iterable[str], world: int, rank: int,
                 axis: int = 0) -> Dict[str, np.ndarray]:
    """Slice the batch-carrying arrays for this rank; everything else is replicated."""
    keys = set(sharded_keys)
    n = None
    for k in keys:
        if n is None:
            n = arrays[k].shape[axis]
        elif arrays[k].shape[axis] != n:
            raise ValueError(f"sharded inputs disagree on the batch extent: {k}")
    out: Dict[str, np.ndarray] = {}
    for k, v in arrays.items():
        if k in keys:
            lo, hi = shard_bounds(n, world, rank)
            index = [slice(None)] * v.ndim
            index[axis] = slice(lo, hi)
            out[k] = np.ascontiguousarray(v[tuple(index)])
        else:
            out[k] = v
    return out


def _dist() -> Any:
    import torch.distributed as dist
    return dist


def gather_rows(local: np.ndarray, total_rows: int, group: Any = None, device: Optional[str] = None) -> np.ndarray:
    """All-gather per-rank row blocks (possibly of unequal height) into the full array on every rank."""
    import torch
    dist = _dist()
    world = dist.get_world_size(group)
    heights = [shard_bounds(total_rows, world, r) for r in range(world)]
    max_h = max(hi - lo for lo, hi in heights)
    pad_shape = (max_h,) + tuple(local.shape[1:])
    dtype_view = local.dtype
    buf = np.zeros(pad_shape, dtype=dtype_view)
    buf[: local.shape[0]] = local
    # bool / float16 etc. travel as raw bytes so that every backend accepts them
    raw = torch.from_numpy(buf.view(np.uint8).reshape(-1) if buf.size else np.zeros((0,), np.uint8))
    if device is not None:
        raw = raw.to(device)
    parts = [torch.empty_like(raw) for _ in range(world)]
    dist.all_gather(parts, raw, group=group)
    rows: List[np.ndarray] = []
    for r, (lo, hi) in enumerate(heights):
        arr = parts[r].cpu().numpy().view(dtype_view).reshape(pad_shape)
        rows.append(arr[: hi - lo])
    return np.concatenate(rows, axis=0) if rows else buf[:0]


class _DeviceView:
    """Exposes the device buffer behind a bridge handle through ``__cuda_array_interface__`` so that
    ``torch.as_tensor`` wraps it without a copy (raw bytes; the caller reinterprets)."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3}


def device_bytes(bridge: Any, handle: int, nbytes: int, device: int) -> Any:
    """The bytes behind ``handle`` as a uint8 CUDA tensor sharing the bridge's memory (no copy).  The tensor is only
    valid while the handle lives, and work on it must be ordered on the bridge's stream."""
    import torch
    return torch.as_tensor(_DeviceView(bridge.device_pointer(handle), nbytes), device=torch.device("cuda", device))


def gather_rows_device(bridge: Any, handle: int, local_shape: Sequence[int], dtype: str, total_rows: int, *,
                       group: Any = None, device: int = 0) -> int:
    """All-gather the row blocks the ranks hold on their devices into the full array on every rank's device and
    return a bridge handle to it: ``torch.distributed.all_gather_into_tensor`` (NCCL over NVLink) reads the bridge's
    own buffer and writes straight into a buffer the bridge allocated (``bridge.alloc``) -- nothing passes through
    host memory, and no kernel is handed a peer's pointer (NCCL moves the bytes).  Blocks of unequal height are padded
    to the tallest inside the exchange.  The collective is ordered on the bridge's stream."""
    import torch
    from . import _lib
    dist = _dist()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    itemsize = _lib.DTYPE_SIZE[dtype]
    row_bytes = itemsize
    for d in local_shape[1:]:
        row_bytes *= int(d)
    spans = [shard_bounds(total_rows, world, r) for r in range(world)]
    heights = [hi - lo for lo, hi in spans]
    if int(local_shape[0]) != heights[rank]:
        raise ValueError(f"gather_rows_device: rank {rank} holds {local_shape[0]} rows, its share of {total_rows} is {heights[rank]}")
    max_h = max(heights)
    dev = torch.device("cuda", device)
    stream = torch.cuda.ExternalStream(bridge.stream(), device=dev)
    out_shape = (total_rows,) + tuple(int(d) for d in local_shape[1:])
    out = bridge.alloc(out_shape, dtype)
    try:
        with torch.cuda.stream(stream):
            mine = device_bytes(bridge, handle, heights[rank] * row_bytes, device) if heights[rank] * row_bytes else \
                torch.empty(0, dtype=torch.uint8, device=dev)
            full = device_bytes(bridge, out, total_rows * row_bytes, device) if total_rows * row_bytes else \
                torch.empty(0, dtype=torch.uint8, device=dev)
            if min(heights) == max_h:
                dist.all_gather_into_tensor(full, mine, group=group)
            else:
                padded = torch.zeros(max_h * row_bytes, dtype=torch.uint8, device=dev)
                padded[: mine.numel()] = mine
                parts = torch.empty(world * max_h * row_bytes, dtype=torch.uint8, device=dev)
                dist.all_gather_into_tensor(parts, padded, group=group)
                for r, (lo, hi) in enumerate(spans):
                    full[lo * row_bytes: hi * row_bytes] = parts[r * max_h * row_bytes: r * max_h * row_bytes + (hi - lo) * row_bytes]
                # torch frees the temporaries once this returns; they were used on the bridge's stream
                padded.record_stream(stream)
                parts.record_stream(stream)
    except BaseException:
        bridge.release(out)
        raise
    return out


def resident_handle(tensor: Any) -> int:
    """Bridge handle behind a tensor returned by ``front.realize_cuda_resident``."""
    buf = tensor._uop.inputs[0] if tensor._uop.op == "LOAD" else tensor._uop
    h = tensor._store._table.get(buf.arg)
    if h is None:
        raise ValueError(f"buffer {buf.arg!r} is not resident on the device")
    return h


def weight_block(weight: np.ndarray, store: Any, group: Any = None) -> Any:
    """This rank's block of ``N / world`` rows of ``weight`` [N, ...] as a graph leaf of ``store``.  Made once and
    passed to ``column_split_linear`` call after call, it is uploaded once and then stays in this rank's HBM."""
    from . import graph
    dist = _dist()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_total = int(weight.shape[0])
    if n_total % world:
        raise ValueError(f"weight_block: {n_total} rows do not divide over {world} ranks")
    n_r = n_total // world
    return graph.from_numpy(np.ascontiguousarray(weight[rank * n_r:(rank + 1) * n_r]), store)


def column_split_linear(bridge: Any, x: Any, weight: Any, bias: Any, *, group: Any = None, device: int = 0) -> Any:
    """``x @ weight.T + bias`` for a very wide ``weight`` [N, K] (an LM head), split along N over the ranks: every rank
    multiplies the same ``x`` [M, K] (a graph tensor; device-resident or not) by its own block of ``N / world`` rows of
    ``weight`` held in its own HBM, the [M, N / world] blocks are all-gathered on the devices (NCCL; no kernel reads a
    peer's memory) and one strided copy per rank lays them side by side.  ``weight`` / ``bias`` are either the whole
    arrays (this rank's block is cut out and uploaded by this call) or the leaves ``weight_block`` made from them (the
    block is uploaded once and reused).  Returns a device-resident graph tensor [M, N] on every rank
    (``front.materialize_resident`` fetches it).  The per-element products and their order are those of the unsplit
    Linear, so the result is bit-identical to it."""
    from . import front, graph
    dist = _dist()
    world = dist.get_world_size(group)
    m = int(x.shape[0])
    store = x._store
    w_r = weight if isinstance(weight, graph.Tensor) else weight_block(weight, store, group)
    b_r = bias if bias is None or isinstance(bias, graph.Tensor) else weight_block(bias, store, group)
    n_r = int(w_r.shape[0])
    n_total = n_r * world
    local = front.realize_cuda_resident(graph.linear(x, w_r, b_r), bridge)          # [M, n_r] on this rank's device
    h_local = resident_handle(local)
    # all-gather as row blocks of a [world * M, n_r] array, then [world, M, n_r] -> [M, world, n_r] = [M, N]
    h_all = gather_rows_device(bridge, h_local, (m, n_r), local.dtype, world * m, group=group, device=device)
    local._store._table.release(local._uop.inputs[0].arg)
    table = local._store._table
    bid = f"resident_{h_all}"
    table.register(bid, h_all)
    buf = graph.Node("BUFFER", (), (world, m, n_r), local.dtype, bid)
    blocks = graph.Tensor(graph.Node("LOAD", (buf,), buf.shape, buf.dtype, None), local._store)
    out = front.realize_cuda_resident(blocks.permute(1, 0, 2).reshape(m, n_total), bridge)
    table.release(bid)
    return out


def combine_mean(local_mean: np.ndarray, local_count: int, group: Any = None, device: Optional[str] = None) -> np.ndarray:
    """Global mean from per-rank means over ``local_count`` contributing positions (one all-reduce of
    (sum, count)).  A rank with no contributing position (its local mean is 0/0 = NaN) adds (0, 0); the
    result is NaN only when no rank contributes, as a single-device mean over nothing is.  The summation
    order differs from a single-device reduction: tolerance, not bit-exact."""
    import torch
    dist = _dist()
    local_sum = float(local_mean) * local_count if local_count > 0 else 0.0
    pair = torch.tensor([local_sum, float(local_count)], dtype=torch.float64)
    if device is not None:
        pair = pair.to(device)
    dist.all_reduce(pair, op=dist.ReduceOp.SUM, group=group)
    pair = pair.cpu()
    total, count = pair[0].item(), pair[1].item()
    return np.asarray(total / count if count > 0 else float("nan"), dtype=np.asarray(local_mean).dtype)


def realize_sharded(build: Callable[[Dict[str, Any]], Any], arrays: Dict[str, np.ndarray], sharded_keys: Sequence[str],
                    realize: Callable[[Any], np.ndarray], make_tensor: Callable[[np.ndarray], Any], *,
                    gather: bool = True, reduce: str = "rows", group: Any = None,
                    device: Optional[str] = None,
                    valid_count: Optional[Callable[[Dict[str, np.ndarray]], int]] = None) -> np.ndarray:
    """Run ``build`` on this rank's shard and combine the results.

    ``realize`` maps a graph tensor to an ndarray (``realize_cuda`` in production), ``make_tensor``
    wraps an ndarray as a leaf.  ``reduce`` = "rows" concatenates row blocks (``gather=False`` keeps
    the local block), "mean" combines a mean-reduced scalar from per-rank (sum, count) pairs.  The count
    is what the local mean divided by: ``valid_count(local_arrays)`` when given -- for cross entropy the
    number of targets that differ from ``ignore_index`` (packages/browsergrad-jit/src/python/
    _framework_contracts.py:3725-3753 divides by exactly that) -- else the shard's row count.
    """
    dist = _dist()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    keys = list(sharded_keys)
    total = arrays[keys[0]].shape[0]
    local = shard_inputs(arrays, keys, world, rank)
    tensors = {k: make_tensor(v) for k, v in local.items()}
    out = realize(build(tensors))
    if world == 1:
        return out
    if reduce == "mean":
        lo, hi = shard_bounds(total, world, rank)
        count = int(valid_count(local)) if valid_count is not None else hi - lo
        return combine_mean(out, count, group, device)
    if not gather:
        return out
    return gather_rows(out, total, group, device)


class RowPipeline:
    """Streams one row-independent realization through a single GPU in row chunks so that the
    host->device copy of chunk i+1, the kernels of chunk i and the device->host copy of chunk i-1
    overlap.  PCIe is full duplex, and a bridge call is synchronous, so the overlap comes from
    running the chunks on ``lanes`` independent bridges (one CUDA stream each), one host thread per
    lane; ctypes releases the GIL for the duration of every C call.

    The premise is the one row sharding across GPUs rests on: every root is independent along the
    leading axis of the ``sharded_keys`` inputs.  ``build(tensors)`` returns a tensor or a dict of
    named tensors; every root's leading axis must be the row axis.  The chunk graphs are built once;
    ``run`` may be called repeatedly (the host arrays are read again on every call).

    ``realize(tensor, lane, out)`` realizes into ``out`` (a row block of the caller's array) and
    ``release(lane, row_tensors)`` drops the chunk's row-carrying leaves from the lane's device
    table (replicated leaves stay resident on every lane until the caller drops them); the CUDA
    front end's ``realize_cuda(..., resident_leaves=True, out=...)`` and its device buffer table are
    the production pair (see ``cuda_row_pipeline``).  The reference has no counterpart.
    """

    def __init__(self, build: Callable[[Dict[str, Any]], Any], arrays: Dict[str, np.ndarray], sharded_keys: Sequence[str],
                 make_tensor: Callable[[np.ndarray], Any], realize: Callable[[Any, int, np.ndarray], Any],
                 release: Callable[[int, Dict[str, Any]], None], *, lanes: int = 2, n_chunks: int = 8) -> None:
        keys = list(sharded_keys)
        if not keys:
            raise ValueError("RowPipeline: no row-carrying inputs named")
        self.total = int(arrays[keys[0]].shape[0])
        for k in keys:
            if arrays[k].shape[0] != self.total:
                raise ValueError(f"row-carrying inputs disagree on the row count: {k}")
        self.lanes = max(1, int(lanes))
        self.n_chunks = max(1, min(int(n_chunks), self.total)) if self.total else 1
        self._realize, self._release = realize, release
        self.chunks: List[Tuple[int, int, Dict[str, Any], Dict[str, Any]]] = []
        replicated = {k: make_tensor(v) for k, v in arrays.items() if k not in keys}
        for j in range(self.n_chunks):
            lo, hi = shard_bounds(self.total, self.n_chunks, j)
            tensors = dict(replicated)
            for k in keys:
                tensors[k] = make_tensor(arrays[k][lo:hi])     # a view: page-locked memory stays page-locked
            roots = build(tensors)
            if not isinstance(roots, dict):
                roots = {"out": roots}
            self.chunks.append((lo, hi, roots, {k: tensors[k] for k in keys}))

    def output_shapes(self) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """Full-size shape and dtype of every root (rows of all chunks stacked)."""
        roots = self.chunks[0][2]
        return {name: ((self.total,) + tuple(t.shape[1:]), str(t.dtype)) for name, t in roots.items()}

    def _lane(self, lane: int, outs: Dict[str, np.ndarray], errors: List[BaseException]) -> None:
        try:
            for j in range(lane, self.n_chunks, self.lanes):
                lo, hi, roots, row_tensors = self.chunks[j]
                try:
                    for name, root in roots.items():
                        self._realize(root, lane, outs[name][lo:hi])
                finally:
                    self._release(lane, row_tensors)
        except BaseException as exc:   # re-raised on the caller's thread
            errors.append(exc)

    def run(self, outs: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        import threading
        for name, (shape, _) in self.output_shapes().items():
            if name not in outs or tuple(outs[name].shape) != shape:
                raise ValueError(f"RowPipeline: output {name!r} must have shape {shape}")
        errors: List[BaseException] = []
        threads = [threading.Thread(target=self._lane, args=(lane, outs, errors)) for lane in range(1, self.lanes)]
        for th in threads:
            th.start()
        self._lane(0, outs, errors)
        for th in threads:
            th.join()
        if errors:
            raise errors[0]
        return outs


def cuda_row_pipeline(build: Callable[[Dict[str, Any]], Any], arrays: Dict[str, np.ndarray], sharded_keys: Sequence[str],
                      bridges: Sequence[Any], *, n_chunks: int = 8, store: Any = None) -> RowPipeline:
    """``RowPipeline`` over ``bridges`` (one lane each, all on the same device) through ``realize_cuda``."""
    from . import front, graph
    st = store if store is not None else graph.BufferStore()

    def realize(tensor: Any, lane: int, out: np.ndarray) -> Any:
        return front.realize_cuda(tensor, bridges[lane], resident_leaves=True, out=out)

    def release(lane: int, row_tensors: Dict[str, Any]) -> None:
        table = front.resident_table(bridges[lane])
        if table is not None:
            for t in row_tensors.values():
                table.release(t._uop.inputs[0].arg)     # LOAD(BUFFER id)

    return RowPipeline(build, arrays, sharded_keys, lambda a: graph.from_numpy(a, st), realize, release,
                       lanes=len(bridges), n_chunks=n_chunks)
