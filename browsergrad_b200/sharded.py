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


def combine_mean(local_mean: np.ndarray, local_count: int, group: Any = None, device: Optional[str] = None) -> np.ndarray:
    """Global mean from per-rank means over ``local_count`` valid positions (one all-reduce of
    (sum, count)).  The summation order differs from a single-device reduction: tolerance, not bit-exact."""
    import torch
    dist = _dist()
    pair = torch.tensor([float(local_mean) * local_count, float(local_count)], dtype=torch.float64)
    if device is not None:
        pair = pair.to(device)
    dist.all_reduce(pair, op=dist.ReduceOp.SUM, group=group)
    pair = pair.cpu()
    return np.asarray(pair[0].item() / pair[1].item(), dtype=np.asarray(local_mean).dtype)


def realize_sharded(build: Callable[[Dict[str, Any]], Any], arrays: Dict[str, np.ndarray], sharded_keys: Sequence[str],
                    realize: Callable[[Any], np.ndarray], make_tensor: Callable[[np.ndarray], Any], *,
                    gather: bool = True, reduce: str = "rows", group: Any = None,
                    device: Optional[str] = None) -> np.ndarray:
    """Run ``build`` on this rank's shard and combine the results.

    ``realize`` maps a graph tensor to an ndarray (``realize_cuda`` in production), ``make_tensor``
    wraps an ndarray as a leaf.  ``reduce`` = "rows" concatenates row blocks (``gather=False`` keeps
    the local block), "mean" combines a mean-reduced scalar.
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
        return combine_mean(out, hi - lo, group, device)
    if not gather:
        return out
    return gather_rows(out, total, group, device)
