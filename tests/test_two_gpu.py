"""GPU, two ranks over NCCL (skipped when fewer than two devices are visible): the device-side all-gather of row
shards and the column-split Linear give, on every rank, the bits one GPU computes for the whole problem.

Each rank is a child process with its own device and its own ``CudaBridge``; results come back as files."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _device_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from browsergrad_b200 import CudaBridge, configs, front, graph, sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    bridge = CudaBridge(rank)
    try:
        store = graph.BufferStore()
        # rows: 7 rows over 2 ranks (4 + 3: unequal blocks), softmax chain, gathered on the devices
        arrays = configs.chain_inputs(7, 37)
        local = sharded.shard_inputs(arrays, list("abcd"), world, rank)
        t = {k: graph.from_numpy(v, store) for k, v in local.items()}
        res = front.realize_cuda_resident(configs.chain_rowsoftmax(graph, t), bridge)
        h = sharded.gather_rows_device(bridge, sharded.resident_handle(res), res.shape, res.dtype, 7, device=rank)
        np.save(os.path.join(out_dir, f"rows_{rank}.npy"), bridge.materialize_array(h, (7, 37), res.dtype))
        bridge.release(h)
        # equal blocks of a larger array (the one-collective path)
        arrays = configs.chain_inputs(256, 512)
        local = sharded.shard_inputs(arrays, list("abcd"), world, rank)
        t = {k: graph.from_numpy(v, store) for k, v in local.items()}
        res = front.realize_cuda_resident(configs.chain_y(graph, t), bridge)
        h = sharded.gather_rows_device(bridge, sharded.resident_handle(res), res.shape, res.dtype, 256, device=rank)
        np.save(os.path.join(out_dir, f"y_{rank}.npy"), bridge.materialize_array(h, (256, 512), res.dtype))
        bridge.release(h)
        # a wide Linear split along its output columns
        lin = configs.linear_inputs(256, 512, 256)
        x = graph.from_numpy(lin["x"], store)
        out = sharded.column_split_linear(bridge, x, lin["w"], lin["bias"], device=rank)
        np.save(os.path.join(out_dir, f"lin_{rank}.npy"), front.materialize_resident(out))
        front.release_resident_leaves(bridge)
    finally:
        bridge.close()
        dist.destroy_process_group()


@pytest.mark.skipif(_device_count() < 2, reason="needs two GPUs")
def test_device_side_gather_and_column_split_match_one_gpu(tmp_path):
    import torch.multiprocessing as mp
    from browsergrad_b200 import CudaBridge, configs, graph, realize_cuda
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    bridge = CudaBridge(0)
    try:
        store = graph.BufferStore()
        t = {k: graph.from_numpy(v, store) for k, v in configs.chain_inputs(7, 37).items()}
        want_rows = realize_cuda(configs.chain_rowsoftmax(graph, t), bridge)
        t = {k: graph.from_numpy(v, store) for k, v in configs.chain_inputs(256, 512).items()}
        want_y = realize_cuda(configs.chain_y(graph, t), bridge)
        lin = configs.linear_inputs(256, 512, 256)
        tl = {k: graph.from_numpy(v, store) for k, v in lin.items()}
        want_lin = realize_cuda(graph.linear(tl["x"], tl["w"], tl["bias"]), bridge)
    finally:
        bridge.close()
    for r in range(world):
        assert np.load(tmp_path / f"rows_{r}.npy").tobytes() == want_rows.tobytes()
        assert np.load(tmp_path / f"y_{r}.npy").tobytes() == want_y.tobytes()
        assert np.load(tmp_path / f"lin_{r}.npy").tobytes() == want_lin.tobytes()
