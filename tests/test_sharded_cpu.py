"""CPU, world_size 2 over gloo: the row-sharding host logic (partition, all-gather of unequal
blocks, mean combine) with the CPU oracle standing in for the device realizer."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from browsergrad_b200 import configs, graph, passes, sharded
    from oracle import port as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        store = graph.BufferStore()
        realize = lambda t: oracle.realize(passes.prepare(t._uop), store)
        make = lambda a: graph.from_numpy(a, store)
        # rows: 7 rows over 2 ranks (4 + 3), softmax chain
        arrays = configs.chain_inputs(7, 37)
        got = sharded.realize_sharded(lambda t: configs.chain_rowsoftmax(graph, t), arrays, list("abcd"), realize, make)
        np.save(os.path.join(out_dir, f"rows_{rank}.npy"), got)
        # mean cross entropy over a sharded batch, weights replicated
        mlp = configs.mlp_inputs(batch=10)
        loss = sharded.realize_sharded(lambda t: configs.mlp_loss(graph, t), mlp, ["x", "y"], realize, make, reduce="mean")
        np.save(os.path.join(out_dir, f"loss_{rank}.npy"), loss)
        # bool output travels as bytes
        got_b = sharded.realize_sharded(lambda t: t["a"] > t["b"], arrays, list("abcd"), realize, make)
        np.save(os.path.join(out_dir, f"bool_{rank}.npy"), got_b)
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_everything():
    from browsergrad_b200 import sharded
    for n in (0, 1, 7, 8, 64, 1001):
        for world in (1, 2, 3, 8):
            spans = [sharded.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_two_rank_gloo_matches_single_process(tmp_path):
    sys.path.insert(0, ROOT)
    from browsergrad_b200 import configs, graph, passes
    from oracle import port as oracle
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    store = graph.BufferStore()
    arrays = configs.chain_inputs(7, 37)
    t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
    want = oracle.realize(passes.prepare(configs.chain_rowsoftmax(graph, t)._uop), store)
    want_b = oracle.realize(passes.prepare((t["a"] > t["b"])._uop), store)
    mlp = configs.mlp_inputs(batch=10)
    tm = {k: graph.from_numpy(v, store) for k, v in mlp.items()}
    want_loss = oracle.realize(passes.prepare(configs.mlp_loss(graph, tm)._uop), store)
    for r in range(world):
        got = np.load(tmp_path / f"rows_{r}.npy")
        assert got.tobytes() == want.tobytes()      # row-wise ops shard bit-exactly
        assert np.load(tmp_path / f"bool_{r}.npy").tobytes() == want_b.tobytes()
        loss = np.load(tmp_path / f"loss_{r}.npy")
        assert abs(float(loss) - float(want_loss)) <= 1e-5 * abs(float(want_loss))
