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
        # the same with ignored targets: rank 1's shard (rows 5..9) is all ignore_index, rank 0 holds two of them
        ign = configs.mlp_inputs(batch=10)
        ign["y"] = ign["y"].copy()
        ign["y"][[1, 3, 5, 6, 7, 8, 9]] = -100
        loss_ign = sharded.realize_sharded(lambda t: configs.mlp_loss(graph, t), ign, ["x", "y"], realize, make, reduce="mean",
                                           valid_count=lambda local: int((local["y"] != -100).sum()))
        np.save(os.path.join(out_dir, f"loss_ign_{rank}.npy"), loss_ign)
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
    ign = configs.mlp_inputs(batch=10)
    ign["y"] = ign["y"].copy()
    ign["y"][[1, 3, 5, 6, 7, 8, 9]] = -100
    ti = {k: graph.from_numpy(v, store) for k, v in ign.items()}
    want_ign = oracle.realize(passes.prepare(configs.mlp_loss(graph, ti)._uop), store)
    assert np.isfinite(want_ign)
    for r in range(world):
        loss_ign = np.load(tmp_path / f"loss_ign_{r}.npy")
        assert abs(float(loss_ign) - float(want_ign)) <= 1e-5 * abs(float(want_ign)), (loss_ign, want_ign)
        got = np.load(tmp_path / f"rows_{r}.npy")
        assert got.tobytes() == want.tobytes()      # row-wise ops shard bit-exactly
        assert np.load(tmp_path / f"bool_{r}.npy").tobytes() == want_b.tobytes()
        loss = np.load(tmp_path / f"loss_{r}.npy")
        assert abs(float(loss) - float(want_loss)) <= 1e-5 * abs(float(want_loss))


def test_row_pipeline_matches_unchunked_realization():
    """Chunked, multi-lane streaming of a row-independent realization gives the same rows as one
    realization of the whole input (host logic only; the oracle stands in for the device)."""
    from browsergrad_b200 import configs, graph, passes
    from browsergrad_b200.sharded import RowPipeline
    from oracle import port

    arrays = configs.chain_inputs(37, 64)
    store = graph.BufferStore()
    released = []

    def build(t):
        return {"y": configs.chain_y(graph, t), "rowsum": configs.chain_rowsum(graph, t),
                "rowsoftmax": configs.chain_rowsoftmax(graph, t)}

    def realize(tensor, lane, out):
        out[...] = port.realize(passes.prepare(tensor._uop), store)

    pipe = RowPipeline(build, arrays, list(arrays), lambda a: graph.from_numpy(a, store), realize,
                       lambda lane, row_tensors: released.append((lane, sorted(row_tensors))), lanes=3, n_chunks=5)
    shapes = pipe.output_shapes()
    assert shapes["y"] == ((37, 64), "float32") and shapes["rowsum"] == ((37,), "float32")
    outs = {k: np.empty(shape, dtype) for k, (shape, dtype) in shapes.items()}
    pipe.run(outs)
    whole = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
    for name, root in build(whole).items():
        want = port.realize(passes.prepare(root._uop), store)
        if name == "rowsum":
            np.testing.assert_allclose(outs[name], want, rtol=1e-6)
        else:
            assert outs[name].tobytes() == want.tobytes(), name
    assert len(released) == 5 and {lane for lane, _ in released} == {0, 1, 2}
    with pytest.raises(ValueError):
        pipe.run({"y": outs["y"]})


def test_row_pipeline_propagates_lane_errors():
    from browsergrad_b200 import configs, graph
    from browsergrad_b200.sharded import RowPipeline

    arrays = configs.chain_inputs(8, 16)
    store = graph.BufferStore()

    def realize(tensor, lane, out):
        if lane == 1:
            raise RuntimeError("lane failed")
        out[...] = 0

    pipe = RowPipeline(lambda t: configs.chain_y(graph, t), arrays, list(arrays), lambda a: graph.from_numpy(a, store),
                       realize, lambda lane, rt: None, lanes=2, n_chunks=4)
    with pytest.raises(RuntimeError, match="lane failed"):
        pipe.run({"out": np.empty((8, 16), np.float32)})
