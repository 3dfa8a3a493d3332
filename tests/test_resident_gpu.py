"""GPU: roots that stay on the device between plans.

``realize_cuda_resident`` registers the root of one plan with the bridge's device table as a new leaf buffer; a
second plan built on that leaf reads it from HBM with no upload in between, and ``materialize_resident`` fetches the
bytes at the end -- the protocol of ``realize_tensor_plan_webgpu_resident`` and ``GpuBufferTable``
(packages/browsergrad-jit/src/python/_realize_webgpu.py:557-596, _gpu_buffer_table.py:82-98)."""
import numpy as np
import pytest

from browsergrad_b200 import graph
from browsergrad_b200.front import materialize_resident, realize_cuda_resident, release_resident_leaves, resident_table
from tests.util import oracle_value

pytestmark = pytest.mark.gpu


def _oracle(t):
    return oracle_value(t, t._store)


def test_second_plan_reads_the_resident_root_without_an_upload(bridge):
    rng = np.random.default_rng(7)
    store = graph.BufferStore()
    a = graph.from_numpy(rng.standard_normal((96, 130), dtype=np.float32), store)
    b = graph.from_numpy(rng.standard_normal((96, 130), dtype=np.float32), store)
    row = graph.from_numpy(rng.standard_normal((130,), dtype=np.float32), store)
    first_graph = graph.relu(a * b + row)
    table = resident_table(bridge)
    uploads_before = table.stats()["uploads"] if table is not None else 0
    first = realize_cuda_resident(first_graph, bridge)
    table = resident_table(bridge)
    uploads_after_first = table.stats()["uploads"]
    assert uploads_after_first - uploads_before == 3
    # the second plan consumes the resident root and one leaf that is already on the device: nothing is uploaded
    second = realize_cuda_resident((first * a).sum(axis=-1), bridge)
    assert table.stats()["uploads"] == uploads_after_first
    got_second = materialize_resident(second)
    got_first = materialize_resident(first)
    want_first = _oracle(first_graph)
    assert got_first.dtype == want_first.dtype and got_first.shape == want_first.shape
    np.testing.assert_array_equal(got_first, want_first)          # multiply, add, select: one rounding each
    want_second = _oracle((first_graph * a).sum(axis=-1))
    assert got_second.shape == want_second.shape
    scale = np.abs(want_second).max()
    assert np.abs(got_second - want_second).max() <= 1e-5 * scale
    release_resident_leaves(bridge)
    assert bridge.aliveHandleCount() == 0


def test_resident_root_feeds_a_contraction_and_a_view(bridge):
    rng = np.random.default_rng(8)
    store = graph.BufferStore()
    x = graph.from_numpy(rng.standard_normal((64, 48), dtype=np.float32), store)
    w = graph.from_numpy(rng.standard_normal((48, 40), dtype=np.float32), store)
    hidden_graph = x @ w
    hidden = realize_cuda_resident(hidden_graph, bridge)
    table = resident_table(bridge)
    before = table.stats()["uploads"]
    out = realize_cuda_resident(hidden.permute(1, 0).exp() * 0.5, bridge)
    assert table.stats()["uploads"] == before
    got = materialize_resident(out)
    want = _oracle(hidden_graph.permute(1, 0).exp() * 0.5)
    assert got.shape == want.shape and got.dtype == want.dtype
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    # a resident buffer cannot be read through the host-side store: the caller has to ask for it
    from browsergrad_b200.errors import RealizationError
    with pytest.raises(RealizationError):
        out._store.get(out._uop.inputs[0].arg)
    release_resident_leaves(bridge)
    assert bridge.aliveHandleCount() == 0


def test_replace_rebinds_a_buffer_id_for_the_next_realization(bridge):
    """``replace`` (_gpu_buffer_table.py:92-99): a graph that names a buffer id reads whatever the table binds to it
    at realization time, and the handle it had is released."""
    from browsergrad_b200 import front
    rng = np.random.default_rng(9)
    first = rng.standard_normal((40, 24), dtype=np.float32)
    second = rng.standard_normal((40, 24), dtype=np.float32)
    store = graph.BufferStore()
    table = front.DeviceBufferTable(bridge)
    bridge._front_table = table
    table.register("state", bridge.upload(first, first.shape, "float32"))
    buf = graph.Node("BUFFER", (), first.shape, "float32", "state")
    x = graph.Tensor(graph.Node("LOAD", (buf,), buf.shape, buf.dtype, None), front._ResidentStore(store, table, bridge))
    out = front.materialize_resident(front.realize_cuda_resident(x * 2.0, bridge))
    np.testing.assert_array_equal(out, first * np.float32(2.0))
    alive = bridge.aliveHandleCount()
    table.replace("state", bridge.upload(second, second.shape, "float32"))
    assert bridge.aliveHandleCount() == alive                      # one uploaded, the old one released
    out = front.materialize_resident(front.realize_cuda_resident(x * 2.0, bridge))
    np.testing.assert_array_equal(out, second * np.float32(2.0))
    kept = table.detach("state")                                   # ours now: the table no longer releases it
    release_resident_leaves(bridge)
    table.release_all()
    assert bridge.aliveHandleCount() == 1
    bridge.release(kept)
    assert bridge.aliveHandleCount() == 0
