"""GPU: the allocation-free cross entropy entry point against the regular plan path.

Collected last on purpose (file name): a run that stops at the first failure has then already
executed every other test.  The entry point serves hosts that may not allocate device memory while
running; it keeps its scratch in a static device array shared by all calls, so the test calls it
twice in a row with different data to show that nothing stale leaks from one call into the next.
"""
import ctypes as C

import numpy as np
import pytest

from browsergrad_b200 import _lib, graph, realize_cuda

pytestmark = pytest.mark.gpu


def _plan_path(bridge, logits, targets, reduction):
    store = graph.BufferStore()
    t = graph.cross_entropy(graph.from_numpy(logits, store), graph.from_numpy(targets, store), reduction=reduction)
    return realize_cuda(t, bridge)


def _noalloc_path(bridge, logits, targets, reduction):
    lib = _lib.load()
    rows, classes = logits.shape[0], logits.shape[1]
    inner = int(np.prod(logits.shape[2:])) if logits.ndim > 2 else 1
    h_l = bridge.upload(logits, logits.shape, "float32")
    h_t = bridge.upload(targets, targets.shape, "int64")
    h_o = bridge.upload(np.full((1,), 123.0, np.float32), (1,), "float32")
    try:
        err = C.create_string_buffer(256)
        rc = lib.bg_cross_entropy_noalloc(bridge.device_pointer(h_l), bridge.device_pointer(h_t), bridge.device_pointer(h_o),
                                          rows, classes, inner, {"mean": 1, "sum": 2}[reduction], -100, bridge.stream(),
                                          err, len(err))
        assert rc == 0, err.value.decode()
        return bridge.materialize_array(h_o, (1,), "float32").reshape(())
    finally:
        for h in (h_l, h_t, h_o):
            bridge.release(h)


def test_noalloc_cross_entropy_matches_plan_path_twice(bridge):
    rng = np.random.default_rng(7)
    first = (rng.standard_normal((4096, 50), dtype=np.float32) * np.float32(3), rng.integers(0, 50, (4096,), dtype=np.int64))
    second_logits = rng.standard_normal((33, 7, 5), dtype=np.float32)
    second_targets = rng.integers(0, 7, (33, 5), dtype=np.int64)
    second_targets[::4] = -100                      # ignored positions
    for logits, targets, reduction in ((first[0], first[1], "mean"), (second_logits, second_targets, "sum"),
                                       (second_logits, second_targets, "mean")):
        want = _plan_path(bridge, logits, targets, reduction)
        got = _noalloc_path(bridge, logits, targets, reduction)
        assert abs(float(got) - float(want)) <= 1e-5 * max(abs(float(want)), 1e-30), (got, want)


def test_noalloc_refuses_oversize_and_bad_targets(bridge):
    lib = _lib.load()
    h = bridge.upload(np.zeros((8, 4), np.float32), (8, 4), "float32")
    ht = bridge.upload(np.array([0, 1, 2, 3, 9, 0, 1, 2], np.int64), (8,), "int64")
    ho = bridge.upload(np.zeros((1,), np.float32), (1,), "float32")
    try:
        err = C.create_string_buffer(256)
        rc = lib.bg_cross_entropy_noalloc(bridge.device_pointer(h), bridge.device_pointer(ht), bridge.device_pointer(ho),
                                          (1 << 20) + 1, 4, 1, 1, -100, bridge.stream(), err, len(err))
        assert rc == 2 and b"exceed the static scratch" in err.value
        rc = lib.bg_cross_entropy_noalloc(bridge.device_pointer(h), bridge.device_pointer(ht), bridge.device_pointer(ho),
                                          8, 4, 1, 1, -100, bridge.stream(), err, len(err))
        assert rc == 7 and b"outside" in err.value
    finally:
        for x in (h, ht, ho):
            bridge.release(x)
