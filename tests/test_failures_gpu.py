"""GPU: the failure paths of the bridge, each provoked on the host or by a wait that is allowed to run out -- never by
a fault.  After every failure the same bridge must go on working and hold no stray handles.

* an index outside its axis (gather, cross-entropy target) through ``realize_cuda``: status 7, as the reference raises
  (packages/browsergrad-jit/src/python/_realize.py:1476-1485, _framework_contracts.py:3677-3682);
* device memory exhausted (injected at the allocator): status 4;
* a bounded device wait that gives up (a barrier nothing arrives on, a limit of about a millisecond): status 6;
* a fully masked attention row: NaN, as NumPy's exp(-inf - -inf) gives the reference."""
import numpy as np
import pytest

from browsergrad_b200 import configs, graph, realize_cuda
from browsergrad_b200.errors import KernelError
from tests.cases import CASES
from tests.util import build_case, check, oracle_value

pytestmark = pytest.mark.gpu


def _still_works(bridge):
    case = CASES["c2_y"]
    t, store, _ = build_case(case)
    check(case, realize_cuda(t, bridge), oracle_value(t, store), "c2_y after a failure")
    assert bridge.aliveHandleCount() == 0


def test_gather_index_out_of_range_is_refused_and_the_bridge_survives(bridge):
    store = graph.BufferStore()
    x = graph.from_numpy(np.arange(12, dtype=np.float32).reshape(3, 4), store)
    idx = np.zeros((2, 4), np.int64)
    idx[1, 2] = 3                      # rows are 0..2
    with pytest.raises(KernelError) as exc:
        realize_cuda(x.gather(0, graph.from_numpy(idx, store)), bridge)
    assert exc.value.status == 7
    idx[1, 2] = -1
    with pytest.raises(KernelError) as exc:
        realize_cuda(x.gather(0, graph.from_numpy(idx, store)), bridge)
    assert exc.value.status == 7
    _still_works(bridge)


@pytest.mark.parametrize("classes", [7, 4100])        # thread-per-position kernel, CTA-per-row kernel
def test_cross_entropy_target_out_of_range_is_refused(bridge, classes):
    store = graph.BufferStore()
    logits = graph.from_numpy(np.random.default_rng(5).standard_normal((6, classes), dtype=np.float32), store)
    tgt = np.array([0, 1, 2, classes, 1, 0], dtype=np.int64)
    with pytest.raises(KernelError) as exc:
        realize_cuda(graph.cross_entropy(logits, graph.from_numpy(tgt, store)), bridge)
    assert exc.value.status == 7
    tgt[3] = -100                      # ignore_index is not an error
    got = realize_cuda(graph.cross_entropy(logits, graph.from_numpy(tgt, store)), bridge)
    assert np.isfinite(got)
    _still_works(bridge)


def test_refusal_in_a_plan_whose_root_stays_on_the_device_is_raised_before_any_byte_reaches_the_host(bridge):
    """A plan that keeps its root on the device does not wait for the device: the refusal is raised by the call
    that fetches the buffer (or by the next plan), never later than the first byte read back."""
    from browsergrad_b200.front import materialize_resident, realize_cuda_resident, release_resident_leaves
    store = graph.BufferStore()
    x = graph.from_numpy(np.arange(12, dtype=np.float32).reshape(3, 4), store)
    idx = np.zeros((2, 4), np.int64)
    idx[0, 1] = 5
    kept = realize_cuda_resident(x.gather(0, graph.from_numpy(idx, store)) * 2.0, bridge)
    with pytest.raises(KernelError) as exc:
        materialize_resident(kept)
    assert exc.value.status == 7
    release_resident_leaves(bridge)
    _still_works(bridge)


def test_exhausted_device_memory_is_reported_as_out_of_memory(bridge):
    case = CASES["c2_rowsoftmax"]
    t, _, _ = build_case(case)
    for nth in (1, 2, 3):              # the failing allocation is an upload, an intermediate or the root
        bridge.set_option("fail_allocation_after", nth)
        try:
            with pytest.raises(KernelError) as exc:
                realize_cuda(t, bridge)
            assert exc.value.status == 4, exc.value
        finally:
            bridge.set_option("fail_allocation_after", 0)
        assert bridge.aliveHandleCount() == 0
    _still_works(bridge)


def test_a_device_wait_that_gives_up_is_reported_and_the_context_stays_usable(bridge):
    with pytest.raises(KernelError) as exc:
        bridge.selftest_wait_timeout(2_000_000)       # about a millisecond of SM cycles
    assert exc.value.status == 6
    _still_works(bridge)
    # a tensor-core plan right after: its own status check must not see a stale word
    case = CASES["c3_tc_f32"]
    t, store, _ = build_case(case)
    check(case, realize_cuda(t, bridge), oracle_value(t, store), "c3_tc_f32 after a timed-out wait")


@pytest.mark.parametrize("amp", ["", "float16"])
def test_fully_masked_attention_rows_are_nan_like_the_reference(bridge, amp):
    """Rows whose every key is masked: the reference's softmax computes exp(-inf - -inf) = NaN; so does the fused kernel
    (0 / 0), and the other rows are unaffected."""
    arrays = configs.attention_inputs(1, 2, 160, 64)
    mask = np.zeros((160, 160), np.float32)
    mask[5, :] = -np.inf
    mask[130:135, :] = -np.inf
    mask[:, 150:] = -np.inf
    arrays["mask"] = mask
    store = graph.BufferStore()
    t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
    root = configs.attention(graph, t, "mask", amp)
    with np.errstate(invalid="ignore"):
        want = oracle_value(root, store)
    got = realize_cuda(root, bridge)
    assert any(ln.startswith("attention_tc") for ln in bridge.last_plan_trace())
    assert np.isnan(want[0, :, 5]).all() and np.isnan(want[0, :, 130:135]).all()
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    tol = 2e-2 if amp else 1e-5
    scale = float(np.max(np.abs(want[ok])))
    assert float(np.max(np.abs(got[ok].astype(np.float64) - want[ok].astype(np.float64)))) <= tol * scale
