"""Parity at the baseline's full sizes, through properties that do not need the oracle to run the whole
problem: the configurations are independent along their leading axis, so a sample of rows / heads /
sequences of the full-size GPU result is compared with the oracle run on exactly that sample, and
whole-tensor invariants (softmax rows sum to one, attention outputs are convex combinations of V rows,
a causal first query copies V's first row, batch entries do not influence each other) are checked on
the full result.  Tolerances: 1e-5 relative for fp32 / 3xTF32, 2e-2 for the bf16 autocast path.
"""
import numpy as np
import pytest

from browsergrad_b200 import configs, graph, passes, realize_cuda
from oracle import port
from tests.util import rel_err

pytestmark = pytest.mark.gpu


def _tensors(arrays, store):
    return {k: graph.from_numpy(v, store) for k, v in arrays.items()}


def _oracle(root, store):
    return port.realize(passes.prepare(root._uop), store)


def _sample(n, count, seed):
    idx = np.random.default_rng(seed).choice(n, size=count, replace=False)
    idx[0], idx[-1] = 0, n - 1          # always include both ends
    return np.sort(np.unique(idx))


def test_config2_full_size_rows_and_invariants(bridge):
    rows, cols = 16384, 4096
    arrays = configs.chain_inputs(rows, cols)
    store = graph.BufferStore()
    t = _tensors(arrays, store)
    y = realize_cuda(configs.chain_y(graph, t), bridge, resident_leaves=True)
    rowsum = realize_cuda(configs.chain_rowsum(graph, t), bridge, resident_leaves=True)
    soft = realize_cuda(configs.chain_rowsoftmax(graph, t), bridge, resident_leaves=True)
    from browsergrad_b200 import release_resident_leaves
    release_resident_leaves(bridge)
    assert y.shape == (rows, cols) and rowsum.shape == (rows,) and soft.shape == (rows, cols)
    # the oracle on a sample of rows (every realization is row-independent)
    pick = _sample(rows, 96, 1)
    sub_store = graph.BufferStore()
    sub = _tensors({k: np.ascontiguousarray(v[pick]) for k, v in arrays.items()}, sub_store)
    want_y = _oracle(configs.chain_y(graph, sub), sub_store)
    assert rel_err(y[pick], want_y) <= 1e-5
    assert rel_err(rowsum[pick], _oracle(configs.chain_rowsum(graph, sub), sub_store)) <= 1e-5
    assert rel_err(soft[pick], _oracle(configs.chain_rowsoftmax(graph, sub), sub_store)) <= 1e-5
    # invariants over all 16384 rows
    assert np.all(y >= 0)                                                # relu(.) * exp(.) is non-negative
    np.testing.assert_allclose(rowsum, y.sum(axis=-1, dtype=np.float64), rtol=1e-5)
    np.testing.assert_allclose(soft.sum(axis=-1, dtype=np.float64), 1.0, atol=1e-5)
    assert np.all((soft >= 0) & (soft <= 1))
    assert np.array_equal(soft.argmax(axis=-1), y.argmax(axis=-1))       # softmax is monotone
    assert bridge.aliveHandleCount() == 0


@pytest.mark.parametrize("n,amp,tol", [(8192, "", 1e-5), (8192, "bfloat16", 2e-2), (4096, "", 1e-5), (4096, "bfloat16", 2e-2),
                                       (1024, "", 1e-5), (1024, "bfloat16", 2e-2)])
def test_config3_full_size_rows(bridge, n, amp, tol):
    arrays = configs.linear_inputs(n, n, n)
    store = graph.BufferStore()
    got = realize_cuda(configs.linear_gelu(graph, _tensors(arrays, store), amp), bridge)
    assert got.shape == (n, n)
    trace = bridge.last_plan_trace()
    assert any(ln.startswith("gemm_tc") and "+bias+gelu" in ln for ln in trace), trace
    # rows of x are independent: the oracle multiplies a sample of them by the full weight matrix
    pick = _sample(n, 48, n)
    sub_store = graph.BufferStore()
    sub = dict(arrays)
    sub["x"] = np.ascontiguousarray(arrays["x"][pick])
    want = _oracle(configs.linear_gelu(graph, _tensors(sub, sub_store), amp), sub_store)
    assert got.dtype == want.dtype
    assert rel_err(got[pick], want) <= tol
    assert np.all(np.isfinite(got))


@pytest.mark.parametrize("amp,tol", [("", 1e-5), ("bfloat16", 2e-2)])
def test_config4_full_size_heads_and_invariants(bridge, amp, tol):
    b, h, s, d = 16, 12, 2048, 64
    arrays = configs.attention_inputs(b, h, s, d)
    arrays["mask"] = configs.causal_mask(s)
    store = graph.BufferStore()
    got = realize_cuda(configs.attention(graph, _tensors(arrays, store), "mask", amp), bridge)
    assert got.shape == (b, h, s, d)
    assert any(ln.startswith("attention_tc") for ln in bridge.last_plan_trace())
    g64 = got.astype(np.float64)
    v64 = arrays["v"].astype(np.float64)
    # every output row is a convex combination of V rows of its head
    slack = tol * 8
    assert np.all(g64 <= v64.max(axis=2, keepdims=True) + slack) and np.all(g64 >= v64.min(axis=2, keepdims=True) - slack)
    # under the causal mask the first query sees only the first key, the second a mix of the first two
    first = arrays["v"][:, :, 0, :]
    if amp:
        first = port.to_bfloat16(first).astype(np.float32)
    assert rel_err(got[:, :, 0, :].astype(np.float32), first) <= tol
    lo, hi = np.minimum(v64[:, :, 0], v64[:, :, 1]), np.maximum(v64[:, :, 0], v64[:, :, 1])
    assert np.all(g64[:, :, 1] <= hi + slack) and np.all(g64[:, :, 1] >= lo - slack)
    # the oracle on three (batch, head) pairs
    for bi, hi_ in ((0, 0), (7, 5), (15, 11)):
        sub = {k: np.ascontiguousarray(arrays[k][bi:bi + 1, hi_:hi_ + 1]) for k in "qkv"}
        sub["mask"] = arrays["mask"]
        sub_store = graph.BufferStore()
        want = _oracle(configs.attention(graph, _tensors(sub, sub_store), "mask", amp), sub_store)
        assert rel_err(got[bi:bi + 1, hi_:hi_ + 1], want) <= tol, (bi, hi_)


def test_config5_full_depth_sequences_are_independent_and_match_the_oracle(bridge):
    """One GPU's shard (batch 8) of the 12-layer decoder: its first sequence equals the same sequence run
    alone (batch sharding changes nothing), and that run matches the oracle on hidden states and logits."""
    arrays = configs.gpt_inputs(batch=8)
    meta = arrays.pop("_meta")
    store = graph.BufferStore()
    full = realize_cuda(configs.gpt_forward(graph, _tensors(arrays, store), meta, logits=False), bridge)
    layers, d_model, heads, d_mlp, vocab, seq, batch = (int(v) for v in meta)
    assert full.shape == (batch * seq, d_model)
    one = configs.gpt_inputs(batch=1)
    one_meta = one.pop("_meta")
    for k in ("ids", "tok_index", "pos_index"):
        assert np.array_equal(one[k], arrays[k][: one[k].shape[0]])      # the first sequence of the shard
    one_store = graph.BufferStore()
    alone = realize_cuda(configs.gpt_forward(graph, _tensors(one, one_store), one_meta, logits=False), bridge)
    assert rel_err(full[:seq], alone) <= 1e-6
    want = _oracle(configs.gpt_forward(graph, _tensors(one, one_store), one_meta, logits=False), one_store)
    assert alone.dtype == want.dtype
    assert rel_err(alone, want) <= 1e-5
    # logits of the last 64 positions (LM head shares the embedding table)
    logits = realize_cuda(configs.gpt_forward(graph, _tensors(one, one_store), one_meta), bridge)
    assert logits.shape == (seq, vocab)
    want_tail = want[-64:].astype(np.float64) @ one["wte"].astype(np.float64).T
    assert rel_err(logits[-64:], want_tail.astype(logits.dtype)) <= 1e-5


@pytest.mark.parametrize("amp", ["float16", "bfloat16"])
def test_config5_full_depth_under_autocast_matches_the_oracle(bridge, amp):
    """The 12-layer decoder built under autocast (float16 is the dtype the reference's AMP pass pins,
    packages/browsergrad-jit/src/python/_amp.py:183-261; bfloat16 follows the same cast rule): one sequence, hidden
    states and the logits of the last 64 positions against the oracle, at the 2e-2 of the 16-bit path."""
    one = configs.gpt_inputs(batch=1)
    meta = one.pop("_meta")
    layers, d_model, heads, d_mlp, vocab, seq, batch = (int(v) for v in meta)
    store = graph.BufferStore()
    t = _tensors(one, store)
    hidden = realize_cuda(configs.gpt_forward(graph, t, meta, logits=False, amp=amp), bridge)
    trace = bridge.last_plan_trace()
    assert any(ln.startswith("gemm_tc") and "3xtf32" not in ln for ln in trace), trace      # the 16-bit tensor-core path ran
    want = _oracle(configs.gpt_forward(graph, t, meta, logits=False, amp=amp), store)
    assert hidden.shape == want.shape == (seq, d_model)
    assert rel_err(hidden, want) <= 2e-2
    logits = realize_cuda(configs.gpt_forward(graph, t, meta, amp=amp), bridge)
    assert logits.shape == (seq, vocab)
    want_logits = _oracle(configs.gpt_forward(graph, t, meta, amp=amp), store)
    assert rel_err(logits[-64:], want_logits[-64:]) <= 2e-2
