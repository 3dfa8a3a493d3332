"""Helpers shared by the parity tests."""
from __future__ import annotations

import os
from typing import Any, Dict, Tuple

import numpy as np

from browsergrad_b200 import graph, passes
from oracle import port
from tests.cases import CASES, Case

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
_GOLDEN = None


def golden() -> Any:
    global _GOLDEN
    if _GOLDEN is None:
        _GOLDEN = np.load(os.path.join(GOLDEN_DIR, "outputs.npz"))
    return _GOLDEN


def build_case(case: Case) -> Tuple[Any, graph.BufferStore, Dict[str, np.ndarray]]:
    raw = case.inputs()
    store = graph.BufferStore()
    t = {k: graph.from_numpy(v, store) for k, v in raw.items() if not k.startswith("_")}
    return case.build(graph, t, raw), store, raw


def oracle_value(tensor: Any, store: graph.BufferStore) -> np.ndarray:
    return port.realize(passes.prepare(tensor._uop), store)


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """max |got - want| / max |want| over the tensor (0 for empty tensors); non-finite entries
    must match exactly."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    if want.size == 0:
        return 0.0
    fin = np.isfinite(want)
    if not np.array_equal(fin, np.isfinite(got)):
        return float("inf")
    if not np.array_equal(got[~fin], want[~fin], equal_nan=True):
        return float("inf")
    if not fin.any():
        return 0.0
    scale = max(float(np.max(np.abs(want[fin]))), 1e-30)
    return float(np.max(np.abs(got[fin] - want[fin]))) / scale


# Element-wise gate: |got_i - want_i| <= rtol * (|want_i| + max|want| * 2^-k) for every finite element, beside the
# max-norm gate.  The floor max|want| * 2^-k keeps an element that is zero by cancellation from being held to a
# relative error no evaluation order can meet; k says how small an element may be and still have to be right to
# rtol by itself:
#   k = 8 (1/256 of the largest element) for graphs without a contraction -- elementwise chains, reductions,
#         softmax, layer norm, gathers: every operation there is accurate relative to its own result;
#   k = 0 for graphs with a MATMUL or attention (and for cases that mark a cancelling difference): the error of a
#         dot product is bounded relative to sum |a_k b_k|, not to the result, so an output near zero among outputs
#         of order one carries the absolute error of its neighbours whatever the accumulation order.  With k = 0
#         the gate says: no element is off by more than rtol * (its own size + the largest size).
FLOOR_BITS_POINTWISE = 8
FLOOR_BITS_CONTRACTION = 0
_CONTRACTIONS = {"MATMUL", "ATTENTION_FORWARD"}
_FLOOR_CACHE: Dict[int, int] = {}


def floor_bits_for(case: Case) -> int:
    """The k of the element-wise gate for this case (see above), from the case's own graph."""
    if case.floor_bits is not None:
        return case.floor_bits
    hit = _FLOOR_CACHE.get(id(case))
    if hit is None:
        t, _, _ = build_case(case)
        ops = {n.op for n in graph.toposort(t._uop)}
        hit = FLOOR_BITS_CONTRACTION if ops & _CONTRACTIONS else FLOOR_BITS_POINTWISE
        _FLOOR_CACHE[id(case)] = hit
    return hit


def elementwise_err(got: np.ndarray, want: np.ndarray, floor_bits: int) -> float:
    """max_i |got_i - want_i| / (|want_i| + max|want| * 2^-floor_bits) over the finite entries."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    fin = np.isfinite(want)
    if want.size == 0 or not fin.any():
        return 0.0
    if not np.array_equal(fin, np.isfinite(got)):
        return float("inf")
    scale = max(float(np.max(np.abs(want[fin]))), 1e-30)
    denom = np.abs(want[fin]) + scale * 2.0 ** -floor_bits
    return float(np.max(np.abs(got[fin] - want[fin]) / denom))


# every comparison made through check(), written out by the session hook in conftest.py
ERROR_LOG: list = []


def check(case: Case, got: np.ndarray, want: np.ndarray, name: str) -> None:
    assert got.shape == want.shape, f"{name}: shape {got.shape} != {want.shape}"
    assert got.dtype == want.dtype, f"{name}: dtype {got.dtype} != {want.dtype}"
    if case.kind == "exact":
        same = got.tobytes() == want.tobytes()
        ERROR_LOG.append({"name": name, "kind": "exact", "ok": bool(same)})
        assert same, f"{name}: not bit-exact"
    else:
        k = floor_bits_for(case)
        e = rel_err(got, want)
        ew = elementwise_err(got, want, k)
        ERROR_LOG.append({"name": name, "kind": "float", "rtol": case.rtol, "max_norm_err": e, "elementwise_err": ew,
                          "floor_bits": k, "dtype": str(np.asarray(want).dtype), "numel": int(np.asarray(want).size)})
        assert e <= case.rtol, f"{name}: rel err {e:.3e} > {case.rtol:.1e}"
        assert ew <= case.rtol, f"{name}: element-wise err {ew:.3e} > {case.rtol:.1e} (floor 2^-{k} of max|ref|)"
