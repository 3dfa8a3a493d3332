"""CPU: the oracle port, the graph builders and the restated passes against the fixtures that
``tests/golden/make_golden.py`` generated from the unmodified reference."""
import json
import os

import numpy as np
import pytest

from browsergrad_b200 import graph, passes
from oracle import port
from tests.cases import CASES, signature
from tests.util import GOLDEN_DIR, build_case, golden

with open(os.path.join(GOLDEN_DIR, "graphs.json")) as _fh:
    GRAPHS = json.load(_fh)

PINNED = [n for n, c in CASES.items() if c.reference_has_it]


def test_fixture_covers_every_pinned_case():
    assert sorted(GRAPHS["cases"]) == sorted(PINNED)
    assert sorted(golden().files) == sorted(PINNED)


@pytest.mark.parametrize("name", PINNED)
def test_builder_and_passes_match_reference_graph(name):
    t, store, _ = build_case(CASES[name])
    pre = signature(graph.toposort(t._uop))
    post = signature(graph.toposort(passes.prepare(t._uop)))
    want = GRAPHS["cases"][name]
    assert json.loads(json.dumps(pre)) == want["pre"]
    assert json.loads(json.dumps(post)) == want["post"]


@pytest.mark.parametrize("name", PINNED)
def test_oracle_port_is_bit_identical_to_reference(name):
    if np.__version__ != GRAPHS["numpy"]:
        pytest.skip(f"fixtures were generated with NumPy {GRAPHS['numpy']}, this is {np.__version__}")
    t, store, _ = build_case(CASES[name])
    got = port.realize(passes.prepare(t._uop), store)
    want = golden()[name]
    assert got.dtype == want.dtype and got.shape == want.shape
    assert got.tobytes() == want.tobytes()


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.005859375, -3.1415927, 65504.0, 1e-40], dtype=np.float32)
    r = port.to_bfloat16(x)
    assert (r.view(np.uint32) & 0xFFFF == 0).all()
    assert r[0] == 1.0 and r[1] == 1.0  # tie rounds to even
    assert abs(r[3] - x[3]) <= abs(x[3]) * 2 ** -8
