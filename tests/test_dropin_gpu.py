"""Drop-in check: the UNMODIFIED reference front end drives ``CudaBridge`` through its own
``register_webgpu_bridge`` seam, and the seam contract the reference's integration tests state for
a bridge (packages/browsergrad-jit/tests-integration/webgpu_realizer.test.ts:1026-1281 and
:2399-2507) holds: which bridge methods are called, how often, what stays resident, and that the
values agree with the reference's own NumPy realizer.

The reference package is assembled from its sources by ``oracle/build_ref.py`` into ``oracle/_ref``;
where that folder is absent the module is skipped (the case parity tests do not need it).
"""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


class CountingBridge:
    """Forwards every protocol method to a ``CudaBridge`` and counts the calls, like the mock
    bridge of the reference's integration tests (webgpu_realizer.test.ts:60-330)."""

    COUNTED = ("upload", "materialize", "release", "matmul", "fused_elementwise", "cast",
               "flash_attention", "run_tensor_plan", "run_tensor_plan_semantic",
               "run_tensor_plan_resident", "run_tensor_plan_resident_semantic")

    def __init__(self, inner):
        self._inner = inner
        self.counts = {name: 0 for name in self.COUNTED}

    def __getattr__(self, name):
        target = getattr(self._inner, name)
        if name not in self.COUNTED:
            return target

        def call(*args, **kwargs):
            self.counts[name] += 1
            return target(*args, **kwargs)
        return call

    def reset(self):
        for name in self.counts:
            self.counts[name] = 0


@pytest.fixture(scope="module")
def bg():
    if not os.path.isdir(os.path.join(REF_DIR, "browsergrad_jit")):
        pytest.skip("reference package not assembled under oracle/_ref")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import browsergrad_jit
    return browsergrad_jit


@pytest.fixture()
def seam(bg, bridge):
    counting = CountingBridge(bridge)
    bg.register_webgpu_bridge(counting)
    try:
        yield counting
    finally:
        bg.unregister_webgpu_bridge()


def test_single_matmul_per_op_walk(bg, seam):
    rng = np.random.RandomState(0)
    A = rng.uniform(-1, 1, size=(4, 8)).astype(np.float32)
    B = rng.uniform(-1, 1, size=(8, 6)).astype(np.float32)
    out = bg.from_numpy(A.copy()) @ bg.from_numpy(B.copy())
    ref = out.numpy()
    gpu = bg.realize_webgpu(out)
    assert gpu.shape == (4, 6) and gpu.dtype == np.float32
    assert float(np.max(np.abs(ref - gpu))) < 1e-6
    assert seam.counts["upload"] == 2
    assert seam.counts["matmul"] == 1
    assert seam.counts["materialize"] == 1


def test_chained_matmul_keeps_the_intermediate_resident(bg, seam):
    rng = np.random.RandomState(1)
    A = rng.uniform(-1, 1, size=(4, 4)).astype(np.float32)
    B = rng.uniform(-1, 1, size=(4, 4)).astype(np.float32)
    C = rng.uniform(-1, 1, size=(4, 4)).astype(np.float32)
    alive_before = seam.aliveHandleCount()
    out = (bg.from_numpy(A.copy()) @ bg.from_numpy(B.copy())) @ bg.from_numpy(C.copy())
    ref = out.numpy()
    gpu = bg.realize_webgpu(out)
    assert float(np.max(np.abs(ref - gpu))) < 1e-5
    assert seam.counts["upload"] == 3
    assert seam.counts["matmul"] == 2
    assert seam.counts["materialize"] == 1          # only the root crosses back
    assert seam.counts["release"] == 2              # the intermediate and the root
    table = bg._realize_webgpu.get_registered_gpu_buffer_table()
    assert table.stats()["handles_alive"] == 3      # the three seeds stay cached
    assert seam.aliveHandleCount() - alive_before == 3


def test_second_realize_reuses_uploaded_seeds(bg, seam):
    a = bg.from_numpy(np.eye(4, dtype=np.float32))
    b = bg.from_numpy(np.eye(4, dtype=np.float32) * 2.0)
    first = bg.realize_webgpu(a @ b)
    assert seam.counts["upload"] == 2
    second = bg.realize_webgpu(a @ b)
    assert seam.counts["upload"] == 2
    assert seam.counts["matmul"] == 2
    assert np.array_equal(first, second)
    assert np.array_equal(first, np.eye(4, dtype=np.float32) * 2.0)


def test_plan_path_is_one_bridge_call(bg, seam):
    rng = np.random.RandomState(11)
    A = rng.uniform(-0.5, 0.5, size=(3, 4)).astype(np.float32)
    B = rng.uniform(-0.5, 0.5, size=(4, 5)).astype(np.float32)
    y = bg.from_numpy(A.copy()) @ bg.from_numpy(B.copy())
    out = bg.exp(y) * y
    ref = out.numpy()
    gpu = bg.realize_tensor_plan_webgpu(out)
    plan = bg.gpu_plan_summary(out)
    assert float(np.max(np.abs(ref - gpu))) < 1e-6
    assert seam.counts["run_tensor_plan"] == 1
    for name in ("upload", "matmul", "fused_elementwise", "materialize"):
        assert seam.counts[name] == 0, name
    assert "FUSED_ELEMENTWISE" in plan["ops"] and "EXP" not in plan["ops"]


def test_plan_path_softmax_template(bg, seam):
    import browsergrad_jit.nn.functional as F
    x = bg.from_numpy(np.array([[1.0, 2.0, 3.0], [-2.0, 0.5, 1.5]], dtype=np.float32))
    out = F.softmax(x, dim=-1)
    ref = out.numpy()
    gpu = bg.realize_tensor_plan_webgpu(out)
    plan = bg.gpu_plan_summary(out)
    assert float(np.max(np.abs(ref - gpu))) < 1e-6
    assert seam.counts["run_tensor_plan"] == 1
    assert "FUSED_SOFTMAX" in plan["ops"]
    assert "REDUCE" not in plan["ops"] and "EXP" not in plan["ops"]


def test_plan_path_sdpa_uses_the_semantic_method(bg, seam):
    import browsergrad_jit.nn.functional as F
    q = bg.from_numpy(np.array([[1.0, 0.5], [0.25, -0.75]], dtype=np.float32))
    k = bg.from_numpy(np.array([[0.5, -0.25], [1.25, 0.75]], dtype=np.float32))
    v = bg.from_numpy(np.array([[2.0, 3.0], [5.0, 7.0]], dtype=np.float32))
    out = F.scaled_dot_product_attention(q, k, v)
    ref = out.numpy()
    gpu = bg.realize_tensor_plan_webgpu(out)
    plan = bg.gpu_plan_summary(out)
    assert float(np.max(np.abs(ref - gpu))) < 1e-6
    assert seam.counts["run_tensor_plan"] == 0
    assert seam.counts["run_tensor_plan_semantic"] == 1
    assert not plan["has_custom_ops"]
    assert "MATMUL" in plan["ops"] and "FUSED_SOFTMAX" in plan["ops"]


def test_resident_roots_stay_on_the_device_until_numpy(bg, seam):
    a = bg.tensor([[1.0, 2.0], [3.0, 4.0]])
    b = bg.tensor([[2.0, 0.0], [1.0, 2.0]])
    offset = bg.tensor([[3.0, 3.0], [3.0, 3.0]])
    first = bg.realize_tensor_plan_webgpu_resident(a @ b)
    first_id = first._uop.inputs[0].arg
    second = bg.realize_tensor_plan_webgpu_resident(first + offset)
    second_id = second._uop.inputs[0].arg
    host_table = second._get_session().buffer_table
    device_table = bg._realize_webgpu.get_registered_gpu_buffer_table()
    assert seam.counts["materialize"] == 0
    assert not host_table.is_materialized(first_id)
    assert device_table.has(first_id) and device_table.has(second_id)
    arr = second.numpy()
    assert seam.counts["materialize"] == 1
    assert seam.counts["run_tensor_plan"] == 0
    assert seam.counts["run_tensor_plan_resident"] == 2
    assert arr.tolist() == [[7.0, 7.0], [13.0, 11.0]]


def test_typed_attention_is_one_flash_attention_call(bg, seam):
    B, H, Sq, Sk, D = 2, 4, 8, 8, 16
    rng = np.random.RandomState(2)
    Q = rng.standard_normal((B, H, Sq, D)).astype(np.float32)
    K = rng.standard_normal((B, H, Sk, D)).astype(np.float32)
    V = rng.standard_normal((B, H, Sk, D)).astype(np.float32)
    out = bg.kernels.attention_forward(bg.from_numpy(Q.copy()), bg.from_numpy(K.copy()),
                                       bg.from_numpy(V.copy()))
    gpu = bg.realize_webgpu(out)
    scores = np.matmul(Q, np.swapaxes(K, -1, -2)) * (1.0 / np.sqrt(D))
    e = np.exp(scores - scores.max(axis=-1, keepdims=True))
    ref = np.matmul(e / e.sum(axis=-1, keepdims=True), V)
    assert out._uop.op == "ATTENTION_FORWARD"
    assert seam.counts["flash_attention"] == 1
    assert gpu.shape == (2, 4, 8, 16)
    assert float(np.max(np.abs(gpu - ref))) < 1e-4


def test_reference_side_refusals_are_unchanged(bg, seam):
    """The per-op walk's whitelist lives in the reference; a CUDA bridge must not widen it."""
    a = bg.from_numpy(np.ones((3, 3), dtype=np.float32))
    with pytest.raises(bg.JitNotImplementedError, match="REDUCE"):
        bg.realize_webgpu(a.sum())


def test_larger_plan_through_the_reference_front_end(bg, seam):
    """A tensor-core sized linear + tanh + softmax plan (the reference's plan builder refuses
    WHERE, so no relu here), built and planned by the reference,
    executed here; compared with the reference's NumPy realizer at the fp32 tolerance."""
    import browsergrad_jit.nn.functional as F
    rng = np.random.RandomState(5)
    x = rng.standard_normal((512, 256)).astype(np.float32)
    w = (rng.standard_normal((256, 384)) * 0.05).astype(np.float32)
    bias = rng.standard_normal((384,)).astype(np.float32)
    h = bg.tanh(bg.from_numpy(x) @ bg.from_numpy(w) + bg.from_numpy(bias))
    out = F.softmax(h, dim=-1)
    ref = out.numpy()
    gpu = bg.realize_tensor_plan_webgpu(out)
    assert seam.counts["run_tensor_plan"] + seam.counts["run_tensor_plan_semantic"] == 1
    denom = max(float(np.max(np.abs(ref))), 1e-30)
    assert float(np.max(np.abs(ref - gpu))) / denom < 1e-5
