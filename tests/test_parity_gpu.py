"""GPU: every parity case through the C ABI (``realize_cuda`` -> ``bg_run_tensor_plan``) against
the CPU oracle on the same seeded inputs, and against the committed golden vectors.

Tolerances: bit-exact for integer / bool / index / copy cases (``kind == "exact"``);
max|diff| / max|ref| <= 1e-5 for fp32 and fp64 graphs; <= 2e-2 for the f16 / bf16 autocast path;
the per-case value is ``Case.rtol``.
"""
import numpy as np
import pytest

from browsergrad_b200 import realize_cuda
from tests.cases import CASES
from tests.util import build_case, check, golden, oracle_value

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(CASES))
def test_case_matches_oracle_and_golden(bridge, name):
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    got = realize_cuda(t, bridge)
    check(case, got, want, name + " vs oracle")
    if case.reference_has_it:
        check(case, got, golden()[name], name + " vs golden")
    assert bridge.aliveHandleCount() == 0


@pytest.mark.parametrize("name", ["c2_y", "c2_rowsoftmax", "c3_linear_gelu", "c4_attn_mask", "c5_gpt_tiny", "int_arith"])
def test_unfused_execution_matches_too(bridge, name):
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    bridge.set_option("fusion", 0)
    try:
        got = realize_cuda(t, bridge)
    finally:
        bridge.set_option("fusion", 1)
    check(case, got, want, name + " (fusion off)")


@pytest.mark.parametrize("name", ["c2_y", "c2_y_static", "c2_rowsum_static", "c2_rowsoftmax_static", "c2_rowsoftmax_long",
                                  "ln_residual_static", "ln_plain_static", "ln_stream_static", "ln_stream_f64_static"])
def test_pattern_kernels_and_interpreter_agree(bridge, name):
    """The specialised pattern kernels and the generic interpreter compute the same bits."""
    case = CASES[name]
    t, store, _ = build_case(case)
    got_static = realize_cuda(t, bridge)
    static_trace = bridge.last_plan_trace()
    bridge.set_option("static_patterns", 0)
    try:
        got_generic = realize_cuda(t, bridge)
        generic_trace = bridge.last_plan_trace()
    finally:
        bridge.set_option("static_patterns", 1)
    assert not any(ln.startswith("static_") for ln in generic_trace)
    if name.endswith("_static"):
        assert any(ln.startswith("static_") for ln in static_trace), static_trace
    if "rowsum" in name or "softmax" in name or name.startswith("ln_"):
        check(case, got_static, got_generic, name)      # summation order / exp2-based tail differ within tolerance
    else:
        assert got_static.tobytes() == got_generic.tobytes()


@pytest.mark.parametrize("name", ["c1_mlp_ce", "c3_chain_gelu_planes", "ln_then_qkv_f16", "c4_attn_block_f64", "c4_attn_merge_heads_bf16",
                                  "gather_rows_by4"])
def test_dependent_launch_changes_no_bit(bridge, name):
    """Option dependent_launch: the decoder's kernels may be set up on the SMs while the kernel before them drains and
    wait for it before they touch global memory; the results are those of plain stream order."""
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    got_on = realize_cuda(t, bridge)
    bridge.set_option("dependent_launch", 0)
    try:
        got_off = realize_cuda(t, bridge)
    finally:
        bridge.set_option("dependent_launch", 1)
    assert got_on.tobytes() == got_off.tobytes()
    check(case, got_on, want, f"{name} (dependent launch)")


@pytest.mark.parametrize("name,expect", [
    ("c3_tc_f32", "gemm_tc_3xtf32+bias+gelu[float32]"),
    ("c3_tc_f16", "gemm_tc+bias+gelu[float16]"),
    ("c3_tc_bf16", "gemm_tc+bias+gelu[bfloat16]"),
    ("c3_tc_ragged", "gemm_tc_3xtf32+bias[float32]"),
    ("c3_tc_relu", "gemm_tc_3xtf32+bias+relu[float32]"),
    ("c3_tc_rowmajor_b", "gemm_tc_3xtf32[float32]"),
])
def test_linear_runs_on_tensor_cores_with_folded_epilogue(bridge, name, expect):
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    got = realize_cuda(t, bridge)
    trace = bridge.last_plan_trace()
    assert expect in trace, trace
    assert not any(ln.startswith(("ew[", "static_ew[")) and "CAST" not in ln for ln in trace), trace
    check(case, got, want, name)
    bridge.set_option("tensor_cores", 0)
    try:
        simt = realize_cuda(t, bridge)
    finally:
        bridge.set_option("tensor_cores", 1)
    check(case, simt, want, name + " (SIMT)")


@pytest.mark.parametrize("name,expect", [
    ("c4_attn_mask_d64", "attention_tc_3xtf32+mask[float32]"),
    ("c4_attn_causal_d64", "attention_tc_3xtf32+boolmask[float32]"),
    ("c4_attn_causal_tiles", "attention_tc_3xtf32+boolmask[float32]"),
    ("c4_attn_mask_tiles", "attention_tc_3xtf32+mask[float32]"),
    ("c4_attn_nomask_d64", "attention_tc_3xtf32[float32]"),
    ("typed_attention_d64", "attention_tc_3xtf32[float32]"),
    ("c4_attn_mask_f16", "attention_tc+mask[float16]"),
    ("c4_attn_causal_f16", "attention_tc+boolmask[float16]"),
    ("c4_attn_mask_bf16", "attention_tc+mask[bfloat16]"),
])
def test_sdpa_runs_as_one_fused_attention_kernel(bridge, name, expect):
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    got = realize_cuda(t, bridge)
    trace = bridge.last_plan_trace()
    assert expect in trace, trace
    assert not any(ln.startswith(("gemm", "row[", "static_row[")) for ln in trace), trace
    check(case, got, want, name)
    bridge.set_option("tensor_cores", 0)        # composed path: batched GEMM + fused softmax + batched GEMM
    try:
        composed = realize_cuda(t, bridge)
    finally:
        bridge.set_option("tensor_cores", 1)
    check(case, composed, want, name + " (composed)")


ATTN16_CASES = ["c4_attn_mask_f16", "c4_attn_causal_f16", "c4_attn_mask_bf16", "c4_attn_growing_f16", "c4_attn_growing_causal_f16",
                "c4_attn_merge_heads_bf16"]


@pytest.mark.parametrize("variant", [0, 1, 3, 5, 7, 15])
@pytest.mark.parametrize("name", ATTN16_CASES)
def test_every_16bit_attention_kernel_matches_oracle(bridge, name, variant):
    """Option attention16_kernel: 0 = one query tile per CTA; bit 0 = two query tiles per CTA, bit 1 = V consumed as an
    MN-major operand (no transposing pass), bit 2 = P kept in tensor memory, bit 3 = fp32 K / V rounded to the operand
    type inside the kernel (no staging pass at all for autocast graphs)."""
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    bridge.set_option("attention16_kernel", variant)
    try:
        got = realize_cuda(t, bridge)
    finally:
        bridge.set_option("attention16_kernel", -1)       # back to the library's default
    assert any(ln.startswith("attention_tc") for ln in bridge.last_plan_trace())
    check(case, got, want, f"{name} (attention16_kernel={variant})")


ATTN32_CASES = ["c4_attn_mask_d64", "c4_attn_causal_d64", "c4_attn_causal_tiles", "c4_attn_mask_tiles", "c4_attn_nomask_d64",
                "typed_attention_d64", "c4_attn_merge_heads", "c4_attn_growing_f32", "c4_attn_long_f32",
                # results stored as operand planes of the projection behind them; fp64-typed q / k / v stored as fp32
                "c4_attn_proj_planes", "c4_attn_block_f64"]


@pytest.mark.parametrize("variant", [0, 1, 3])
@pytest.mark.parametrize("name", ATTN32_CASES)
def test_every_3xtf32_attention_kernel_matches_oracle(bridge, name, variant):
    """Option attention32_kernel: 0 = two threads per query row, P through shared memory, P.V folded into registers
    every tile; 1 = one thread per row, P and O in tensor memory, O folded into registers every eighth tile; 3 = as 1, with
    fp32 Q and K rows split into hi / lo planes by converter warps of the kernel instead of a staging pass."""
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    bridge.set_option("attention32_kernel", variant)
    try:
        got = realize_cuda(t, bridge)
    finally:
        bridge.set_option("attention32_kernel", -1)
    assert any(ln.startswith("attention_tc_3xtf32") for ln in bridge.last_plan_trace())
    check(case, got, want, f"{name} (attention32_kernel={variant})")


@pytest.mark.parametrize("name", ["c3_tc_f32", "c3_tc_f16", "c3_tc_bf16", "c3_tc_ragged", "c3_tc_relu", "c3_tc_rowmajor_b",
                                  "c3_tc_f32_long_k"])
def test_cta_pair_gemm_matches_oracle(bridge, name):
    """The two-CTA (cta_group::2) kernel with 256 x 256, 256 x 192 and 256 x 128 tiles, forced on shapes with
    ragged edges in M, N and K."""
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    single = realize_cuda(t, bridge)
    bridge.set_option("gemm_cta_pairs", 2)
    try:
        for width in (256, 192, 128):
            bridge.set_option("gemm_pair_tile_width", width)
            got = realize_cuda(t, bridge)
            check(case, got, want, f"{name} (CTA pairs, {width} columns)")
            # same products, same accumulation order per output element: every tiling agrees to the bit
            assert got.tobytes() == single.tobytes(), width
    finally:
        bridge.set_option("gemm_cta_pairs", 1)
        bridge.set_option("gemm_pair_tile_width", 0)


@pytest.mark.parametrize("name,unit,members", [
    ("c3_group_qkv_f32", "gemm_tc_3xtf32+bias[float32] x3", 3),
    ("c3_group_pair_f32_long_k", "gemm_tc_3xtf32+bias[float32] x2", 2),
    ("c3_group_qkv_f16", "gemm_tc+bias[float16] x3", 3),
    ("c3_group_four_bf16", "gemm_tc+bias[bfloat16] x3", 3),
])
def test_projections_of_one_activation_launch_together(bridge, name, unit, members):
    """Linear layers that read the same activation (q / k / v) run as one CTA-pair launch whose grid holds the tiles
    of all of them; the activation is split / converted once.  Same products and order as separate launches."""
    case = CASES[name]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    for width in (0, 192):
        bridge.set_option("gemm_pair_tile_width", width)
        try:
            got = realize_cuda(t, bridge)
        finally:
            bridge.set_option("gemm_pair_tile_width", 0)
        trace = bridge.last_plan_trace()
        assert unit in trace and sum(ln.startswith("gemm_operands[") for ln in trace) == members - 1, trace
        assert sum(ln.startswith("convert16[") for ln in trace) <= 1, trace
        check(case, got, want, f"{name} (joint launch, width {width})")
    bridge.set_option("gemm_groups", 0)
    try:
        apart = realize_cuda(t, bridge)
        assert not any(ln.startswith("gemm_operands[") for ln in bridge.last_plan_trace())
    finally:
        bridge.set_option("gemm_groups", 1)
    assert got.tobytes() == apart.tobytes()


@pytest.mark.parametrize("name", ["c3_chain_relu_f32", "c3_chain_gelu_f64", "c3_chain_kept_hidden"])
def test_gemm_feeding_a_gemm(bridge, name):
    """Two chained Linear layers on tensor cores (the hidden activation is the A operand of the second GEMM, in fp32
    after relu and in fp64 after gelu), fused and unfused."""
    case = CASES[name]
    t, store, _ = build_case(case)
    got = realize_cuda(t, bridge)
    assert sum(ln.startswith("gemm_tc_3xtf32") for ln in bridge.last_plan_trace()) == 2, bridge.last_plan_trace()
    check(case, got, oracle_value(t, store), name)
    bridge.set_option("fusion", 0)
    try:
        plain = realize_cuda(t, bridge)
    finally:
        bridge.set_option("fusion", 1)
    check(case, plain, oracle_value(t, store), name + " (unfused)")


def test_autocast_attention_is_one_unit_and_keeps_mask_classes_with_the_handle(bridge):
    """The fp32 -> 16-bit casts of Q, K, V are folded into the operand staging of the fused kernel, and the
    mask tile classes computed for a mask bound by handle live exactly as long as that handle."""
    from browsergrad_b200 import release_resident_leaves
    case = CASES["c4_attn_mask_bf16"]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    base = bridge.resourceSnapshot()["currentBytes"]
    first = realize_cuda(t, bridge, resident_leaves=True)
    trace = bridge.last_plan_trace()
    assert trace == ["attention_tc+mask[bfloat16]"], trace
    held = bridge.resourceSnapshot()["currentBytes"]
    second = realize_cuda(t, bridge, resident_leaves=True)       # classes come from the cache this time
    assert bridge.resourceSnapshot()["currentBytes"] == held
    check(case, first, want, "autocast attention")
    assert first.tobytes() == second.tobytes()
    release_resident_leaves(bridge)
    assert bridge.resourceSnapshot()["currentBytes"] == base
    assert bridge.aliveHandleCount() == 0


@pytest.mark.parametrize("name,unit", [("c4_attn_merge_heads", "attention_tc_3xtf32+mask+merge[float32]"),
                                       ("c4_attn_merge_heads_bf16", "attention_tc+boolmask+merge[bfloat16]")])
def test_head_merge_after_attention_is_written_by_the_attention_kernel(bridge, name, unit):
    """permute(0, 2, 1, 3).reshape(...) of the attention result needs no copy: the kernel stores its rows at the
    merged layout's addresses."""
    case = CASES[name]
    t, store, _ = build_case(case)
    got = realize_cuda(t, bridge)
    trace = bridge.last_plan_trace()
    assert unit in trace and "copy[strided]" not in trace, trace
    check(case, got, oracle_value(t, store), "merged heads")


@pytest.mark.parametrize("bad", ["range", "duplicate"])
def test_scatter_refuses_what_the_reference_refuses(bridge, bad):
    """An index outside the axis, or two index entries naming one destination, end the plan with an index error
    (the reference raises RealizationError for both, _realize.py:1184-1186); the bridge stays usable."""
    from browsergrad_b200 import graph
    from browsergrad_b200.errors import KernelError
    store = graph.BufferStore()
    x = graph.from_numpy(np.zeros((4, 6), np.float32), store)
    idx = np.tile(np.arange(6, dtype=np.int64), (4, 1))
    if bad == "range":
        idx[2, 3] = 6
    else:
        idx[1, 0] = idx[1, 5]
    src = graph.from_numpy(np.ones((4, 6), np.float32), store)
    with pytest.raises(KernelError, match="scatter") as info:
        realize_cuda(x.scatter(1, graph.from_numpy(idx, store), src), bridge)
    assert info.value.status == 7
    good = np.tile(np.arange(6, dtype=np.int64)[::-1], (4, 1))
    got = realize_cuda(x.scatter(1, graph.from_numpy(np.ascontiguousarray(good), store), src), bridge)
    assert np.array_equal(got, np.ones((4, 6), np.float32))
    assert bridge.aliveHandleCount() == 0


def test_row_pipeline_equals_one_realization(bridge):
    """Row chunks streamed over three bridges of the device give the rows of one whole realization."""
    from browsergrad_b200 import CudaBridge, configs, graph
    from browsergrad_b200.sharded import cuda_row_pipeline
    arrays = configs.chain_inputs(1500, 1028)
    store = graph.BufferStore()
    t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}

    def build(tt):
        return {"y": configs.chain_y(graph, tt), "rowsum": configs.chain_rowsum(graph, tt),
                "rowsoftmax": configs.chain_rowsoftmax(graph, tt)}
    whole = {name: realize_cuda(root, bridge) for name, root in build(t).items()}
    lanes = [bridge, CudaBridge(0), CudaBridge(0)]
    try:
        pipe = cuda_row_pipeline(build, arrays, list(arrays), lanes, n_chunks=7)
        outs = {name: np.empty(shape, dtype) for name, (shape, dtype) in pipe.output_shapes().items()}
        for _ in range(2):
            pipe.run(outs)
            for name in whole:
                if name == "rowsum":      # small chunks take the generic row kernel: another summation order
                    np.testing.assert_allclose(outs[name], whole[name], rtol=1e-6)
                else:
                    assert outs[name].tobytes() == whole[name].tobytes(), name
        for lane in lanes:
            assert lane.aliveHandleCount() == 0
    finally:
        for lane in lanes[1:]:
            lane.close()


def test_weight_planes_live_and_die_with_their_handle(bridge):
    """A 3xTF32 Linear with resident leaves keeps the hi / lo planes of its weight with the weight's handle:
    the second realization allocates nothing new, releasing the leaves returns every byte."""
    from browsergrad_b200 import release_resident_leaves
    case = CASES["c3_tc_f32"]
    t, store, _ = build_case(case)
    want = oracle_value(t, store)
    base = bridge.resourceSnapshot()["currentBytes"]
    first = realize_cuda(t, bridge, resident_leaves=True)
    held = bridge.resourceSnapshot()["currentBytes"]
    second = realize_cuda(t, bridge, resident_leaves=True)
    assert bridge.resourceSnapshot()["currentBytes"] == held
    check(case, first, want, "resident linear")
    assert first.tobytes() == second.tobytes()
    release_resident_leaves(bridge)
    assert bridge.resourceSnapshot()["currentBytes"] == base


def test_autocast_linear_is_one_unit_and_keeps_the_weight_copy_with_its_handle(bridge):
    """The fp32 -> 16-bit casts of x and W leave the interpreter: x is converted by a vectorised unit, the converted weight lives
    with the weight's handle (second realization allocates nothing, release returns every byte)."""
    from browsergrad_b200 import release_resident_leaves
    for name, expect in (("c3_tc_bf16", ["convert16[bfloat16]", "gemm_tc+bias+gelu[bfloat16]"]),
                         ("c3_tc_f16", ["convert16[float16]", "gemm_tc+bias+gelu[float16]"])):
        case = CASES[name]
        t, store, _ = build_case(case)
        want = oracle_value(t, store)
        base = bridge.resourceSnapshot()["currentBytes"]
        first = realize_cuda(t, bridge, resident_leaves=True)
        assert bridge.last_plan_trace() == expect
        held = bridge.resourceSnapshot()["currentBytes"]
        second = realize_cuda(t, bridge, resident_leaves=True)
        assert bridge.resourceSnapshot()["currentBytes"] == held
        check(case, first, want, name)
        assert first.tobytes() == second.tobytes()
        third = realize_cuda(t, bridge)                  # leaves passed by value: converted into temporaries
        assert third.tobytes() == first.tobytes()
        release_resident_leaves(bridge)
        assert bridge.resourceSnapshot()["currentBytes"] == base
