"""CPU: the C-ABI library loads, exports every symbol ``include/bgcuda.h`` declares, refuses to
create a context without a GPU, and its plan compiler lowers every parity case (dry run)."""
import ctypes as C
import os
import re

import pytest

from browsergrad_b200 import _lib, front, wire
from browsergrad_b200.errors import JitNotImplementedError, KernelError
from tests.cases import CASES
from tests.util import build_case

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "bgcuda.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bg_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in bgcuda.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.bg_abi_version() == 1


def test_struct_layout_matches_header():
    assert C.sizeof(_lib.PlanStep) == 4 * 4 + 8 * 8 + 4 * 8 + 8 * 8 + 2 * 8 + 2 * 4
    assert C.sizeof(_lib.PlanInput) == 32
    assert C.sizeof(_lib.ResourceStats) == 72


def dry(plan, fusion=1):
    lib = _lib.load()
    ep = wire.encode_plan(plan)
    buf = C.create_string_buffer(1 << 16)
    rc = lib.bg_compile_plan_dry(C.byref(ep.plan), fusion, buf, len(buf))
    return rc, [ln for ln in buf.value.decode().split("\n") if ln]


@pytest.mark.parametrize("name", sorted(CASES))
def test_plan_compiler_lowers_case(name):
    t, store, _ = build_case(CASES[name])
    _, plan = front.plan_for(t._uop)
    rc, lines = dry(plan)
    assert rc == 0, lines
    assert lines
    rc2, lines2 = dry(plan, fusion=0)
    assert rc2 == 0, lines2
    assert len(lines2) >= len(lines)


def test_config2_chains_compile_to_one_kernel_each():
    for name, kind in (("c2_y", "ew["), ("c2_rowsum", "row["), ("c2_rowsoftmax", "row[")):
        t, _, _ = build_case(CASES[name])
        _, plan = front.plan_for(t._uop)
        rc, lines = dry(plan)
        assert rc == 0 and len(lines) == 1 and lines[0].replace("static_", "").startswith(kind), lines


def test_full_size_config2_takes_the_pattern_kernels():
    import numpy as np
    from browsergrad_b200 import configs, graph
    store = graph.BufferStore()
    t = {k: graph.from_numpy(np.zeros((16384, 4096), np.float32), store) for k in "abcd"}
    for build in (configs.chain_y, configs.chain_rowsum, configs.chain_rowsoftmax):
        _, plan = front.plan_for(build(graph, t)._uop)
        rc, lines = dry(plan)
        assert rc == 0 and len(lines) == 1 and lines[0].startswith("static_"), lines


def test_autocast_decoder_block_leaves_nothing_on_the_interpreter():
    """The casts the AMP pass inserts around every MATMUL are removed or absorbed by the plan compiler: a decoder block
    built under autocast lowers to tensor-core GEMMs (bias + GELU + narrowing cast in the epilogue, q / k / v as one
    grid), the fused attention and the specialised LayerNorm kernel, which stores its rows in the 16-bit type the next
    Linears read (no conversion pass of its own)."""
    import collections
    from browsergrad_b200 import configs, graph
    arrays = configs.gpt_inputs(layers=2, batch=8)
    meta = arrays.pop("_meta")
    store = graph.BufferStore()
    t = {k: graph.from_numpy(v, store) for k, v in arrays.items()}
    for amp in ("float16", "bfloat16"):
        _, plan = front.plan_for(configs.gpt_forward(graph, t, meta, amp=amp)._uop)
        rc, lines = dry(plan, fusion=3)
        assert rc == 0, lines
        units = collections.Counter(lines)
        assert not any(ln.startswith(("ew[", "row[")) for ln in lines), units
        assert units[f"gemm_tc+bias+gelu[{amp}]"] == 2 and units[f"gemm_tc+bias[{amp}] x3"] == 2, units
        assert units[f"attention_tc+mask+merge[{amp}]"] == 2 and units["static_row[CAST,ADD,ADD|LAYER_NORM]+cast16"] == 4, units
        assert not any(ln.startswith("convert16") for ln in lines), units


def test_small_fp32_products_take_the_split_k_kernel_with_their_epilogue():
    for name, expect in (("small_gemm_relu", ["gemm_small+bias+relu[float32]"]), ("small_gemm_bias", ["gemm_small+bias[float32]"]),
                         ("small_gemm_plain", ["gemm_small[float32]"]), ("c1_mlp_ce", None)):
        t, _, _ = build_case(CASES[name])
        _, plan = front.plan_for(t._uop)
        rc, lines = dry(plan, fusion=3)
        assert rc == 0, lines
        if expect is not None:
            assert lines == expect, lines
        else:
            assert lines == ["gemm_small+bias+relu[float32]", "gemm_small+bias[float32]", "cross_entropy"], lines


def test_values_read_only_by_products_leave_their_producer_in_the_operand_format():
    """A value that nothing but split products read (as their dense A operand, K a multiple of 8) is stored by its
    producer as those products' operand planes (+split); LayerNorm rows that only autocast Linears read are stored in
    their 16-bit type (+cast16, no convert16 unit); fp64-typed products that only a fused fp32 attention reads are
    stored as the fp32 numbers they hold (+f32store).  A second reader of another kind keeps the plain store."""
    expect = {
        "c3_chain_relu_planes": ["gemm_tc_3xtf32+bias+relu+split[float32]", "gemm_tc_3xtf32+bias[float32]"],
        "c3_chain_gelu_planes": ["gemm_tc_3xtf32+bias+gelu+split[float32]", "gemm_tc_3xtf32+bias[float64]"],
        "c3_chain_plain_planes": ["gemm_tc_3xtf32+split[float32]", "gemm_tc_3xtf32[float32]"],
        "c3_chain_gelu_f64": ["gemm_tc_3xtf32+bias+gelu[float32]", "gemm_tc_3xtf32+bias[float64]"],     # K = 300: fp32 residual planes
        "c3_chain_kept_hidden": ["gemm_tc_3xtf32+bias+gelu[float32]", "gemm_tc_3xtf32+bias[float64]", "place[CONCAT]"],
        "ln_then_linear_planes": ["static_row[ADD|LAYER_NORM]+split", "gemm_tc_3xtf32+bias[float32]"],
        "c4_attn_proj_planes": ["attention_tc_3xtf32+mask+merge[float32]+split", "gemm_tc_3xtf32+bias[float32]"],
    }
    for name, want in expect.items():
        t, _, _ = build_case(CASES[name])
        _, plan = front.plan_for(t._uop)
        rc, lines = dry(plan, fusion=3)
        assert rc == 0 and lines == want, (name, lines)
    for name, has, has_not in (("ln_then_qkv_planes", "static_row[ADD|LAYER_NORM]+split", "split["),
                               ("ln_then_qkv_f16", "static_row[ADD|LAYER_NORM]+cast16", "convert16"),
                               ("ln_then_qkv_f16_kept", "convert16[float16]", "+cast16"),
                               ("c4_attn_block_f64", "gemm_tc_3xtf32+bias+f32store[float64]", "convert16"),
                               ("c4_attn_block_f64_kept_q", "gemm_tc_3xtf32+bias[float64] x2", "convert16")):
        t, _, _ = build_case(CASES[name])
        _, plan = front.plan_for(t._uop)
        rc, lines = dry(plan, fusion=3)
        assert rc == 0 and has in lines and not any(has_not in ln for ln in lines), (name, lines)


def test_unsupported_opcode_mentions_numpy_fallback():
    plan = {"step_count": 1, "root_id": 0, "steps": [
        {"step": 0, "value_id": 0, "op": "CONV2D", "input_ids": [], "shape": [1], "dtype": "float32", "arg": None}]}
    with pytest.raises(JitNotImplementedError, match=r"bg\.realize\(\)"):
        wire.encode_plan(plan)


def test_malformed_plans_are_refused():
    t, _, _ = build_case(CASES["c2_y"])
    _, plan = front.plan_for(t._uop)
    bad = dict(plan, root_id=10 ** 6)
    with pytest.raises(KernelError):
        wire.encode_plan(bad)
    bad = dict(plan, steps=[dict(s) for s in plan["steps"]])
    bad["steps"][3]["value_id"] = 99
    with pytest.raises(KernelError):
        wire.encode_plan(bad)
    # an input that does not precede its user is caught by the compiler
    bad = dict(plan, steps=[dict(s) for s in plan["steps"]])
    for s in bad["steps"]:
        if s["op"] == "MUL":
            s["input_ids"] = [len(bad["steps"]) - 1, s["input_ids"][1]]
            break
    rc, lines = dry(bad)
    assert rc != 0 and "precede" in lines[0]


def test_semantic_requests_validation():
    from browsergrad_b200 import graph
    import numpy as np
    st = graph.BufferStore()
    x = graph.from_numpy(np.zeros((3, 5), np.float32), st)
    _, plan = front.plan_for(x.permute(1, 0)._uop)
    vid = [s["value_id"] for s in plan["steps"] if s["op"] == "PERMUTE"][0]
    import json
    ok = {"schema": wire.SEMANTIC_SCHEMA, "version": {"major": 1, "minor": 0},
          "requests": [{"kind": wire.VIEW_COPY_KIND, "valueId": vid, "inputShape": ["3", "5"], "axes": [1, 0],
                        "dtype": "f32"}]}
    assert wire.validate_semantic_requests(plan, json.dumps(ok)) == {vid: (1, 0)}
    for mutate in (lambda d: d.update(schema="x"), lambda d: d["requests"][0].update(axes=[0, 0]),
                   lambda d: d["requests"][0].update(inputShape=["5", "3"]),
                   lambda d: d["requests"][0].update(valueId=0)):
        bad = json.loads(json.dumps(ok))
        mutate(bad)
        with pytest.raises(KernelError):
            wire.validate_semantic_requests(plan, json.dumps(bad))


def test_no_gpu_means_loud_failure():
    import ctypes
    lib = _lib.load()
    ctx = ctypes.c_void_p()
    rc = lib.bg_create(0, ctypes.byref(ctx))
    if rc == 0:
        lib.bg_destroy(ctx)
        pytest.skip("a GPU is present")
    from browsergrad_b200 import CudaBridge
    with pytest.raises(KernelError, match="no CPU fallback"):
        CudaBridge(0)


def _lines_for(name, flags=3):
    t, _, _ = build_case(CASES[name])
    _, plan = front.plan_for(t._uop)
    rc, lines = dry(plan, fusion=flags)
    assert rc == 0, lines
    return lines


def test_b200_lowering_of_linear_and_attention():
    """With tensor-core kernels selectable the Linear cases fold their epilogue into one GEMM and the
    SDPA graphs collapse into one attention kernel."""
    assert _lines_for("c3_tc_f32") == ["gemm_tc_3xtf32+bias+gelu[float32]"]
    assert _lines_for("c3_tc_relu") == ["gemm_tc_3xtf32+bias+relu[float32]"]
    assert _lines_for("c3_tc_ragged") == ["gemm_tc_3xtf32+bias[float32]"]
    f16 = _lines_for("c3_tc_f16")
    assert f16[-1] == "gemm_tc+bias+gelu[float16]" and all(ln.startswith(("ew[CAST", "static_ew[CAST", "convert16[")) for ln in f16[:-1]), f16
    assert _lines_for("c4_attn_mask_d64") == ["attention_tc_3xtf32+mask[float32]"]
    assert _lines_for("c4_attn_causal_tiles") == ["attention_tc_3xtf32+boolmask[float32]"]
    assert _lines_for("typed_attention_d64") == ["attention_tc_3xtf32[float32]"]
    amp = _lines_for("c4_attn_mask_f16")
    assert amp[-1] == "attention_tc+mask[float16]", amp
    # head dimension 16 is outside the fused kernel: composed path
    assert any(ln.startswith("gemm_simt") for ln in _lines_for("c4_attn_mask"))
