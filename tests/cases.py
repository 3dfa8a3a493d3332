"""Parity cases shared by the golden generator, the CPU tests and the GPU tests.

A case = seeded inputs + a builder that takes an ``api`` namespace, so the same definition
produces the reference's graph (``RefApi`` over ``browsergrad_jit``), this build's graph
(``browsergrad_b200.graph``) and the oracle's input.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List

import numpy as np

from browsergrad_b200 import configs


from oracle.ref_api import RefApi  # noqa: E402,F401  (the adapter lives beside the recipe that assembles the reference)


def canonical_arg(op: str, arg: Any) -> Any:
    if op == "BUFFER":
        return "buffer"
    if isinstance(arg, dict):
        return {k: canonical_arg("", v) for k, v in sorted(arg.items()) if k != "vjp_of"}
    if isinstance(arg, (tuple, list)):
        return [canonical_arg("", v) for v in arg]
    if isinstance(arg, slice):
        return ["slice", arg.start, arg.stop, arg.step]
    if isinstance(arg, float):
        return repr(arg)
    if isinstance(arg, (np.integer,)):
        return int(arg)
    if isinstance(arg, (np.floating,)):
        return repr(float(arg))
    return arg


def signature(order: List[Any]) -> List[Any]:
    pos = {id(n): i for i, n in enumerate(order)}
    return [[n.op, [pos[id(i)] for i in n.inputs], list(n.shape), n.dtype,
             canonical_arg(n.op, n.arg)] for n in order]


@dataclass
class Case:
    inputs: Callable[[], Dict[str, np.ndarray]]
    build: Callable[[Any, Dict[str, Any], Dict[str, np.ndarray]], Any]
    kind: str = "float"          # "float" (tolerance) or "exact" (bit-exact)
    rtol: float = 1e-5
    reference_has_it: bool = True
    floor_bits: Any = None       # overrides the k of the element-wise gate (tests/util.py); None = from the graph


def _rng(seed: int) -> np.random.Generator:
    return np.random.default_rng(seed)


def _misc_inputs() -> Dict[str, np.ndarray]:
    r = _rng(100)
    return {
        "x": r.standard_normal((6, 5, 33), dtype=np.float32),
        "p": (r.standard_normal((6, 5, 33), dtype=np.float32) ** 2 + np.float32(0.1)),
        "row": r.standard_normal((33,), dtype=np.float32),
        "col": r.standard_normal((5, 1), dtype=np.float32),
        "i": r.integers(-1000, 1000, (6, 5, 33), dtype=np.int64),
        "j": r.integers(-50, 50, (5, 33), dtype=np.int64),
        "i32": r.integers(-2 ** 30, 2 ** 30, (6, 5, 33), dtype=np.int32),
        "big": r.integers(-2 ** 62, 2 ** 62, (6, 5, 33), dtype=np.int64),
        "d": r.standard_normal((6, 5, 33)),
        "h": r.standard_normal((6, 5, 33)).astype(np.float16),
        "g": np.linspace(0.5, 1.5, 33, dtype=np.float32),
        "be": np.linspace(-0.2, 0.2, 33, dtype=np.float32),
        "table": r.standard_normal((17, 33), dtype=np.float32),
        "tidx": np.ascontiguousarray(np.broadcast_to(r.integers(0, 17, (9, 1), dtype=np.int64), (9, 33))),
        "cidx": r.integers(0, 33, (17, 4), dtype=np.int64),
        # rows of 36 four-byte values: the lookup kernel that moves four neighbours of a row at a time, with every
        # output row repeating one table row (an embedding lookup) and with a different table row per element
        "table36": r.standard_normal((17, 36), dtype=np.float32),
        "tidx36": np.ascontiguousarray(np.broadcast_to(r.integers(0, 17, (9, 1), dtype=np.int64), (9, 36))),
        "tidx36_mixed": r.integers(0, 17, (9, 36), dtype=np.int64),
        "bm": r.standard_normal((2, 1, 7, 9), dtype=np.float32),
        "bn": r.standard_normal((3, 9, 4), dtype=np.float32),
        "v9": r.standard_normal((9,), dtype=np.float32),
        "m79": r.standard_normal((7, 9), dtype=np.float32),
        "logits": r.standard_normal((12, 7), dtype=np.float32) * np.float32(3),
        "tgt": np.array([0, 6, 3, -100, 2, 2, 5, -100, 1, 0, 4, 6], dtype=np.int64),
        "perm_last": np.argsort(r.standard_normal((6, 5, 33)), axis=2).astype(np.int64),
        "perm_mid_part": np.argsort(r.standard_normal((6, 5, 33)), axis=1).astype(np.int64)[:, :3, :],
        "perm_first_i": np.argsort(r.standard_normal((6, 5, 33)), axis=0).astype(np.int64),
        "src_part": r.standard_normal((6, 3, 33), dtype=np.float32),
        "logits3": r.standard_normal((4, 7, 5), dtype=np.float32),
        "tgt3": r.integers(0, 7, (4, 5), dtype=np.int64),
        "cw": np.linspace(0.25, 2.0, 7, dtype=np.float32),
        "probs": _softmax_rows(r.standard_normal((12, 7), dtype=np.float32)),
    }


def _softmax_rows(a: np.ndarray) -> np.ndarray:
    e = np.exp(a - a.max(axis=1, keepdims=True))
    return (e / e.sum(axis=1, keepdims=True)).astype(a.dtype)


def _long_ce_inputs(rows: int, classes: int, dtype: Any = np.float32) -> Callable[[], Dict[str, np.ndarray]]:
    def make() -> Dict[str, np.ndarray]:
        r = _rng(700 + classes)
        tgt = r.integers(0, classes, (rows,), dtype=np.int64)
        tgt[rows // 2] = -100
        return {"logits": (r.standard_normal((rows, classes)) * 4).astype(dtype), "tgt": tgt,
                "cw": r.uniform(0.5, 1.5, (classes,)).astype(dtype),
                "probs": _softmax_rows(r.standard_normal((rows, classes)).astype(dtype))}
    return make


def _attn_small(b: int, h: int, s: int, d: int) -> Callable[[], Dict[str, np.ndarray]]:
    def make() -> Dict[str, np.ndarray]:
        t = configs.attention_inputs(b, h, s, d)
        t["mask"] = configs.causal_mask(s)
        return t
    return make


def _qkv_inputs(m: int, n: int, k: int) -> Callable[[], Dict[str, np.ndarray]]:
    def make() -> Dict[str, np.ndarray]:
        r = _rng(77)
        out = {"x": r.standard_normal((m, k), dtype=np.float32)}
        for name in "qkv":
            out["w" + name] = (r.standard_normal((n, k), dtype=np.float32) / np.float32(np.sqrt(k)))
            out["b" + name] = r.standard_normal((n,), dtype=np.float32) * np.float32(0.1)
        return out
    return make


def _qkv(api: Any, t: Dict[str, Any], names: str, amp: str = "") -> Any:
    def build() -> Any:
        return api.cat([api.linear(t["x"], t["w" + c], t["b" + c]) for c in names], 1)
    if amp:
        with api.autocast(dtype=amp):
            return build()
    return build()


def _mlp2_inputs() -> Dict[str, np.ndarray]:
    r = _rng(78)
    return {"x": r.standard_normal((264, 272), dtype=np.float32),
            "w1": r.standard_normal((300, 272), dtype=np.float32) / np.float32(16), "b1": r.standard_normal((300,), dtype=np.float32) * np.float32(0.1),
            "w2": r.standard_normal((272, 300), dtype=np.float32) / np.float32(17), "b2": r.standard_normal((272,), dtype=np.float32) * np.float32(0.1)}


def _split_chain_inputs() -> Dict[str, np.ndarray]:
    """Two Linears whose hidden width (304) lets the second product take the first one's result as operand planes
    stored by the producing kernel; rows for a LayerNorm and heads for an attention in front of a projection."""
    r = _rng(91)
    out = {"x": r.standard_normal((264, 272), dtype=np.float32), "y": r.standard_normal((264, 272), dtype=np.float32),
           "w1": r.standard_normal((304, 272), dtype=np.float32) / np.float32(16), "b1": r.standard_normal((304,), dtype=np.float32) * np.float32(0.1),
           "w2": r.standard_normal((272, 304), dtype=np.float32) / np.float32(17), "b2": r.standard_normal((272,), dtype=np.float32) * np.float32(0.1),
           "w1t": r.standard_normal((272, 304), dtype=np.float32) / np.float32(16), "w2t": r.standard_normal((304, 280), dtype=np.float32) / np.float32(17),
           "g": np.linspace(0.5, 1.5, 272, dtype=np.float32), "be": np.linspace(-0.2, 0.2, 272, dtype=np.float32),
           "wp": r.standard_normal((264, 256), dtype=np.float32) / np.float32(16), "bp": r.standard_normal((264,), dtype=np.float32) * np.float32(0.1)}
    for name in "qkv":
        out["w" + name] = r.standard_normal((320, 272), dtype=np.float32) / np.float32(16)
        out["b" + name] = r.standard_normal((320,), dtype=np.float32) * np.float32(0.1)
    out.update(configs.attention_inputs(2, 4, 192, 64))
    out["mask"] = configs.causal_mask(192)
    return out


def _f64_block_inputs() -> Dict[str, np.ndarray]:
    r = _rng(93)
    out = {"x": r.standard_normal((384, 256), dtype=np.float32), "mask": configs.causal_mask(192),
           "wp": r.standard_normal((264, 256), dtype=np.float32) / np.float32(16), "bp": r.standard_normal((264,), dtype=np.float32) * np.float32(0.1)}
    for name in "qkv":
        out["w" + name] = r.standard_normal((256, 256), dtype=np.float32) / np.float32(16)
        out["b" + name] = r.standard_normal((256,), dtype=np.float32) * np.float32(0.1)
    return out


def _f64_attention_block(api: Any, t: Dict[str, Any], keep_q: bool = False) -> Any:
    """q / k / v projections of a float64 activation (the GELU of an fp32 tensor, as after the first MLP of a decoder),
    heads split by views, attention, heads merged, output projection."""
    h = api.gelu(t["x"])
    q, k, v = (api.linear(h, t["w" + c], t["b" + c]).reshape(2, 192, 4, 64).permute(0, 2, 1, 3) for c in "qkv")
    o = api.scaled_dot_product_attention(q, k, v, attn_mask=t["mask"]).permute(0, 2, 1, 3).reshape(384, 256)
    out = api.linear(o, t["wp"], t["bp"])
    return api.cat([out, q.permute(0, 2, 1, 3).reshape(384, 256)], 1) if keep_q else out


def _ln_qkv_amp(api: Any, t: Dict[str, Any], amp: str, keep: bool) -> Any:
    with api.autocast(dtype=amp):
        h = api.layer_norm(t["x"] + t["y"], (272,), t["g"], t["be"])
        out = api.cat([api.linear(h, t["w" + c], t["b" + c]) for c in "qkv"], 1)
        return api.cat([out, h], 1) if keep else out


def _small_gemm_inputs(m: int, n: int, k: int) -> Callable[[], Dict[str, np.ndarray]]:
    def make() -> Dict[str, np.ndarray]:
        r = _rng(79 + m + n + k)
        return {"x": r.standard_normal((m, k), dtype=np.float32), "w": r.standard_normal((n, k), dtype=np.float32) / np.float32(k ** 0.5),
                "wt": r.standard_normal((k, n), dtype=np.float32) / np.float32(k ** 0.5), "bias": r.standard_normal((n,), dtype=np.float32)}
    return make


def _ln_inputs(rows: int, cols: int) -> Callable[[], Dict[str, np.ndarray]]:
    def make() -> Dict[str, np.ndarray]:
        r = _rng(300 + cols)
        return {
            "x": r.standard_normal((rows, cols), dtype=np.float32),
            "y": r.standard_normal((rows, cols), dtype=np.float32),
            "yd": r.standard_normal((rows, cols)),
            "bias": r.standard_normal((cols,), dtype=np.float32),
            "g": np.linspace(0.5, 1.5, cols, dtype=np.float32),
            "be": np.linspace(-0.2, 0.2, cols, dtype=np.float32),
        }
    return make


def _attn_growing(b: int, h: int, s: int, d: int) -> Callable[[], Dict[str, np.ndarray]]:
    """Keys whose scale grows along the sequence: the running row maximum keeps rising by many e-folds from
    one key tile to the next, which forces the fused kernels to rescale what they have accumulated."""
    def make() -> Dict[str, np.ndarray]:
        t = configs.attention_inputs(b, h, s, d)
        ramp = (1.0 + 40.0 * np.arange(s, dtype=np.float32) / s).reshape(1, 1, s, 1)
        t["k"] = (t["k"] * ramp).astype(np.float32)
        t["mask"] = configs.causal_mask(s)
        return t
    return make


def _sort_inputs() -> Dict[str, np.ndarray]:
    r = _rng(400)
    special = r.standard_normal((5, 40), dtype=np.float32)
    special[:, ::7] = np.nan
    special[:, 1::9] = 0.0
    special[:, 2::9] = -0.0
    special[:, 3::11] = np.inf
    special[:, 5::13] = -np.inf
    return {
        "x": r.standard_normal((4, 9, 37), dtype=np.float32),
        "d": r.standard_normal((6, 100)),
        "ties": r.integers(0, 4, (33, 50), dtype=np.int64),
        "special": special,
        "long": r.standard_normal((3, 3000), dtype=np.float32),
    }


def _gpt_tiny() -> Dict[str, np.ndarray]:
    return configs.gpt_inputs(layers=2, d_model=64, heads=4, d_mlp=128, vocab=211, seq=32, batch=2)


def _ln_stream(api: Any, t: Dict[str, Any], other: str, cols: int) -> Any:
    """Pre-LayerNorm block step: the residual stream h is both normalised and carried on."""
    h = t["x"] + (t[other] + t["bias"])
    return api.layer_norm(h, (cols,), t["g"], t["be"]) * t["g"] + h


CASES: Dict[str, Case] = {
    # -- the five configurations at sizes the CPU oracle finishes in well under a second ----
    "c1_mlp_ce": Case(lambda: configs.mlp_inputs(), lambda api, t, raw: configs.mlp_loss(api, t)),
    "c2_y": Case(lambda: configs.chain_inputs(64, 512), lambda api, t, raw: configs.chain_y(api, t)),
    "c2_rowsum": Case(lambda: configs.chain_inputs(64, 512),
                      lambda api, t, raw: configs.chain_rowsum(api, t)),
    "c2_rowsoftmax": Case(lambda: configs.chain_inputs(64, 512),
                          lambda api, t, raw: configs.chain_rowsoftmax(api, t)),
    "c2_y_ragged": Case(lambda: configs.chain_inputs(7, 37),
                        lambda api, t, raw: configs.chain_y(api, t)),
    "c2_rowsum_ragged": Case(lambda: configs.chain_inputs(7, 37),
                             lambda api, t, raw: configs.chain_rowsum(api, t)),
    "c2_rowsoftmax_ragged": Case(lambda: configs.chain_inputs(7, 37),
                                 lambda api, t, raw: configs.chain_rowsoftmax(api, t)),
    "c2_rowsoftmax_long": Case(lambda: configs.chain_inputs(3, 9001),
                               lambda api, t, raw: configs.chain_rowsoftmax(api, t)),
    # shapes large enough to take the specialised pattern kernels (warp-per-row sum, CTA-per-row softmax)
    "c2_y_static": Case(lambda: configs.chain_inputs(96, 1030),
                        lambda api, t, raw: configs.chain_y(api, t)),
    "c2_rowsum_static": Case(lambda: configs.chain_inputs(1280, 388),
                             lambda api, t, raw: configs.chain_rowsum(api, t)),
    "c2_rowsoftmax_static": Case(lambda: configs.chain_inputs(160, 1028),
                                 lambda api, t, raw: configs.chain_rowsoftmax(api, t)),
    "c3_linear_gelu": Case(lambda: configs.linear_inputs(96, 80, 72),
                           lambda api, t, raw: configs.linear_gelu(api, t)),
    "c3_linear_gelu_128": Case(lambda: configs.linear_inputs(256, 128, 192),
                               lambda api, t, raw: configs.linear_gelu(api, t)),
    "c3_linear_gelu_f16": Case(lambda: configs.linear_inputs(96, 80, 72),
                               lambda api, t, raw: configs.linear_gelu(api, t, "float16"), rtol=2e-2),
    "c3_linear_gelu_f16_128": Case(lambda: configs.linear_inputs(256, 128, 192),
                                   lambda api, t, raw: configs.linear_gelu(api, t, "float16"),
                                   rtol=2e-2),
    "c3_linear_gelu_bf16": Case(lambda: configs.linear_inputs(256, 128, 192),
                                lambda api, t, raw: configs.linear_gelu(api, t, "bfloat16"),
                                rtol=2e-2, reference_has_it=False),
    # large enough for the tensor-core GEMM (>= 2^24 multiply-adds), with ragged M / N tiles
    "c3_tc_f32": Case(lambda: configs.linear_inputs(256, 384, 320),
                      lambda api, t, raw: configs.linear_gelu(api, t)),
    "c3_tc_f16": Case(lambda: configs.linear_inputs(256, 384, 320),
                      lambda api, t, raw: configs.linear_gelu(api, t, "float16"), rtol=2e-2),
    "c3_tc_bf16": Case(lambda: configs.linear_inputs(256, 384, 320),
                       lambda api, t, raw: configs.linear_gelu(api, t, "bfloat16"), rtol=2e-2,
                       reference_has_it=False),
    # K = 1100: three accumulation chunks (16 + 16 + 3 blocks of 32) in the 3xTF32 kernels
    "c3_tc_f32_long_k": Case(lambda: configs.linear_inputs(264, 272, 1100),
                             lambda api, t, raw: configs.linear_gelu(api, t, "")),
    "c3_tc_ragged": Case(lambda: configs.linear_inputs(300, 264, 296),
                         lambda api, t, raw: api.linear(t["x"], t["w"], t["bias"])),
    "c3_tc_relu": Case(lambda: configs.linear_inputs(300, 264, 296),
                       lambda api, t, raw: api.relu(api.linear(t["x"], t["w"], t["bias"]))),
    "c3_tc_rowmajor_b": Case(lambda: configs.linear_inputs(256, 256, 256),
                             lambda api, t, raw: t["x"] @ t["w"]),
    "c3_group_qkv_f32": Case(_qkv_inputs(300, 272, 264), lambda api, t, raw: _qkv(api, t, "qkv")),
    "c3_group_pair_f32_long_k": Case(_qkv_inputs(264, 192, 1100), lambda api, t, raw: _qkv(api, t, "qk")),
    "c3_group_qkv_f16": Case(_qkv_inputs(300, 272, 264), lambda api, t, raw: _qkv(api, t, "qkv", "float16"), rtol=2e-2),
    "c3_group_four_bf16": Case(_qkv_inputs(520, 160, 264), lambda api, t, raw: _qkv(api, t, "qkvq", "bfloat16"), rtol=2e-2,
                               reference_has_it=False),
    "c3_chain_relu_f32": Case(_mlp2_inputs, lambda api, t, raw: api.linear(api.relu(api.linear(t["x"], t["w1"], t["b1"])), t["w2"], t["b2"])),
    "c3_chain_gelu_f64": Case(_mlp2_inputs, lambda api, t, raw: api.linear(api.gelu(api.linear(t["x"], t["w1"], t["b1"])), t["w2"], t["b2"])),
    # the hidden value only feeds the next product: the first kernel's epilogue stores its operand planes (tf32(x),
    # bf16(x), bf16(x - tf32(x))) instead of the value; likewise a LayerNorm and an attention in front of products
    "c3_chain_relu_planes": Case(_split_chain_inputs, lambda api, t, raw: api.linear(api.relu(api.linear(t["x"], t["w1"], t["b1"])), t["w2"], t["b2"])),
    "c3_chain_gelu_planes": Case(_split_chain_inputs, lambda api, t, raw: api.linear(api.gelu(api.linear(t["x"], t["w1"], t["b1"])), t["w2"], t["b2"])),
    "c3_chain_plain_planes": Case(_split_chain_inputs, lambda api, t, raw: (t["x"] @ t["w1t"]) @ t["w2t"]),
    "c3_chain_two_readers_planes": Case(_split_chain_inputs, lambda api, t, raw: (lambda h: api.cat(
        [api.linear(h, t["w2"], t["b2"]), h.reshape(2, 132, 304).reshape(264, 304) @ t["w2t"]], 1))(api.gelu(api.linear(t["x"], t["w1"], t["b1"])))),
    # the reader's rows (240) are a multiple of 8, the producer's (300) are not: the value keeps its plain store
    "c3_chain_reshaped_reader": Case(_mlp2_inputs, lambda api, t, raw: api.relu(api.linear(t["x"], t["w1"], t["b1"])).reshape(330, 240)
                                     @ t["w2"].reshape(340, 240).permute(1, 0)),
    "ln_then_linear_planes": Case(_split_chain_inputs, lambda api, t, raw: api.linear(
        api.layer_norm(t["x"] + t["y"], (272,), t["g"], t["be"]), t["w1"], t["b1"])),
    "ln_then_qkv_planes": Case(_split_chain_inputs, lambda api, t, raw: (lambda h: api.cat(
        [api.linear(h, t["w" + c], t["b" + c]) for c in "qkv"], 1))(api.layer_norm(t["x"] + t["y"], (272,), t["g"], t["be"]))),
    "c4_attn_proj_planes": Case(_split_chain_inputs, lambda api, t, raw: api.linear(
        configs.attention(api, t, "mask").permute(0, 2, 1, 3).reshape(2 * 192, 4 * 64), t["wp"], t["bp"])),
    # autocast: a LayerNorm whose rows only feed Linears stores them in the 16-bit type itself; one that something else
    # reads too keeps its fp32 store and the conversion pass
    "ln_then_qkv_f16": Case(_split_chain_inputs, lambda api, t, raw: _ln_qkv_amp(api, t, "float16", False), rtol=2e-2),
    "ln_then_qkv_bf16": Case(_split_chain_inputs, lambda api, t, raw: _ln_qkv_amp(api, t, "bfloat16", False), rtol=2e-2,
                             reference_has_it=False),
    "ln_then_qkv_f16_kept": Case(_split_chain_inputs, lambda api, t, raw: _ln_qkv_amp(api, t, "float16", True), rtol=2e-2),
    # fp64-typed q / k / v products read by nothing but the attention are stored as the fp32 values they hold; a
    # projection that something else reads too keeps its fp64 store
    "c4_attn_block_f64": Case(_f64_block_inputs, lambda api, t, raw: _f64_attention_block(api, t)),
    "c4_attn_block_f64_kept_q": Case(_f64_block_inputs, lambda api, t, raw: _f64_attention_block(api, t, True)),
    "c3_chain_kept_hidden": Case(_mlp2_inputs, lambda api, t, raw: (lambda h: api.cat([api.linear(h, t["w2"], t["b2"]), h], 1))(
        api.gelu(api.linear(t["x"], t["w1"], t["b1"])))),
    "c4_attn_mask": Case(_attn_small(2, 3, 64, 16),
                         lambda api, t, raw: configs.attention(api, t, "mask")),
    "c4_attn_causal": Case(_attn_small(2, 3, 64, 16),
                           lambda api, t, raw: configs.attention(api, t, "causal")),
    "c4_attn_mask_d64": Case(_attn_small(1, 2, 160, 64),
                             lambda api, t, raw: configs.attention(api, t, "mask")),
    "c4_attn_causal_d64": Case(_attn_small(1, 2, 160, 64),
                               lambda api, t, raw: configs.attention(api, t, "causal")),
    "c4_attn_causal_tiles": Case(_attn_small(2, 2, 320, 64),
                                 lambda api, t, raw: configs.attention(api, t, "causal")),
    "c4_attn_mask_tiles": Case(_attn_small(2, 2, 320, 64),
                               lambda api, t, raw: configs.attention(api, t, "mask")),
    "c4_attn_merge_heads": Case(_attn_small(2, 3, 200, 64),
                                lambda api, t, raw: configs.attention(api, t, "mask").permute(0, 2, 1, 3).reshape(2 * 200, 3 * 64) * 2.0),
    "c4_attn_merge_heads_bf16": Case(_attn_small(2, 2, 320, 64),
                                     lambda api, t, raw: configs.attention(api, t, "causal", "bfloat16").permute(0, 2, 1, 3).reshape(2, 320, 128),
                                     rtol=2e-2, reference_has_it=False),
    "c4_attn_nomask_d64": Case(_attn_small(1, 3, 200, 64),
                               lambda api, t, raw: configs.attention(api, t, "none")),
    "c4_attn_mask_f16": Case(_attn_small(2, 2, 320, 64),
                             lambda api, t, raw: configs.attention(api, t, "mask", "float16"), rtol=2e-2),
    "c4_attn_causal_f16": Case(_attn_small(1, 2, 160, 64),
                               lambda api, t, raw: configs.attention(api, t, "causal", "float16"), rtol=2e-2),
    "c4_attn_mask_bf16": Case(_attn_small(2, 2, 320, 64),
                              lambda api, t, raw: configs.attention(api, t, "mask", "bfloat16"), rtol=2e-2,
                              reference_has_it=False),
    "c4_attn_growing_f16": Case(_attn_growing(1, 2, 640, 64),
                                lambda api, t, raw: configs.attention(api, t, "none", "float16"), rtol=2e-2),
    "c4_attn_growing_causal_f16": Case(_attn_growing(1, 2, 640, 64),
                                       lambda api, t, raw: configs.attention(api, t, "mask", "float16"), rtol=2e-2),
    "c4_attn_growing_f32": Case(_attn_growing(1, 2, 640, 64),
                                lambda api, t, raw: configs.attention(api, t, "mask")),
    # 1280 keys = 20 key tiles of 64: crosses two folds of the tensor-memory accumulator into registers
    "c4_attn_long_f32": Case(_attn_growing(1, 1, 1280, 64), lambda api, t, raw: configs.attention(api, t, "mask")),
    "typed_attention_d64": Case(_attn_small(2, 2, 136, 64),
                                lambda api, t, raw: api.attention_forward(t["q"], t["k"], t["v"])),
    "c4_attn_full": Case(_attn_small(1, 2, 96, 32),
                         lambda api, t, raw: configs.attention(api, t, "none")),
    "c5_gpt_tiny": Case(_gpt_tiny, lambda api, t, raw: configs.gpt_forward(api, t, raw["_meta"]),
                        rtol=1e-4),
    "c5_gpt_tiny_f16": Case(_gpt_tiny, lambda api, t, raw: configs.gpt_forward(api, t, raw["_meta"], amp="float16"),
                            rtol=2e-2),
    "c5_gpt_tiny_bf16": Case(_gpt_tiny, lambda api, t, raw: configs.gpt_forward(api, t, raw["_meta"], amp="bfloat16"),
                             rtol=2e-2, reference_has_it=False),
    # -- single ops and edge cases -----------------------------------------------------
    "typed_attention": Case(_attn_small(2, 2, 40, 24),
                            lambda api, t, raw: api.attention_forward(t["q"], t["k"], t["v"])),
    "layer_norm": Case(_misc_inputs, lambda api, t, raw: api.layer_norm(t["x"], (33,), t["g"], t["be"])),
    # residual adds + bias feeding a layer norm: the warp-per-row kernel (cols % 4 == 0, <= 1024)
    "ln_residual_static": Case(_ln_inputs(75, 768), lambda api, t, raw: api.layer_norm(
        t["x"] + (t["y"] + t["bias"]), (768,), t["g"], t["be"])),
    "ln_plain_static": Case(_ln_inputs(9, 1024), lambda api, t, raw: api.layer_norm(t["x"], (1024,), t["g"], t["be"])),
    "ln_stream_static": Case(_ln_inputs(33, 200), lambda api, t, raw: _ln_stream(api, t, "y", 200)),
    "ln_stream_f64_static": Case(_ln_inputs(41, 520), lambda api, t, raw: _ln_stream(api, t, "yd", 520)),
    "layer_norm_2axes": Case(_misc_inputs, lambda api, t, raw: api.layer_norm(t["x"], (5, 33))),
    # -- data-movement and composite opcodes beyond the five configurations ----------------
    "tril_causal": Case(_misc_inputs, lambda api, t, raw: t["bm"].tril(), kind="exact"),
    "triu_diag2": Case(_misc_inputs, lambda api, t, raw: t["x"].triu(2), kind="exact"),
    "tril_int_neg": Case(_misc_inputs, lambda api, t, raw: t["i"].tril(-1), kind="exact"),
    "tril_of_permute": Case(_misc_inputs, lambda api, t, raw: t["x"].permute(0, 2, 1).tril(1), kind="exact"),
    "flip_last": Case(_misc_inputs, lambda api, t, raw: t["x"].flip(2), kind="exact"),
    "flip_first_int": Case(_misc_inputs, lambda api, t, raw: t["i"].flip(0), kind="exact"),
    "cat_rows": Case(_misc_inputs, lambda api, t, raw: api.cat([t["x"], t["p"], t["x"]], 0), kind="exact"),
    "cat_last_mixed": Case(_misc_inputs, lambda api, t, raw: api.cat([t["x"], t["d"]], 2), kind="exact"),
    "cat_then_sum": Case(_misc_inputs, lambda api, t, raw: api.cat([t["x"] * t["p"], t["x"] + t["row"]], 1).sum(axis=-1)),
    "stack_mid": Case(_misc_inputs, lambda api, t, raw: api.stack([t["x"], t["p"]], 1), kind="exact"),
    "prod_last": Case(_misc_inputs, lambda api, t, raw: t["p"].prod(-1)),
    "prod_mid_keepdims": Case(_misc_inputs, lambda api, t, raw: t["x"].prod(1, keepdims=True)),
    "prod_two_axes_f64": Case(_misc_inputs, lambda api, t, raw: t["d"].prod((0, 1))),
    "prod_after_chain": Case(_misc_inputs, lambda api, t, raw: (t["x"] * t["row"] + 1.0).prod(2)),
    "prod_int_wraps": Case(_misc_inputs, lambda api, t, raw: t["i"].prod(2), kind="exact"),
    "prod_int_first": Case(_misc_inputs, lambda api, t, raw: t["j"].prod(0), kind="exact"),
    "pad_last": Case(_misc_inputs, lambda api, t, raw: api.pad(t["x"], (2, 3)), kind="exact"),
    "pad_two_axes_value": Case(_misc_inputs, lambda api, t, raw: api.pad(t["x"], (1, 0, 0, 2), value=-1.5), kind="exact"),
    "pad_all_axes_int": Case(_misc_inputs, lambda api, t, raw: api.pad(t["i"], (0, 4, 3, 0, 1, 1), value=7), kind="exact"),
    "pad_f64_then_chain": Case(_misc_inputs, lambda api, t, raw: api.relu(api.pad(t["d"], (1, 1)) * 2.0)),
    "scatter_last_perm": Case(_misc_inputs, lambda api, t, raw: t["x"].scatter(2, t["perm_last"], t["p"]), kind="exact"),
    "scatter_mid_partial": Case(_misc_inputs, lambda api, t, raw: t["x"].scatter(1, t["perm_mid_part"], t["src_part"]), kind="exact"),
    "scatter_scalar_source": Case(_misc_inputs, lambda api, t, raw: t["x"].scatter(-2, t["perm_mid_part"], -2.5), kind="exact"),
    "scatter_int_first": Case(_misc_inputs, lambda api, t, raw: t["i"].scatter(0, t["perm_first_i"], t["big"]), kind="exact"),
    "scatter_then_chain": Case(_misc_inputs, lambda api, t, raw: api.relu(t["x"].scatter(2, t["perm_last"], t["p"]) * t["row"])),
    "cumsum_last": Case(_misc_inputs, lambda api, t, raw: api.cumsum(t["x"], 2), kind="exact"),
    "cumsum_first_int": Case(_misc_inputs, lambda api, t, raw: api.cumsum(t["i32"], 0), kind="exact"),
    "cumsum_mid_f64": Case(_misc_inputs, lambda api, t, raw: api.cumsum(t["d"], 1), kind="exact"),
    "clamp_both": Case(_misc_inputs, lambda api, t, raw: t["x"].clamp(-0.5, 0.75), kind="exact"),
    "clamp_min_chain": Case(_misc_inputs, lambda api, t, raw: (t["x"] * t["p"]).clamp(min=0.0) + t["row"]),
    "var_last": Case(_misc_inputs, lambda api, t, raw: t["x"].var(axis=-1)),
    "var_biased_keep": Case(_misc_inputs, lambda api, t, raw: t["x"].var(axis=(0, 2), keepdims=True, correction=0)),
    "var_all_f64": Case(_misc_inputs, lambda api, t, raw: t["d"].var()),
    # stable orderings: ties (small integer keys, repeated floats, signed zeros, NaNs) must keep their original order
    "sort_idx_last": Case(_sort_inputs, lambda api, t, raw: api.sort(t["x"], 2)[1], kind="exact"),
    "sort_val_desc_mid": Case(_sort_inputs, lambda api, t, raw: api.sort(t["x"], 1, True)[0], kind="exact"),
    "sort_idx_ties_desc": Case(_sort_inputs, lambda api, t, raw: api.sort(t["ties"], 1, True)[1], kind="exact"),
    "sort_idx_ties_first": Case(_sort_inputs, lambda api, t, raw: api.sort(t["ties"], 0)[1], kind="exact"),
    "sort_idx_special": Case(_sort_inputs, lambda api, t, raw: api.sort(t["special"], 1)[1], kind="exact"),
    "sort_idx_special_desc": Case(_sort_inputs, lambda api, t, raw: api.sort(t["special"], 1, True)[1], kind="exact"),
    "sort_idx_long": Case(_sort_inputs, lambda api, t, raw: api.sort(t["long"], 1)[1], kind="exact"),
    "sort_val_f64": Case(_sort_inputs, lambda api, t, raw: api.sort(t["d"], 1)[0], kind="exact"),
    "topk_val_last": Case(_sort_inputs, lambda api, t, raw: api.topk(t["x"], 5, 2)[0], kind="exact"),
    "topk_idx_smallest_mid": Case(_sort_inputs, lambda api, t, raw: api.topk(t["x"], 3, 1, False)[1], kind="exact"),
    "topk_then_softmax": Case(_sort_inputs, lambda api, t, raw: api.softmax(api.topk(t["long"], 64, 1)[0], dim=-1)),
    "repeat_tile": Case(_misc_inputs, lambda api, t, raw: t["x"].repeat(2, 1, 3), kind="exact"),
    "repeat_new_axis": Case(_misc_inputs, lambda api, t, raw: t["row"].repeat(4, 2), kind="exact"),
    "repeat_interleave_mid": Case(_misc_inputs, lambda api, t, raw: t["i"].repeat_interleave(3, 1), kind="exact"),
    "repeat_interleave_fused": Case(_misc_inputs, lambda api, t, raw: (t["x"] * t["p"]).repeat_interleave(2, 2) + 1.0),
    "gather_rows": Case(_misc_inputs, lambda api, t, raw: t["table"].gather(0, t["tidx"]), kind="exact"),
    "gather_rows_by4": Case(_misc_inputs, lambda api, t, raw: t["table36"].gather(0, t["tidx36"]), kind="exact"),
    "gather_rows_by4_mixed": Case(_misc_inputs, lambda api, t, raw: t["table36"].gather(0, t["tidx36_mixed"]), kind="exact"),
    "gather_cols": Case(_misc_inputs, lambda api, t, raw: t["table"].gather(1, t["cidx"]), kind="exact"),
    "int_arith": Case(_misc_inputs, lambda api, t, raw: (t["i"] * t["j"] + t["i"]) * 3 + (-t["j"]),
                      kind="exact"),
    "int_wrap64": Case(_misc_inputs, lambda api, t, raw: t["big"] * t["i"] + t["big"], kind="exact"),
    "int32_arith": Case(_misc_inputs, lambda api, t, raw: t["i32"] * t["i32"] + t["i32"], kind="exact"),
    "int_cmp_where": Case(_misc_inputs,
                          lambda api, t, raw: api.where(t["i"] > t["j"], t["i"], t["j"] * 2),
                          kind="exact"),
    "bool_cmp": Case(_misc_inputs, lambda api, t, raw: t["x"] >= t["row"], kind="exact"),
    "argmax_last": Case(_misc_inputs, lambda api, t, raw: t["x"].argmax(axis=-1), kind="exact"),
    "argmax_mid": Case(_misc_inputs, lambda api, t, raw: t["x"].argmax(axis=1), kind="exact"),
    "argmax_all": Case(_misc_inputs, lambda api, t, raw: t["x"].argmax(), kind="exact"),
    "int_sum": Case(_misc_inputs, lambda api, t, raw: t["i"].sum(axis=0), kind="exact"),
    "int_max_last": Case(_misc_inputs, lambda api, t, raw: t["i"].max(axis=-1), kind="exact"),
    "reduce_max_keep": Case(_misc_inputs, lambda api, t, raw: t["x"].max(axis=-1, keepdims=True),
                            kind="exact"),
    "reduce_min_axis0": Case(_misc_inputs, lambda api, t, raw: t["x"].min(axis=0), kind="exact"),
    "reduce_mean_mid": Case(_misc_inputs, lambda api, t, raw: t["x"].mean(axis=1)),
    "reduce_sum_all": Case(_misc_inputs, lambda api, t, raw: t["p"].sum()),
    "reduce_sum_two_axes": Case(_misc_inputs, lambda api, t, raw: t["p"].sum(axis=(0, 2))),
    "broadcast_chain": Case(_misc_inputs,
                            lambda api, t, raw: (t["x"] * t["row"] + t["col"]) / t["p"]),
    "log_exp": Case(_misc_inputs, lambda api, t, raw: (t["p"].log() * 0.5).exp()),
    "f64_chain": Case(_misc_inputs, lambda api, t, raw: (t["d"] * t["d"] + t["x"]).exp() / 3.0),
    # F.gelu of an fp32 value: Python scalars make its tail float64 under NumPy 2.  Without a float64 leaf in the plan
    # the tail is evaluated in fp32 and widened (inputs span the saturated ends: 9 * x); with one it stays float64.
    "gelu_f64_tail": Case(_misc_inputs, lambda api, t, raw: api.gelu(t["x"] * t["p"] + t["row"])),
    "gelu_f64_tail_wide": Case(_misc_inputs, lambda api, t, raw: api.gelu(t["x"] * 9.0)),
    "gelu_f64_tail_rows": Case(_misc_inputs, lambda api, t, raw: api.gelu(t["x"] * t["p"]).sum(axis=-1)),
    "gelu_f64_leaf": Case(_misc_inputs, lambda api, t, raw: api.gelu(t["x"] * t["p"]) + t["d"], rtol=1e-12),
    "f16_chain": Case(_misc_inputs, lambda api, t, raw: t["h"] * t["h"] + t["h"], rtol=2e-3),
    "cast_chain": Case(_misc_inputs,
                       lambda api, t, raw: (t["x"] * 100.0).cast("int32").cast("float32") + t["row"]),
    "cast_f16": Case(_misc_inputs, lambda api, t, raw: t["x"].cast("float16"), kind="exact"),
    "cast_bool": Case(_misc_inputs, lambda api, t, raw: t["j"].cast("bool"), kind="exact"),
    "softmax_mid_axis": Case(_misc_inputs, lambda api, t, raw: api.softmax(t["x"], dim=1)),
    "softmax_axis0": Case(_misc_inputs, lambda api, t, raw: api.softmax(t["x"], dim=0)),
    "permute_copy": Case(_misc_inputs, lambda api, t, raw: t["x"].permute(2, 0, 1), kind="exact"),
    "permute_add": Case(_misc_inputs, lambda api, t, raw: t["x"].permute(1, 0, 2) + t["row"]),
    "reshape_reduce": Case(_misc_inputs, lambda api, t, raw: t["x"].reshape(30, 33).sum(axis=0)),
    # 2-D fp32 products below the tensor-core threshold: the split-K kernel (32 x 32 tiles, ragged edges, one to many
    # K slices, a K that leaves a short last slice), with and without its folded bias / ReLU, row-major and transposed B
    "small_gemm_relu": Case(_small_gemm_inputs(70, 100, 300), lambda api, t, raw: api.relu(api.linear(t["x"], t["w"], t["bias"]))),
    "small_gemm_bias": Case(_small_gemm_inputs(33, 65, 1000), lambda api, t, raw: api.linear(t["x"], t["w"], t["bias"])),
    "small_gemm_plain": Case(_small_gemm_inputs(64, 10, 128), lambda api, t, raw: t["x"] @ t["wt"]),
    "small_gemm_one_slice": Case(_small_gemm_inputs(500, 300, 32), lambda api, t, raw: api.relu(t["x"] @ t["wt"] + t["bias"])),
    "small_gemm_kept_product": Case(_small_gemm_inputs(48, 40, 96),
                                    lambda api, t, raw: (lambda p: api.cat([api.relu(p + t["bias"]), p], 1))(t["x"] @ t["wt"])),
    "matmul_batched_bcast": Case(_misc_inputs, lambda api, t, raw: t["bm"] @ t["bn"]),
    "matmul_vec_rhs": Case(_misc_inputs, lambda api, t, raw: t["m79"] @ t["v9"]),
    "matmul_vec_lhs": Case(_misc_inputs, lambda api, t, raw: t["v9"] @ t["bn"]),
    "matmul_dot": Case(_misc_inputs, lambda api, t, raw: t["v9"] @ t["v9"]),
    "matmul_f64": Case(_misc_inputs, lambda api, t, raw: t["d"] @ t["d"].permute(0, 2, 1), rtol=1e-12),
    "matmul_int": Case(_misc_inputs, lambda api, t, raw: t["i"] @ t["i"].permute(0, 2, 1), kind="exact"),
    "relu_linear_relu": Case(lambda: configs.linear_inputs(33, 17, 129),
                             lambda api, t, raw: api.relu(api.linear(t["x"], t["w"], t["bias"]))),
    "linear_nobias_odd": Case(lambda: configs.linear_inputs(130, 70, 250),
                              lambda api, t, raw: api.linear(t["x"], t["w"])),
    "ce_mean_ignore": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"])),
    "ce_sum": Case(_misc_inputs,
                   lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], reduction="sum")),
    "ce_none": Case(_misc_inputs,
                    lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], reduction="none")),
    "ce_spatial": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits3"], t["tgt3"])),
    # (e^x - e^-x) / (e^x + e^-x): the numerator cancels near zero, so small outputs carry the absolute error of exp
    # class weights, label smoothing, probability targets (_framework_contracts.py:3756-3835)
    "ce_weight_mean": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], weight=t["cw"])),
    "ce_weight_sum": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], weight=t["cw"], reduction="sum")),
    "ce_weight_none": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], weight=t["cw"], reduction="none")),
    "ce_smooth": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], label_smoothing=0.1)),
    "ce_weight_smooth": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], weight=t["cw"], reduction="sum",
                                                                                 label_smoothing=0.25)),
    "ce_prob": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["probs"])),
    "ce_prob_smooth_weight": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits"], t["probs"], weight=t["cw"],
                                                                                      reduction="none", label_smoothing=0.2)),
    "ce_spatial_weight": Case(_misc_inputs, lambda api, t, raw: api.cross_entropy(t["logits3"], t["tgt3"], weight=t["cw"])),
    # long contiguous class axes: one CTA per position (vector loads; a class count that is no multiple of four;
    # float64; every optional term at once)
    "ce_long_row": Case(_long_ce_inputs(6, 4100), lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], reduction="none")),
    "ce_long_row_odd": Case(_long_ce_inputs(5, 1030), lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], label_smoothing=0.1)),
    "ce_long_row_f64": Case(_long_ce_inputs(3, 2050, np.float64),
                            lambda api, t, raw: api.cross_entropy(t["logits"], t["tgt"], weight=t["cw"], label_smoothing=0.3)),
    "ce_long_prob": Case(_long_ce_inputs(4, 4096), lambda api, t, raw: api.cross_entropy(t["logits"], t["probs"], weight=t["cw"],
                                                                                        label_smoothing=0.05)),
    "tanh": Case(_misc_inputs, lambda api, t, raw: api.tanh(t["x"]), floor_bits=0),
    "scalar_only": Case(_misc_inputs, lambda api, t, raw: t["row"].sum() * 2.0 + 1.0),
    "empty_rows": Case(lambda: {"a": np.zeros((0, 8), np.float32), "b": np.ones((0, 8), np.float32)},
                       lambda api, t, raw: api.relu(t["a"] * t["b"])),
    "prod_empty_axis": Case(lambda: {"a": np.zeros((0, 8), np.float32)}, lambda api, t, raw: t["a"].prod(0) + 1.0),
    "prod_empty_rows": Case(lambda: {"a": np.zeros((0, 8), np.float32)}, lambda api, t, raw: t["a"].prod(1), kind="exact"),
    "pad_empty_rows": Case(lambda: {"a": np.zeros((0, 8), np.float32)}, lambda api, t, raw: api.pad(t["a"], (1, 2, 2, 1), value=3.0),
                           kind="exact"),
    "scatter_empty_index": Case(lambda: {"a": np.arange(12, dtype=np.float32).reshape(3, 4), "i": np.zeros((0, 4), np.int64),
                                         "s": np.zeros((0, 4), np.float32)},
                                lambda api, t, raw: t["a"].scatter(0, t["i"], t["s"]), kind="exact"),
    # NARROW / SLICE: strided views on the device, built through the node constructor (no public builder emits them)
    "narrow_rows_chain": Case(_misc_inputs, lambda api, t, raw: api.relu(api.narrow(t["x"], 0, 2, 3) * 2.0)),
    "narrow_last_softmax": Case(_misc_inputs, lambda api, t, raw: api.softmax(api.narrow(t["x"], 2, 1, 32), dim=-1)),
    "narrow_root_copy": Case(_misc_inputs, lambda api, t, raw: api.narrow(t["x"], 1, 1, 3), kind="exact"),
    "narrow_int": Case(_misc_inputs, lambda api, t, raw: api.narrow(t["i"], 2, 5, 20),
                       kind="exact"),
    "narrow_empty": Case(_misc_inputs, lambda api, t, raw: api.narrow(t["x"], 1, 2, 0), kind="exact"),
    "slice_steps_root": Case(_misc_inputs, lambda api, t, raw: api.take_slice(t["x"], (slice(1, 6, 2), slice(None), slice(3, 33, 3))),
                             kind="exact"),
    "slice_rows_matmul": Case(_misc_inputs, lambda api, t, raw: api.take_slice(t["m79"], (slice(2, 7),)) @ t["bn"]),
    "slice_mid_rowsum": Case(_misc_inputs, lambda api, t, raw: api.take_slice(t["x"], (slice(None), slice(1, 4))).sum(-1)),
    "slice_then_reshape": Case(_misc_inputs, lambda api, t, raw: api.take_slice(t["x"], (slice(None), slice(0, 5, 2))).reshape(6, 99) + 1.0),
    "slice_undoes_pad": Case(_misc_inputs, lambda api, t, raw: api.take_slice(api.pad(t["x"], (1, 2), value=0.5),
                                                                          (slice(None), slice(None), slice(1, 34))), kind="exact"),
    "slice_of_permuted": Case(_misc_inputs, lambda api, t, raw: api.exp(api.take_slice(t["x"].permute(2, 0, 1), (slice(4, 20, 5), slice(1, 5))) * 0.5)),
    "single_element": Case(lambda: {"a": np.array([[2.5]], np.float32)},
                           lambda api, t, raw: api.softmax(t["a"] * t["a"], dim=-1)),
}
