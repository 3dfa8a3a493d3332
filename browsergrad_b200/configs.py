"""Seeded synthetic workloads: the five benchmark configurations as graph builders.

Each builder takes an ``api`` namespace (``browsergrad_b200.graph`` or an adapter over the
reference's ``browsergrad_jit``) so that one definition produces the graph for the CUDA
realizer, for the CPU oracle and for the reference itself.  Inputs come from
``np.random.default_rng(seed)`` with fixed seeds per tensor; sizes are parameters so the tests
run reduced shapes and the benchmark the full ones.
"""
from __future__ import annotations

from typing import Any, Dict, Tuple

import numpy as np


def _normal(seed: int, shape: Tuple[int, ...], std: float = 1.0) -> np.ndarray:
    a = np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)
    return a if std == 1.0 else (a * np.float32(std)).astype(np.float32)


def _uniform(seed: int, shape: Tuple[int, ...], bound: float) -> np.ndarray:
    return np.random.default_rng(seed).uniform(-bound, bound, shape).astype(np.float32)


def mlp_inputs(batch: int = 64, d_in: int = 784, d_h: int = 128, d_out: int = 10) -> Dict[str, np.ndarray]:
    return {
        "x": _normal(1, (batch, d_in)),
        "y": np.random.default_rng(2).integers(0, d_out, (batch,), dtype=np.int64),
        "w1": _uniform(3, (d_h, d_in), 1.0 / np.sqrt(d_in)),
        "b1": _uniform(4, (d_h,), 1.0 / np.sqrt(d_in)),
        "w2": _uniform(5, (d_out, d_h), 1.0 / np.sqrt(d_h)),
        "b2": _uniform(6, (d_out,), 1.0 / np.sqrt(d_h)),
    }


def mlp_loss(api: Any, t: Dict[str, Any]) -> Any:
    """Config 1: 784->128(ReLU)->10 + mean cross entropy."""
    h = api.relu(api.linear(t["x"], t["w1"], t["b1"]))
    return api.cross_entropy(api.linear(h, t["w2"], t["b2"]), t["y"])


def chain_inputs(rows: int = 16384, cols: int = 4096) -> Dict[str, np.ndarray]:
    return {k: _normal(s, (rows, cols)) for k, s in zip("abcd", (10, 11, 12, 13))}


def chain_y(api: Any, t: Dict[str, Any]) -> Any:
    """Config 2: y = relu(a*b+c) * exp(-d)."""
    return api.relu(t["a"] * t["b"] + t["c"]) * api.exp(-t["d"])


def chain_rowsum(api: Any, t: Dict[str, Any]) -> Any:
    return chain_y(api, t).sum(axis=-1)


def chain_rowsoftmax(api: Any, t: Dict[str, Any]) -> Any:
    return api.softmax(chain_y(api, t), dim=-1)


def linear_inputs(m: int, n: int, k: int) -> Dict[str, np.ndarray]:
    return {"x": _normal(20, (m, k)), "w": _uniform(21, (n, k), 1.0 / np.sqrt(k)),
            "bias": _uniform(22, (n,), 1.0 / np.sqrt(k))}


def linear_gelu(api: Any, t: Dict[str, Any], amp: str = "") -> Any:
    """Config 3: gelu(x @ W.T + bias); ``amp`` = "", "float16" or "bfloat16"."""
    if amp:
        with api.autocast(dtype=amp):
            return api.gelu(api.linear(t["x"], t["w"], t["bias"]))
    return api.gelu(api.linear(t["x"], t["w"], t["bias"]))


def attention_inputs(b: int = 16, h: int = 12, s: int = 2048, d: int = 64) -> Dict[str, np.ndarray]:
    return {"q": _normal(30, (b, h, s, d)), "k": _normal(31, (b, h, s, d)),
            "v": _normal(32, (b, h, s, d))}


def causal_mask(s: int) -> np.ndarray:
    return np.triu(np.full((s, s), -np.inf, dtype=np.float32), k=1)


def attention(api: Any, t: Dict[str, Any], variant: str = "mask", amp: str = "") -> Any:
    """Config 4: causal SDPA, as an additive -inf mask ("mask") or ``is_causal`` ("causal");
    ``amp`` = "", "float16" or "bfloat16" runs it under autocast."""
    if amp:
        with api.autocast(dtype=amp):
            return attention(api, t, variant)
    if variant == "mask":
        return api.scaled_dot_product_attention(t["q"], t["k"], t["v"], attn_mask=t["mask"])
    if variant == "causal":
        return api.scaled_dot_product_attention(t["q"], t["k"], t["v"], is_causal=True)
    return api.scaled_dot_product_attention(t["q"], t["k"], t["v"])


def gpt_inputs(layers: int = 12, d_model: int = 768, heads: int = 12, d_mlp: int = 3072,
               vocab: int = 32000, seq: int = 1024, batch: int = 8) -> Dict[str, np.ndarray]:
    """Config 5 weights ~N(0, 0.02), LN gamma=1 beta=0, token ids uniform."""
    t: Dict[str, np.ndarray] = {}
    ids = np.random.default_rng(40).integers(0, vocab, (batch, seq), dtype=np.int64)
    t["ids"] = ids
    # gather needs an index of the output's full shape: each row repeats the token id.
    t["tok_index"] = np.ascontiguousarray(np.broadcast_to(ids.reshape(-1, 1), (batch * seq, d_model)))
    pos = np.tile(np.arange(seq, dtype=np.int64), batch)
    t["pos_index"] = np.ascontiguousarray(np.broadcast_to(pos.reshape(-1, 1), (batch * seq, d_model)))
    seed = 41
    t["wte"] = _normal(seed, (vocab, d_model), 0.02); seed += 1
    t["wpe"] = _normal(seed, (seq, d_model), 0.02); seed += 1
    for i in range(layers):
        for name, shape in (("q_w", (d_model, d_model)), ("q_b", (d_model,)),
                            ("k_w", (d_model, d_model)), ("k_b", (d_model,)),
                            ("v_w", (d_model, d_model)), ("v_b", (d_model,)),
                            ("proj_w", (d_model, d_model)), ("proj_b", (d_model,)),
                            ("fc_w", (d_mlp, d_model)), ("fc_b", (d_mlp,)),
                            ("out_w", (d_model, d_mlp)), ("out_b", (d_model,))):
            t[f"l{i}.{name}"] = _normal(seed, shape, 0.02); seed += 1
        for name in ("ln1", "ln2"):
            t[f"l{i}.{name}_g"] = np.ones((d_model,), np.float32)
            t[f"l{i}.{name}_b"] = np.zeros((d_model,), np.float32)
    t["lnf_g"] = np.ones((d_model,), np.float32)
    t["lnf_b"] = np.zeros((d_model,), np.float32)
    t["mask"] = causal_mask(seq)
    t["_meta"] = np.array([layers, d_model, heads, d_mlp, vocab, seq, batch], dtype=np.int64)
    return t


def gpt_forward(api: Any, t: Dict[str, Any], meta: Tuple[int, ...], logits: bool = True, amp: str = "") -> Any:
    """Config 5: pre-LayerNorm GPT decoder forward built from gather, layer_norm, linear,
    scaled_dot_product_attention, gelu and residual adds; the LM head shares ``wte``.  ``amp`` = "", "float16" or
    "bfloat16" builds it under autocast."""
    if amp:
        with api.autocast(dtype=amp):
            return gpt_forward(api, t, meta, logits)
    layers, d_model, heads, d_mlp, vocab, seq, batch = (int(v) for v in meta)
    dh = d_model // heads
    x = t["wte"].gather(0, t["tok_index"]) + t["wpe"].gather(0, t["pos_index"])
    for i in range(layers):
        p = lambda n: t[f"l{i}.{n}"]
        h = api.layer_norm(x, (d_model,), p("ln1_g"), p("ln1_b"))
        q, k, v = (api.linear(h, p(n + "_w"), p(n + "_b")).reshape(batch, seq, heads, dh)
                   .permute(0, 2, 1, 3) for n in "qkv")
        a = api.scaled_dot_product_attention(q, k, v, attn_mask=t["mask"])
        a = a.permute(0, 2, 1, 3).reshape(batch * seq, d_model)
        x = x + api.linear(a, p("proj_w"), p("proj_b"))
        h = api.layer_norm(x, (d_model,), p("ln2_g"), p("ln2_b"))
        x = x + api.linear(api.gelu(api.linear(h, p("fc_w"), p("fc_b"))), p("out_w"), p("out_b"))
    x = api.layer_norm(x, (d_model,), t["lnf_g"], t["lnf_b"])
    if not logits:
        return x
    return api.linear(x, t["wte"])
