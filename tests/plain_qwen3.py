"""A plain, slow implementation of the Qwen3 dense decoder for the tests: whole sequences,
no cache, one function per part, float64 on the CPU by default.

It rests on the reference's formulas only: mashriram/llm-rs is Rust on top of the candle
crate and cannot be compiled or imported here (no Rust toolchain, no vendored crates),
so there is no golden output from the reference's own model code. Every function cites
the reference lines (paths within mashriram/llm-rs) it restates. It shares no code with
the package under test: it reads config.json with ``json`` and the weights with the
``safetensors`` package.

Two deliberate differences from the reference, which the engine shares: the rotation
pairs (x[i], x[i + d/2]) as the published Qwen3 weights assume (the reference pairs
(x[2i], x[2i+1]), llm-core/src/backends/attention.rs:216-233), and the per-head q/k
norms are always applied with eps = rms_norm_eps (the reference only finds them under
GGUF-derived names and fixes eps 1e-6, llm-core/src/graph/scan.rs:159-176,
llm-core/src/graph/builder.rs:130,144).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


def load_model_dir(model_dir: str, dtype=torch.float64):
    """config.json as a dict and every tensor of model.safetensors widened to ``dtype``."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def layer_windows(config: dict) -> List[int]:
    """Per layer: 0 = all earlier keys, w = the last w keys. The reference reads none of
    these keys; this follows the config.json fields of the architecture
    (use_sliding_window, sliding_window, max_window_layers, layer_types)."""
    L = config["num_hidden_layers"]
    w = config.get("sliding_window")
    if config.get("layer_types"):
        return [w if t == "sliding_attention" else 0 for t in config["layer_types"]]
    if config.get("use_sliding_window") and w:
        first = config.get("max_window_layers", L)
        first = L if first is None else first
        return [w if i >= first else 0 for i in range(L)]
    return [0] * L


def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """h0[t] = E[id_t], no scale: llm-core/src/graph/builder.rs:8-14,
    llm-core/src/backends/candle.rs:1238-1261."""
    return table[torch.as_tensor(list(ids), dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the last axis, plain weight:
    llm-core/src/backends/attention.rs:55-68,98-104."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(var + eps) * weight


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x @ W^T (+ b) with W stored [out, in]: llm-core/src/backends/candle.rs:1276-1340."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def rope_angles(positions: Sequence[int], head_dim: int, theta: float, dtype, device=None) -> torch.Tensor:
    """ang[t, i] = pos_t * theta^(-2i/d), i < d/2:
    llm-core/src/backends/attention.rs:178-214."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = float(theta) ** (-2.0 * i / head_dim)
    pos = torch.as_tensor(list(positions), dtype=torch.float64)
    return (pos[:, None] * inv_freq[None, :]).to(dtype).to(device)


def rotate_half(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d]. out[i] = x[i] cos_i - x[i+d/2] sin_i; out[i+d/2] = x[i+d/2] cos_i + x[i] sin_i.
    Same angles as llm-core/src/backends/attention.rs:216-233, pairing (i, i+d/2)."""
    half = x.shape[-1] // 2
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int = 0,
              scale: Optional[float] = None) -> torch.Tensor:
    """q: [T, nq, d], k, v: [T, nkv, d] -> [T, nq*d].
    Key head j serves query heads j*G..j*G+G-1 (llm-core/src/backends/attention.rs:240-248);
    scores / sqrt(d), -inf where key > query, softmax, times values
    (llm-core/src/backends/candle.rs:1587-1640). With ``window`` w > 0 a query at p sees
    keys p-w+1..p."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    G = nq // nkv
    kk = k.repeat_interleave(G, dim=1)
    vv = v.repeat_interleave(G, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, kk)
    s = s / math.sqrt(d) if scale is None else s * scale
    qi = torch.arange(T, device=q.device)[:, None]
    ki = torch.arange(T, device=q.device)[None, :]
    hidden = ki > qi
    if window and window > 0:
        hidden = hidden | (ki <= qi - window)
    s = s.masked_fill(hidden[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hqk,khd->qhd", p, vv)
    return o.reshape(T, nq * d)


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, config: dict, positions,
                    window: int, use_rope: bool = True) -> torch.Tensor:
    """Projections, per-head q/k norm before the rotation, rotation, attention, output
    projection: llm-core/src/graph/builder.rs:97-243."""
    nq, nkv = config["num_attention_heads"], config.get("num_key_value_heads", config["num_attention_heads"])
    d = config.get("head_dim") or config["hidden_size"] // nq
    eps = config.get("rms_norm_eps", 1e-5)
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).reshape(T, nq, d)
    k = linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).reshape(T, nkv, d)
    v = linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).reshape(T, nkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    if use_rope:
        ang = rope_angles(positions, d, config.get("rope_theta", 10000.0), x.dtype, x.device)
        q, k = rotate_half(q, ang), rotate_half(k, ang)
    o = attention(q, k, v, window)
    return linear(o, w[prefix + "o_proj.weight"], w.get(prefix + "o_proj.bias"))


def swiglu(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down( g * sigmoid(g) * u ), g = gate(x), u = up(x):
    llm-core/src/graph/builder.rs:256-297, llm-core/src/backends/candle.rs:1645-1663."""
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    return linear(g * torch.sigmoid(g) * u, w[prefix + "down_proj.weight"])


def decoder_layer(h: torch.Tensor, w, i: int, config: dict, positions, window: int, use_rope: bool = True):
    """h += attn(norm(h)); h += mlp(norm(h)): llm-core/src/graph/builder.rs:74-88,223-254,322-333."""
    p = f"model.layers.{i}."
    eps = config.get("rms_norm_eps", 1e-5)
    h = h + attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", config,
                            positions, window, use_rope)
    h = h + swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return h


def forward(config: dict, w: Dict[str, torch.Tensor], token_ids: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.
    Final norm and head: llm-core/src/graph/builder.rs:408-437; a tied head uses the
    embedding table (llm-core/src/backends/weights.rs:144-157)."""
    h = embedding(w["model.embed_tokens.weight"], token_ids)
    positions = list(range(len(token_ids)))
    windows = layer_windows(config)
    no_rope = config.get("no_rope_layers") or [False] * config["num_hidden_layers"]
    for i in range(config["num_hidden_layers"]):
        h = decoder_layer(h, w, i, config, positions, windows[i], not no_rope[i])
    h = rms_norm(h, w["model.norm.weight"], config.get("rms_norm_eps", 1e-5))
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head)


# ---------------------------------------------------------------------------------------
# Sampling
# ---------------------------------------------------------------------------------------
def philox4x32_10(key, counter):
    """Philox4x32 with 10 rounds (Salmon et al., SC'11), on Python integers."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, \
                         ((p0 >> 32) ^ c3 ^ k1) & 0xFFFFFFFF, p0 & 0xFFFFFFFF
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def uniform(seed: int, request_id: int, index: int) -> float:
    """The engine's draw for (seed, request, index of the generated token): 24 bits in [0, 1)."""
    r = philox4x32_10((seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF),
                      (request_id & 0xFFFFFFFF, (request_id >> 32) & 0xFFFFFFFF, index & 0xFFFFFFFF, 0))
    return (r[0] >> 8) / 16777216.0


def kept_probabilities(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0,
                       repetition_penalty: float = 1.0, history: Sequence[int] = ()) -> np.ndarray:
    """The distribution the sampler draws from (zeros for tokens that were cut), in the
    order of llm-core/src/sampler.rs:36-124: repetition penalty on distinct history
    tokens (divide if positive else multiply), temperature, softmax, top-k, top-p, each
    cut followed by renormalisation. Ties at a cut-off value are all kept."""
    x = np.asarray(logits, dtype=np.float64).copy()
    if repetition_penalty != 1.0:
        for t in set(int(t) for t in history):
            if 0 <= t < len(x):
                x[t] = x[t] / repetition_penalty if x[t] > 0 else x[t] * repetition_penalty
    x = x / temperature
    p = np.exp(x - x.max())
    p /= p.sum()
    if 0 < top_k < len(p):
        kth = np.sort(p)[::-1][top_k - 1]
        p = np.where(p >= kth, p, 0.0)
        p /= p.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cum = np.cumsum(p[order])
        n = int(np.searchsorted(cum, top_p, side="left")) + 1  # smallest prefix with mass >= top_p
        cut = p[order[min(n, len(p)) - 1]]
        p = np.where(p >= cut, p, 0.0)
        p /= p.sum()
    return p


def sample(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0,
           repetition_penalty: float = 1.0, history: Sequence[int] = (), seed: int = 0, request_id: int = 0,
           index: int = 0) -> int:
    """Greedy when temperature <= 1e-5 (first maximum, llm-core/src/sampler.rs:40-49), else a
    draw in vocabulary order from ``kept_probabilities`` with the Philox uniform."""
    x = np.asarray(logits, dtype=np.float64).copy()
    if temperature <= 1e-5:
        if repetition_penalty != 1.0:
            for t in set(int(t) for t in history):
                if 0 <= t < len(x):
                    x[t] = x[t] / repetition_penalty if x[t] > 0 else x[t] * repetition_penalty
        return int(np.argmax(x))
    p = kept_probabilities(logits, temperature, top_k, top_p, repetition_penalty, history)
    u = uniform(seed, request_id, index)
    cum = np.cumsum(p)
    return int(min(np.searchsorted(cum, u * cum[-1], side="right"), len(p) - 1))


def greedy_generate(config: dict, w, prompt: Sequence[int], n_new: int) -> List[int]:
    """Whole-sequence recomputation for every new token (no cache)."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward(config, w, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


def greedy_gap(config: dict, w, prompt: Sequence[int], generated: Sequence[int]) -> float:
    """How far the tokens someone else generated greedily are from this implementation's
    choice: the largest (max logit - logit of the generated token) along the sequence.
    0 means the same tokens; a reduced-precision engine may pick another token only where
    two logits are closer than its rounding."""
    ids = list(prompt) + list(generated)
    logits = forward(config, w, ids[:-1])
    worst = 0.0
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        worst = max(worst, float(row.max() - row[tok]))
    return worst
