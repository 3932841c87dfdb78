"""A plain, slow implementation of the Qwen3 dense decoder, for tests only.

Whole sequences, no cache, no pages, no batching: every call recomputes the full
sequence with dense torch CPU operations in float32 (or float64).  It shares no code
with the package: it reads config.json with ``json`` and the weights with the
``safetensors`` library, and has one function for each part of the model.

It restates the formulas of the reference (paths within tylerguest/infurnace); each
function cites the lines it restates.  It is compared once with the reference's own model
file, src/infurnace/executor/tinygrad/model.py, run unmodified over a torch stand-in for the
tinygrad Tensor (tinygrad itself is neither installed here nor installable offline): the
outputs are stored under tests/golden/ with the script that made them, and
tests/test_golden.py holds this file to them (5e-6 on logits of size 2 to 3).

The window (a key at position k is visible to the query at position p when
0 <= p - k < window) has no counterpart in the reference, which has full attention only
(model.py:117-132); it is this engine's definition, stated here independently.
"""
from __future__ import annotations

import json
import math
import os

import torch


def read_model(model_dir, dtype=torch.float32):
    """config.json as a dict and all tensors widened to ``dtype``."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    for name in sorted(os.listdir(model_dir)):
        if name.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, name), framework="pt") as f:
                for k in f.keys():
                    tensors[k] = f.get_tensor(k).to(dtype)
    return cfg, tensors


def rms_norm(x, weight, eps):
    """x * rsqrt(mean(x^2, last axis) + eps) * weight; eps inside the root
    (src/infurnace/executor/tinygrad/model.py:11-13)."""
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def linear(x, weight):
    """x @ W^T with W stored [out, in] (model.py:15-16; tests/test_qwen3_model.py:97-102)."""
    return x @ weight.t()


def rope_table(head_dim, positions, theta, dtype):
    """cos and sin of position * theta^(-2i/d), i = 0 .. d/2-1 (model.py:18-22).
    The frequencies and angles are formed in float32 as the reference forms them."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.arange(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
    if dtype == torch.float64:
        ang = ang.double()
    return ang.cos(), ang.sin()


def apply_rope(x, cos, sin):
    """Half-split rotation: (x1*cos - x2*sin, x2*cos + x1*sin) with x1, x2 the two halves
    of the head (model.py:24-27; convention pinned by tests/test_qwen3_model.py:111-124).
    x: [heads, T, d]; cos, sin: [T, d/2]."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def attention(q, k, v, scale, window=None):
    """Causal grouped-query attention: softmax(q k^T * scale) v with the key at position j
    visible to the query at position p when j <= p (model.py:117-118,128-132); query head h
    uses key/value head h // (heads / kv_heads) (the grouped form that model.py:118 asks of
    its attention routine).  q: [nq, T, d]; k, v: [nkv, T, d].  Returns [nq, T, d]."""
    nq, T, d = q.shape
    group = nq // k.shape[0]
    k = k.repeat_interleave(group, dim=0)
    v = v.repeat_interleave(group, dim=0)
    scores = (q @ k.transpose(-1, -2)) * scale
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= (pos[:, None] - pos[None, :]) < window
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def attention_block(x, w, prefix, cfg, cos, sin, window):
    """q/k/v projections, head split, per-head RMSNorm of q and k, rotation, attention,
    head merge and output projection (model.py:102-114,140-143)."""
    T = x.shape[0]
    nq, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    eps = cfg.get("rms_norm_eps", 1e-6)
    q = linear(x, w[f"{prefix}.q_proj.weight"]).view(T, nq, d).transpose(0, 1)
    k = linear(x, w[f"{prefix}.k_proj.weight"]).view(T, nkv, d).transpose(0, 1)
    v = linear(x, w[f"{prefix}.v_proj.weight"]).view(T, nkv, d).transpose(0, 1)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = attention(q, k, v, 1.0 / math.sqrt(d), window)
    return linear(out.transpose(0, 1).reshape(T, nq * d), w[f"{prefix}.o_proj.weight"])


def mlp_block(x, w, prefix):
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z) (model.py:146-148)."""
    g = linear(x, w[f"{prefix}.gate_proj.weight"])
    u = linear(x, w[f"{prefix}.up_proj.weight"])
    return linear(g * torch.sigmoid(g) * u, w[f"{prefix}.down_proj.weight"])


def layer_windows(cfg):
    """The window of each layer (None: full attention), from config.json's own keys."""
    n = cfg["num_hidden_layers"]
    types = cfg.get("layer_types")
    if types is None:
        first = cfg.get("max_window_layers", n)
        on = cfg.get("use_sliding_window", False) and cfg.get("sliding_window") is not None
        types = ["sliding_attention" if on and i >= first else "full_attention" for i in range(n)]
    return [cfg["sliding_window"] if t == "sliding_attention" else None for t in types]


def forward(cfg, w, token_ids, dtype=torch.float32, return_hidden=False):
    """Logits [T, vocab] at every position of one whole sequence (model.py:90-151, except
    that the final norm and the head are applied to every row, not only to the last)."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    eps = cfg.get("rms_norm_eps", 1e-6)
    nq = cfg["num_attention_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    cos, sin = rope_table(d, len(ids), cfg.get("rope_theta", 10000.0), dtype)
    cos, sin = cos.to(dtype), sin.to(dtype)
    windows = layer_windows(cfg)
    x = w["model.embed_tokens.weight"][ids].to(dtype)                       # model.py:95
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        h = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)               # model.py:101
        x = x + attention_block(h, w, f"{p}.self_attn", cfg, cos, sin, windows[i])  # model.py:143
        h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)      # model.py:145
        x = x + mlp_block(h, w, f"{p}.mlp")                                  # model.py:148
    hidden = x
    x = rms_norm(x, w["model.norm.weight"], eps)                             # model.py:150
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    logits = linear(x, head)                                                 # model.py:151
    return (logits, hidden) if return_hidden else logits


def greedy(cfg, w, prompt, n, dtype=torch.float32):
    """n greedy tokens after ``prompt``: argmax of the last row, lowest index on ties
    (src/infurnace/sampler/greedy.py:21-22), recomputing the whole sequence each time."""
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(forward(cfg, w, ids, dtype)[-1]).item()))
    return ids[len(prompt):]


def temperature_probs(logits, temperature):
    """softmax(logits / temperature) in float32."""
    return torch.softmax(logits.float() / temperature, dim=-1)
