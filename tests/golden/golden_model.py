"""The tiny models of the golden comparison: their sizes, their weights (a fixed function of a seed,
independent of the package's own random-weights writer), and the two namings of the same tensors: the
names of a model folder (``model.layers.N.self_attn.q_proj.weight``, ...) that the plain implementation
reads, and the GGUF names (``blk.N.attn_q.weight``, ...) that the reference's model reads
(src/infurnace/executor/tinygrad/model.py:97-148).  The reference has tied heads and full attention only,
so both models are tied and windowless."""
from __future__ import annotations

import torch

MODELS = {
    # 2 layers, 4 query heads over 2 key/value heads of 16
    "g1": dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
               intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
               tie_word_embeddings=True, max_position_embeddings=64, seed=101, tokens=40),
    # 3 layers, 6 query heads over 3 key/value heads of 48 (q width 288 != hidden 72), nothing a power of two
    "g2": dict(num_hidden_layers=3, hidden_size=72, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
               intermediate_size=136, vocab_size=333, rope_theta=500000.0, rms_norm_eps=3e-6,
               tie_word_embeddings=True, max_position_embeddings=48, seed=202, tokens=33),
}

_HF_TO_GGUF = {"self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
               "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm",
               "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate",
               "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}


def shapes(cfg):
    h, i, nq, nkv, d = (cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"],
                        cfg["num_key_value_heads"], cfg["head_dim"])
    out = {"model.embed_tokens.weight": (cfg["vocab_size"], h), "model.norm.weight": (h,)}
    for n in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{n}"
        out.update({f"{p}.self_attn.q_proj.weight": (nq * d, h), f"{p}.self_attn.k_proj.weight": (nkv * d, h),
                    f"{p}.self_attn.v_proj.weight": (nkv * d, h), f"{p}.self_attn.o_proj.weight": (h, nq * d),
                    f"{p}.self_attn.q_norm.weight": (d,), f"{p}.self_attn.k_norm.weight": (d,),
                    f"{p}.input_layernorm.weight": (h,), f"{p}.post_attention_layernorm.weight": (h,),
                    f"{p}.mlp.gate_proj.weight": (i, h), f"{p}.mlp.up_proj.weight": (i, h),
                    f"{p}.mlp.down_proj.weight": (h, i)})
    return out


def weights(cfg):
    """float32 tensors by model-folder name.  Matrices N(0, 0.08) (large enough that attention and the
    feed-forward matter in a model this narrow), norm weights 1 + N(0, 0.1), q_norm weights three times
    that, so that attention is peaked and a wrong key shows."""
    g = torch.Generator().manual_seed(cfg["seed"])
    out = {}
    for name, shape in sorted(shapes(cfg).items()):
        if len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
            if name.endswith("q_norm.weight"):
                t = t * 3.0
        else:
            t = 0.08 * torch.randn(shape, generator=g)
        out[name] = t
    return out


def tokens(cfg):
    g = torch.Generator().manual_seed(cfg["seed"] + 1)
    return torch.randint(0, cfg["vocab_size"], (cfg["tokens"],), generator=g).tolist()


def gguf_name(name):
    if name == "model.embed_tokens.weight":
        return "token_embd.weight"
    if name == "model.norm.weight":
        return "output_norm.weight"
    _, _, n, rest = name.split(".", 3)
    part, _ = rest.rsplit(".", 1)
    return f"blk.{n}.{_HF_TO_GGUF[part]}.weight"
