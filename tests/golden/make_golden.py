#!/usr/bin/env python3
"""Writes tests/golden/reference_logits.npz: the logits of the reference's own model code on two tiny models.

    python tests/golden/make_golden.py --reference-src <tylerguest/infurnace checkout>/src

The reference's model (src/infurnace/executor/tinygrad/model.py) is imported unmodified; tinygrad, which cannot
be installed here, is replaced by tests/golden/tinygrad_standin.py (see its header for what that does and does
not vouch for).  For each model of tests/golden/golden_model.py this records, in float32:

* ``<name>/whole``: the logits after every prefix of the token sequence, each computed by one call of
  ``Qwen3Model.forward(ids)`` without a cache (model.py:137-138): [tokens, vocab];
* ``<name>/cached``: the same places computed through the reference's cache (model.py:115-136): a prompt
  portion at position 0, a second portion on top of it, then one token per call; keys and values are stored
  in float16 as the reference stores them, so these differ from ``whole`` by that rounding: [places, vocab],
  with ``<name>/cached_places`` the positions.

tests/test_golden.py compares tests/plain_qwen3.py with this file.
"""
from __future__ import annotations

import argparse
import os
import sys
from types import MappingProxyType

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import golden_model as G          # noqa: E402
import tinygrad_standin           # noqa: E402


def reference_model(cfg, src):
    tg = tinygrad_standin.install()
    if src not in sys.path:
        sys.path.insert(0, src)
    from infurnace.executor.tinygrad.buffers import ContiguousKVCache
    from infurnace.executor.tinygrad.model import Qwen3Model
    from infurnace.executor.tinygrad.weights import Qwen3Weights, WeightPolicy
    from infurnace.models.config import Qwen3Config, TensorSpec
    w = G.weights(cfg)
    tensors = {G.gguf_name(k): tg.Tensor(v) for k, v in w.items()}
    specs = tuple(TensorSpec(n, tuple(t.shape), "F32", "float") for n, t in tensors.items())
    rc = Qwen3Config(architecture="qwen3", block_count=cfg["num_hidden_layers"], context_length=cfg["max_position_embeddings"],
                     embedding_length=cfg["hidden_size"], feed_forward_length=cfg["intermediate_size"],
                     attention_head_count=cfg["num_attention_heads"], attention_head_count_kv=cfg["num_key_value_heads"],
                     key_length=cfg["head_dim"], value_length=cfg["head_dim"], rope_dimension_count=cfg["head_dim"],
                     rope_freq_base=cfg["rope_theta"], rms_norm_epsilon=cfg["rms_norm_eps"], vocab_size=cfg["vocab_size"],
                     quantization_version=2, file_type=0, quantization="F32", qk_norm=True, attention_bias=False,
                     mlp_bias=False, tied_embeddings=True, mlp_type="swiglu", tensors=specs)
    tensors["output.weight"] = tensors["token_embd.weight"]          # tied: the same object (model.py:34-36)
    model = Qwen3Model(Qwen3Weights(rc, MappingProxyType(tensors), WeightPolicy.LAZY_FP16))
    return tg, model, lambda: ContiguousKVCache(rc, cfg["max_position_embeddings"], 2)


def run(cfg, src):
    tg, model, new_cache = reference_model(cfg, src)
    toks = G.tokens(cfg)
    ids = lambda t: tg.Tensor([t], dtype=tg.dtypes.int32)        # noqa: E731
    whole = torch.stack([model.forward(ids(toks[:n])).t[0] for n in range(1, len(toks) + 1)])
    cache = new_cache()
    first, second = len(toks) // 3, len(toks) // 3 + 7
    places, rows = [], []
    rows.append(model.prefill(ids(toks[:first]), cache, slot=1, start_position=0).t[0]); places.append(first - 1)
    rows.append(model.prefill(ids(toks[first:second]), cache, slot=1, start_position=first).t[0]); places.append(second - 1)
    for p in range(second, len(toks)):
        rows.append(model.decode(ids(toks[p:p + 1]), p, cache, slot=1).t[0]); places.append(p)
    return whole.float().numpy(), torch.stack(rows).float().numpy(), np.asarray(places, dtype=np.int32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True, help="the src folder of a tylerguest/infurnace checkout")
    ap.add_argument("--out", default=os.path.join(HERE, "reference_logits.npz"))
    args = ap.parse_args()
    out = {}
    for name, cfg in G.MODELS.items():
        whole, cached, places = run(cfg, os.path.abspath(args.reference_src))
        out[f"{name}/whole"], out[f"{name}/cached"], out[f"{name}/cached_places"] = whole, cached, places
        print(f"{name}: whole {whole.shape}, cached {cached.shape}, largest logit {np.abs(whole).max():.3f}, "
              f"cached against whole {np.abs(cached - whole[places]).max():.2e}")
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
