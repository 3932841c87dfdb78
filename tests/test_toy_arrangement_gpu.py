"""Other arrangements of the same parts, defined here and registered from outside: a block whose mixer
and feed-forward read one norm and are added together (parallel residual), a block that normalises after
the addition (post-norm), an embedding with a scale, and a head whose logits are soft-capped.  Nothing
under infurnace_b200/ is changed for them: a block, an embedding and a head are parts like any other,
built from their spec by the registry, and the decoder only knows their ``forward``.  They are test
devices, not a model of anyone's.

The model is stepped through the engine's own step function whole, in portions and mixed with other
requests (pages reused), in 32-bit and in bfloat16, and compared with a plain whole-sequence computation."""
from dataclasses import asdict, dataclass
from typing import Mapping

import pytest
import torch

import plain_qwen3 as P
import tiny
from infurnace_b200.config.specs import (AttentionSpec, GatedMLPSpec, LayerCall, ModelPlan, RMSNormSpec, RotarySpec,
                                         TensorSpec)
from infurnace_b200.engine import EngineOptions, build_runner
from infurnace_b200.models import register_architecture
from infurnace_b200.parts import build_part, register_part
from infurnace_b200.weights.random_init import write_random_model

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ the parts
@dataclass(frozen=True)
class ScaledEmbeddingSpec:
    """x[t] = table[id_t] * scale."""
    vocab_size: int
    hidden_size: int
    weight: str
    scale: float

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


class ScaledEmbedding:
    def __init__(self, spec, weights, runtime):
        self.spec, self.table, self.k = spec, weights[spec.weight], runtime.kernels

    def forward(self, ids, out):
        self.k.embed(self.table, ids, out)          # the framework's kernel, then the scale in place
        out.mul_(self.spec.scale)
        return out


@dataclass(frozen=True)
class CappedHeadSpec:
    """logits = cap * tanh(h W^T / cap), W a tensor of its own."""
    vocab_size: int
    hidden_size: int
    weight: str
    cap: float
    tied: bool = False
    stored_as: object = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


class CappedHead:
    def __init__(self, spec, weights, runtime):
        self.spec, self.weight, self.k = spec, weights[spec.weight], runtime.kernels

    def forward(self, h, out):
        self.k.linear(h, self.weight, out)
        out.div_(self.spec.cap).tanh_().mul_(self.spec.cap)
        return out


@dataclass(frozen=True)
class ParallelBlockSpec:
    """h = norm(x); x += mixer(h) + ffn(h)."""
    norm: object
    mixer: object
    ffn: object

    def tensors(self):
        t = {}
        for part in (self.norm, self.mixer, self.ffn):
            t.update(part.tensors())
        return t

    def cache_need(self):
        return self.mixer.cache_need()


class ParallelBlock:
    """Takes the delta the block before left (``pending``), lets its norm add it, and hands on the sum of
    its two branches as the next pending delta."""

    def __init__(self, spec, weights, runtime):
        self.rt = runtime
        self.norm = build_part(spec.norm, weights, runtime)
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.ffn = build_part(spec.ffn, weights, runtime)

    def forward(self, x, pending, ctx, call):
        h = ctx.buffer("h", x.shape, self.rt.act_dtype)
        self.norm.forward(x, h, delta=pending)
        a = self.mixer.forward(h, ctx, call)
        m = self.ffn.forward(h, ctx)
        return a.add_(m)


@dataclass(frozen=True)
class PostNormBlockSpec:
    """x = norm1(x + mixer(x)); x = norm2(x + ffn(x)): the residual stream itself is normalised."""
    mixer: object
    mixer_norm: object
    ffn: object
    ffn_norm: object

    def tensors(self):
        t = {}
        for part in (self.mixer, self.mixer_norm, self.ffn, self.ffn_norm):
            t.update(part.tensors())
        return t

    def cache_need(self):
        return self.mixer.cache_need()


class PostNormBlock:
    def __init__(self, spec, weights, runtime):
        self.rt = runtime
        self.mixer = build_part(spec.mixer, weights, runtime)
        self.mixer_norm = build_part(spec.mixer_norm, weights, runtime)
        self.ffn = build_part(spec.ffn, weights, runtime)
        self.ffn_norm = build_part(spec.ffn_norm, weights, runtime)

    def forward(self, x, pending, ctx, call):
        if pending is not None:
            x.add_(pending)
        h = ctx.buffer("h", x.shape, self.rt.act_dtype)
        for part, norm, args in ((self.mixer, self.mixer_norm, (ctx, call)), (self.ffn, self.ffn_norm, (ctx,))):
            h.copy_(x)                                           # the branch reads the stream in the activation dtype
            d = part.forward(h, *args)
            y = ctx.buffer("post", x.shape, torch.float32)
            norm.forward(x, y, delta=d)                          # x += d; y = norm(x)
            x.copy_(y)
        return None


register_part(ScaledEmbeddingSpec, ScaledEmbedding)
register_part(CappedHeadSpec, CappedHead)
register_part(ParallelBlockSpec, ParallelBlock)
register_part(PostNormBlockSpec, PostNormBlock)


# ------------------------------------------------------------------ the toy architecture
@dataclass(frozen=True)
class Toy3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    eps: float
    theta: float
    max_positions: int
    embed_scale: float
    logit_cap: float

    @classmethod
    def from_dict(cls, d):
        return cls(d["architectures"][0], *(d[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_heads",
                                                            "num_kv_heads", "head_dim", "eps", "theta", "max_positions",
                                                            "embed_scale", "logit_cap")))

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        return d


def toy3_plan(c):
    def norm(name):
        return RMSNormSpec(c.hidden_size, c.eps, name)

    def attn(p):
        return AttentionSpec(c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim, c.head_dim ** -0.5, f"{p}.q", f"{p}.k",
                             f"{p}.v", f"{p}.o", position=RotarySpec(c.head_dim, c.head_dim, c.theta))

    def mlp(p):
        return GatedMLPSpec(c.hidden_size, c.intermediate_size, "silu", f"{p}.gate", f"{p}.up", f"{p}.down")

    parallel = ParallelBlockSpec(norm("p.n"), attn("p"), mlp("p"))
    post = PostNormBlockSpec(attn("s"), norm("s.n1"), mlp("s"), norm("s.n2"))
    return ModelPlan(c.architecture, c.vocab_size, c.hidden_size, c.max_positions,
                     ScaledEmbeddingSpec(c.vocab_size, c.hidden_size, "embed", c.embed_scale), (parallel, post),
                     (LayerCall(0), LayerCall(1), LayerCall(0)), norm("final"),
                     CappedHeadSpec(c.vocab_size, c.hidden_size, "head", c.logit_cap))


register_architecture("ToyParallelPostNormLM", Toy3Config, toy3_plan, replace=True)
CONFIG3 = dict(architectures=["ToyParallelPostNormLM"], vocab_size=101, hidden_size=48, intermediate_size=72, num_heads=4,
               num_kv_heads=2, head_dim=16, eps=1e-5, theta=50.0, max_positions=256, embed_scale=48 ** 0.5, logit_cap=2.5)


def plain_toy3(cfg, w, ids):
    T, nh, nkv, d = len(ids), cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    cos, sin = P.rope_table(d, T, cfg["theta"], torch.float32)

    def attn(h, p):
        q = P.apply_rope((h @ w[f"{p}.q"].t()).view(T, nh, d).transpose(0, 1), cos, sin)
        k = P.apply_rope((h @ w[f"{p}.k"].t()).view(T, nkv, d).transpose(0, 1), cos, sin)
        v = (h @ w[f"{p}.v"].t()).view(T, nkv, d).transpose(0, 1)
        return P.attention(q, k, v, d ** -0.5).transpose(0, 1).reshape(T, nh * d) @ w[f"{p}.o"].t()

    def mlp(h, p):
        g = h @ w[f"{p}.gate"].t()
        return (g * torch.sigmoid(g) * (h @ w[f"{p}.up"].t())) @ w[f"{p}.down"].t()

    def parallel(x):
        h = P.rms_norm(x, w["p.n"], cfg["eps"])
        return x + attn(h, "p") + mlp(h, "p")

    def post(x):
        x = P.rms_norm(x + attn(x, "s"), w["s.n1"], cfg["eps"])
        return P.rms_norm(x + mlp(x, "s"), w["s.n2"], cfg["eps"])

    x = w["embed"][torch.as_tensor(ids)] * cfg["embed_scale"]
    x = parallel(post(parallel(x)))
    z = P.rms_norm(x, w["final"], cfg["eps"]) @ w["head"].t()
    return cfg["logit_cap"] * torch.tanh(z / cfg["logit_cap"])


@pytest.mark.parametrize("dtype,tolerance", [("float32", 3e-5), ("bfloat16", 6e-2)])
def test_parallel_and_post_norm_blocks_a_scaled_embedding_and_a_capped_head(tmp_path, dtype, tolerance):
    cfg = Toy3Config.from_dict(CONFIG3)
    d = write_random_model(cfg, 21, str(tmp_path / "toy3"), store_dtype="float32")
    w = {k: v.clone() for k, v in P.read_model(d)[1].items()}
    w["head"] = w["head"] * 6.0                   # logits beyond the cap, so that the cap matters
    from safetensors.torch import save_file
    import os
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(d, "model.safetensors"))
    opts = EngineOptions(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=3, max_num_batched_tokens=128)
    _, plan, runner = build_runner(d, opts)
    assert len(plan.resolved_schedule()) == 3 and len(runner.cache.kv_groups) == 1
    reqs = {f"v{i}": tiny.random_tokens(101, n, 400 + i) for i, n in enumerate([50, 90, 7, 64, 33])}
    ref = {r: plain_toy3(CONFIG3, w, t) for r, t in reqs.items()}
    assert max(float(r.abs().max()) for r in ref.values()) > 2.0          # the cap was reached
    for steps in (tiny.schedule_whole(reqs), tiny.schedule_portions(reqs, seed=5),
                  tiny.schedule_mixed(reqs, max_live=3, max_tokens=320, seed=6)):
        out = tiny.collect(steps, tiny.run_inprocess(runner, steps), 101)
        for r in reqs:
            err = (out[r] - ref[r]).abs().max(dim=-1).values
            assert float(err.max()) <= tolerance, (r, int(err.argmax()), float(err.max()))
    runner.cache.check()
