"""Parts and an architecture that the package does not have, defined here and registered from
outside: a mixer with per-request state of fixed size (a running mean of its inputs), used in one
layer beside an attention layer, in a schedule that calls the stateful layer twice.  Nothing under
infurnace_b200/ is changed for it.  It is a test device, not a model of anyone's.

The model is stepped through the engine's own step function in different cuttings (whole, in
portions, mixed with another request so that state slots and pages are reused) and compared with
a plain whole-sequence computation."""
import json
import os
from dataclasses import asdict, dataclass

import pytest
import torch

import plain_qwen3 as P
import tiny
from infurnace_b200.config.specs import (AttentionSpec, EmbeddingSpec, GatedMLPSpec, LayerCall, LMHeadSpec, ModelPlan,
                                         PreNormBlockSpec, RMSNormSpec, RotarySpec, StateNeed, TensorSpec)
from infurnace_b200.engine import EngineOptions, build_runner
from infurnace_b200.models import register_architecture
from infurnace_b200.parts import register_part
from infurnace_b200.weights.random_init import write_random_model

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------ the toy mixer
@dataclass(frozen=True)
class RunningMeanSpec:
    hidden_size: int
    out_proj: str

    def tensors(self):
        return {self.out_proj: TensorSpec((self.hidden_size, self.hidden_size))}

    def cache_need(self):
        return StateNeed((self.hidden_size,))          # the running sum of the inputs


class RunningMean:
    """delta[t] = W (mean of h[0..t]).  The running sum lives in the request's state slot."""

    def __init__(self, spec, weights, runtime):
        self.spec, self.w, self.rt = spec, weights[spec.out_proj], runtime

    def forward(self, h, ctx, call):
        state = ctx.state(call.cache)                  # [slots, hidden] float32
        mean = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        for r, slot in enumerate(ctx.host_state_slots):
            q0, q1 = ctx.host_cu_q[r], ctx.host_cu_q[r + 1]
            run = state[slot] + torch.cumsum(h[q0:q1].float(), dim=0)
            state[slot] = run[-1]
            mean[q0:q1] = run / (ctx.positions[q0:q1].float() + 1.0)[:, None]
        delta = ctx.buffer("toy_delta", (h.shape[0], self.spec.hidden_size), torch.float32)
        self.rt.kernels.linear(mean.to(self.rt.act_dtype), self.w, delta)
        return delta


register_part(RunningMeanSpec, RunningMean)


# ------------------------------------------------------------------ the toy architecture
@dataclass(frozen=True)
class ToyConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    head_dim: int
    eps: float
    theta: float
    max_positions: int

    @classmethod
    def from_dict(cls, d):
        return cls(d["architectures"][0], d["vocab_size"], d["hidden_size"], d["intermediate_size"], d["num_heads"],
                   d["head_dim"], d["eps"], d["theta"], d["max_positions"])

    def to_dict(self):
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        return d


def toy_plan(c: ToyConfig) -> ModelPlan:
    def mlp(p):
        return GatedMLPSpec(c.hidden_size, c.intermediate_size, "silu", f"{p}.gate", f"{p}.up", f"{p}.down")

    def norm(name):
        return RMSNormSpec(c.hidden_size, c.eps, name)

    stateful = PreNormBlockSpec(norm("l0.n1"), RunningMeanSpec(c.hidden_size, "l0.mix.out"), norm("l0.n2"), mlp("l0.mlp"))
    attention = PreNormBlockSpec(
        norm("l1.n1"),
        AttentionSpec(c.hidden_size, c.num_heads, c.num_heads, c.head_dim, c.head_dim ** -0.5, "l1.q", "l1.k", "l1.v",
                      "l1.o", position=RotarySpec(c.head_dim, c.head_dim // 2, c.theta, interleaved=True)),
        norm("l1.n2"), mlp("l1.mlp"))
    return ModelPlan(c.architecture, c.vocab_size, c.hidden_size, c.max_positions,
                     EmbeddingSpec(c.vocab_size, c.hidden_size, "embed"), (stateful, attention),
                     (LayerCall(0), LayerCall(1), LayerCall(0)),       # the stateful layer runs twice
                     norm("final"), LMHeadSpec(c.vocab_size, c.hidden_size, "embed", tied=True))


register_architecture("ToyRunningMeanLM", ToyConfig, toy_plan, replace=True)

CONFIG = dict(architectures=["ToyRunningMeanLM"], vocab_size=97, hidden_size=48, intermediate_size=80, num_heads=3,
              head_dim=16, eps=1e-5, theta=100.0, max_positions=128)


# ------------------------------------------------------------------ its plain statement
def plain_toy(cfg, w, ids):
    T = len(ids)
    x = w["embed"][torch.as_tensor(ids)]

    def mlp(h, p):
        g = h @ w[f"{p}.gate"].t()
        return (g * torch.sigmoid(g) * (h @ w[f"{p}.up"].t())) @ w[f"{p}.down"].t()

    def stateful(x):
        h = P.rms_norm(x, w["l0.n1"], cfg["eps"])
        mean = torch.cumsum(h, 0) / torch.arange(1, T + 1)[:, None]
        x = x + mean @ w["l0.mix.out"].t()
        return x + mlp(P.rms_norm(x, w["l0.n2"], cfg["eps"]), "l0.mlp")

    def attention(x):
        nh, d = cfg["num_heads"], cfg["head_dim"]
        h = P.rms_norm(x, w["l1.n1"], cfg["eps"])
        q = (h @ w["l1.q"].t()).view(T, nh, d).transpose(0, 1)
        k = (h @ w["l1.k"].t()).view(T, nh, d).transpose(0, 1)
        v = (h @ w["l1.v"].t()).view(T, nh, d).transpose(0, 1)
        rd = d // 2                                     # the first half of each head, adjacent pairs
        inv = 1.0 / (cfg["theta"] ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        ang = torch.arange(T, dtype=torch.float32)[:, None] * inv[None]

        def rot(t):
            a, b = t[..., 0:rd:2], t[..., 1:rd:2]
            o = torch.stack((a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin()), -1).flatten(-2)
            return torch.cat((o, t[..., rd:]), -1)

        o = P.attention(rot(q), rot(k), v, d ** -0.5)
        x = x + o.transpose(0, 1).reshape(T, nh * d) @ w["l1.o"].t()
        return x + mlp(P.rms_norm(x, w["l1.n2"], cfg["eps"]), "l1.mlp")

    x = stateful(attention(stateful(x)))
    return P.rms_norm(x, w["final"], cfg["eps"]) @ w["embed"].t()


@pytest.mark.parametrize("dtype,tolerance", [("float32", 3e-5), ("bfloat16", 6e-2)])
def test_a_stateful_mixer_from_outside_the_package(tmp_path, dtype, tolerance):
    cfg = ToyConfig.from_dict(CONFIG)
    d = write_random_model(cfg, 9, str(tmp_path / "toy"), store_dtype="float32")
    _, w = P.read_model(d)
    with open(os.path.join(d, "config.json")) as f:
        assert json.load(f)["architectures"] == ["ToyRunningMeanLM"]
    opts = EngineOptions(dtype=dtype, page_size=8, num_pages=24, max_num_seqs=2, max_num_batched_tokens=128)
    _, plan, runner = build_runner(d, opts)
    assert len(runner.cache.state_groups) == 1 and len(runner.cache.state_groups[0].cache_ids) == 2
    assert len(runner.cache.kv_groups) == 1 and not runner.use_graphs
    reqs = {f"t{i}": tiny.random_tokens(97, n, 200 + i) for i, n in enumerate([40, 75, 9, 64])}
    ref = {r: plain_toy(CONFIG, w, t) for r, t in reqs.items()}
    for steps in (tiny.schedule_whole(reqs), tiny.schedule_portions(reqs, seed=3),
                  tiny.schedule_mixed(reqs, max_live=2, max_tokens=192, seed=4)):
        out = tiny.collect(steps, tiny.run_inprocess(runner, steps), 97)
        for r in reqs:
            err = (out[r] - ref[r]).abs().max(dim=-1).values
            assert float(err.max()) <= tolerance, (r, int(err.argmax()), float(err.max()))
    assert runner.cache.num_free_slots == 2
