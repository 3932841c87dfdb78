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


# ----------------------------------------------------------------------------------------------------------------
# More parts from outside the package, each a test device and nothing else: a feed-forward that routes every token
# to one of several small experts and runs its own CUDA kernel (compiled from a source file that this test writes,
# through register_library), a position code that is no rotation the fused kernel knows (so the attention part runs
# norm -> apply -> store as three steps), and a mixer whose per-token cache entries are a narrow "key" and a wider
# "value" of different shapes (a cache need with unequal streams).
# ----------------------------------------------------------------------------------------------------------------
ROUTE_CU = r"""
#include "common.cuh"
// out[t, :] = sum_e gate[t, e] * y[e, t, :]   (gate: [T, E] float32 with zeros for experts not chosen; y: [E, T, H])
__global__ void toy_combine_kernel(const float* gate, const float* y, float* out, int T, int E, int H) {
  ifb_pdl_wait();
  ifb_pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * H) return;
  const int t = i / H;
  float acc = 0.f;
  for (int e = 0; e < E; ++e) acc += gate[t * E + e] * y[(size_t)e * T * H + i];
  out[i] = acc;
}
IFB_EXPORT int toy_combine(const float* gate, const float* y, float* out, int T, int E, int H, cudaStream_t stream) {
  if (T <= 0) return IFB_OK;
  return ifb_launch(toy_combine_kernel, dim3((T * H + 255) / 256), dim3(256), 0, stream, gate, y, out, T, E, H);
}
"""


@dataclass(frozen=True)
class RoutedMLPSpec:
    hidden_size: int
    inner: int
    experts: int
    prefix: str

    def tensors(self):
        t = {f"{self.prefix}.router": TensorSpec((self.experts, self.hidden_size))}
        for e in range(self.experts):
            t[f"{self.prefix}.e{e}.up"] = TensorSpec((self.inner, self.hidden_size))
            t[f"{self.prefix}.e{e}.down"] = TensorSpec((self.hidden_size, self.inner))
        return t

    def cache_need(self):
        return None


class RoutedMLP:
    """Top-1 routing on float32 router logits; every expert runs on all tokens (a toy) through the engine's own
    product kernel, and the part's own kernel combines them with the one-hot gate times the softmax weight."""
    graph_safe = True
    library = None

    def __init__(self, spec, weights, runtime):
        import ctypes
        from infurnace_b200.kernels import load_library
        self.spec, self.rt, self.k = spec, runtime, runtime.kernels
        self.router = weights[f"{spec.prefix}.router"].float()
        self.up = [weights[f"{spec.prefix}.e{e}.up"] for e in range(spec.experts)]
        self.down = [weights[f"{spec.prefix}.e{e}.down"] for e in range(spec.experts)]
        self.lib = load_library(RoutedMLP.library)
        self.lib.toy_combine.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_void_p]

    def forward(self, h, ctx):
        s, n = self.spec, h.shape[0]
        logits = h.float() @ self.router.t()                               # router logits in 32-bit
        probs = torch.softmax(logits, dim=-1)
        top = probs.argmax(dim=-1, keepdim=True)
        gate = torch.zeros_like(probs).scatter_(1, top, probs.gather(1, top)).contiguous()
        y = ctx.buffer("toy_expert_out", (s.experts * n, s.hidden_size), torch.float32, rows=s.experts * n)
        for e in range(s.experts):
            mid = ctx.buffer("toy_expert_mid", (n, s.inner), self.rt.act_dtype)
            self.k.linear(h, self.up[e], mid)
            mid.copy_(torch.relu(mid.float()).to(mid.dtype))
            self.k.linear(mid, self.down[e], y[e * n:(e + 1) * n])
        out = ctx.buffer("toy_routed", (n, s.hidden_size), torch.float32)
        status = self.lib.toy_combine(gate.data_ptr(), y.data_ptr(), out.data_ptr(), n, s.experts, s.hidden_size,
                                      torch.cuda.current_stream().cuda_stream)
        assert status == 0
        return out


@dataclass(frozen=True)
class SquarePhaseSpec:
    """A position code that rotates adjacent pairs of the whole head by position^2 * inv_freq_i mod 2 pi."""
    head_dim: int
    theta: float

    def tensors(self):
        return {}


class SquarePhase:
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec = spec
        self.inv = (1.0 / (spec.theta ** (torch.arange(0, spec.head_dim, 2, dtype=torch.float32) / spec.head_dim))).to(runtime.device)

    def fused_rotary(self):
        return None                                  # not a rotation by position * frequency: no fused form

    def apply(self, qkv, num_heads, num_kv_heads, head_dim, positions):
        n = qkv.shape[0]
        ang = (positions.float() ** 2)[:, None] * self.inv[None]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        heads = qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)[:, :num_heads + num_kv_heads].float()
        a, b = heads[..., 0::2], heads[..., 1::2]
        rot = torch.stack((a * cos - b * sin, b * cos + a * sin), -1).flatten(-2)
        qkv.view(n, num_heads + 2 * num_kv_heads, head_dim)[:, :num_heads + num_kv_heads] = rot.to(qkv.dtype)


@dataclass(frozen=True)
class NarrowKeySpec:
    """One head: keys of width ``key_dim``, values of width ``hidden_size`` (unequal cache streams)."""
    hidden_size: int
    key_dim: int
    prefix: str

    def tensors(self):
        return {f"{self.prefix}.q": TensorSpec((self.key_dim, self.hidden_size)),
                f"{self.prefix}.k": TensorSpec((self.key_dim, self.hidden_size))}

    def cache_need(self):
        from infurnace_b200.config.specs import PagedCacheNeed, PagedStream
        return PagedCacheNeed((PagedStream("key", 1, self.key_dim), PagedStream("value", 1, self.hidden_size)))


class NarrowKey:
    """delta[t] = softmax_j<=t(q_t . k_j / sqrt(key_dim)) h_j: the value is the input itself."""

    def __init__(self, spec, weights, runtime):
        self.spec, self.rt = spec, runtime
        self.wq, self.wk = weights[f"{spec.prefix}.q"].float(), weights[f"{spec.prefix}.k"].float()

    def forward(self, h, ctx, call):
        kv = ctx.kv(call.cache)
        assert kv.pages is None and set(kv.streams) == {"key", "value"}
        keys, values = kv.streams["key"], kv.streams["value"]              # [pages, 1, page_size, width]
        ps = kv.page_size
        hf = h.float()
        q, k = hf @ self.wq.t(), hf @ self.wk.t()
        slots = kv.slot_mapping.long()
        keys[slots // ps, 0, slots % ps] = k.to(keys.dtype)
        values[slots // ps, 0, slots % ps] = h.to(values.dtype)
        out = torch.zeros((h.shape[0], self.spec.hidden_size), dtype=torch.float32, device=h.device)
        for r in range(ctx.num_requests):
            q0, q1, L = ctx.host_cu_q[r], ctx.host_cu_q[r + 1], ctx.host_seq_lens[r]
            table = kv.block_tables[r, : -(-L // ps)].long()
            kk = keys[table, 0].reshape(-1, self.spec.key_dim)[:L].float()
            vv = values[table, 0].reshape(-1, self.spec.hidden_size)[:L].float()
            scores = q[q0:q1] @ kk.t() / self.spec.key_dim ** 0.5
            pos = ctx.positions[q0:q1].long()[:, None]
            scores = scores.masked_fill(torch.arange(L, device=h.device)[None, :] > pos, float("-inf"))
            out[q0:q1] = torch.softmax(scores, -1) @ vv
        return out


register_part(RoutedMLPSpec, RoutedMLP)
register_part(SquarePhaseSpec, SquarePhase)
register_part(NarrowKeySpec, NarrowKey)


@dataclass(frozen=True)
class Toy2Config(ToyConfig):
    experts: int = 3
    key_dim: int = 12

    @classmethod
    def from_dict(cls, d):
        return cls(d["architectures"][0], d["vocab_size"], d["hidden_size"], d["intermediate_size"], d["num_heads"],
                   d["head_dim"], d["eps"], d["theta"], d["max_positions"], d["experts"], d["key_dim"])


def toy2_plan(c):
    def norm(name):
        return RMSNormSpec(c.hidden_size, c.eps, name)
    attention = PreNormBlockSpec(
        norm("a.n1"),
        AttentionSpec(c.hidden_size, c.num_heads, c.num_heads, c.head_dim, c.head_dim ** -0.5, "a.q", "a.k", "a.v", "a.o",
                      position=SquarePhaseSpec(c.head_dim, c.theta)),
        norm("a.n2"), RoutedMLPSpec(c.hidden_size, c.intermediate_size, c.experts, "a.moe"))
    narrow = PreNormBlockSpec(norm("b.n1"), NarrowKeySpec(c.hidden_size, c.key_dim, "b.mix"), norm("b.n2"),
                              GatedMLPSpec(c.hidden_size, c.intermediate_size, "silu", "b.gate", "b.up", "b.down"))
    return ModelPlan(c.architecture, c.vocab_size, c.hidden_size, c.max_positions,
                     EmbeddingSpec(c.vocab_size, c.hidden_size, "embed"), (attention, narrow), (LayerCall(0), LayerCall(1)),
                     norm("final"), LMHeadSpec(c.vocab_size, c.hidden_size, "embed", tied=True))


register_architecture("ToyRoutedNarrowLM", Toy2Config, toy2_plan, replace=True)
CONFIG2 = dict(CONFIG, architectures=["ToyRoutedNarrowLM"], experts=3, key_dim=12)


def plain_toy2(cfg, w, ids):
    T, H = len(ids), cfg["hidden_size"]
    x = w["embed"][torch.as_tensor(ids)]
    nh, d = cfg["num_heads"], cfg["head_dim"]
    h = P.rms_norm(x, w["a.n1"], cfg["eps"])
    q, k, v = [(h @ w[f"a.{n}"].t()).view(T, nh, d).transpose(0, 1) for n in "qkv"]
    inv = 1.0 / (cfg["theta"] ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = (torch.arange(T, dtype=torch.float32) ** 2)[:, None] * inv[None]

    def rot(t):
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack((a * ang.cos() - b * ang.sin(), b * ang.cos() + a * ang.sin()), -1).flatten(-2)
    o = P.attention(rot(q), rot(k), v, d ** -0.5)
    x = x + o.transpose(0, 1).reshape(T, nh * d) @ w["a.o"].t()
    h = P.rms_norm(x, w["a.n2"], cfg["eps"])
    probs = torch.softmax(h @ w["a.moe.router"].t(), -1)
    top = probs.argmax(-1)
    y = torch.zeros(T, H)
    for t in range(T):
        e = int(top[t])
        y[t] = probs[t, e] * (torch.relu(h[t] @ w[f"a.moe.e{e}.up"].t()) @ w[f"a.moe.e{e}.down"].t())
    x = x + y
    h = P.rms_norm(x, w["b.n1"], cfg["eps"])
    scores = (h @ w["b.mix.q"].t()) @ (h @ w["b.mix.k"].t()).t() / cfg["key_dim"] ** 0.5
    scores = scores.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
    x = x + torch.softmax(scores, -1) @ h
    h = P.rms_norm(x, w["b.n2"], cfg["eps"])
    g = h @ w["b.gate"].t()
    x = x + (g * torch.sigmoid(g) * (h @ w["b.up"].t())) @ w["b.down"].t()
    return P.rms_norm(x, w["final"], cfg["eps"]) @ w["embed"].t()


def test_routing_another_position_code_unequal_cache_streams_and_a_kernel_library_from_outside(tmp_path):
    from infurnace_b200.kernels import register_library
    src = tmp_path / "toy_route.cu"
    src.write_text(ROUTE_CU)
    register_library("toy_route", [str(src)], replace=True)
    RoutedMLP.library = "toy_route"
    cfg = Toy2Config.from_dict(CONFIG2)
    d = write_random_model(cfg, 12, str(tmp_path / "toy2"), store_dtype="float32")
    w = {k: v.clone() for k, v in P.read_model(d)[1].items()}        # copies: the file they were mapped from is rewritten below
    for k in list(w):                     # spread the router logits and the scores, so that routing and masks matter
        if k.endswith(".router") or k.endswith("mix.q"):
            w[k] = w[k] * 40.0
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(d, "model.safetensors"))
    opts = EngineOptions(dtype="float32", page_size=8, num_pages=24, max_num_seqs=2, max_num_batched_tokens=128)
    _, plan, runner = build_runner(d, opts)
    groups = runner.cache.kv_groups
    assert len(groups) == 2 and sorted(g.uniform for g in groups) == [False, True]
    odd = [g for g in groups if not g.uniform][0]
    shapes = {n: tuple(t.shape[1:]) for n, t in odd.streams[odd.cache_ids[0]].items()}
    assert shapes == {"key": (1, 8, 12), "value": (1, 8, 48)}
    assert runner.cache.bytes_per_token() == 4 * (2 * 3 * 16 + 12 + 48)
    reqs = {f"u{i}": tiny.random_tokens(97, n, 300 + i) for i, n in enumerate([40, 75, 9, 64])}
    ref = {r: plain_toy2(CONFIG2, w, t) for r, t in reqs.items()}
    experts_used = set()
    for t in reqs.values():
        x = w["embed"][torch.as_tensor(t)]
        experts_used |= set((x @ w["a.moe.router"].t()).argmax(-1).tolist())
    for steps in (tiny.schedule_whole(reqs), tiny.schedule_portions(reqs, seed=3),
                  tiny.schedule_mixed(reqs, max_live=2, max_tokens=192, seed=4)):
        out = tiny.collect(steps, tiny.run_inprocess(runner, steps), 97)
        for r in reqs:
            err = (out[r] - ref[r]).abs().max(dim=-1).values
            assert float(err.max()) <= 5e-5, (r, int(err.argmax()), float(err.max()))
    assert len(experts_used) > 1
