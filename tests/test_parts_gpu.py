"""Each part of a layer alone (norm, position code, attention mixer, feed-forward, block,
embedding, head), built from its own description and weights, against the plain functions."""
import pytest
import torch

import plain_qwen3 as P
import tiny
from infurnace_b200.cache import CacheManager
from infurnace_b200.engine.runner import ModelRunner, StepEntry
from infurnace_b200.models import plan_for, read_config
from infurnace_b200.parts import Runtime, build_part
from infurnace_b200.weights.loader import load_weights

pytestmark = pytest.mark.gpu


class OnePart:
    """Stands where a model stands in the runner and runs one function on the step's context."""

    graph_safe = False

    def __init__(self, plan, fn):
        self.plan, self.fn = plan, fn

    def forward(self, ctx):
        self.fn(ctx)
        return None


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def setup(request, tmp_path_factory):
    from infurnace_b200.kernels import load_cuda_kernels
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[request.param]
    d = tiny.make_model_dir("B", str(tmp_path_factory.mktemp("parts")))
    cfg, w = P.read_model(d)
    plan = plan_for(read_config(d))
    rt = Runtime(torch.device("cuda"), dtype, load_cuda_kernels())
    weights = load_weights(d, plan, dtype, rt.device)
    tol = dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    return cfg, w, plan, rt, weights, dtype, tol


def run_part(plan, rt, fn, portions, page_size=8):
    cache = CacheManager(plan, page_size, 64, 2, dtype=rt.act_dtype, device=rt.device)
    runner = ModelRunner(OnePart(plan, fn), cache, rt, 256, 256)
    cache.add_request("a")
    for toks in portions:
        runner.step([StepEntry("a", toks, [])])
    torch.cuda.synchronize()


def test_norm_part(setup):
    cfg, w, plan, rt, weights, dtype, tol = setup
    spec = plan.layers[0].mixer_norm
    part = build_part(spec, weights, rt)
    x = torch.randn(9, cfg["hidden_size"])
    delta = torch.randn(9, cfg["hidden_size"])
    xg, out = x.cuda(), torch.empty((9, cfg["hidden_size"]), dtype=dtype, device="cuda")
    part.forward(xg, out, delta=delta.cuda())
    want = P.rms_norm(x + delta, w[spec.weight], spec.eps)
    torch.testing.assert_close(xg.cpu(), x + delta)
    torch.testing.assert_close(out.cpu().float(), want, **tol)


def test_rotary_part(setup):
    cfg, w, plan, rt, weights, dtype, tol = setup
    a = plan.layers[0].mixer
    part = build_part(a.position, weights, rt)
    n, nq, nkv, d = 7, a.num_heads, a.num_kv_heads, a.head_dim
    qkv = torch.randn(n, (nq + 2 * nkv) * d).to(dtype)
    pos = torch.tensor([0, 1, 5, 17, 100, 200, 255], dtype=torch.int32)
    g = qkv.cuda()
    part.apply(g, nq, nkv, d, pos.cuda())
    cos, sin = P.rope_table(d, 256, cfg["rope_theta"], torch.float32)
    q = qkv[:, : nq * d].float().view(n, nq, d).transpose(0, 1)
    k = qkv[:, nq * d:(nq + nkv) * d].float().view(n, nkv, d).transpose(0, 1)
    qr = P.apply_rope(q, cos[pos.long()], sin[pos.long()]).transpose(0, 1).reshape(n, nq * d)
    kr = P.apply_rope(k, cos[pos.long()], sin[pos.long()]).transpose(0, 1).reshape(n, nkv * d)
    torch.testing.assert_close(g[:, : nq * d].cpu().float(), qr, **tol)
    torch.testing.assert_close(g[:, nq * d:(nq + nkv) * d].cpu().float(), kr, **tol)
    assert torch.equal(g[:, (nq + nkv) * d:].cpu(), qkv[:, (nq + nkv) * d:])      # v is not rotated
    assert torch.equal(g[0, : nq * d].cpu(), qkv[0, : nq * d])                     # position 0 is the identity


@pytest.mark.parametrize("layer", [0, 1])      # full attention, and the layer with a window of 24
def test_attention_part_in_portions(setup, layer):
    cfg, w, plan, rt, weights, dtype, tol = setup
    spec = plan.layers[layer].mixer
    part = build_part(spec, weights, rt)
    call = plan.resolved_schedule()[layer]
    T, H = 60, cfg["hidden_size"]
    h = torch.randn(T, H)
    hg = h.to(dtype).cuda()
    outs = []

    def fn(ctx):
        s = int(ctx.positions[0])
        outs.append(part.forward(hg[s:s + ctx.num_tokens], ctx, call).clone())

    run_part(plan, rt, fn, [[1] * 33, [1] * 2, [1] * 24, [1]])
    got = torch.cat(outs).cpu()
    cos, sin = P.rope_table(spec.head_dim, T, cfg["rope_theta"], torch.float32)
    want = P.attention_block(hg.float().cpu(), w, f"model.layers.{layer}.self_attn", cfg, cos, sin, spec.window)
    torch.testing.assert_close(got, want, **tol)


def test_feed_forward_and_block_parts(setup):
    cfg, w, plan, rt, weights, dtype, tol = setup
    T, H = 21, cfg["hidden_size"]
    ffn = build_part(plan.layers[2].ffn, weights, rt)
    block = build_part(plan.layers[2], weights, rt)
    call = plan.resolved_schedule()[2]
    h = torch.randn(T, H)
    x0 = torch.randn(T, H) * 0.1
    seen = {}

    def fn(ctx):
        seen["ffn"] = ffn.forward(h.to(dtype).cuda(), ctx).clone()
        x = x0.cuda()
        pending = block.forward(x, None, ctx, call)
        seen["block"] = (x + pending).clone()

    run_part(plan, rt, fn, [[1] * T])
    torch.testing.assert_close(seen["ffn"].cpu(), P.mlp_block(h.to(dtype).float(), w, "model.layers.2.mlp"), **tol)
    eps = cfg["rms_norm_eps"]
    cos, sin = P.rope_table(cfg["head_dim"], T, cfg["rope_theta"], torch.float32)
    x = x0 + P.attention_block(P.rms_norm(x0, w["model.layers.2.input_layernorm.weight"], eps), w,
                               "model.layers.2.self_attn", cfg, cos, sin, None)
    x = x + P.mlp_block(P.rms_norm(x, w["model.layers.2.post_attention_layernorm.weight"], eps), w, "model.layers.2.mlp")
    torch.testing.assert_close(seen["block"].cpu(), x, **tol)


def test_embedding_and_head_parts(setup):
    cfg, w, plan, rt, weights, dtype, tol = setup
    emb = build_part(plan.embedding, weights, rt)
    head = build_part(plan.lm_head, weights, rt)
    ids = torch.tensor([0, 5, 319, 7], dtype=torch.int32)
    out = torch.empty((4, cfg["hidden_size"]), dtype=torch.float32, device="cuda")
    emb.forward(ids.cuda(), out)
    assert torch.equal(out.cpu(), w["model.embed_tokens.weight"][ids.long()])
    h = torch.randn(4, cfg["hidden_size"]).to(dtype)
    logits = torch.empty((4, cfg["vocab_size"]), dtype=torch.float32, device="cuda")
    head.forward(h.cuda(), logits)
    torch.testing.assert_close(logits.cpu(), h.float() @ w["lm_head.weight"].t(), **tol)
