"""The plain implementation itself: each part against a hand formula, as the reference tests
its own helpers (tests/test_qwen3_model.py:80-124), plus causality, grouping and the window."""
import math

import pytest
import torch

import plain_qwen3 as P
import tiny


def test_rms_norm_formula():
    x = torch.tensor([[1.0, -2.0, 3.0, 0.5]])
    w = torch.tensor([0.5, 1.0, 2.0, 1.5])
    eps = 1e-3
    r = 1.0 / math.sqrt((1 + 4 + 9 + 0.25) / 4 + eps)
    want = torch.tensor([[1.0 * r * 0.5, -2.0 * r, 3.0 * r * 2.0, 0.5 * r * 1.5]])
    torch.testing.assert_close(P.rms_norm(x, w, eps), want)


def test_linear_uses_out_in_orientation():
    w = torch.tensor([[1.0, 0.0, 2.0], [0.0, 3.0, 0.0]])          # [out=2, in=3]
    x = torch.tensor([[1.0, 2.0, 3.0]])
    assert P.linear(x, w).tolist() == [[7.0, 6.0]]


def test_rope_is_identity_at_position_zero_and_half_split():
    d = 8
    cos, sin = P.rope_table(d, 3, 10000.0, torch.float32)
    x = torch.arange(1.0, d + 1).view(1, 1, d).expand(1, 3, d).clone()
    y = P.apply_rope(x, cos, sin)
    torch.testing.assert_close(y[0, 0], x[0, 0])
    # position 1: element i pairs with i + d/2, not with i + 1
    inv = [1.0 / (10000.0 ** (2 * i / d)) for i in range(d // 2)]
    for i in range(d // 2):
        a, b = float(x[0, 1, i]), float(x[0, 1, i + d // 2])
        assert abs(float(y[0, 1, i]) - (a * math.cos(inv[i]) - b * math.sin(inv[i]))) < 1e-5
        assert abs(float(y[0, 1, i + d // 2]) - (b * math.cos(inv[i]) + a * math.sin(inv[i]))) < 1e-5
    adjacent = x[0, 1, 0] * math.cos(inv[0]) - x[0, 1, 1] * math.sin(inv[0])
    assert abs(float(y[0, 1, 0]) - float(adjacent)) > 1e-3


def test_attention_is_causal_grouped_and_scaled():
    torch.manual_seed(0)
    nq, nkv, T, d = 4, 2, 6, 8
    q, k, v = torch.randn(nq, T, d), torch.randn(nkv, T, d), torch.randn(nkv, T, d)
    out = P.attention(q, k, v, d ** -0.5)
    for h in range(nq):
        g = h // (nq // nkv)
        for t in range(T):
            s = (q[h, t] @ k[g, :t + 1].t()) * d ** -0.5
            want = torch.softmax(s, -1) @ v[g, :t + 1]
            torch.testing.assert_close(out[h, t], want)
    # a window of 3 keys
    outw = P.attention(q, k, v, d ** -0.5, window=3)
    s = (q[1, 5] @ k[0, 3:6].t()) * d ** -0.5
    torch.testing.assert_close(outw[1, 5], torch.softmax(s, -1) @ v[0, 3:6])
    torch.testing.assert_close(outw[:, :3], out[:, :3])


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d = tiny.make_model_dir("B", str(tmp_path_factory.mktemp("m")))
    return P.read_model(d)


def test_logits_do_not_depend_on_later_tokens(model):
    cfg, w = model
    a = tiny.random_tokens(cfg["vocab_size"], 40, 1)
    b = a[:25] + tiny.random_tokens(cfg["vocab_size"], 15, 2)
    la, lb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    torch.testing.assert_close(la[:25], lb[:25], rtol=0, atol=1e-6)
    assert (la[25:] - lb[25:]).abs().max() > 1e-3


def test_the_window_matters_and_only_beyond_its_reach(model):
    cfg, w = model
    toks = tiny.random_tokens(cfg["vocab_size"], 60, 3)
    full = dict(cfg, layer_types=["full_attention"] * 3)
    lw, lf = P.forward(cfg, w, toks), P.forward(full, w, toks)
    torch.testing.assert_close(lw[:24], lf[:24], rtol=0, atol=1e-6)      # up to 24 keys nothing is cut off
    assert (lw[30:] - lf[30:]).abs().max() > 1e-3


def test_float32_and_float64_agree(model):
    cfg, w = model
    toks = tiny.random_tokens(cfg["vocab_size"], 50, 4)
    l32 = P.forward(cfg, w, toks)
    l64 = P.forward(cfg, {k: v.double() for k, v in w.items()}, toks, dtype=torch.float64)
    assert (l32.double() - l64).abs().max() < 2e-5


def test_tied_and_untied_heads(tmp_path):
    da = tiny.make_model_dir("A", str(tmp_path))
    cfg, w = P.read_model(da)
    assert "lm_head.weight" not in w
    toks = tiny.random_tokens(cfg["vocab_size"], 9, 5)
    logits, hidden = P.forward(cfg, w, toks, return_hidden=True)
    want = P.rms_norm(hidden, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["model.embed_tokens.weight"].t()
    torch.testing.assert_close(logits, want)


def test_greedy_takes_the_lowest_index_on_ties():
    assert int(torch.argmax(torch.tensor([1.0, 3.0, 3.0, 2.0]))) == 1
