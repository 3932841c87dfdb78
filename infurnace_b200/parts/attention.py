"""The attention mixer: projections, q/k norm, position code, paged cache, attention."""
from __future__ import annotations

import torch

from ..config.specs import AttentionSpec
from .registry import build_part, fold_residual_norm, register_part, unfolded


class PagedAttention:
    """h -> o_proj(attention(q, K, V)) over the request's pages.

    The three projections (src/infurnace/executor/tinygrad/model.py:102-104) run as one
    product against their row-wise concatenation, which is exact.  One fused kernel then
    normalises the q and k heads (model.py:110-111), rotates them (model.py:113-114) and
    writes k and v into the pages (model.py:134-138); the attention kernel reads every
    key, this step's included, from the pages, so there is one rule for all ways of
    cutting the work: the query at position p sees the keys at positions <= p
    (model.py:117-132 has three cases for the same rule)."""

    graph_safe = True     # launches depend on the step's sizes only, never on values read on the host

    def __init__(self, spec: AttentionSpec, weights, runtime):
        self.spec = spec
        self.rt = runtime
        self.k = runtime.kernels
        wq, wk, wv = weights[spec.q_proj], weights[spec.k_proj], weights[spec.v_proj]
        self.w_qkv = torch.cat((wq, wk, wv), dim=0).contiguous()
        self.w_o = weights[spec.o_proj]
        self.q_norm_w = weights[spec.q_norm.weight] if spec.q_norm is not None else None
        self.k_norm_w = weights[spec.k_norm.weight] if spec.k_norm is not None else None
        eps = [n.eps for n in (spec.q_norm, spec.k_norm) if n is not None]
        if len(set(eps)) > 1:
            raise ValueError("q_norm and k_norm must share eps: one kernel normalises both")
        self.eps = eps[0] if eps else 0.0
        self.position = build_part(spec.position, weights, runtime) if spec.position is not None else None
        self.qkv_width = (spec.num_heads + 2 * spec.num_kv_heads) * spec.head_dim

    can_fold_output = True

    def can_take_folded(self, n):
        can = getattr(self.k, "can_fold_norm", None)
        return bool(can and can(n, self.rt.act_dtype, self.w_qkv))

    def forward(self, h, ctx, call, fold=None):
        s, k = self.spec, self.k
        h, row_scale = unfolded(h)
        n = h.shape[0]
        qkv = ctx.buffer("qkv", (n, self.qkv_width), self.rt.act_dtype)
        kv = ctx.kv(call.cache)
        slots = kv.slot_mapping if call.store else None
        fused = self.position.fused_rotary() if self.position is not None else None
        has_table = fused is not None and hasattr(self.position, "table")
        one_launch = getattr(k, "can_fuse_qkv", None)
        if (self.position is None or has_table) and one_launch and one_launch(
                n, h.dtype, self.w_qkv, s.head_dim, fused[1] if fused is not None else 0,
                bool(fused[2]) if fused is not None else False, kv.pages):
            # few rows: the projection's own kernel finishes norm, rotation and store
            k.linear_qkv_rope_store(h, self.w_qkv, qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.q_norm_w, self.k_norm_w,
                                    self.eps, self.position.table(ctx) if fused is not None else None, slots, kv.pages,
                                    row_scale=row_scale)
        else:
            if row_scale is not None:
                k.linear(h, self.w_qkv, qkv, row_scale=row_scale)
            else:
                k.linear(h, self.w_qkv, qkv)
            self._norm_rotate_store(qkv, ctx, kv, slots, fused)
        attn = ctx.buffer("attn", (n, s.num_heads * s.head_dim), self.rt.act_dtype)
        k.paged_attention(qkv, s.num_heads, s.num_kv_heads, s.head_dim, kv.pages, kv.block_tables,
                          ctx.cu_q, ctx.seq_lens, attn, s.scale, s.window or 0, ctx.max_q_len, ctx.max_seq_len,
                          min_q_len=ctx.min_q_len)
        folded = fold_residual_norm(k, ctx, "mixer", attn, self.w_o, fold, self.rt.act_dtype)
        if folded is not None:
            return folded
        delta = ctx.buffer("delta_mixer", (n, s.hidden_size), torch.float32)
        k.linear(attn, self.w_o, delta)
        return delta

    def _norm_rotate_store(self, qkv, ctx, kv, slots, fused):
        s, k = self.spec, self.k
        if self.position is None or fused is not None:
            inv_freq, rdim, inter = fused if fused is not None else (None, 0, False)
            table = self.position.table(ctx) if fused is not None and hasattr(self.position, "table") else None
            k.qk_norm_rope_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.q_norm_w, self.k_norm_w,
                                 self.eps, inv_freq, rdim, inter, ctx.positions, slots, kv.pages, rope_table=table)
        else:   # a position code without a fused form: norm, then the code, then the store
            k.qk_norm_rope_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, self.q_norm_w, self.k_norm_w,
                                 self.eps, None, 0, False, ctx.positions, None, None)
            self.position.apply(qkv, s.num_heads, s.num_kv_heads, s.head_dim, ctx.positions)
            if slots is not None:
                k.qk_norm_rope_store(qkv, s.num_heads, s.num_kv_heads, s.head_dim, None, None, 0.0,
                                     None, 0, False, ctx.positions, slots, kv.pages)


register_part(AttentionSpec, PagedAttention)
