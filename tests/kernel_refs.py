"""Plain torch statements of what each CUDA kernel computes, for tests only.

Two uses.  The ``-m gpu`` tests call each kernel alone and compare it with the function of
the same name here, computed in float32 (or float64) on the CPU.  The CPU tests put an
instance of :class:`ReferenceKernels` in the place of the CUDA kernel set, so that the
step function, the cache manager and the scheduler can be exercised on a machine
without a GPU; the package itself never does that and fails if its CUDA libraries
cannot be loaded.

Every function takes the same arguments as the method of the same name of
``infurnace_b200.kernels.cuda.CudaKernels``.
"""
from __future__ import annotations

import torch


class ReferenceKernels:
    name = "reference"

    def __init__(self, compute_dtype=torch.float32, fold=True):
        self.cd = compute_dtype
        self.fold = fold          # offer the folded norm (for few rows, as the CUDA kernels do)

    # ------------------------------------------------------------------ embedding
    def embed(self, table, ids, out):
        out.copy_(table[ids.long()].to(out.dtype))

    def random_normal(self, out, seed64, mean, std):
        """out[i] = mean + std * z_i, the counter-based values of weights/random_init.py."""
        from infurnace_b200.weights.random_init import normal_values
        out.copy_(normal_values(seed64, out.numel(), mean, std).view(out.shape).to(out.dtype))

    # ------------------------------------------------------------------ norm
    def rmsnorm(self, x, weight, eps, out, delta=None, rows=None):
        """x is the float32 residual stream [N, H]; delta ([N, H] or [S, N, H], summed over S)
        is what the previous part adds to it.  Without ``rows``: x += delta in place and
        out[n] = norm(x[n]).  With ``rows`` (int32 [M]): x is left as it is and
        out[m] = norm(x[rows[m]] + delta[rows[m]]).  norm(v) = v * rsqrt(mean(v^2) + eps) *
        weight, statistics in 32-bit, rounded to out's dtype."""
        d = None
        if delta is not None:
            d = delta.to(torch.float32)
            if d.dim() == 3:
                d = d.sum(0)
        if rows is None:
            if d is not None:
                x.add_(d)
            src = x
        else:
            src = x[rows.long()]
            if d is not None:
                src = src + d[rows.long()]
        s = src.to(self.cd)
        y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.cd)
        out.copy_(y.to(out.dtype))

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out, epilogue="none", row_scale=None):
        """out = x @ w^T (w is [out_features, in_features]); accumulation in 32-bit.
        epilogue "silu_gate": w is [2I, K] with the gate rows first; out[n, j] =
        silu(y[n, j]) * y[n, I + j].  row_scale (partials, parts, eps, width): row n of the
        product is multiplied by rsqrt(sum_p partials[p, n] / width + eps) first."""
        y = x.to(self.cd) @ w.to(self.cd).t()
        if row_scale is not None:
            partials, parts, eps, width = row_scale
            r = torch.rsqrt(partials[:parts].to(self.cd).sum(dim=0) / width + eps)
            y = y * r[:, None]
        if epilogue == "silu_gate":
            half = y.shape[1] // 2
            g, u = y[:, :half], y[:, half:]
            y = g * torch.sigmoid(g) * u
        out.copy_(y.to(out.dtype))

    def can_fold_norm(self, n, dtype, w, epilogue="none"):
        return bool(self.fold) and 0 < n <= 64

    def fold_parts(self, out_features, n=None, w=None):
        return -(-out_features // 16)

    def linear_residual_norm(self, a, w, x, norm_weight, out, partials):
        """x += a @ w^T; out = x * norm_weight; partials[p, n] = sum of x[n, 16p:16p+16]^2."""
        x.add_((a.to(self.cd) @ w.to(self.cd).t()).to(x.dtype))
        v = x.to(self.cd)
        out.copy_((v * norm_weight.to(self.cd)[None, :]).to(out.dtype))
        o = v.shape[1]
        parts = self.fold_parts(o)
        sq = torch.zeros(v.shape[0], parts * 16, dtype=self.cd)
        sq[:, :o] = v * v
        partials[:parts].copy_(sq.view(v.shape[0], parts, 16).sum(dim=2).t().to(partials.dtype))

    # ------------------------------------------------------------------ q/k norm, rotation, store
    def rope_table(self, positions, inv_freq, out):
        """out[tok] = (cos, sin) pairs of positions[tok] * inv_freq[i], interleaved: [tokens, 2 * len(inv_freq)]."""
        ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
        out.copy_(torch.stack((ang.cos(), ang.sin()), dim=-1).flatten(-2))

    def qk_norm_rope_store(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps,
                           inv_freq, rotary_dim, interleaved, positions, slot_mapping, kv_pages, rope_table=None):
        """In place on qkv [N, (nq + 2 nkv) d]: per-head RMSNorm of the q and k heads (when
        the weights are given), rotation of q and k by the token's position (when inv_freq
        is given), then k and v are written to the pages at ``slot_mapping`` (slot =
        page * page_size + offset; -1: not stored).  kv_pages: [pages, 2, nkv, page_size, d]."""
        N = qkv.shape[0]
        nq, nkv, d = num_heads, num_kv_heads, head_dim
        q = qkv[:, : nq * d].to(self.cd).reshape(N, nq, d).clone()
        k = qkv[:, nq * d: (nq + nkv) * d].to(self.cd).reshape(N, nkv, d).clone()
        v = qkv[:, (nq + nkv) * d:].view(N, nkv, d)

        def norm(t, w):
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.to(self.cd)

        if q_weight is not None:
            q = norm(q, q_weight)
        if k_weight is not None:
            k = norm(k, k_weight)
        if inv_freq is not None:
            if rope_table is not None:
                pairs = rope_table.view(N, rotary_dim // 2, 2)
                cos, sin = pairs[..., 0].to(self.cd)[:, None, :], pairs[..., 1].to(self.cd)[:, None, :]
            else:
                ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]
                cos, sin = ang.cos().to(self.cd)[:, None, :], ang.sin().to(self.cd)[:, None, :]

            def rot(t):
                r, rest = t[..., :rotary_dim], t[..., rotary_dim:]
                if interleaved:
                    a, b = r[..., 0::2], r[..., 1::2]
                    o = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)
                else:
                    a, b = r[..., : rotary_dim // 2], r[..., rotary_dim // 2:]
                    o = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
                return torch.cat((o, rest), dim=-1)

            q, k = rot(q), rot(k)
        qkv[:, : nq * d] = q.reshape(N, nq * d).to(qkv.dtype)
        qkv[:, nq * d: (nq + nkv) * d] = k.reshape(N, nkv * d).to(qkv.dtype)
        if slot_mapping is not None:
            ps = kv_pages.shape[3]
            kk = k.to(kv_pages.dtype)
            for n in range(N):
                s = int(slot_mapping[n])
                if s < 0:
                    continue
                kv_pages[s // ps, 0, :, s % ps, :] = kk[n]
                kv_pages[s // ps, 1, :, s % ps, :] = v[n].to(kv_pages.dtype)

    # ------------------------------------------------------------------ attention over pages
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q,
                        seq_lens, out, scale, window, max_q_len, max_seq_len, min_q_len=1):
        """For request r the query tokens are rows cu_q[r] .. cu_q[r+1]-1 of qkv (their q
        heads are the first nq*d columns); the last of them stands at position
        seq_lens[r]-1.  A query at position p attends to the keys at positions
        max(0, p-window+1) .. p (window 0: from 0), read from the pages that
        block_tables[r] names.  Softmax in 32-bit.  A query with no visible key gives 0."""
        nq, nkv, d = num_heads, num_kv_heads, head_dim
        ps = kv_pages.shape[3]
        R = cu_q.numel() - 1
        g = nq // nkv
        for r in range(R):
            q0, q1 = int(cu_q[r]), int(cu_q[r + 1])
            n, L = q1 - q0, int(seq_lens[r])
            if n == 0:
                continue
            if L <= 0:
                out[q0:q1] = 0
                continue
            first = 0
            if window:
                first = max(0, (L - n) - window + 1)
            pos = torch.arange(first, L)
            pages = block_tables[r].long()[pos // ps]
            k = kv_pages[pages, 0, :, pos % ps, :].to(self.cd)      # [keys, nkv, d]
            v = kv_pages[pages, 1, :, pos % ps, :].to(self.cd)
            q = qkv[q0:q1, : nq * d].to(self.cd).view(n, nq, d)
            k = k.repeat_interleave(g, dim=1)
            v = v.repeat_interleave(g, dim=1)
            s = torch.einsum("nhd,khd->hnk", q, k) * scale
            qpos = torch.arange(L - n, L)
            vis = pos[None, :] <= qpos[:, None]
            if window:
                vis &= (qpos[:, None] - pos[None, :]) < window
            s = s.masked_fill(~vis[None], float("-inf"))
            p = torch.softmax(s.float(), dim=-1).to(self.cd)
            o = torch.einsum("hnk,khd->nhd", p, v)
            out[q0:q1] = o.reshape(n, nq * d).to(out.dtype)

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, uniform, out):
        """Row m: temperature[m] == 0 -> the index of the largest logit (the lowest such
        index); else the smallest index i with cumsum(softmax(logits/temperature))[i] >
        uniform[m] (the last index with non-zero probability if rounding leaves none)."""
        for m in range(logits.shape[0]):
            t = 0.0 if temperature is None else float(temperature[m])
            row = logits[m].double()
            if t == 0.0:
                out[m] = int(torch.argmax(row))
            else:
                p = torch.softmax(row / t, dim=-1)
                c = torch.cumsum(p, 0)
                idx = int(torch.searchsorted(c, torch.tensor(float(uniform[m]), dtype=torch.float64), right=True))
                out[m] = min(idx, row.numel() - 1)
