"""The CUDA kernel set: thin, checked calls into the compiled libraries.

Every method takes device tensors, checks what the kernel assumes (dtype, contiguity,
matching sizes) and launches on torch's current stream.  There is no CPU path: without
a CUDA device or without the compiled library the constructor raises
:class:`~infurnace_b200.errors.KernelError`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..errors import KernelError
from .build import load_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
_ERRORS = {1: "a dtype (or combination of dtypes) has no kernel", 2: "a size is outside what the kernel takes",
           3: "an address or row length breaks the kernel's alignment rule", 4: "arguments contradict each other"}


def _code(t):
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} has no kernel; float32 and bfloat16 do") from None


def _ptr(t):
    return 0 if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
if _raw_stream is None:                       # an older torch: the public, slower way
    def _raw_stream(device_index):
        return torch.cuda.current_stream(device_index).cuda_stream


def _check(status, what):
    if status == 0:
        return
    if status > 0:
        raise KernelError(f"{what}: refused: {_ERRORS.get(status, status)}")
    raise KernelError(f"{what}: CUDA launch failed with error {-status}")


def _dense(t, name, dtype=None):
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t


class CudaKernels:
    name = "cuda"

    def __init__(self, progress=None):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; this engine has no CPU path")
        self._progress = progress
        self.launches = 0          # kernels launched through this object
        self.scratch_generation = 0  # bumped when a scratch buffer moves: captured graphs go stale
        self.core = load_library("core", progress=progress)
        c = self.core
        c.ifb_embed.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
        c.ifb_random_normal.argtypes = [c_void_p, c_int, c_longlong, ctypes.c_ulonglong, c_float, c_float, c_void_p]
        c.ifb_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int, c_float, c_void_p, c_int,
                                  c_void_p, c_int, c_int, c_void_p]
        c.ifb_qk_norm_rope_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                             c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                             c_void_p]
        c.ifb_rope_table.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]
        c.ifb_sample.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
        c.ifb_argmax_rows.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        self._argmax_scratch = None    # (values, indices, counters) of the several-blocks-per-row argmax
        c.ifb_linear_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p]
        c.ifb_linear_skinny.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p]
        c.ifb_linear_gemv.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                      c_float, c_int, c_void_p]
        c.ifb_linear_gemv_residual_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                    c_int, c_int, c_int, c_void_p]
        c.ifb_linear_gemv_qkv.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                          c_float, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p,
                                          c_int, c_void_p]
        self.fused_qkv = os.environ.get("INFURNACE_FUSED_QKV", "1") != "0"
        self.fused_qkv_calls = 0
        c.ifb_linear_gemv_set_plan.argtypes = [c_int]
        c.ifb_linear_gemv_set_plan.restype = None
        c.ifb_linear_skinny_scratch.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        c.ifb_linear_skinny_scratch.restype = None
        self._lin_partials = None
        self._lin_counters = None
        self.gemv_max_rows = 64        # up to here: the kernel without global partial sums
        # up to here norms are folded into products (the kernels take 64 rows; beyond 32 the separate norm measured faster)
        self.fold_max_rows = int(os.environ.get("INFURNACE_FOLD_MAX_ROWS", "32"))
        self.split_min_keys = int(os.environ.get("INFURNACE_SPLIT_MIN_KEYS", "256"))   # fewest keys a split of a context gets
        self._tc = None                # the tcgen05 library, loaded when a product first has more than tc_min_rows rows
        # device int: non-zero after a kernel recorded a fault it contained (a bounded barrier wait that gave up, a
        # token id outside the vocabulary); read by check_device_errors
        self._dev_err = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.attention_tma = True      # keys and values by TMA where the sizes allow (else 16-byte async copies)
        self.attention_tc = True       # prompts on tcgen05 where the sizes allow (head size 128, pages of 16/32/64)
        self._attn_tc = None
        self.tc_attention_calls = 0    # launches of the tcgen05 attention kernel, of the small-q kernel, and of the latter
        self.small_q_calls = 0         # with keys and values by TMA (what ran is what tests of the product path ask)
        self.small_q_tma_calls = 0
        self.tc_shared_k_calls = 0     # tcgen05 products with the k range shared by a cluster; with a folded norm
        self.tc_folded_calls = 0
        self._err_armed = False
        self.tc_min_rows = 65
        if os.environ.get("INFURNACE_GATE_PLAN"):
            self.core.ifb_linear_gemv_set_gate_plan(int(os.environ["INFURNACE_GATE_PLAN"]))
        self.tc_split_min_k = int(os.environ.get("INFURNACE_TC_SPLIT_MIN_K", "256"))
        self.fused_qkv_tc = os.environ.get("INFURNACE_FUSED_QKV_TC", "1") != "0"
        self.tc_split_min_rows = int(os.environ.get("INFURNACE_TC_SPLIT_MIN_ROWS", "0"))     # 0: by the matrix
        self.tc_fold_max_rows = int(os.environ.get("INFURNACE_TC_FOLD_MAX_ROWS", "128"))
        self._tc_clusters = {}         # CTAs per cluster -> clusters of the split product that run at a time
        self._route_memo = {}          # what _on_tcgen05 and tcgen05_splits answered (asked several times per launch)
        self._splits_memo = {}
        self._attn_mma = {}        # head size -> library
        self._attn_scratch = None
        self._attn_counters = None
        self.sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self.attention_scratch_cap = 64 << 20     # bytes of split scratch beyond which a step runs unsplit
        c.ifb_paged_attention_simt.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                               c_void_p]

    @staticmethod
    def _stream():
        # the raw handle of torch's current stream on the current device (torch.cuda.current_stream() builds a Stream
        # object around it on every call, which was a fifth of an eager step's host time)
        return _raw_stream(torch._C._cuda_getDevice())

    # ------------------------------------------------------------------ embedding
    def embed(self, table, ids, out):
        _dense(table, "table"), _dense(ids, "ids", torch.int32), _dense(out, "out", torch.float32)
        n, hidden = out.shape
        if table.shape[1] != hidden or ids.numel() != n:
            raise KernelError("embed: sizes of table, ids and out do not match")
        self.launches += 1
        self._err_armed = True
        _check(self.core.ifb_embed(table.data_ptr(), _code(table), ids.data_ptr(), out.data_ptr(), n, hidden,
                                   table.shape[0], self._dev_err.data_ptr(), self._stream()), "embed")

    def random_normal(self, out, seed64, mean, std):
        """out[i] = mean + std * z_i with z_i approximately N(0, 1), a pure function of (seed64, i): the
        same bits as ``weights.random_init.normal_values``."""
        _dense(out, "out")
        self.launches += 1
        _check(self.core.ifb_random_normal(out.data_ptr(), _code(out), out.numel(), int(seed64) & ((1 << 64) - 1),
                                           float(mean), float(std), self._stream()), "random_normal")

    # ------------------------------------------------------------------ norm
    def rmsnorm(self, x, weight, eps, out, delta=None, rows=None):
        _dense(x, "x", torch.float32), _dense(weight, "weight"), _dense(out, "out")
        hidden = x.shape[1]
        n_out = out.shape[0]
        if weight.numel() != hidden or out.shape[1] != hidden:
            raise KernelError("rmsnorm: widths of x, weight and out do not match")
        splits, stride = 0, 0
        if delta is not None:
            _dense(delta, "delta", torch.float32)
            if delta.dim() == 3:
                splits, stride = delta.shape[0], delta.stride(0)
                drows = delta.shape[1]
            else:
                splits, stride, drows = 1, 0, delta.shape[0]
            if delta.shape[-1] != hidden or drows != x.shape[0]:
                raise KernelError("rmsnorm: delta does not match x")
        if rows is not None:
            _dense(rows, "rows", torch.int32)
            if rows.numel() != n_out:
                raise KernelError("rmsnorm: out has a row for each entry of rows")
        elif n_out != x.shape[0]:
            raise KernelError("rmsnorm: out has a row for each row of x")
        self.launches += 1
        _check(self.core.ifb_rmsnorm(x.data_ptr(), _ptr(delta), splits, stride, weight.data_ptr(), _code(weight),
                                     float(eps), out.data_ptr(), _code(out), _ptr(rows), n_out, hidden,
                                     self._stream()), "rmsnorm")

    # ------------------------------------------------------------------ matrix products
    def linear(self, x, w, out, epilogue="none", row_scale=None):
        """out = x w^T with the epilogue.  ``row_scale`` (partials, parts, eps, width), from
        :meth:`linear_residual_norm`, multiplies row n by rsqrt(sum_p partials[p, n] / width + eps)
        before the epilogue; only where :meth:`can_fold_norm` says so."""
        _dense(x, "x"), _dense(w, "w"), _dense(out, "out")
        n, k = x.shape
        o = out.shape[1]
        epi = {"none": 0, "silu_gate": 1}[epilogue]
        if w.shape[1] != k or out.shape[0] != n or w.shape[0] != (2 * o if epi else o):
            raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not match")
        if row_scale is not None:
            if not self.can_fold_norm(n, x.dtype, w, epilogue) or out.dtype not in (torch.bfloat16, torch.float32):
                raise KernelError("linear: a row scale is taken only by the bfloat16 kernels (see can_fold_norm)")
            partials, parts = row_scale[0], row_scale[1]
            _dense(partials, "row_scale partials", torch.float32)
            if partials.dim() != 2 or partials.shape[0] < parts or partials.shape[1] != n:
                raise KernelError("linear: row_scale partials must be [parts, rows]")
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 8 == 0 \
                and out.dtype in (torch.bfloat16, torch.float32):
            if self._on_tcgen05(n, w, epilogue):
                return self._linear_tcgen05(x, w, out, n, o, k, epi, splits=self.tcgen05_splits(n, o, k, epi),
                                            row_scale=row_scale)
            return self._linear_gemv(x, w, out, n, o, k, epi, row_scale)
        self.launches += 1
        _check(self.core.ifb_linear_simt(x.data_ptr(), _code(x), w.data_ptr(), _code(w), out.data_ptr(), _code(out),
                                         n, o, k, epi, self._stream()), "linear")

    def _on_tcgen05(self, n, w, epilogue="none", shared_k=True):
        key = (n, w.shape[0], w.shape[1], w.dtype, epilogue, shared_k)
        hit = self._route_memo.get(key)
        if hit is None:
            hit = self._route_memo[key] = self._on_tcgen05_rule(n, w, epilogue, shared_k)
        return hit

    def _on_tcgen05_rule(self, n, w, epilogue, shared_k):
        """Which kernel a bfloat16 product of n rows against w runs on.  More than 64 rows: the tcgen05 kernel.
        From ``tc_split_min_rows`` rows, a product with the plain epilogue whose few tiles can share their k
        range in clusters (:meth:`tcgen05_splits`): the tcgen05 kernel in that form, which streams a long k
        faster than the few-rows kernel.  Else up to 8 rows: the few-rows kernel.  Between, by measurement:
        the few-rows kernel re-reads the rows from L2 in every CTA, so for a large weight matrix (from 2^24
        elements, or from 33 rows and 4,096 features) the tcgen05 kernel, which streams the weights once
        through its tiles, is the faster one although most of its 128-row tile is empty."""
        if n >= self.tc_min_rows:
            return True
        if shared_k and epilogue == "none" and n >= self._shared_k_min_rows(w) and w.dtype == torch.bfloat16 \
                and w.shape[1] % 8 == 0 and self.tcgen05_splits(n, w.shape[0], w.shape[1]) > 1:
            return True
        if n <= 8:
            return False
        return w.numel() >= (1 << 24) or (n >= 33 and w.shape[0] >= 4096)

    def _shared_k_min_rows(self, w):
        """From how many rows the tcgen05 kernel with a shared k range beats the few-rows kernel, by
        measurement in a step's graph (o and down products of the 0.6B, 8B and 32B sizes): 17 for a small
        matrix (the few-rows kernel is bound by its round trips, not by its bytes); 9 for a large one (a
        second block of 8 rows costs the few-rows kernel a third more); 1 where the few-rows kernel with
        its one CTA of 16 features per SM (long k) leaves most of its last wave empty (5,120 features:
        320 CTAs on 148 SMs; a decode step of one row of the 32B sizes 14.13 against 13.74 ms)."""
        if self.tc_split_min_rows:
            return self.tc_split_min_rows
        o, k = w.shape
        waves = -(-o // 16) / self.sm_count
        if k > 3072 and -(-waves // 1) / waves > 1.25:
            return 1
        return 9 if w.numel() >= (1 << 23) else 17

    def _linear_tcgen05(self, x, w, out, n, o, k, epi, shape=0, splits=1, row_scale=None, residual=None):
        """shape: 0 lets the library choose its tile shape; 1 narrow, 2 deep, 3 wide, 4 and 5 persistent.
        splits > 1: the k range of a tile is shared by a cluster of that many CTAs.  row_scale: as in
        :meth:`linear`.  residual (x, norm_weight, partials): as in :meth:`linear_residual_norm`."""
        partials, parts, eps, width = row_scale if row_scale is not None else (None, 0, 0.0, 0)
        res_x, res_g, res_partials = residual if residual is not None else (None, None, None)
        self.launches += 1
        self.tc_shared_k_calls += splits > 1
        self.tc_folded_calls += partials is not None or res_x is not None
        self._err_armed = True
        _check(self._tc_lib().ifb_linear_tcgen05_ex(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), n, o, k, epi, int(shape), int(splits),
            _ptr(partials), int(parts), float(eps), int(width), _ptr(res_x), _ptr(res_g),
            _code(res_g) if res_g is not None else 0, _ptr(res_partials), self._dev_err.data_ptr(), self._stream()), "linear")

    def _tc_lib(self):
        if self._tc is None:
            self._tc = load_library("linear_tcgen05", progress=self._progress)
            self._tc.ifb_linear_tcgen05_ex.argtypes = [
                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float,
                c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]
            self._tc.ifb_linear_tcgen05_split_clusters.argtypes = [c_int]
            self._tc.ifb_linear_tcgen05_fold_parts.argtypes = [c_int, c_int, c_int]
            self._tc.ifb_linear_tcgen05_qkv.argtypes = [
                c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int,
                c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        return self._tc

    def tcgen05_splits(self, n, o, k, epi=0):
        """How many CTAs (a cluster) share the k range of a tile in the tcgen05 product of up to 512 rows
        (128 with the silu_gate epilogue): the most, up to 8, whose clusters for all tiles of 128 x 128
        run at the same time, each CTA with at least ``tc_split_min_k`` of k; 1 if that is none."""
        key = (n, o, k, bool(epi))
        hit = self._splits_memo.get(key)
        if hit is None:
            hit = self._splits_memo[key] = self._tcgen05_splits_rule(n, o, k, epi)
        return hit

    def _tcgen05_splits_rule(self, n, o, k, epi):
        if n > (128 if epi else 512):
            return 1
        tiles = -(-o // 128) * -(-n // 128)
        for splits in range(min(8, k // self.tc_split_min_k), 1, -1):
            if splits not in self._tc_clusters:
                self._tc_clusters[splits] = int(self._tc_lib().ifb_linear_tcgen05_split_clusters(splits))
            if tiles <= self._tc_clusters[splits]:
                return splits
        return 1

    def _linear_tcgen05_split(self, x, w, out, n, o, k, splits):
        """The one-tile kernel with the k range of a tile shared by a cluster of ``splits`` CTAs."""
        self._linear_tcgen05(x, w, out, n, o, k, 0, splits=splits)

    def check_device_errors(self):
        """Raise if a kernel recorded a fault that it contained: a bounded wait on a barrier that gave
        up, or a token id outside the vocabulary at the embedding (synchronises)."""
        if self._err_armed:
            self._err_armed = False
            code = int(self._dev_err.item())
            if code:
                self._dev_err.zero_()
                if code == 900:
                    raise KernelError("a token id outside the vocabulary reached the embedding (code 900): the step "
                                      "that sampled it had no valid logits; its output is not valid")
                raise KernelError(f"a kernel gave up waiting on a barrier (code {code}); its output is not valid")

    def _linear_gemv(self, x, w, out, n, o, k, epi, row_scale=None):
        self.launches += 1
        partials, parts, eps, width = row_scale if row_scale is not None else (None, 0, 0.0, 0)
        if partials is not None:
            _dense(partials, "row_scale partials", torch.float32)
            if partials.dim() != 2 or partials.shape[0] < parts or partials.shape[1] != n:
                raise KernelError("linear: row_scale partials must be [parts, rows]")
        _check(self.core.ifb_linear_gemv(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), n, o, k, epi,
                                         _ptr(partials), int(parts), float(eps), int(width), self._stream()), "linear")

    # A norm folded into the products around it: RMSNorm(v) = v * g * r with one r per row, so the product that
    # makes v writes v * g and partial sums of v^2, and the product that reads it multiplies by r at its end.
    def can_fold_norm(self, n, dtype, w, epilogue="none"):
        """Whether a product of ``n`` rows of ``dtype`` against ``w`` (with that epilogue) takes or makes a
        folded norm: on the tcgen05 kernel up to ``tc_fold_max_rows`` rows (one tile of rows: with many
        rows the longer epilogue costs what the norm's own launch did), on the few-rows kernel up to
        ``fold_max_rows``."""
        if not (dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and n > 0
                and self.fold_max_rows > 0):
            return False
        if self._on_tcgen05(n, w, epilogue):
            return n <= self.tc_fold_max_rows
        return n <= min(self.gemv_max_rows, self.fold_max_rows)

    def fold_parts(self, out_features, n=None, w=None):
        """Partial sums per row that :meth:`linear_residual_norm` writes for a product of ``n`` rows against
        ``w`` (without them: on the few-rows kernel)."""
        if n is not None and w is not None and self._on_tcgen05(n, w):
            splits = self.tcgen05_splits(n, w.shape[0], w.shape[1])
            return int(self._tc_lib().ifb_linear_tcgen05_fold_parts(int(n), int(out_features), int(splits)))
        return int(self.core.ifb_linear_gemv_parts(int(out_features), int(n) if n is not None else 1 << 20))

    def linear_residual_norm(self, a, w, x, norm_weight, out, partials):
        """x += a w^T (x float32, in place); out = x * norm_weight (bfloat16); partials[p, n] = the sum
        of squares of row n of x over part p's features.  With ``linear(..., row_scale=(partials,
        fold_parts(o, n, w), eps, o))`` after it this is x += a w^T followed by an RMSNorm of x."""
        _dense(a, "a", torch.bfloat16), _dense(w, "w", torch.bfloat16), _dense(x, "x", torch.float32)
        _dense(out, "out", torch.bfloat16), _dense(partials, "partials", torch.float32), _dense(norm_weight, "norm_weight")
        n, k = a.shape
        o = w.shape[0]
        parts = self.fold_parts(o, n, w)
        if w.shape[1] != k or x.shape != (n, o) or out.shape != (n, o) or norm_weight.numel() != o \
                or partials.dim() != 2 or partials.shape[0] < parts or partials.shape[1] != n:
            raise KernelError("linear_residual_norm: sizes of a, w, x, norm_weight, out and partials do not match")
        if not self.can_fold_norm(n, a.dtype, w):
            raise KernelError("linear_residual_norm: only for bfloat16 (see can_fold_norm)")
        if self._on_tcgen05(n, w):
            return self._linear_tcgen05(a, w, out, n, o, k, 0, splits=self.tcgen05_splits(n, o, k),
                                        residual=(x, norm_weight, partials))
        self.launches += 1
        _check(self.core.ifb_linear_gemv_residual_norm(
            a.data_ptr(), w.data_ptr(), x.data_ptr(), norm_weight.data_ptr(), _code(norm_weight), out.data_ptr(),
            partials.data_ptr(), n, o, k, self._stream()), "linear_residual_norm")

    # The split-k product with scratch from the caller: not on linear()'s path (tcgen05 takes 65 rows and more, the
    # kernel above 64 and fewer); it is the kernel whose static-scratch variant the library linear_skinny_static exports.
    def linear_splits(self, n, o, k):
        """CTAs that share the k range of one 64-feature tile: enough to cover the SMs twice, and
        at least 256 of k each."""
        blocks = 1 if n <= 8 else 2 if n <= 16 else 4 if n <= 32 else 8
        tiles = -(-o // 64) * -(-n // (blocks * 8))
        return max(1, min(-(-2 * self.sm_count // tiles), k // 256))

    def _linear_skinny(self, x, w, out, n, o, k, epi, splits=None):
        if splits is None:
            splits = self.linear_splits(n, o, k)
        partials = counters = None
        if splits > 1:
            nf, nc = ctypes.c_longlong(), ctypes.c_longlong()
            self.core.ifb_linear_skinny_scratch(n, o, epi, splits, ctypes.byref(nf), ctypes.byref(nc))
            if self._lin_partials is None or self._lin_partials.numel() < nf.value:
                self._lin_partials = torch.empty(max(nf.value, 1 << 20), dtype=torch.float32, device="cuda")
                self.scratch_generation += 1
            if self._lin_counters is None or self._lin_counters.numel() < nc.value:
                self._lin_counters = torch.zeros(max(nc.value, 1 << 14), dtype=torch.int32, device="cuda")
                self.scratch_generation += 1
            partials, counters = self._lin_partials, self._lin_counters
        self.launches += 1
        _check(self.core.ifb_linear_skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), _code(out), _ptr(partials),
                                           _ptr(counters), n, o, k, epi, splits, self._stream()), "linear")

    # The q | k | v projection of a decode step with the head norm, the rotation and the page store in its epilogue.
    def can_fuse_qkv(self, n, dtype, w_qkv, head_dim, rotary_dim, interleaved, kv_pages):
        """Whether :meth:`linear_qkv_rope_store` takes a step of ``n`` rows: bfloat16, heads rotated whole in
        the half-split pairing (or not rotated); up to 16 rows on the few-rows kernel (heads of 64, 128 or
        256), or up to 128 rows on the tcgen05 kernel in its shared-k form (heads of 128)."""
        if not (self.fused_qkv and n > 0 and dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16
                and w_qkv.shape[1] % 8 == 0 and (rotary_dim == 0 or (rotary_dim == head_dim and not interleaved))
                and (kv_pages is None or kv_pages.dtype == torch.bfloat16)):
            return False
        return self._fused_qkv_route(n, w_qkv, head_dim) is not None

    def _fused_qkv_route(self, n, w_qkv, head_dim):
        """"gemv", "tcgen05" or None for the fused q | k | v product of ``n`` rows."""
        if n <= 16 and head_dim in (64, 128, 256) and not self._on_tcgen05(n, w_qkv, shared_k=False):
            return "gemv"
        if n <= 128 and head_dim == 128 and self.fused_qkv_tc and self._on_tcgen05(n, w_qkv) \
                and self.tcgen05_splits(n, w_qkv.shape[0], w_qkv.shape[1]) > 1:
            return "tcgen05"
        return None

    def linear_qkv_rope_store(self, x, w_qkv, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, rope_table,
                              slot_mapping, kv_pages, row_scale=None):
        """qkv = x w_qkv^T, then per head what :meth:`qk_norm_rope_store` does (RMSNorm of the q and k heads,
        rotation by the angles of ``rope_table``, k and v into the pages at ``slot_mapping``), in one launch."""
        _dense(x, "x", torch.bfloat16), _dense(w_qkv, "w_qkv", torch.bfloat16), _dense(qkv, "qkv", torch.bfloat16)
        n, k = x.shape
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if w_qkv.shape != (width, k) or qkv.shape != (n, width):
            raise KernelError("linear_qkv_rope_store: sizes of x, w_qkv and qkv do not match the heads")
        wd = F32
        for wt in (q_weight, k_weight):
            if wt is not None:
                _dense(wt, "norm weight")
                if wt.numel() != head_dim:
                    raise KernelError("linear_qkv_rope_store: norm weight length is not head_dim")
                wd = _code(wt)
        if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("linear_qkv_rope_store: q and k norm weights differ in dtype")
        if rope_table is not None:
            _dense(rope_table, "rope_table", torch.float32)
            if rope_table.shape != (n, head_dim):
                raise KernelError("linear_qkv_rope_store: rope_table is [tokens, head_dim]")
        page_size = 1
        if slot_mapping is not None:
            _dense(slot_mapping, "slot_mapping", torch.int32), _dense(kv_pages, "kv_pages", torch.bfloat16)
            if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads \
                    or kv_pages.shape[4] != head_dim or slot_mapping.numel() != n:
                raise KernelError("linear_qkv_rope_store: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
            page_size = kv_pages.shape[3]
        partials, parts, seps, swidth = row_scale if row_scale is not None else (None, 0, 0.0, 0)
        self.launches += 1
        self.fused_qkv_calls += 1
        route = self._fused_qkv_route(n, w_qkv, head_dim)
        if route is None:
            raise KernelError("linear_qkv_rope_store: no kernel takes these sizes (see can_fuse_qkv)")
        if route == "tcgen05":
            self._err_armed = True
            self.tc_shared_k_calls += 1
            self.tc_folded_calls += partials is not None
            _check(self._tc_lib().ifb_linear_tcgen05_qkv(
                x.data_ptr(), w_qkv.data_ptr(), qkv.data_ptr(), n, num_heads, num_kv_heads, head_dim, k,
                self.tcgen05_splits(n, width, k), _ptr(partials), int(parts), float(seps), int(swidth), _ptr(q_weight),
                _ptr(k_weight), wd, float(eps), _ptr(rope_table), _ptr(slot_mapping),
                _ptr(kv_pages) if slot_mapping is not None else 0, page_size, self._dev_err.data_ptr(), self._stream()),
                "linear_qkv_rope_store")
            return
        _check(self.core.ifb_linear_gemv_qkv(
            x.data_ptr(), w_qkv.data_ptr(), qkv.data_ptr(), n, num_heads, num_kv_heads, head_dim, k, _ptr(partials),
            int(parts), float(seps), int(swidth), _ptr(q_weight), _ptr(k_weight), wd, float(eps), _ptr(rope_table),
            _ptr(slot_mapping), _ptr(kv_pages) if slot_mapping is not None else 0, page_size, self._stream()),
            "linear_qkv_rope_store")

    # ------------------------------------------------------------------ q/k norm, rotation, store
    def rope_table(self, positions, inv_freq, out):
        """out[tok, i] = (cos, sin)(positions[tok] * inv_freq[i]), float32 ``[tokens, 2 * len(inv_freq)]``."""
        _dense(positions, "positions", torch.int32), _dense(inv_freq, "inv_freq", torch.float32)
        _dense(out, "out", torch.float32)
        n, half = positions.numel(), inv_freq.numel()
        if out.shape != (n, 2 * half):
            raise KernelError("rope_table: out is [tokens, 2 * len(inv_freq)]")
        self.launches += 1
        _check(self.core.ifb_rope_table(positions.data_ptr(), inv_freq.data_ptr(), half, out.data_ptr(), n, self._stream()),
               "rope_table")

    def qk_norm_rope_store(self, qkv, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, inv_freq,
                           rotary_dim, interleaved, positions, slot_mapping, kv_pages, rope_table=None):
        _dense(qkv, "qkv")
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("qk_norm_rope_store: qkv width is not (heads + 2 kv_heads) * head_dim")
        wd = F32
        for wt in (q_weight, k_weight):
            if wt is not None:
                _dense(wt, "norm weight")
                if wt.numel() != head_dim:
                    raise KernelError("qk_norm_rope_store: norm weight length is not head_dim")
                wd = _code(wt)
        if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("qk_norm_rope_store: q and k norm weights differ in dtype")
        if inv_freq is not None:
            _dense(inv_freq, "inv_freq", torch.float32), _dense(positions, "positions", torch.int32)
            if inv_freq.numel() != rotary_dim // 2 or positions.numel() != n:
                raise KernelError("qk_norm_rope_store: inv_freq or positions has the wrong length")
            if rope_table is not None:
                _dense(rope_table, "rope_table", torch.float32)
                if rope_table.shape != (n, rotary_dim):
                    raise KernelError("qk_norm_rope_store: rope_table is [tokens, rotary_dim]")
        page_size = 1
        if slot_mapping is not None:
            _dense(slot_mapping, "slot_mapping", torch.int32), _dense(kv_pages, "kv_pages", qkv.dtype)
            if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads \
                    or kv_pages.shape[4] != head_dim or slot_mapping.numel() != n:
                raise KernelError("qk_norm_rope_store: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
            page_size = kv_pages.shape[3]
        self.launches += 1
        _check(self.core.ifb_qk_norm_rope_store(
            qkv.data_ptr(), _code(qkv), n, num_heads, num_kv_heads, head_dim, _ptr(q_weight), _ptr(k_weight), wd,
            float(eps), _ptr(inv_freq), _ptr(rope_table) if inv_freq is not None else 0, int(rotary_dim),
            int(bool(interleaved)), _ptr(positions), _ptr(slot_mapping),
            _ptr(kv_pages) if slot_mapping is not None else 0, page_size, self._stream()), "qk_norm_rope_store")

    # ------------------------------------------------------------------ attention
    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out,
                        scale, window, max_q_len, max_seq_len, min_q_len=1):
        _dense(qkv, "qkv"), _dense(kv_pages, "kv_pages", qkv.dtype), _dense(out, "out", qkv.dtype)
        _dense(cu_q, "cu_q", torch.int32), _dense(seq_lens, "seq_lens", torch.int32)
        if block_tables.dtype != torch.int32 or block_tables.stride(1) != 1:
            raise KernelError("paged_attention: block_tables must be int32 with unit stride along pages")
        n = qkv.shape[0]
        r = seq_lens.numel()
        if cu_q.numel() != r + 1 or block_tables.shape[0] < r or out.shape != (n, num_heads * head_dim):
            raise KernelError("paged_attention: sizes of cu_q, seq_lens, block_tables and out do not match")
        if kv_pages.dim() != 5 or kv_pages.shape[1] != 2 or kv_pages.shape[2] != num_kv_heads \
                or kv_pages.shape[4] != head_dim:
            raise KernelError("paged_attention: kv_pages is not [pages, 2, kv_heads, page_size, head_dim]")
        group = num_heads // num_kv_heads
        if qkv.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256 and group <= 16 \
                and num_heads % num_kv_heads == 0:
            return self._paged_attention_mma(qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q,
                                             seq_lens, out, scale, window, max_q_len, max_seq_len, n, r,
                                             min_q_len=min_q_len)
        self.launches += 1
        _check(self.core.ifb_paged_attention_simt(
            qkv.data_ptr(), _code(qkv), qkv.stride(0), kv_pages.data_ptr(), block_tables.data_ptr(),
            block_tables.stride(0), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), n, r, num_heads,
            num_kv_heads, head_dim, kv_pages.shape[3], float(scale), int(window), self._stream()), "paged_attention")

    def _attention_tc(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out, scale,
                      window, max_q_len, n, r):
        if self._attn_tc is None:
            self._attn_tc = load_library("attention_tc", progress=self._progress)
            self._attn_tc.ifb_attention_tc.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                                       c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                                       c_int, c_int, c_void_p]
        self._err_armed = True
        self.launches += 1
        self.tc_attention_calls += 1
        _check(self._attn_tc.ifb_attention_tc(
            qkv.data_ptr(), qkv.stride(0), kv_pages.data_ptr(), kv_pages.shape[0], block_tables.data_ptr(),
            block_tables.stride(0), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), self._dev_err.data_ptr(), n, r,
            num_heads, num_kv_heads, head_dim, kv_pages.shape[3], float(scale), int(window), int(max_q_len), self._stream()),
            "paged_attention")

    def attention_library(self, head_dim):
        lib = self._attn_mma.get(head_dim)
        if lib is None:
            lib = load_library("attention_mma", {"HEAD_DIM": head_dim}, progress=self._progress)
            lib.ifb_attention_mma.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                              c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
            lib.ifb_attention_mma_scratch_floats.restype = c_longlong
            lib.ifb_attention_mma_scratch_floats.argtypes = [c_int, c_int, c_int]
            self._attn_mma[head_dim] = lib
        return lib

    def attention_splits(self, num_requests, num_kv_heads, max_seq_len, window=0):
        """How many CTAs share one (request, key/value head) of the small-q kernel: as many as
        keep the whole grid resident at once (two CTAs fit on an SM), so that no second wave
        runs, and no fewer than ``split_min_keys`` keys per split (256, four tiles: with 128 a lone
        request's 32 partial results cost more to merge than the shorter splits saved)."""
        reach = min(max_seq_len, window + 16) if window else max_seq_len
        fit = (2 * self.sm_count) // max(1, num_requests * num_kv_heads)
        return max(1, min(fit, -(-reach // self.split_min_keys), 32))

    def attention_scratch(self, floats):
        if self._attn_scratch is None or self._attn_scratch.numel() < floats:
            self._attn_scratch = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device="cuda")
            self.scratch_generation += 1
        return self._attn_scratch

    def _paged_attention_mma(self, qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out,
                             scale, window, max_q_len, max_seq_len, n, r, num_splits=None, min_q_len=1):
        lib = self.attention_library(head_dim)
        group = num_heads // num_kv_heads
        only_small = max_q_len * group <= 16
        if num_splits is None:
            num_splits = self.attention_splits(r, num_kv_heads, max_seq_len, window)
        need = lib.ifb_attention_mma_scratch_floats(n, num_heads, num_splits)
        if need * 4 > self.attention_scratch_cap:
            num_splits, need = 1, 0
        scratch = self.attention_scratch(need) if need else None
        counters = None
        if need:
            if self._attn_counters is None or self._attn_counters.numel() < r * num_kv_heads:
                self._attn_counters = torch.zeros(max(r * num_kv_heads, 4096), dtype=torch.int32, device="cuda")
                self.scratch_generation += 1
            counters = self._attn_counters
        use_tc = (not only_small and self.attention_tc and head_dim == 128 and 128 % group == 0
                  and kv_pages.shape[3] in (16, 32, 64) and kv_pages.data_ptr() % 128 == 0)
        if use_tc:
            self._attention_tc(qkv, num_heads, num_kv_heads, head_dim, kv_pages, block_tables, cu_q, seq_lens, out, scale,
                               window, max_q_len, n, r)
            if min_q_len * group > 16:
                return                 # no request of this step is left for the small-q kernel
            only_small = True          # the tile kernel's requests are done; the small-q kernel takes the rest
        self.launches += 1 + (0 if only_small else 1)
        self.small_q_calls += 1
        if self.attention_tma and head_dim % 64 == 0 and kv_pages.shape[3] in (16, 32, 64) \
                and kv_pages.data_ptr() % 128 == 0 and kv_pages.numel() // head_dim < 0x7fffffff:
            self.small_q_tma_calls += 1        # the library's own condition for its TMA path
        self._err_armed = True
        _check(lib.ifb_attention_mma(
            qkv.data_ptr(), qkv.stride(0), kv_pages.data_ptr(), kv_pages.shape[0], block_tables.data_ptr(),
            block_tables.stride(0), cu_q.data_ptr(), seq_lens.data_ptr(), out.data_ptr(), _ptr(scratch), _ptr(counters),
            self._dev_err.data_ptr(), n, r, num_heads, num_kv_heads, head_dim, kv_pages.shape[3], float(scale), int(window),
            int(max_q_len), int(num_splits), 1, 0 if only_small else 1, 1 if self.attention_tma else 0, self._stream()),
            "paged_attention")

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, uniform, out):
        _dense(logits, "logits", torch.float32), _dense(out, "out", torch.int32)
        m, vocab = logits.shape
        if temperature is not None:
            _dense(temperature, "temperature", torch.float32), _dense(uniform, "uniform", torch.float32)
            if temperature.numel() != m or uniform.numel() != m:
                raise KernelError("sample: one temperature and one uniform number per row")
        if out.numel() != m:
            raise KernelError("sample: out has one entry per row")
        self.launches += 1
        if temperature is None and vocab >= 16384 and m <= 4096:
            # greedy over a large vocabulary: several blocks per row, enough to fill the device about twice
            bpr = max(1, min(64, (2 * self.sm_count) // m, vocab // 2048))
            if bpr > 1:
                if self._argmax_scratch is None:
                    self._argmax_scratch = (torch.empty(4096 * 64, dtype=torch.float32, device="cuda"),
                                            torch.empty(4096 * 64, dtype=torch.int32, device="cuda"),
                                            torch.zeros(4096, dtype=torch.int32, device="cuda"))
                    self.scratch_generation += 1
                vals, idxs, counters = self._argmax_scratch
                return _check(self.core.ifb_argmax_rows(logits.data_ptr(), m, vocab, bpr, vals.data_ptr(), idxs.data_ptr(),
                                                        counters.data_ptr(), out.data_ptr(), self._stream()), "sample")
        _check(self.core.ifb_sample(logits.data_ptr(), m, vocab, _ptr(temperature), _ptr(uniform), out.data_ptr(),
                                    self._stream()), "sample")
