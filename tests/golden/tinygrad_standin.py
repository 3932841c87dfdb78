"""A stand-in for the part of tinygrad's ``Tensor`` interface that the reference's model file uses,
written on torch CPU tensors, so that src/infurnace/executor/tinygrad/model.py of tylerguest/infurnace can
be imported and run, unmodified, on a machine where tinygrad itself cannot be installed.

What this buys.  With it, the order of operations, the head split and merge, which norm is applied
where, the pairing of the rotation, the causal mask in its three forms (whole prompt, portion on top
of a cache, one decoded token), the grouping of query heads over key/value heads, the rounding of the
stored keys and values, and the tying of the head are the reference's own code, not a restatement.

What it does not buy.  The elementary operations (matrix product, mean, rsqrt, softmax, cos, sin) are
torch's, and the meaning of each method below is written from tinygrad's public documentation of the
method of the same name: ``linear`` is ``x @ w``; ``transpose()`` without arguments swaps the first two
axes; ``scaled_dot_product_attention`` divides the scores by sqrt(head size), masks with -inf under
``is_causal`` (lower triangle) or where a boolean ``attn_mask`` is False, takes the softmax over keys and,
with ``enable_gqa``, repeats each key/value head over its group of query heads; ``assign`` on a sliced
view writes through to the sliced tensor.  Only what the model file, its cache and its weights file touch
is here.

``install()`` puts modules named ``tinygrad``, ``tinygrad.helpers`` and ``tinygrad.llm.gguf`` into
``sys.modules``; nothing of the product imports this file.
"""
from __future__ import annotations

import math
import sys
import types

import torch


class DType:
    def __init__(self, name, torch_dtype):
        self.name, self.torch = name, torch_dtype
        self.itemsize = torch.empty((), dtype=torch_dtype).element_size()

    def __repr__(self):
        return f"dtypes.{self.name}"


class dtypes:  # noqa: N801  (the name is tinygrad's)
    float32 = float = DType("float", torch.float32)
    float16 = half = DType("half", torch.float16)
    float64 = double = DType("double", torch.float64)
    int32 = int = DType("int", torch.int32)
    int64 = long = DType("long", torch.int64)
    uint8 = DType("uchar", torch.uint8)
    bool = DType("bool", torch.bool)
    ints = (int32, int64, uint8)


_BY_TORCH = {d.torch: d for d in (dtypes.float32, dtypes.float16, dtypes.float64, dtypes.int32, dtypes.int64,
                                  dtypes.uint8, dtypes.bool)}


def _t(x):
    return x.t if isinstance(x, Tensor) else x


class Tensor:
    def __init__(self, data, dtype=None, device=None):
        if isinstance(data, Tensor):
            data = data.t
        if not isinstance(data, torch.Tensor):
            data = torch.tensor(data)
            if data.dtype == torch.float64:
                data = data.float()
            if data.dtype == torch.int64:
                data = data.int()
        if dtype is not None:
            data = data.to(dtype.torch)
        self.t = data

    # ------------------------------------------------------------------ properties
    @property
    def shape(self):
        return tuple(self.t.shape)

    @property
    def ndim(self):
        return self.t.dim()

    @property
    def dtype(self):
        return _BY_TORCH[self.t.dtype]

    @property
    def device(self):
        return "CPU"

    def numel(self):
        return self.t.numel()

    # ------------------------------------------------------------------ creation
    @staticmethod
    def arange(start, stop=None, step=1, dtype=None, **kw):
        if stop is None:
            start, stop = 0, start
        out = torch.arange(start, stop, step)
        return Tensor(out.to((dtype or dtypes.int32).torch))

    @staticmethod
    def zeros(*shape, dtype=None, device=None):
        return Tensor(torch.zeros(*shape, dtype=(dtype or dtypes.float32).torch))

    @staticmethod
    def ones(*shape, dtype=None, device=None):
        return Tensor(torch.ones(*shape, dtype=(dtype or dtypes.float32).torch))

    @staticmethod
    def stack(*tensors, dim=0):
        return Tensor(torch.stack([_t(x) for x in tensors], dim=dim))

    # ------------------------------------------------------------------ movement, no arithmetic
    def to(self, device):
        return self

    def contiguous(self):
        return Tensor(self.t.contiguous()) if not self.t.is_contiguous() else self

    def realize(self, *others):
        return self

    def cast(self, dtype):
        return Tensor(self.t.to(dtype.torch))

    def float(self):
        return Tensor(self.t.float())

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        return Tensor(self.t.reshape(*shape))

    def transpose(self, dim0=1, dim1=0):
        return Tensor(self.t.transpose(dim0, dim1))

    def permute(self, *order):
        return Tensor(self.t.permute(*order))

    def unsqueeze(self, dim):
        return Tensor(self.t.unsqueeze(dim))

    def chunk(self, n, dim=0):
        return tuple(Tensor(c) for c in self.t.chunk(n, dim=dim))

    def cat(self, *others, dim=0):
        return Tensor(torch.cat([self.t] + [_t(o) for o in others], dim=dim))

    def __getitem__(self, idx):
        if not isinstance(idx, tuple):
            idx = (idx,)
        idx = tuple(i.t.long() if isinstance(i, Tensor) else i for i in idx)
        return Tensor(self.t[idx])           # basic indexing gives a view, which is what assign() relies on

    def assign(self, other):
        self.t.copy_(_t(other))
        return self

    def tolist(self):
        return self.t.tolist()

    def item(self):
        return self.t.item()

    def argmax(self, axis=None):
        return Tensor(self.t.argmax() if axis is None else self.t.argmax(dim=axis))

    # ------------------------------------------------------------------ arithmetic (torch's type promotion is tinygrad's
    # for the pairs that occur here: float32 with float16 or with a Python number gives float32)
    def __mul__(self, o):
        return Tensor(self.t * _t(o))

    __rmul__ = __mul__

    def __add__(self, o):
        return Tensor(self.t + _t(o))

    __radd__ = __add__

    def __sub__(self, o):
        return Tensor(self.t - _t(o))

    def __truediv__(self, o):
        return Tensor(self.t / _t(o))

    def __rtruediv__(self, o):
        return Tensor(o / self.t)

    def __rpow__(self, base):
        return Tensor(torch.pow(torch.tensor(float(base), dtype=self.t.dtype), self.t))

    def __le__(self, o):
        return Tensor(self.t <= _t(o))

    def square(self):
        return Tensor(self.t * self.t)

    def mean(self, axis=None, keepdim=False):
        return Tensor(self.t.mean(dim=axis, keepdim=keepdim))

    def rsqrt(self):
        return Tensor(torch.rsqrt(self.t))

    def cos(self):
        return Tensor(torch.cos(self.t))

    def sin(self):
        return Tensor(torch.sin(self.t))

    def silu(self):
        return Tensor(self.t * torch.sigmoid(self.t))

    def linear(self, weight, bias=None):
        w = _t(weight)
        x = self.t
        if x.dtype != w.dtype:
            common = torch.promote_types(x.dtype, w.dtype)
            x, w = x.to(common), w.to(common)
        out = x @ w
        return Tensor(out if bias is None else out + _t(bias))

    def scaled_dot_product_attention(self, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, enable_gqa=False):
        q, k, v = self.t, _t(key), _t(value)
        if enable_gqa:
            rep = q.shape[-3] // k.shape[-3]
            k, v = k.repeat_interleave(rep, dim=-3), v.repeat_interleave(rep, dim=-3)
        common = torch.promote_types(torch.promote_types(q.dtype, k.dtype), v.dtype)
        q, k, v = q.to(common), k.to(common), v.to(common)
        scores = q @ k.transpose(-2, -1) / math.sqrt(q.shape[-1])
        if is_causal:
            if attn_mask is not None:
                raise ValueError("is_causal and attn_mask are exclusive")
            rows, cols = scores.shape[-2], scores.shape[-1]
            attn_mask = Tensor(torch.ones(rows, cols, dtype=torch.bool).tril())
        if attn_mask is not None:
            m = _t(attn_mask)
            scores = scores.masked_fill(~m, float("-inf")) if m.dtype == torch.bool else scores + m
        return Tensor(torch.softmax(scores, dim=-1) @ v)


class UOp:
    """Only named in a type annotation of the model file."""


class Variable(UOp):
    pass


def TinyJit(fn):  # noqa: N802
    return fn


class Context:
    def __init__(self, **kw):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def install():
    """Register the stand-in under tinygrad's module names (only if tinygrad itself is absent)."""
    if "tinygrad" in sys.modules:
        return sys.modules["tinygrad"]
    root = types.ModuleType("tinygrad")
    root.Tensor, root.UOp, root.Variable, root.TinyJit, root.dtypes = Tensor, UOp, Variable, TinyJit, dtypes
    root.__stand_in__ = True
    helpers = types.ModuleType("tinygrad.helpers")
    helpers.Context = Context
    llm = types.ModuleType("tinygrad.llm")
    gguf = types.ModuleType("tinygrad.llm.gguf")

    def gguf_load(*a, **kw):
        raise NotImplementedError("the stand-in reads no GGUF files")
    gguf.gguf_load = gguf_load
    llm.gguf = gguf
    root.helpers, root.llm = helpers, llm
    sys.modules.update({"tinygrad": root, "tinygrad.helpers": helpers, "tinygrad.llm": llm, "tinygrad.llm.gguf": gguf})
    return root
