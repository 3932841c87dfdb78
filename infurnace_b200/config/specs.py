"""Architecture-independent descriptions of a model: parts, layers and their order.

A model's ``config.json`` is turned, by the architecture's plan builder, into a
:class:`ModelPlan`: a tuple of layer descriptions, each put together from part
descriptions (norm, mixer, feed-forward, position encoding), and a *schedule*: the
list of layer calls in the order in which they run.  Everything below is plain data
(frozen dataclasses, no tensors), so it imports without torch, as the reference's
model contract does (tests/test_model_config.py:118).

Every part description

* carries its sizes and constants as fields (nothing is a literal in a kernel call),
* names its tensors (``tensors()``: name -> :class:`TensorSpec`), which is what the
  weight loader checks a model folder against, and
* says what it needs from the cache manager (``cache_need()``).

The implementation class of a description is looked up in
``infurnace_b200.parts.registry`` by the description's type, so a new mixer is a new
dataclass plus a class registered for it; neither this file nor the engine changes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


# --------------------------------------------------------------------------- tensors
@dataclass(frozen=True)
class TensorSpec:
    """One tensor of a model folder.  ``kind`` is "float" (kept in the engine's weight
    dtype, see weights/loader.py) or "int" (an integer table, kept as int32)."""
    shape: Tuple[int, ...]
    kind: str = "float"


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedStream:
    """One thing a mixer keeps per token in the pages: ``heads`` rows of ``width`` elements."""
    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class KVCacheNeed:
    """Keys and values that grow with the sequence, kept in pages.

    ``window`` None: every earlier key stays visible.  ``window`` w: a query at
    position p sees keys at positions p-w+1 .. p, and pages that lie wholly below
    that range are given back while the request still runs.  ``value_head_dim``: the
    width of a value head where it differs from a key head's."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_head_dim: Optional[int] = None

    @property
    def streams(self) -> Tuple[PagedStream, ...]:
        return (PagedStream("k", self.num_kv_heads, self.head_dim),
                PagedStream("v", self.num_kv_heads, self.value_head_dim or self.head_dim))

    @property
    def group_key(self):
        return ("kv", self.streams, self.window)


@dataclass(frozen=True)
class PagedCacheNeed:
    """Per-token entries of any shape, kept in pages: a tuple of streams (a compressed latent and a
    small rotated key, say, instead of full keys and values), with the same window rule as
    :class:`KVCacheNeed`.  A cache entry then has one tensor per stream,
    ``[pages, heads, page_size, width]``; streams of equal shape share one tensor
    ``[pages, streams, heads, page_size, width]`` (which is the layout of keys and values)."""
    streams: Tuple[PagedStream, ...]
    window: Optional[int] = None

    @property
    def group_key(self):
        return ("kv", self.streams, self.window)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (``shape`` float32 elements per request)."""
    shape: Tuple[int, ...]

    @property
    def group_key(self):
        return ("state", self.shape)


# --------------------------------------------------------------------------- parts
@dataclass(frozen=True)
class RMSNormSpec:
    """y = x * rsqrt(mean(x^2) + eps) * weight, statistics in 32-bit
    (src/infurnace/executor/tinygrad/model.py:11-13)."""
    size: int
    eps: float
    weight: str  # tensor name

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.size,))}


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding of the first ``rotary_dim`` elements of a head.

    ``interleaved`` False pairs element i with i + rotary_dim/2 (the half-split form
    of model.py:24-27); True pairs 2i with 2i+1.  ``theta`` is the base of the
    frequencies inv_freq_i = theta^(-2i/rotary_dim) (model.py:18-22)."""
    head_dim: int
    rotary_dim: int
    theta: float
    interleaved: bool = False

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {}


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over the paged cache.

    q/k/v/o projections without bias (model.py:102-104,143); optional per-head
    RMSNorm of q and k before the position encoding (model.py:110-114); scores are
    scaled by ``scale`` (the reference leaves it at its attention routine's default,
    1/sqrt(head_dim), model.py:118); causal; optional window."""
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    q_proj: str
    k_proj: str
    v_proj: str
    o_proj: str
    q_norm: Optional[RMSNormSpec] = None
    k_norm: Optional[RMSNormSpec] = None
    position: Optional[RotarySpec] = None
    window: Optional[int] = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {
            self.q_proj: TensorSpec((self.num_heads * self.head_dim, self.hidden_size)),
            self.k_proj: TensorSpec((self.num_kv_heads * self.head_dim, self.hidden_size)),
            self.v_proj: TensorSpec((self.num_kv_heads * self.head_dim, self.hidden_size)),
            self.o_proj: TensorSpec((self.hidden_size, self.num_heads * self.head_dim)),
        }
        for part in (self.q_norm, self.k_norm, self.position):
            if part is not None:
                t.update(part.tensors())
        return t

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class GatedMLPSpec:
    """x -> down(act(gate(x)) * up(x)), no bias (model.py:146-148).  ``activation``
    names the gate's function; "silu" is z * sigmoid(z)."""
    hidden_size: int
    intermediate_size: int
    activation: str
    gate_proj: str
    up_proj: str
    down_proj: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {
            self.gate_proj: TensorSpec((self.intermediate_size, self.hidden_size)),
            self.up_proj: TensorSpec((self.intermediate_size, self.hidden_size)),
            self.down_proj: TensorSpec((self.hidden_size, self.intermediate_size)),
        }

    def cache_need(self):
        return None


@dataclass(frozen=True)
class PreNormBlockSpec:
    """x += mixer(norm1(x)); x += ffn(norm2(x))  (model.py:101,143,145,148)."""
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = {}
        for part in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn):
            t.update(part.tensors())
        return t

    def cache_need(self):
        return self.mixer.cache_need()


@dataclass(frozen=True)
class EmbeddingSpec:
    """x[t] = table[id_t], no scaling (model.py:95)."""
    vocab_size: int
    hidden_size: int
    weight: str

    def tensors(self) -> Mapping[str, TensorSpec]:
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


@dataclass(frozen=True)
class LMHeadSpec:
    """logits = x @ W^T in 32-bit (model.py:151).  ``tied`` True: ``weight`` names the
    embedding table, which is read in place (weights.py:68), and is no tensor of its own;
    ``stored_as`` is then the name under which a model folder may nevertheless store the
    head, which is accepted only as an exact copy of the table (the reference's rule is
    identity of the two, model.py:34-36)."""
    vocab_size: int
    hidden_size: int
    weight: str
    tied: bool
    stored_as: Optional[str] = None

    def tensors(self) -> Mapping[str, TensorSpec]:
        if self.tied:
            return {}
        return {self.weight: TensorSpec((self.vocab_size, self.hidden_size))}


# --------------------------------------------------------------------------- the order
@dataclass(frozen=True)
class LayerCall:
    """One entry of the schedule: run ``layer`` (an index into ``ModelPlan.layers``).

    ``cache`` is the id of the cache entry the layer's mixer reads; it defaults to a
    fresh id per call.  Two calls may name the same layer (shared weights, each with a
    cache of its own) and a call may name another call's cache id with ``store`` False:
    then it reads what that call stored and stores nothing itself."""
    layer: int
    cache: Optional[int] = None
    store: bool = True


@dataclass(frozen=True)
class ModelPlan:
    """All of a model that the loader, the cache manager and the engine need."""
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: Tuple[object, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: object
    lm_head: LMHeadSpec
    extra: Mapping[str, object] = field(default_factory=dict)

    def resolved_schedule(self) -> Tuple[LayerCall, ...]:
        """The schedule with every ``cache`` id filled in: a call without one gets the
        smallest id that no call names."""
        named = {c.cache for c in self.schedule if c.cache is not None}
        out, nxt = [], 0
        for call in self.schedule:
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule names layer {call.layer}; the model has {len(self.layers)}")
            if call.cache is None:
                while nxt in named:
                    nxt += 1
                named.add(nxt)
                call = LayerCall(call.layer, nxt, call.store)
            out.append(call)
        stored = {c.cache for c in out if c.store}
        for call in out:
            if not call.store and call.cache not in stored:
                raise ValueError(f"layer call reads cache {call.cache}, which no call stores")
        return tuple(out)

    def duplicates(self) -> Mapping[str, str]:
        """Names a model folder may hold beside the inventory, each with the tensor it must be an exact
        copy of: the head of a tied model stored under a name of its own."""
        if self.lm_head.tied and self.lm_head.stored_as and self.lm_head.stored_as != self.lm_head.weight:
            return {self.lm_head.stored_as: self.lm_head.weight}
        return {}

    def tensors(self) -> Mapping[str, TensorSpec]:
        t = dict(self.embedding.tensors())
        for layer in self.layers:
            for name, spec in layer.tensors().items():
                if name in t and t[name] != spec:
                    raise ValueError(f"tensor {name} is described twice with different shapes")
                t[name] = spec
        t.update(self.final_norm.tensors())
        t.update(self.lm_head.tensors())
        return t
