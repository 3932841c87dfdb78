"""The step function: one batch of (request, its next tokens) through the model.

The reference's runner contract has two calls for one request at a time,
``prefill(ids[1,T], slot, start_position)`` and ``decode(ids[1,1], position, slot)``
(src/infurnace/executor/runner.py:22-37), and its documents ask for the packed batch
contract to be written down before it is built (docs/architecture.md:178-182).  This is
that contract: a step is a list of entries; an entry is a live request, its next
tokens (a whole prompt, a portion of one cut anywhere, or one decoded token) and the
places among them whose logits are wanted.  All entries run as one batch on one flat
token axis.  A step runs only the tokens it is given; everything earlier is read from
the pages.

What the kernels see of a step (all int32, on the device):

* ``token_ids[N]``, ``positions[N]``: the tokens and their absolute positions;
* ``cu_q[R+1]``: request r's tokens are rows cu_q[r] .. cu_q[r+1]-1;
* ``seq_lens[R]``: request r's length after this step;
* ``state_slots[R]``, ``first_portion[R]``: the request's row in fixed-size state
  tensors, and whether this is the first step of its life;
* per key/value group: ``slot_mapping[N]`` (page * page_size + offset of each token)
  and ``block_tables[R, P]``;
* ``logit_rows[M]``: the rows of the token axis whose logits are returned, in the order
  of the entries and of their ``want`` lists.

Order inside a layer: the step's keys and values are stored before attention reads
(the write-before-read rule of docs/architecture.md:249-250), on one stream.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..cache import CacheManager, RELEASED
from ..errors import BatchError, OutOfPages


@dataclass
class StepEntry:
    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = ()


class SampledTokens:
    """The token ids one step sampled, on their way to the host: a device copy that the next step may
    take its input tokens from, and a pinned host copy that ``tolist`` waits for."""

    def __init__(self, device, host, event, count, slot):
        self.device, self.host, self.event, self.count, self.slot = device, host, event, count, slot

    def tolist(self):
        if self.event is not None:
            self.event.synchronize()
        return self.host[: self.count].tolist()


@dataclass
class KVView:
    """What a mixer gets for its cache entry: the entry's pages and its group's tables.  ``pages`` is the
    entry's one tensor ``[pages, streams, heads, page_size, width]`` when all its streams have one shape
    (keys and values), else None; ``streams`` has each stream's ``[pages, heads, page_size, width]`` by name."""
    pages: Optional[torch.Tensor]
    block_tables: torch.Tensor
    slot_mapping: torch.Tensor
    page_size: int
    window: Optional[int]
    streams: Optional[Dict[str, torch.Tensor]] = None


class _Arena:
    """Named device buffers that keep their address from step to step."""

    def __init__(self, device, max_rows):
        import os
        self.device, self.max_rows = device, max_rows
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self.generation = 0          # bumped whenever a buffer is (re)allocated: captured graphs go stale
        # a debugging aid: new buffers start as NaN (floating) or as a large negative number (integer), so that a
        # kernel that reads what no kernel wrote shows in the logits instead of depending on what the memory held
        self.poison = os.environ.get("INFURNACE_POISON_BUFFERS", "0") not in ("", "0")

    def get(self, name, shape, dtype, rows=None):
        cap = max(rows or self.max_rows, shape[0])
        key = (name, tuple(shape[1:]), dtype)
        buf = self._bufs.get(key)
        if buf is None or buf.shape[0] < cap:
            buf = torch.empty((cap, *shape[1:]), dtype=dtype, device=self.device)
            if self.poison:
                buf.fill_(float("nan") if dtype.is_floating_point else -(1 << 30))
            self._bufs[key] = buf
            self.generation += 1
        return buf[: shape[0]]


class StepContext:
    """One step as the parts see it."""

    def __init__(self, runner: "ModelRunner"):
        self._runner = runner
        self.num_tokens = 0
        self.num_requests = 0
        self.num_logit_rows = 0
        self.max_logit_rows = runner.max_tokens
        self.max_q_len = 0
        self.min_q_len = 1
        self.max_seq_len = 0
        self.token_ids = self.positions = self.cu_q = self.seq_lens = None
        self.state_slots = self.first_portion = self.logit_rows = self.req_index = None
        self.shared: Dict[tuple, torch.Tensor] = {}       # what parts compute once per step and share (keyed by the part)
        self.group_slot_mapping: List[torch.Tensor] = []
        self.group_block_tables: List[torch.Tensor] = []
        # host copies, for parts written with torch operations
        self.host_cu_q: List[int] = []
        self.host_seq_lens: List[int] = []
        self.host_state_slots: List[int] = []
        self.host_first_portion: List[bool] = []

    def buffer(self, name, shape, dtype, rows=None):
        return self._runner.arena.get(name, shape, dtype, rows)

    def kv(self, cache_id: int) -> KVView:
        cache = self._runner.cache
        gi = cache.kv_group_of(cache_id)
        g = cache.kv_groups[gi]
        return KVView(g.tensors[cache_id], self.group_block_tables[gi], self.group_slot_mapping[gi],
                      g.page_size, g.need.window, g.streams.get(cache_id))

    def state(self, cache_id: int) -> torch.Tensor:
        """The fixed-size state tensor ``[slots, *shape]`` of a cache entry; request r of this
        step owns row ``state_slots[r]``."""
        cache = self._runner.cache
        return cache.state_groups[cache.state_group_of(cache_id)].tensors[cache_id]


class ModelRunner:
    def __init__(self, model, cache: CacheManager, runtime, max_tokens: int, max_model_len: int):
        self.model = model
        self.cache = cache
        self.rt = runtime
        self.max_tokens = max_tokens
        self.max_model_len = max_model_len
        self.max_requests = cache.max_requests
        self.max_pages = -(-max_model_len // cache.page_size)
        # rows of the flat token axis that the staging regions and buffers hold: a decode-only step is padded to
        # a power-of-two number of requests (at most max_requests), which may exceed the token budget
        self._n_cap = max(max_tokens, self.max_requests)
        self.arena = _Arena(runtime.device, self._n_cap)
        dev = runtime.device
        self._pin = dev is not None and torch.device(dev).type == "cuda"
        n, r, g = self._n_cap, self.max_requests, len(cache.kv_groups)
        # one staging area: [ids n][pos n][req n][logit_rows n][cu_q r+1][seq r][slot r][first r] + g * [slots n]
        self._small_len = 4 * n + 4 * r + 1 + g * n + 2 * r      # the last 2r words: temperatures, uniforms (float32)
        # two host staging sets used in turn: a set is rewritten only after the copy that
        # read it last has finished (its event), so the host may run a step ahead
        self._stage = [
            (torch.zeros(self._small_len, dtype=torch.int32, pin_memory=self._pin),
             torch.full((max(g, 1), r, self.max_pages), RELEASED, dtype=torch.int32, pin_memory=self._pin))
            for _ in range(2)]
        self._stage_events = [None, None]
        self._stage_np = [(a.numpy(), b.numpy()) for a, b in self._stage]      # the same memory, for cheap list writes
        # block tables of live requests as arrays that grow with the tables: (epoch, synced length, array) by (rid, group)
        self._table_rows: Dict[tuple, list] = {}
        self._dev_small = torch.zeros(self._small_len, dtype=torch.int32, device=dev)
        self._dev_tables = torch.full((max(g, 1), r, self.max_pages), RELEASED, dtype=torch.int32, device=dev)
        self.steps_run = 0
        self.sampled = torch.zeros(max(r, 1), dtype=torch.int32, device=dev)
        # the sampled ids of the last two steps (a step in flight may feed the next one from the device)
        self._hist = [torch.zeros(max(r, 1), dtype=torch.int32, device=dev) for _ in range(2)]
        self._hist_host = [torch.zeros(max(r, 1), dtype=torch.int32, pin_memory=self._pin) for _ in range(2)]
        self._sampled_steps = 0
        # decode-only steps are replayed from CUDA graphs, one per (batch bucket, context bucket)
        self.use_graphs = self._pin and bool(getattr(model, "graph_safe", False))
        self._graphs: Dict[tuple, tuple] = {}
        self._shapes_seen: Dict[tuple, int] = {}
        self.max_graphs = 64
        self.graph_replays = 0
        self.launches_per_graph_step = 0

    # ------------------------------------------------------------------ the step
    def validate(self, entries: Sequence[StepEntry], placeholders: bool = False, sampled: bool = False) -> None:
        """Refuse a malformed batch before anything is taken or launched.  ``sampled``: the wanted rows
        go through the sampling kernel, whose per-row inputs and outputs hold ``max_requests`` rows."""
        if not entries:
            raise BatchError("a step needs at least one entry")
        if len(entries) > self.max_requests:
            raise BatchError(f"{len(entries)} entries in a step; at most {self.max_requests}")
        seen = set()
        total = 0
        vocab = self.model.plan.vocab_size
        for e in entries:
            if e.request_id in seen:
                raise BatchError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            if not self.cache.has_request(e.request_id):
                raise BatchError(f"request {e.request_id!r} is not live; add it first")
            n = len(e.tokens)
            if n < 1:
                raise BatchError(f"request {e.request_id!r} brings no tokens")
            if not placeholders:
                lo, hi = (min(e.tokens), max(e.tokens)) if n > 1 else (e.tokens[0], e.tokens[0])
                if not 0 <= int(lo) or not int(hi) < vocab:
                    bad = next(t for t in e.tokens if not 0 <= int(t) < vocab)
                    raise BatchError(f"token id {bad} of request {e.request_id!r} is outside the vocabulary of {vocab}")
            if len(e.want) and not (0 <= int(min(e.want)) and int(max(e.want)) < n):
                bad = next(w for w in e.want if not 0 <= int(w) < n)
                raise BatchError(f"request {e.request_id!r} wants logits at place {bad} of {n} tokens")
            if self.cache.num_computed(e.request_id) + n > self.max_model_len:
                raise BatchError(f"request {e.request_id!r} would grow past max_model_len {self.max_model_len}")
            total += n
        if total > self.max_tokens:
            raise BatchError(f"{total} tokens in a step; at most {self.max_tokens}")
        if sampled:
            wanted = sum(len(e.want) for e in entries)
            if wanted > self.max_requests:
                raise BatchError(f"{wanted} rows to sample from in a step; at most {self.max_requests}")

    def _reserve(self, entries) -> None:
        cache = self.cache
        done = []
        try:
            for e in entries:
                cache.allocate(e.request_id, len(e.tokens))
                done.append(e)
        except OutOfPages:
            for e in done:
                cache.release_allocation(e.request_id)
            raise

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` on the device (None if
        nothing is wanted).  The returned tensor is a buffer that the next step overwrites.

        Raises :class:`OutOfPages`, with nothing changed, if the pages for the step's tokens
        cannot all be had."""
        self.validate(entries)
        self._reserve(entries)
        logits = self._run_reserved(entries, None, None, None, sample=False)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        return logits

    def step_and_sample(self, entries: Sequence[StepEntry], temperatures: Sequence[float],
                        uniforms: Sequence[float], feed=None) -> Optional[SampledTokens]:
        """``step`` followed by the sampling kernel on the wanted rows: returns the sampled token
        ids as a :class:`SampledTokens` (None if nothing is wanted); nothing here waits for the
        device.  ``temperatures`` and ``uniforms`` have one entry per wanted row.

        ``feed`` = (previous step's SampledTokens, rows): the step's input tokens are not known
        to the host yet; entry i takes row ``rows[i]`` of what the previous step sampled, on the
        device (every entry then brings exactly one token, whose id in ``tokens`` is ignored)."""
        if feed is not None and (len(feed[1]) != len(entries) or any(len(e.tokens) != 1 for e in entries)):
            raise BatchError("a step fed from the device brings one token per entry and one source row per entry")
        self.validate(entries, placeholders=feed is not None, sampled=True)
        wanted = sum(len(e.want) for e in entries)
        if len(temperatures) != wanted or len(uniforms) != wanted:
            raise BatchError("one temperature and one uniform number per wanted row")
        self._reserve(entries)
        self._run_reserved(entries, temperatures, uniforms, feed, sample=True)
        for e in entries:
            self.cache.commit(e.request_id, len(e.tokens))
        self.steps_run += 1
        if not wanted:
            return None
        slot = self._sampled_steps % 2
        self._sampled_steps += 1
        dev, host = self._hist[slot], self._hist_host[slot]
        dev[:wanted].copy_(self.sampled[:wanted])
        host[:wanted].copy_(dev[:wanted], non_blocking=True)
        event = None
        if self._pin:
            event = torch.cuda.Event()
            event.record()
        return SampledTokens(dev, host, event, wanted, slot)

    def _run_reserved(self, entries, temperatures, uniforms, feed, sample: bool):
        """``_execute`` for a step whose pages are taken: if it raises, the pages go back, so that a caller
        that goes on after the error (the engine fails the step's requests; a replay ends) finds the
        cache as it was before the step."""
        try:
            return self._execute(entries, temperatures, uniforms, feed, sample=sample)
        except BaseException:
            for e in entries:
                if self.cache.has_request(e.request_id):
                    self.cache.release_allocation(e.request_id)
            raise

    def _apply_feed(self, ctx, feed) -> None:
        """Overwrite the step's token ids on the device with rows of the previous step's sampled ids."""
        if feed is None:
            return
        prev, rows = feed
        n = len(rows)
        if list(rows) == list(range(n)):
            ctx.token_ids[:n].copy_(prev.device[:n])
        else:
            idx = torch.tensor(list(rows), dtype=torch.int64, device=prev.device.device)
            ctx.token_ids[:n].copy_(prev.device.index_select(0, idx))

    def _forward(self, ctx, sample: bool, greedy: bool):
        logits = self.model.forward(ctx)
        if sample and logits is not None:
            m = logits.shape[0]
            if greedy:
                self.rt.kernels.sample(logits, None, None, self.sampled[:m])
            else:
                self.rt.kernels.sample(logits, ctx.temperatures[:m], ctx.uniforms[:m], self.sampled[:m])
        return logits

    def _execute(self, entries, temperatures, uniforms, feed, sample: bool):
        """The step's kernels: launched one by one, or replayed from a CUDA graph.

        What a graph fixes is what the launches take from the host: the numbers of tokens, requests
        and wanted rows, the longest portion, a bucket of the longest context (it decides how
        attention is split) and the kind of sampling; token ids, positions, lengths, tables and
        wanted rows are read from device buffers that keep their address.  Plain decoding (one
        token per request) is padded to a power-of-two batch and recorded at its first
        occurrence; any other shape is recorded when it occurs a second time (a prompt cut into
        portions of one size, a benchmark's repeated prompt), so that one-off shapes cost no
        recording.  A graph is dropped when a buffer it points at has moved."""
        greedy = sample and all(t == 0.0 for t in temperatures)
        build = dict(temperatures=temperatures, uniforms=uniforms) if sample else {}
        # The padding and the length bucket are the same whether graphs are used or not, so that a step launches
        # the same kernels with the same parameters either way (the split of a context over CTAs follows the bucket).
        longest = max(self.cache.num_computed(e.request_id) + len(e.tokens) for e in entries)
        seq_bucket = 256
        while seq_bucket < longest:
            seq_bucket *= 2
        decode_only = sample and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)
        r_bucket = 0
        if decode_only:
            r_bucket = 1
            while r_bucket < len(entries):
                r_bucket *= 2
            r_bucket = min(r_bucket, self.max_requests)      # <= _n_cap, which the staging regions are sized by
        if not self.use_graphs:
            ctx = self._build_context(entries, pad_to=r_bucket, seq_bucket=seq_bucket, **build)
            self._apply_feed(ctx, feed)
            return self._forward(ctx, sample, greedy)
        if decode_only:
            key = ("decode", r_bucket, seq_bucket, greedy)
            ctx = self._build_context(entries, pad_to=r_bucket, seq_bucket=seq_bucket, **build)
        else:
            ctx = self._build_context(entries, seq_bucket=seq_bucket, **build)
            key = ("any", ctx.num_tokens, ctx.num_requests, ctx.num_logit_rows, ctx.max_q_len, ctx.min_q_len, seq_bucket,
                   sample, greedy)
        self._apply_feed(ctx, feed)
        stamp = (self.arena.generation, getattr(self.rt.kernels, "scratch_generation", 0))
        held = self._graphs.get(key)
        if held is not None and held[1] == stamp:
            held[0].replay()
            self.graph_replays += 1
            return held[2]
        if len(self._shapes_seen) > 4096:
            self._shapes_seen.clear()
        seen = self._shapes_seen.get(key, 0) + 1
        self._shapes_seen[key] = seen
        # run once as it is (which also makes every allocation) ...
        logits = self._forward(ctx, sample, greedy)
        if not decode_only and seen < 2:
            return logits
        # ... then record the same launches for the next time; the recording runs nothing
        if len(self._graphs) >= self.max_graphs:
            self._graphs.pop(next(iter(self._graphs)))
        torch.cuda.synchronize()
        stamp = (self.arena.generation, getattr(self.rt.kernels, "scratch_generation", 0))
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.rt.kernels, "launches", 0)
        ctx.shared.clear()             # what parts computed once for the step is computed in the recording too
        with torch.cuda.graph(graph):
            recorded = self._forward(ctx, sample, greedy)
        self.launches_per_graph_step = getattr(self.rt.kernels, "launches", 0) - before
        self._graphs[key] = (graph, stamp, recorded)
        return logits

    def _table_row(self, rid, gi):
        """The block table of (request, group) as an int32 array, extended by the pages taken since last
        time.  Entries of pages that a window released are left as they were: nothing reads them."""
        import numpy as np
        cache = self.cache
        table = cache.block_table(rid, gi)
        epoch = cache.epoch_of(rid)
        held = self._table_rows.get((rid, gi))
        if held is None or held[0] != epoch or held[1] > len(table):
            if len(self._table_rows) > 8 * self.max_requests * max(1, len(cache.kv_groups)):
                self._table_rows = {k: v for k, v in self._table_rows.items() if cache.has_request(k[0])}
            held = [epoch, 0, np.empty(self.max_pages, dtype=np.int32)]
            self._table_rows[(rid, gi)] = held
        n = len(table)
        if n > held[1]:
            held[2][held[1]:n] = table[held[1]:n]
            held[1] = n
        return held[2][:n]

    # ------------------------------------------------------------------ metadata
    def _build_context(self, entries, temperatures=None, uniforms=None, pad_to=0, seq_bucket=0) -> StepContext:
        cache = self.cache
        n_max, r_max = self._n_cap, self.max_requests
        turn = self.steps_run % 2
        if self._stage_events[turn] is not None:
            self._stage_events[turn].synchronize()
        host_small, host_tables = self._stage[turn]
        np_small, np_tables = self._stage_np[turn]
        import numpy as np
        n_groups = len(cache.kv_groups)
        o_ids, o_pos, o_req, o_rows = 0, n_max, 2 * n_max, 3 * n_max
        o_cu = 4 * n_max
        o_seq = o_cu + r_max + 1
        o_slot = o_seq + r_max
        o_first = o_slot + r_max
        o_g = o_first + r_max
        h = np_small
        total = sum(len(e.tokens) for e in entries) + max(0, pad_to - len(entries))
        wanted = sum(len(e.want) for e in entries) + max(0, pad_to - len(entries))
        if total > n_max or max(len(entries), pad_to) > r_max or wanted > n_max:
            raise BatchError(f"a step of {total} rows, {max(len(entries), pad_to)} requests and {wanted} wanted rows does not "
                             f"fit the staging regions ({n_max} rows, {r_max} requests)")
        cu, seq, slots, first = [0], [], [], []
        max_q, min_q = 0, 1 << 30
        base = n_rows = 0
        for r, e in enumerate(entries):            # whole spans at a time: a prompt portion costs no Python loop over its tokens
            start = cache.num_computed(e.request_id)
            n = len(e.tokens)
            if n == 1:                              # a decoded token: plain scalar writes beat array calls
                h[o_ids + base] = max(0, int(e.tokens[0]))
                h[o_pos + base] = start
                h[o_req + base] = r
                for w in e.want:
                    h[o_rows + n_rows] = base + int(w)
                    n_rows += 1
            else:
                h[o_ids + base:o_ids + base + n] = np.maximum(np.asarray(e.tokens, dtype=np.int64), 0)
                h[o_pos + base:o_pos + base + n] = np.arange(start, start + n, dtype=np.int32)
                h[o_req + base:o_req + base + n] = r
                k = len(e.want)
                if k:
                    h[o_rows + n_rows:o_rows + n_rows + k] = np.asarray(e.want, dtype=np.int64) + base
                    n_rows += k
            cu.append(base + n)
            seq.append(start + n)
            slots.append(cache.slot_of(e.request_id))
            first.append(1 if start == 0 else 0)
            max_q, min_q = max(max_q, n), min(min_q, n)
            for gi in range(n_groups):
                if n == 1:
                    h[o_g + gi * n_max + base] = cache.slots_for(e.request_id, gi, 1)[0]
                else:
                    h[o_g + gi * n_max + base:o_g + gi * n_max + base + n] = cache.slots_array(e.request_id, gi, n)
                row = self._table_row(e.request_id, gi)
                np_tables[gi, r, : len(row)] = row
            base += n
        real_rows = n_rows
        for j in range(len(entries), pad_to):      # padding of a graph bucket: tokens that store and see nothing
            h[o_ids + base] = 0; h[o_pos + base] = 0; h[o_req + base] = j; h[o_rows + n_rows] = 0
            for gi in range(n_groups):
                h[o_g + gi * n_max + base] = -1
            cu.append(cu[-1] + 1); seq.append(0); slots.append(0); first.append(0)
            base += 1; n_rows += 1
        N, R, M = base, len(cu) - 1, n_rows
        h[o_cu:o_cu + R + 1] = cu
        h[o_seq:o_seq + R] = seq
        h[o_slot:o_slot + R] = slots
        h[o_first:o_first + R] = first
        group_slots = cache.kv_groups
        o_f = o_g + len(group_slots) * n_max
        if temperatures is not None:
            hf = h.view("float32")
            k = len(temperatures)
            hf[o_f:o_f + 2 * r_max] = 0.0
            if k:
                hf[o_f:o_f + k] = temperatures
                hf[o_f + r_max:o_f + r_max + k] = uniforms
        h = host_small
        d = self._dev_small
        d.copy_(h, non_blocking=True)
        if cache.kv_groups:
            self._dev_tables[:, :R].copy_(host_tables[:, :R], non_blocking=True)
        if self._pin:
            ev = torch.cuda.Event()
            ev.record()
            self._stage_events[turn] = ev
        ctx = StepContext(self)
        ctx.num_tokens, ctx.num_requests, ctx.num_logit_rows = N, R, M
        ctx.max_q_len, ctx.max_seq_len = max_q, max(max(seq), seq_bucket)
        ctx.min_q_len = 1 if pad_to > len(entries) else max(1, min(min_q, max_q))
        df = d.view(torch.float32)
        ctx.temperatures, ctx.uniforms = df[o_f:o_f + r_max], df[o_f + r_max:o_f + 2 * r_max]
        ctx.num_real_logit_rows = real_rows
        ctx.token_ids, ctx.positions = d[o_ids:o_ids + N], d[o_pos:o_pos + N]
        ctx.req_index, ctx.logit_rows = d[o_req:o_req + N], d[o_rows:o_rows + M]
        ctx.cu_q, ctx.seq_lens = d[o_cu:o_cu + R + 1], d[o_seq:o_seq + R]
        ctx.state_slots, ctx.first_portion = d[o_slot:o_slot + R], d[o_first:o_first + R]
        ctx.group_slot_mapping = [d[o_g + gi * n_max: o_g + gi * n_max + N] for gi in range(len(cache.kv_groups))]
        ctx.group_block_tables = [self._dev_tables[gi, :R] for gi in range(len(cache.kv_groups))]
        ctx.host_cu_q, ctx.host_seq_lens = cu, seq
        ctx.host_state_slots, ctx.host_first_portion = slots, [bool(f) for f in first]
        return ctx
