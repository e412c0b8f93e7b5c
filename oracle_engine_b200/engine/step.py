"""The step function: runs a batch's next tokens through the model from the cache.

`Stepper.step(seqs)` takes, per sequence, its slot, its next tokens and the places whose
logits are wanted.  It runs exactly those tokens as one packed batch: a sequence's new
keys and values are written at positions start..start+n-1 of its slot, every token
attends to its own sequence's cache up to its own position, and the final norm and the
head run only on the wanted rows.  Prompts of unequal length and single decoded tokens
go through the same code; the sequences of a step need not be aligned in any way.

Steps in which every sequence brings one token are replayed from a CUDA graph, captured
per padded batch size, when every part of the model allows it.

Reference: `Model::forward` (one token, core/model.cpp:340-495) and
`Model::forward_prefill` (n tokens of one sequence from start_pos, reading keys and
values from the cache, core/model.cpp:510-674).
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache.kv_cache import CacheView
from ..csrc import ops
from .batch import SequenceStep, StepBuffers, build_plan, context_class

_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
# A step of up to this many tokens that is no decode step (a short prompt, a piece of one, prompts and single
# tokens mixed) is captured as well, per padded token count, padded batch size and context class: launched
# one by one its 230 kernels cost the host 3.1 ms, twice what the device needs for them.
GRAPH_STEP_TOKENS = 256
MAX_TOKEN_GRAPHS = 64
MAX_GRAPH_WANTED_ROWS = 64
_TOKEN_BUCKETS = (16, 32, 64, 128, 256)


class StepError(ValueError):
    """A step that cannot run; raised before anything is launched."""


def _bucket(n: int) -> int:
    for b in _BUCKETS:
        if n <= b:
            return b
    return (n + 63) // 64 * 64


class _DecodeGraph:
    """The decode step of one padded batch size and context class: its staging buffers, its
    residual stream, and the forward pass as a list of captured graphs and, between them, the
    stages that must run eagerly."""

    def __init__(self, bucket: int, buffers: StepBuffers):
        self.bucket = bucket
        self.buffers = buffers
        self.graph = None              # [(CUDAGraph | None, first stage, one past the last stage)]
        self.x = None                  # the residual stream, [bucket, hidden] float32, kept between the pieces
        self.logits = None
        self.runs = 0
        self.n_kernels = 0
        self.key = None                # slots of the last upload, in order
        self.version = -1              # page-table version of the last upload
        self.ctx = None


class Stepper:
    def __init__(self, model, cache, state, runtime, use_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.state = state
        self.rt = runtime
        self.vocab = model.spec.vocab_size
        self.n_entries = len(model.schedule)
        self._views_storage = [cache.storage_of(e) if e in cache.entry_group else None
                               for e in range(self.n_entries)]
        self._entry_group = [cache.group_of(e) if e in cache.entry_group else -1 for e in range(self.n_entries)]
        self._state_views = [state.views(e) for e in range(self.n_entries)]
        self._stages = model.stages()
        self.use_graphs = bool(use_graphs and any(safe for safe, _, _ in self._stages))
        self._graphs: dict[tuple, _DecodeGraph] = {}      # (padded batch size, long context) -> graph
        self._token_graphs: dict[tuple, _DecodeGraph] = {}    # (padded tokens, batch size, wanted rows; context class) -> graph
        self._eager_buffers: dict[tuple, StepBuffers] = {}
        self.launch_counter = None         # set by the bench to count kernel launches

    # ------------------------------------------------------------------ helpers
    def _table_shapes(self, n_seqs: int):
        return [(n_seqs, self.cache.max_pages_per_seq) for _ in self.cache.groups]

    def _cache_views(self, ctx):
        return [CacheView(self._views_storage[e], ctx.tables[g], g) if g >= 0 else CacheView(None, None, -1)
                for e, g in enumerate(self._entry_group)]

    def _validate(self, seqs):
        if not seqs:
            raise StepError("a step needs at least one sequence")
        seen = set()
        token_arrays = []
        for i, s in enumerate(seqs):
            if not self.cache.slots.is_held(s.slot):
                raise StepError(f"sequence {i}: slot {s.slot} is not allocated")
            if s.slot in seen:
                raise StepError(f"sequence {i}: slot {s.slot} appears twice in one step")
            seen.add(s.slot)
            if len(s.tokens) < 1:
                raise StepError(f"sequence {i}: a step needs at least one token per sequence")
            ids = None
            if len(s.tokens) >= 64:       # a prompt: one pass over its list, and the plan reuses the array
                ids = np.asarray(s.tokens, dtype=np.int64)
                if ids.ndim != 1:
                    raise StepError(f"sequence {i}: tokens must be a flat list of ids")
                lo, hi = int(ids.min()), int(ids.max())
            else:
                lo, hi = min(s.tokens), max(s.tokens)
            if not (0 <= lo and hi < self.vocab):
                bad = [t for t in s.tokens if not 0 <= int(t) < self.vocab]
                raise StepError(f"sequence {i}: token id {bad[0]} is outside the vocabulary [0, {self.vocab})")
            token_arrays.append(ids)
            for w in s.want:
                if not 0 <= int(w) < len(s.tokens):
                    raise StepError(f"sequence {i}: wanted place {w} is outside its {len(s.tokens)} tokens")
            if len(set(s.want)) != len(s.want):
                raise StepError(f"sequence {i}: a place is wanted twice")
            if self.cache.length(s.slot) + len(s.tokens) > self.model.spec.max_positions:
                raise StepError(f"sequence {i}: {self.cache.length(s.slot)} + {len(s.tokens)} tokens exceed the "
                                f"{self.model.spec.max_positions} positions the model was built for")
        return token_arrays

    # ------------------------------------------------------------------ the step
    def step(self, seqs: list[SequenceStep], device_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """Returns float32 logits [wanted, vocab] on the device (order: sequences, then
        each sequence's `want`), or None if nothing is wanted.  The tensor may be reused
        by the next step.

        device_tokens (int32 on the device, one per sequence; only for steps of one token
        each): the tokens are taken from there instead of from `seqs`, whose token values
        are placeholders; the host need not have seen them yet."""
        token_arrays = self._validate(seqs)
        if device_tokens is not None and not all(len(s.tokens) == 1 for s in seqs):
            raise StepError("tokens on the device can only feed a step of one token per sequence")
        starts = [self.cache.length(s.slot) for s in seqs]
        tables_changed = False
        for s, st in zip(seqs, starts):
            tables_changed |= self.cache.reserve(s.slot, st + len(s.tokens))
        decode = all(len(s.tokens) == 1 for s in seqs)
        n_tokens = sum(len(s.tokens) for s in seqs)
        if decode and self.use_graphs:
            logits = self._step_graph(seqs, starts, tables_changed, device_tokens)
        elif self.use_graphs and device_tokens is None and n_tokens <= GRAPH_STEP_TOKENS:
            logits = self._step_graph_tokens(seqs, starts, n_tokens, token_arrays)
        else:
            logits = self._step_eager(seqs, starts, device_tokens, token_arrays)
        for s, st in zip(seqs, starts):
            self.cache.commit(s.slot, st + len(s.tokens))
        return logits

    def _step_eager(self, seqs, starts, device_tokens=None, token_arrays=None):
        plan = build_plan(seqs, starts, token_arrays=token_arrays)
        key = (plan.n_tokens, plan.n_seqs, plan.want_rows.size)
        buf = self._eager_buffers.get(key)
        if buf is None:
            if len(self._eager_buffers) > 64:
                self._eager_buffers.clear()
            buf = StepBuffers(plan.n_tokens, plan.n_seqs, plan.want_rows.size, self._table_shapes(plan.n_seqs),
                              self.rt.device)
            self._eager_buffers[key] = buf
        tables = [self.cache.tables_for(g.index, plan.seq_slot) for g in self.cache.groups]
        ctx = buf.upload(plan, tables)
        if device_tokens is not None:
            ctx.token_ids[:len(seqs)].copy_(device_tokens[:len(seqs)])
        self.last_h2d_bytes = buf.bytes()
        return self.model.forward(ctx, self._cache_views(ctx), self._state_views)

    def _run_graph(self, g, ctx):
        """The forward pass of a step whose shapes are those of `g`: directly at the first use (loads the
        kernels' modules), captured at the second, replayed from then on.  Returns the head's output."""
        views = self._cache_views(ctx)
        if g.graph is None and g.runs == 1:
            # first use of this batch size: run directly (loads the kernels' modules)
            all_logits = self.model.forward(ctx, views, self._state_views)
        else:
            if g.graph is None:
                # Capture (nothing runs yet): every run of graph-safe stages becomes one graph; the
                # stages between them run eagerly at every replay, on the same residual stream.
                torch.cuda.synchronize()
                g.x = self.rt.empty(g.bucket, self.model.spec.hidden_size, dtype=torch.float32)
                pieces, g.n_kernels = [], 0
                for safe, lo, hi in self._stages:
                    if not safe:
                        pieces.append((None, lo, hi))
                        continue
                    graph = torch.cuda.CUDAGraph()
                    before = ops.LAUNCHES[0]
                    with torch.cuda.graph(graph):
                        out = self.model.run_stages(g.x, ctx, views, self._state_views, lo, hi)
                    g.n_kernels += ops.LAUNCHES[0] - before
                    ops.LAUNCHES[0] = before          # captured, not launched
                    pieces.append((graph, lo, hi))
                    if out is not None:
                        g.logits = out                 # the captured head's output buffer
                g.graph = pieces
            logits_now = None
            for graph, lo, hi in g.graph:
                if graph is None:
                    out = self.model.run_stages(g.x, ctx, views, self._state_views, lo, hi)
                    if out is not None:
                        logits_now = out
                else:
                    graph.replay()
            ops.LAUNCHES[0] += g.n_kernels
            all_logits = logits_now if logits_now is not None else g.logits
        return all_logits

    def _step_graph_tokens(self, seqs, starts, n_tokens: int, token_arrays=None):
        """A short step that is no decode step, through a graph of its padded shape.  Everything a kernel's
        launch depends on is the graph's: the token count and the batch size are padded (padding tokens
        belong to no sequence, padding sequences bring no token), the longest sequence's share of the
        step counts as the whole padded step, and the wanted rows are padded with row 0 (to the padded
        batch size when at most one row per sequence is wanted, as in generation, else to the padded
        token count)."""
        tb = next(b for b in _TOKEN_BUCKETS if n_tokens <= b)
        bb = min(_bucket(len(seqs)), tb)
        plan = build_plan(seqs, starts, pad_seqs=bb, pad_tokens=tb, token_arrays=token_arrays)
        n_want = int(plan.want_rows.size)
        if n_want > max(bb, MAX_GRAPH_WANTED_ROWS):            # a graph keeps its logits buffer: [rows, vocabulary] float32
            return self._step_eager(seqs, starts, None, token_arrays)
        wb = bb if n_want <= bb else min(tb, MAX_GRAPH_WANTED_ROWS)
        gkey = (tb, bb, wb, context_class(plan.max_kvlen))
        g = self._token_graphs.get(gkey)
        if g is None:
            if len(self._token_graphs) >= MAX_TOKEN_GRAPHS:     # shapes beyond these run directly
                return self._step_eager(seqs, starts, None, token_arrays)
            g = _DecodeGraph(tb, StepBuffers(tb, bb, wb, self._table_shapes(bb), self.rt.device))
            self._token_graphs[gkey] = g
        want = np.zeros(wb, dtype=np.int32)
        want[:n_want] = plan.want_rows
        plan.want_rows = want
        plan.max_qlen = tb
        tables = [self.cache.tables_for(gr.index, plan.seq_slot) for gr in self.cache.groups]
        ctx = g.buffers.upload(plan, tables)
        self.last_h2d_bytes = g.buffers.bytes()
        g.runs += 1
        all_logits = self._run_graph(g, ctx)
        return all_logits[:n_want] if n_want else None

    def _step_graph(self, seqs, starts, tables_changed=True, device_tokens=None):
        B = len(seqs)
        bucket = _bucket(B)
        # one graph per padded batch size and context class: kernels chosen by the class stay right
        gkey = (bucket, context_class(max(starts) + 1))
        g = self._graphs.get(gkey)
        if g is None:
            g = _DecodeGraph(bucket, StepBuffers(bucket, bucket, bucket, self._table_shapes(bucket), self.rt.device))
            self._graphs[gkey] = g
        key = tuple(s.slot for s in seqs)
        if key == g.key and g.version == self.cache.version:
            # the same sequences one token further: only tokens and positions change
            g.buffers.update_decode(None if device_tokens is not None else [s.tokens[0] for s in seqs], starts, B)
            ctx = g.ctx
        else:
            plan = build_plan(seqs, starts, pad_seqs=bucket, pad_tokens=bucket, want_all_rows=True)
            tables = [self.cache.tables_for(gr.index, plan.seq_slot) for gr in self.cache.groups]
            ctx = g.buffers.upload(plan, tables)
            g.key, g.ctx, g.version = key, ctx, self.cache.version
        if device_tokens is not None:         # after the copy of the step's tables, before the kernels
            ctx.token_ids[:B].copy_(device_tokens[:B])
        self.last_h2d_bytes = g.buffers.bytes()
        g.runs += 1
        all_logits = self._run_graph(g, ctx)
        # rows wanted by the caller, in order
        rows = [b for b, s in enumerate(seqs) if s.want]
        if not rows:
            return None
        if rows == list(range(all_logits.shape[0])):
            return all_logits
        if rows == list(range(len(rows))):
            return all_logits[:len(rows)]
        return all_logits[torch.as_tensor(rows, device=all_logits.device)]
