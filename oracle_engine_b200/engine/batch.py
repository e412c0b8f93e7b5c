"""A step's batch: the host-side plan and the device-side context the parts read.

A step brings, for each of its sequences, the next tokens (a whole prompt, a piece of
one, or one decoded token) and the places among them whose logits are wanted.  The plan
packs all tokens into one list (no padding between sequences) with, per token, the index
of its sequence in the batch and its absolute position, and per sequence its slot, the
length its cache had before the step, and its token count.  Rows can be padded up to a
fixed size for a captured CUDA graph: padding tokens carry sequence index -1, which every
kernel skips, so padding changes no result.

All integers go to the device in ONE copy from pinned host memory (`StepBuffers`).
The reference has no batch: `forward(token, pos)` and `forward_prefill(tokens, n,
start_pos)` take one sequence (core/model.hpp:74-89).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class SequenceStep:
    """One sequence's share of a step."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)      # indices into `tokens`


@dataclass
class StepPlan:
    n_seqs: int
    n_tokens: int                   # with padding
    n_real_tokens: int
    token_ids: np.ndarray           # [T] int32
    tok_seq: np.ndarray             # [T] int32, -1 for padding
    tok_pos: np.ndarray             # [T] int32
    seq_slot: np.ndarray            # [B] int32, -1 for padding
    seq_start: np.ndarray           # [B] int32 cache length before the step
    seq_qlen: np.ndarray            # [B] int32
    cu_q: np.ndarray                # [B+1] int32
    want_rows: np.ndarray           # [n_want] int32 rows of the packed token list
    max_qlen: int
    max_kvlen: int
    all_decode: bool                # every sequence brings exactly one token


def build_plan(seqs: list, starts: list, pad_seqs: int = 0, pad_tokens: int = 0,
               want_all_rows: bool = False, token_arrays: list | None = None) -> StepPlan:
    """seqs: SequenceStep list; starts: each sequence's cache length before the step;
    token_arrays: per sequence its tokens as an array where the caller has one already, else None."""
    B = len(seqs)
    qlens = [len(s.tokens) for s in seqs]
    T_real = sum(qlens)
    Bp = max(B, pad_seqs)
    Tp = max(T_real, pad_tokens)
    token_ids = np.zeros(Tp, dtype=np.int32)
    tok_seq = np.full(Tp, -1, dtype=np.int32)
    tok_pos = np.zeros(Tp, dtype=np.int32)
    seq_slot = np.full(Bp, -1, dtype=np.int32)
    seq_start = np.zeros(Bp, dtype=np.int32)
    seq_qlen = np.zeros(Bp, dtype=np.int32)
    cu_q = np.zeros(Bp + 1, dtype=np.int32)
    want = []
    row = 0
    for b, (s, st, n) in enumerate(zip(seqs, starts, qlens)):
        ids = None if token_arrays is None else token_arrays[b]
        token_ids[row:row + n] = s.tokens if ids is None else ids
        tok_seq[row:row + n] = b
        tok_pos[row:row + n] = np.arange(st, st + n, dtype=np.int32)
        seq_slot[b], seq_start[b], seq_qlen[b] = s.slot, st, n
        cu_q[b + 1] = row + n
        for w in s.want:
            if not 0 <= w < n:
                raise ValueError(f"sequence {b}: wanted place {w} is outside its {n} tokens")
            want.append(row + w)
        row += n
    cu_q[B + 1:] = row
    if want_all_rows:
        want = list(range(Tp))
    return StepPlan(
        n_seqs=Bp, n_tokens=Tp, n_real_tokens=T_real, token_ids=token_ids, tok_seq=tok_seq, tok_pos=tok_pos,
        seq_slot=seq_slot, seq_start=seq_start, seq_qlen=seq_qlen, cu_q=cu_q,
        want_rows=np.asarray(want, dtype=np.int32), max_qlen=max(qlens, default=0),
        max_kvlen=max((st + n for st, n in zip(starts, qlens)), default=0),
        all_decode=all(n == 1 for n in qlens) and B > 0)


# Steps are classed by the longest sequence they touch: kernels may be chosen by the class, and a
# captured decode graph is kept per class, so the choice stays valid as sequences grow.
CONTEXT_CLASS_TOKENS = [768, 1536, 4096]     # class 0 up to the first, 1 up to the second, 2 up to the third, 3 beyond


def context_class(n_tokens: int) -> int:
    """The class of a step by its longest sequence; kernels may be chosen by it, and a decode
    graph is kept per class."""
    return sum(1 for t in CONTEXT_CLASS_TOKENS if n_tokens > t)


@dataclass
class StepContext:
    """Device-side view of a step, handed to every part."""
    n_tokens: int
    n_seqs: int
    n_want: int
    token_ids: torch.Tensor
    tok_seq: torch.Tensor
    tok_pos: torch.Tensor
    seq_slot: torch.Tensor
    seq_start: torch.Tensor
    seq_qlen: torch.Tensor
    cu_q: torch.Tensor
    want_rows: torch.Tensor
    tables: list                    # per cache group: [B, max_pages] int32
    max_qlen: int
    max_kvlen: int
    all_decode: bool
    context_class: int = 0          # context_class() of the longest sequence (kernels may choose by it)


class StepBuffers:
    """Pinned host staging and its device mirror for a step of fixed (padded) sizes."""

    def __init__(self, n_tokens: int, n_seqs: int, n_want: int, table_shapes: list, device):
        self.n_tokens, self.n_seqs, self.n_want = n_tokens, n_seqs, n_want
        self.table_shapes = list(table_shapes)
        sizes = [n_tokens, n_tokens, n_tokens, n_seqs, n_seqs, n_seqs, n_seqs + 1, n_want] + \
                [a * b for a, b in table_shapes]
        # 16-byte aligned sections so that vector loads of any section are legal
        self.offsets = []
        off = 0
        for s in sizes:
            self.offsets.append(off)
            off += (s + 3) // 4 * 4
        self.total = max(off, 4)
        self.host = torch.empty(self.total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.dev = torch.empty(self.total, dtype=torch.int32, device=device)
        self.sizes = sizes
        self._copied = torch.cuda.Event() if torch.cuda.is_available() else None
        self._pending = False
        # the sections as numpy views of the staging buffer and as device views, made once
        self._host_views = [self.host[o: o + n].numpy() for o, n in zip(self.offsets, sizes)]
        self._dev_views = [self.dev[o: o + n] for o, n in zip(self.offsets, sizes)]
        self._dev_tables = [self._dev_views[8 + j].view(*shape) for j, shape in enumerate(self.table_shapes)]

    def _host_view(self, i):
        return self._host_views[i]

    def _dev_view(self, i):
        return self._dev_views[i]

    def upload(self, plan: StepPlan, tables: list) -> StepContext:
        """Fills the staging buffer from the plan and copies it to the device (one
        asynchronous copy on the current stream)."""
        if self._pending:                     # the previous copy must have read the staging buffer
            self._copied.synchronize()
        fields = [plan.token_ids, plan.tok_seq, plan.tok_pos, plan.seq_slot, plan.seq_start, plan.seq_qlen,
                  plan.cu_q, plan.want_rows]
        for i, arr in enumerate(fields):
            if arr.size != self.sizes[i]:
                raise ValueError(f"step buffer section {i} holds {self.sizes[i]} values, the plan has {arr.size}")
            if arr.size:
                self._host_view(i)[:] = arr
        for j, tb in enumerate(tables):
            self._host_view(8 + j)[:] = tb.reshape(-1)
        self.dev.copy_(self.host, non_blocking=True)
        if self._copied is not None:
            self._copied.record(torch.cuda.current_stream())
            self._pending = True
        return self.context(plan)

    def update_decode(self, tokens, starts, n: int) -> None:
        """For a step of the same sequences as the last upload, each one token further: only
        token ids, positions and starts change.  Rewrites those and copies the buffer."""
        if self._pending:
            self._copied.synchronize()
        if tokens is not None:                # else the caller writes them on the device
            self._host_view(0)[:n] = tokens
        self._host_view(2)[:n] = starts
        self._host_view(4)[:n] = starts
        self.dev.copy_(self.host, non_blocking=True)
        if self._copied is not None:
            self._copied.record(torch.cuda.current_stream())
            self._pending = True

    def bytes(self) -> int:
        return self.total * 4

    def context(self, plan: StepPlan) -> StepContext:
        v = self._dev_views
        tabs = list(self._dev_tables)
        return StepContext(
            n_tokens=self.n_tokens, n_seqs=self.n_seqs, n_want=self.n_want, token_ids=v[0], tok_seq=v[1],
            tok_pos=v[2], seq_slot=v[3], seq_start=v[4], seq_qlen=v[5], cu_q=v[6], want_rows=v[7], tables=tabs,
            max_qlen=plan.max_qlen, max_kvlen=plan.max_kvlen, all_decode=plan.all_decode,
            context_class=context_class(plan.max_kvlen))
