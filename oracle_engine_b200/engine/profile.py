"""Device time per kind of kernel, measured with CUDA events around every launch.

    with KernelProfile() as prof:
        engine.generate(prompts, params)
    prof.report(sys.stderr)

Every kernel of this library is launched through csrc/ops.py; while a profile is open it
records an event after each launch, and the time between two consecutive events is
booked on the later launch's kind ("gemm_skinny 8x16384x3072", "attention_decode_warps",
"rmsnorm", ...).  That time is the kernel's own plus the gap before it, so the kinds add
up to the device time of what ran.

Launches that are captured into a CUDA graph while the profile is open get event nodes of
their own inside the graph (`external` events): they are timed on the device at every
replay, free of host gaps, and `report` shows the last replay.  Events between kernels
keep a kernel from starting while its predecessor drains, so a profiled step is a little
slower than a plain one: read shares and per-kernel times, not the total.  Keep to one
batch size and context class while a profile is open (one captured graph), and open the
profile before the graph is captured.

The reference times prefill and generation with host clocks
(benchmark/bench_engine.cpp:225-244); this is the same idea one level down.
"""
from __future__ import annotations

import torch

from ..csrc import ops


class KernelProfile:
    def __init__(self, with_shapes: bool = True):
        self.with_shapes = with_shapes
        self.events: list = []          # launches outside graphs: (kind, event)
        self.graph_events: list = []    # launches captured into graphs: (kind, event)
        self.kinds: list = []           # every launch's (what, detail), in order
        self._start = None

    def __enter__(self):
        if ops.OBSERVER[0] is not None:
            raise RuntimeError("a kernel profile is already open")
        self._start = torch.cuda.Event(enable_timing=True)
        self._start.record()
        ops.OBSERVER[0] = self
        return self

    def __exit__(self, *exc):
        ops.OBSERVER[0] = None
        torch.cuda.synchronize()

    def _kind(self, what, detail) -> str:
        if self.with_shapes and isinstance(detail, tuple):
            return f"{what} {'x'.join(str(d) for d in detail)}"
        return what

    def mark(self, what: str, detail) -> None:
        self.kinds.append((what, detail))
        if torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event(enable_timing=True, external=True)
            ev.record()
            self.graph_events.append((self._kind(what, detail), ev))
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.events.append((self._kind(what, detail), ev))

    @staticmethod
    def _sum(chain, prev) -> dict:
        out: dict = {}
        for kind, ev in chain:
            if prev is not None:
                n, us = out.get(kind, (0, 0.0))
                out[kind] = (n + 1, us + prev.elapsed_time(ev) * 1e3)
            prev = ev
        return out

    def totals(self) -> dict:
        """kind -> (launches, microseconds) of the launches outside graphs, in order of first appearance."""
        return self._sum(self.events, self._start)

    def graph_totals(self) -> dict:
        """The same for the launches inside captured graphs, as timed at their last replay (the
        first launch of the chain has no event before it and is left out)."""
        return self._sum(self.graph_events, None)

    def report(self, file, title: str = "device time per kind of kernel") -> None:
        for name, totals, n in (("outside graphs", self.totals(), len(self.events)),
                                ("inside the captured graph, last replay", self.graph_totals(), len(self.graph_events))):
            if not totals:
                continue
            whole = sum(us for _, us in totals.values()) or 1.0
            print(f"{title}, {name} ({n} launches, {whole / 1e3:.3f} ms)", file=file)
            for kind, (k, us) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
                print(f"  {kind:<44s} {k:6d} x {us / k:9.1f} us  {us / 1e3:9.3f} ms  {100 * us / whole:5.1f} %",
                      file=file)
