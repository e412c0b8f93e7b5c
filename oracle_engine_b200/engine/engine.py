"""Engine: a loaded model with its cache, step function, sampler and generation loop.

The Python entry point of the library, in the manner of the reference's `Engine`
(core/engine.hpp:35-76: load, then generate with `GenParams`), working on token ids:

    engine = Engine.from_pretrained("model_dir", dtype="bfloat16", max_tokens=65536)
    outs = engine.generate([[1, 2, 3], [4, 5]], GenParams(n_predict=16, temperature=0.0))

One engine drives one CUDA stream and is not re-entrant (the reference serialises
`generate` with a mutex, core/engine.cpp:86).
"""
from __future__ import annotations

from pathlib import Path

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..cache.kv_cache import KVCache
from ..cache.state import StateStore
from ..config.base import get_architecture, load_config
from ..csrc import ops
from ..parts.model import DecoderModel
from ..sampling.params import GenParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_weights
from ..weights.random_init import RandomSource
from ..weights.safetensors_io import ModelFiles
from .batch import SequenceStep
from .generate import GenerationResult, run_generation
from .runtime import Runtime, parse_dtype
from .step import Stepper


class Engine:
    def __init__(self, config, arch, source, dtype="bfloat16", max_tokens: int = 8192,
                 max_seq_len: int | None = None, device="cuda:0", use_graphs: bool = True,
                 tensor_cores: bool = True, n_slots: int | None = None):
        ops.require_cuda()
        self.config = config
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.rt = Runtime(parse_dtype(dtype), self.device, tensor_cores)
        page = ops.PAGE
        max_tokens = max(page, (int(max_tokens) + page - 1) // page * page)
        limit = arch.build_spec(config, None).max_positions        # the architecture's own limit
        self.max_seq_len = min(int(max_seq_len or limit), limit, max_tokens)
        self.spec = arch.build_spec(config, self.max_seq_len)
        self.model = DecoderModel(self.spec, self.rt)
        load_weights(self.model, source(self.model) if callable(source) else source)
        self.cache = KVCache(self.model.cache_needs(), max_tokens, self.max_seq_len, self.rt.dtype, self.device,
                             n_slots=n_slots)
        self.state = StateStore(self.cache.n_slots, self.device)
        for e, needs in enumerate(self.model.state_needs()):
            for name, need in needs.items():
                self.state.add(e, name, need)
        self.sampler = Sampler(self.state, self.device)
        self.stepper = Stepper(self.model, self.cache, self.state, self.rt, use_graphs)
        self._row_slot = torch.empty(self.cache.n_slots, dtype=torch.int32, device=self.device)
        self._ahead = None        # token buffers of the generation loop's step ahead (device, pinned host, event) x 2

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, folder, **kw) -> "Engine":
        """A model folder (config.json + model.safetensors or shards)."""
        config, arch = load_config(folder)
        files = ModelFiles(folder)
        try:
            return cls(config, arch, files, **kw)
        finally:
            files.close()

    @classmethod
    def from_config(cls, config, seed: int = 0, std: float = 0.02, norm_std: float = 0.1, **kw) -> "Engine":
        """Seeded random weights generated on the device (the same values that
        `write_model_folder` writes for this configuration and seed)."""
        arch = get_architecture(config.architecture)
        device = kw.get("device", "cuda:0")
        return cls(config, arch, lambda model: RandomSource(model.tensors(), seed, torch.bfloat16, device, std,
                                                            norm_std), **kw)

    # ------------------------------------------------------------------ slots and steps
    def alloc(self) -> int:
        slot = self.cache.alloc_slot()
        self.state.reset(slot)
        return slot

    def free(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def step(self, seqs: list[SequenceStep], device_tokens=None):
        """Float32 logits [wanted, vocab] on the device, or None; see Stepper.step."""
        return self.stepper.step(seqs, device_tokens)

    def check_device_errors(self) -> None:
        err = self.model.embedding.err
        if err is not None and int(err.item()) != 0:
            err.zero_()
            raise RuntimeError("a token id outside the vocabulary reached the embedding kernel")
        from ..csrc import ops_tc
        code = ops_tc.device_error()
        if code:
            raise RuntimeError(f"a bounded wait inside a tensor-core kernel ran out (code {code}); "
                               f"the results of the last steps are not valid")

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, params: GenParams | None = None, batch_size: int | None = None,
                 on_token=None, return_results: bool = False, lookahead: bool = True,
                 max_step_tokens: int | None = None):
        """prompts: lists of token ids.  Returns the new tokens of each request (or
        GenerationResult objects with the finish reason).  lookahead: the next step is queued
        before the host has read the last tokens (same tokens either way; `on_token` then hears
        of a token while the step after it is already running).  max_step_tokens: the most
        prompt tokens a step takes; longer prompts go through in portions (bounds the memory
        of a step's activations; None: every prompt whole).  Raises RuntimeError if a kernel
        reported an error during a batch (the tokens of that batch are then not returned)."""
        params = params or GenParams()
        backend = _Backend(self)
        backend.supports_lookahead = bool(lookahead)
        results = run_generation(backend, prompts, params, batch_size, self.spec.stop_ids, on_token,
                                 max_step_tokens)
        return results if return_results else [r.tokens for r in results]


class _Backend:
    """The engine as the generation loop sees it."""

    def __init__(self, engine: Engine):
        self.e = engine
        self.max_seq_len = engine.max_seq_len
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._last_slots = None
        self._turn = 0

    def alloc(self, request_index, prompt, params):
        slot = self.e.alloc()
        self.e.sampler.start_sequence(slot, params.seed + request_index, prompt, params)
        return slot

    def free(self, slot):
        self.e.free(slot)

    def check(self):
        self.e.check_device_errors()

    def step(self, seqs):
        logits = self.e.step(seqs)
        self.h2d_bytes += self.e.stepper.last_h2d_bytes
        return logits

    def _row_slots(self, slots, params):
        e = self.e
        row_slot = e._row_slot[:len(slots)]
        if params.temperature > 0.0 or params.repeat_penalty > 1.0:      # greedy needs no per-sequence state
            if slots != self._last_slots:
                row_slot.copy_(torch.tensor(slots, dtype=torch.int32))
                self._last_slots = list(slots)
                self.h2d_bytes += len(slots) * 4
        return row_slot

    def sample(self, logits, slots, params):
        rows = len(slots)
        out = self.e.sampler.sample(logits[:rows], self._row_slots(slots, params), params)
        self.d2h_bytes += rows * 4
        return out.tolist()

    # ---- one step ahead of the host (see run_generation)
    supports_lookahead = True

    def sample_async(self, logits, slots, params):
        """Samples on the device and starts the copy of the tokens to pinned host memory;
        returns (tokens on the device, pinned host tensor, event after the copy)."""
        rows = len(slots)
        e = self.e
        self._turn = (self._turn + 1) % 2                          # the host may still read the other pair
        if e._ahead is None:
            n = e._row_slot.numel()
            e._ahead = [(torch.empty(n, dtype=torch.int32, device=e.device),
                         torch.empty(n, dtype=torch.int32, pin_memory=True), torch.cuda.Event()) for _ in range(2)]
        dev, host, event = e._ahead[self._turn]
        self.e.sampler.sample(logits[:rows], self._row_slots(slots, params), params, out=dev[:rows])
        host[:rows].copy_(dev[:rows], non_blocking=True)
        event.record(torch.cuda.current_stream())
        self.d2h_bytes += rows * 4
        return dev[:rows], host[:rows], event

    def read(self, handle):
        handle[2].synchronize()
        return handle[1].tolist()

    def step_ahead(self, slots, handle):
        logits = self.e.step([SequenceStep(s, [0], [0]) for s in slots], device_tokens=handle[0])
        self.h2d_bytes += self.e.stepper.last_h2d_bytes
        return logits
