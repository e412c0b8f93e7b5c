"""The generation loop's decisions, on a scripted backend (no GPU)."""
import pytest

from oracle_engine_b200 import GenParams
from oracle_engine_b200.engine.generate import run_generation


class Scripted:
    """Each request i emits script[i] token by token; records how it is driven."""

    def __init__(self, scripts, n_slots=2, max_seq_len=64):
        self.scripts = scripts
        self.max_seq_len = max_seq_len
        self.free_slots = list(range(n_slots))
        self.owner = {}
        self.pos = {}
        self.steps = []
        self.events = []

    def alloc(self, i, prompt, params):
        slot = self.free_slots.pop(0)          # raises if the loop holds more than the batch
        self.owner[slot] = i
        self.pos[i] = 0
        self.events.append(("alloc", i, slot))
        return slot

    def free(self, slot):
        assert slot in self.owner, "freed twice"
        self.events.append(("free", self.owner.pop(slot), slot))
        self.free_slots.append(slot)

    def step(self, seqs):
        self.steps.append([(self.owner[s.slot], list(s.tokens), list(s.want)) for s in seqs])
        return [self.owner[s.slot] for s in seqs]

    def sample(self, logits, slots, params):
        assert [self.owner[s] for s in slots] == logits
        out = []
        for i in logits:
            out.append(self.scripts[i][self.pos[i]])
            self.pos[i] += 1
        return out


def test_unequal_prompts_stops_and_batches():
    scripts = {0: [5, 6, 99], 1: [7, 99], 2: [8, 9, 10, 11, 12], 3: [99]}
    be = Scripted(scripts)
    prompts = [[1, 2, 3], [4], [1, 1, 1, 1, 1], [2, 2]]
    res = run_generation(be, prompts, GenParams.greedy(4), batch_size=2, stop_ids=(99,))
    assert [r.tokens for r in res] == [[5, 6], [7], [8, 9, 10, 11], []]
    assert [r.finish_reason for r in res] == ["stop", "stop", "length", "stop"]
    # first step of a batch: whole prompts, last place wanted; then one token each
    assert be.steps[0] == [(0, [1, 2, 3], [2]), (1, [4], [0])]
    assert be.steps[1] == [(0, [5], [0]), (1, [7], [0])]
    assert be.steps[2] == [(0, [6], [0])]                         # request 1 ended earlier
    assert be.steps[3] == [(2, [1, 1, 1, 1, 1], [4]), (3, [2, 2], [1])]
    assert be.steps[4] == [(2, [8], [0])]
    # slots are given back when the batch ends, and used again by the next batch
    assert be.events == [("alloc", 0, 0), ("alloc", 1, 1), ("free", 0, 0), ("free", 1, 1),
                         ("alloc", 2, 0), ("alloc", 3, 1), ("free", 2, 0), ("free", 3, 1)]
    # the last sampled token of a request that hit its limit is not fed again
    assert len(be.steps) == 7 and be.steps[-1] == [(2, [10], [0])]


def test_ignore_eos_custom_stops_callback_and_context():
    be = Scripted({0: [99, 3, 4, 5, 6, 7, 8, 9]}, n_slots=1, max_seq_len=6)
    seen = []
    res = run_generation(be, [[1, 2, 3]], GenParams.greedy(8, ignore_eos=True), stop_ids=(99,),
                         on_token=lambda i, t: seen.append((i, t)))
    # the slot holds 6 tokens: 3 of the prompt, then 3 fed back; the 4th new token is still emitted
    assert res[0].tokens == [99, 3, 4, 5] and res[0].finish_reason == "context"
    assert seen == [(0, 99), (0, 3), (0, 4), (0, 5)]
    be = Scripted({0: [5, 6, 7]}, n_slots=1)
    res = run_generation(be, [[1]], GenParams.greedy(8, stop_ids=(6,)), stop_ids=(99,))
    assert res[0].tokens == [5] and res[0].finish_reason == "stop"


def test_refusals_and_cleanup():
    be = Scripted({0: [1]})
    with pytest.raises(ValueError, match="empty prompt"):
        run_generation(be, [[]], GenParams.greedy(2))
    with pytest.raises(ValueError, match="exceeds the context"):
        run_generation(be, [[1] * 100], GenParams.greedy(2))
    with pytest.raises(ValueError, match="top_p"):
        run_generation(be, [[1]], GenParams(top_p=0.0))

    class Failing(Scripted):
        def step(self, seqs):
            raise RuntimeError("boom")
    be = Failing({0: [1], 1: [2]})
    with pytest.raises(RuntimeError, match="boom"):
        run_generation(be, [[1], [2]], GenParams.greedy(2))
    assert sorted(be.free_slots) == [0, 1]                        # slots come back after an error
    be = Scripted({0: [1]}, n_slots=1)
    res = run_generation(be, [[1, 2]], GenParams.greedy(0))
    assert res[0].tokens == [] and be.steps == [] and be.free_slots == [0]


def test_reference_defaults():
    p = GenParams()
    assert (p.n_predict, p.temperature, p.top_p, p.top_k, p.repeat_penalty, p.repeat_last_n) == \
        (256, 0.7, 0.9, 40, 1.15, 64)
