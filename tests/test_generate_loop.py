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
        return [self.owner[s.slot] for s in seqs if s.want]       # one row of "logits" per wanted place

    def sample(self, logits, slots, params):
        assert [self.owner[s] for s in slots] == logits
        out = []
        for i in logits:
            out.append(self.scripts[i][self.pos[i]])
            self.pos[i] += 1
        return out


class ScriptedAhead(Scripted):
    """The same backend with the step ahead: a handle is the list of tokens not yet read."""
    supports_lookahead = True

    def sample_async(self, logits, slots, params):
        return {"tokens": self.sample(logits, slots, params), "read": False}

    def read(self, handle):
        handle["read"] = True
        return handle["tokens"]

    def step_ahead(self, slots, handle):
        assert not handle["read"], "a step ahead is queued before its tokens are read"
        self.steps.append([(self.owner[s], ["ahead"] + [t], [0]) for s, t in zip(slots, handle["tokens"])])
        return [self.owner[s] for s in slots]

    def sample(self, logits, slots, params):
        assert [self.owner[s] for s in slots] == logits
        out = []
        for i in logits:
            sc = self.scripts[i]
            out.append(sc[self.pos[i]] if self.pos[i] < len(sc) else 1000 + self.pos[i])    # beyond a stop: anything
            self.pos[i] += 1
        return out


def test_step_ahead_gives_the_same_results():
    scripts = {0: [5, 6, 99], 1: [7, 99], 2: [8, 9, 10, 11, 12, 13, 14], 3: [99], 4: [3, 4, 5, 6, 7, 8]}
    prompts = [[1, 2, 3], [4], [1, 1, 1, 1, 1], [2, 2], [9]]
    for n_predict, bs, ctx in [(n, b, c) for n in (1, 2, 4, 6) for b in (1, 2, 3, 5) for c in (64, 7)]:
        plain = run_generation(Scripted(scripts, n_slots=5, max_seq_len=ctx), prompts, GenParams.greedy(n_predict),
                               batch_size=bs, stop_ids=(99,))
        be = ScriptedAhead(scripts, n_slots=5, max_seq_len=ctx)
        seen = []
        ahead = run_generation(be, prompts, GenParams.greedy(n_predict), batch_size=bs, stop_ids=(99,),
                               on_token=lambda i, t: seen.append((i, t)))
        assert [r.tokens for r in ahead] == [r.tokens for r in plain]
        assert [r.finish_reason for r in ahead] == [r.finish_reason for r in plain]
        assert sorted(seen) == sorted((i, t) for i, r in enumerate(plain) for t in r.tokens)
        assert sorted(be.free_slots) == list(range(5))
        # no step holds more tokens of a sequence than its slot takes
        fed = {}
        for st in be.steps:
            for (i, toks, _) in st:
                fed[i] = fed.get(i, 0) + (1 if toks[0] == "ahead" else len(toks))
                assert fed[i] <= ctx
    assert any(r.finish_reason == "context" for r in plain)


def test_step_ahead_decisions():
    be = ScriptedAhead({0: [5, 6, 7, 8, 9, 10], 1: [7, 8, 99]})
    res = run_generation(be, [[1, 2], [3]], GenParams.greedy(6), batch_size=2, stop_ids=(99,))
    assert [r.tokens for r in res] == [[5, 6, 7, 8, 9, 10], [7, 8]]
    assert be.steps == [
        [(0, [1, 2], [1]), (1, [3], [0])],                    # the prompts
        [(0, ["ahead", 5], [0]), (1, ["ahead", 7], [0])],     # queued before 5 and 7 were read
        [(0, ["ahead", 6], [0]), (1, ["ahead", 8], [0])],
        [(0, ["ahead", 7], [0]), (1, ["ahead", 99], [0])],    # ran with the sequence that had stopped: its row is dropped
        [(0, [8], [0])],                                      # the survivor alone, its token from the host again
        [(0, ["ahead", 9], [0])],
        # the sixth token ends request 0 by its count: no step is queued for it
    ]


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


def test_prompts_in_portions():
    """A limit on the prompt tokens per step: portions in request order, logits wanted only where a
    prompt ends, finished prompts decode beside later portions, a request without room waits."""
    scripts = {0: [5, 6, 7], 1: [8, 9, 10], 2: [11, 99]}
    prompts = [[1, 2, 3], [4, 5, 6, 7, 8], [9]]
    be = Scripted(scripts, n_slots=3)
    res = run_generation(be, prompts, GenParams.greedy(3), stop_ids=(99,), max_step_tokens=4)
    assert [r.tokens for r in res] == [[5, 6, 7], [8, 9, 10], [11]]
    assert be.steps == [
        [(0, [1, 2, 3], [2]), (1, [4], [])],                       # request 2 got no room
        [(0, [5], [0]), (1, [5, 6, 7, 8], [3])],                   # a decoded token beside a portion that ends
        [(0, [6], [0]), (1, [8], [0]), (2, [9], [0])],             # request 2 starts two steps late
        [(1, [9], [0]), (2, [11], [0])],                           # request 0 ended by its count
    ]
    # two-token portions, and a portion that is the prompt's last token alone
    be = Scripted({0: [5, 6]}, n_slots=1)
    res = run_generation(be, [[1, 2, 3, 4, 5]], GenParams.greedy(2), max_step_tokens=2)
    assert be.steps == [[(0, [1, 2], [])], [(0, [3, 4], [])], [(0, [5], [0])], [(0, [5], [0])]]
    assert res[0].tokens == [5, 6]
    # the tokens do not depend on the limit, with and without the step ahead
    scripts = {0: [5, 6, 99], 1: [7, 99], 2: [8, 9, 10, 11, 12, 13, 14], 3: [99], 4: [3, 4, 5, 6, 7, 8]}
    prompts = [[1, 2, 3], [4], [1, 1, 1, 1, 1], [2, 2], [9]]
    whole = run_generation(Scripted(scripts, n_slots=5), prompts, GenParams.greedy(5), stop_ids=(99,))
    for limit in (1, 2, 3, 100):
        for cls in (Scripted, ScriptedAhead):
            got = run_generation(cls(scripts, n_slots=5), prompts, GenParams.greedy(5), stop_ids=(99,),
                                 max_step_tokens=limit, batch_size=3)
            assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in whole]
    with pytest.raises(ValueError, match="max_step_tokens"):
        run_generation(Scripted(scripts), prompts, GenParams.greedy(1), max_step_tokens=0)


def test_device_errors_end_the_batch():
    """The backend's check (error flags that kernels set) is read once per batch; what it raises
    reaches the caller, and the slots still come back."""
    class Flagged(Scripted):
        checks = 0

        def check(self):
            self.checks += 1
            if self.checks == 2:
                raise RuntimeError("a bounded wait inside a kernel ran out")
    be = Flagged({0: [1, 2], 1: [3, 4], 2: [5, 6]}, n_slots=1)
    with pytest.raises(RuntimeError, match="bounded wait"):
        run_generation(be, [[1], [2], [3]], GenParams.greedy(2), batch_size=1)
    assert be.checks == 2 and be.free_slots == [0]
    assert [e[0] for e in be.events] == ["alloc", "free", "alloc", "free"]      # the third batch never started


def test_reference_defaults():
    p = GenParams()
    assert (p.n_predict, p.temperature, p.top_p, p.top_k, p.repeat_penalty, p.repeat_last_n) == \
        (256, 0.7, 0.9, 40, 1.15, 64)


def test_decode_kernel_rules_depend_on_sizes_only():
    """Which decode attention kernel runs and how many CTAs share a sequence's keys are functions
    of the batch size, the context class and the geometry (a captured graph stays valid), and
    the context classes cut where they say."""
    from oracle_engine_b200.csrc import ops_tc
    from oracle_engine_b200.engine import batch
    assert [batch.context_class(n) for n in (1, 768, 769, 1536, 1537, 4096, 4097, 100000)] == [0, 0, 1, 1, 2, 2, 3, 3]
    uses = lambda n_seqs, cls: ops_tc.decode_uses_warps(n_seqs, cls, 128, 24, 8, sm_count=148)
    assert [uses(b, c) for c in (0, 1, 2, 3) for b in (1, 8, 64, 500)] == [True] * 16       # wherever it can be used
    # few sequences past 768 tokens: 2, 4 or 8 CTAs (a cluster) per (sequence, KV head), at most about 64 CTAs in all
    cluster = lambda n_seqs, cls: ops_tc.decode_warps_cluster(n_seqs, cls, 8, sm_count=148)
    assert [cluster(b, 0) for b in (1, 4, 8, 64)] == [1, 1, 1, 1]
    assert [cluster(b, 1) for b in (1, 2, 3, 4, 5, 8, 64)] == [4, 4, 2, 2, 1, 1, 1]
    assert [cluster(b, 2) for b in (1, 2, 3, 4, 5, 8, 64)] == [4, 4, 2, 2, 1, 1, 1]
    assert [cluster(b, 3) for b in (1, 2, 3, 4, 5, 8, 64)] == [8, 4, 2, 2, 1, 1, 1]
    with ops_tc.knobs(decode_warps_cluster=2):
        assert cluster(64, 0) == 2
    # its form, (warps, tiles in a warp's ring): the most warps whose CTAs are all resident at once (1, 2 or 4 an SM)
    shape = lambda n_seqs, cls, hd=128, kvh=8: ops_tc.decode_warps_shape(n_seqs, cls, hd, kvh, sm_count=148)
    assert [shape(b, 0) for b in (1, 18, 19, 37, 38, 64, 74, 75, 128)] == \
        [(6, 2), (6, 2), (2, 3), (2, 3), (1, 3), (1, 3), (1, 3), (1, 3), (1, 3)]
    assert [shape(b, 1) for b in (18, 19, 38, 128)] == [(6, 2), (2, 3), (1, 3), (1, 3)]         # up to 1,536 tokens alike
    # long contexts: no one-warp form; past one round of CTAs the fullest last round, equal ones to the smaller CTAs
    assert [shape(b, c) for c in (2, 3) for b in (18, 19, 37, 38, 48, 64, 96, 128)] == 2 * \
        [(6, 2), (2, 3), (2, 3), (6, 2), (6, 2), (2, 3), (2, 3), (6, 2)]
    assert shape(4, 0, hd=256, kvh=2) == (2, 3) and shape(100, 2, hd=256, kvh=2) == (2, 3)     # 6 x 2 does not fit an SM there
    assert shape(30, 0, hd=64, kvh=8) == (6, 2) and shape(40, 0, hd=64, kvh=8) == (2, 3)       # two CTAs of 6 x 2 an SM
    with ops_tc.knobs(decode_warps_shape=(4, 3)):
        assert shape(64, 0) == (4, 3)
    assert not ops_tc.decode_uses_warps(8, 0, 128, 64, 2, sm_count=148)                      # 32 heads per KV head
    splits = lambda n_seqs, cls, pages=128: ops_tc.decode_splits(n_seqs, 8, 148, pages, cls, 3)
    assert [splits(b, 0) for b in (1, 8, 24, 64)] == [32, 5, 2, 1]                            # about two CTAs an SM
    assert [splits(b, 1) for b in (1, 8, 24, 64)] == [32, 5, 2, 1]
    assert [splits(b, 3) for b in (1, 8, 24, 32, 40, 64)] == [32, 6, 2, 3, 4, 3]              # the last round filled
    assert splits(8, 3, pages=4) == 4 and splits(1, 0, pages=3) == 3
    # the products: the weight-streaming kernel up to 16 tokens; the two-SM kernel from 129 tokens on, except
    # for weights with few tiles at up to 384 tokens, which the one-SM kernel splits over clusters
    assert [ops_tc.uses_skinny(m, 3072, 3072, 0) for m in (1, 8, 9, 16, 17)] == [True, True, True, True, False]
    shapes = ((3072, 8192), (3072, 3072), (5120, 3072), (16384, 3072))
    assert [ops_tc.uses_pair(128, n, k, 148) for n, k in shapes] == [False] * 4
    assert [ops_tc.uses_pair(200, n, k, 148) for n, k in shapes] == [False, False, True, True]
    assert [ops_tc.uses_pair(385, n, k, 148) for n, k in shapes] == [True] * 4
    # and their places in the launch chain: flags per product and token count
    from oracle_engine_b200.parts.linear import START_EARLY, TRIGGER_LATE, chain_flags
    assert chain_flags("mixer_out", 8) == START_EARLY | TRIGGER_LATE and chain_flags("mixer_out", 9) == TRIGGER_LATE
    assert chain_flags("ffn_out", 1) == START_EARLY and chain_flags("ffn_out", 16) == START_EARLY | TRIGGER_LATE                          # never more than the pages


def test_step_plan_packs_unequal_sequences_with_padding():
    """The packed plan of a step: rows in the order of the sequences, places counted per sequence, padding
    tokens that belong to no sequence and padding sequences that bring no token; a prompt's tokens given as
    an array (what the step's validation hands over) pack to the same plan as the list."""
    import numpy as np
    from oracle_engine_b200.engine.batch import SequenceStep, build_plan
    seqs = [SequenceStep(4, [11, 12, 13], [0, 2]), SequenceStep(1, [21], []), SequenceStep(7, [31, 32], [1])]
    starts = [0, 9, 64]
    plan = build_plan(seqs, starts, pad_seqs=4, pad_tokens=8)
    assert plan.n_seqs == 4 and plan.n_tokens == 8 and plan.n_real_tokens == 6
    assert plan.token_ids.tolist() == [11, 12, 13, 21, 31, 32, 0, 0]
    assert plan.tok_seq.tolist() == [0, 0, 0, 1, 2, 2, -1, -1]
    assert plan.tok_pos.tolist() == [0, 1, 2, 9, 64, 65, 0, 0]
    assert plan.seq_slot.tolist() == [4, 1, 7, -1] and plan.seq_qlen.tolist() == [3, 1, 2, 0]
    assert plan.cu_q.tolist() == [0, 3, 4, 6, 6]
    assert plan.want_rows.tolist() == [0, 2, 5]
    assert (plan.max_qlen, plan.max_kvlen, plan.all_decode) == (3, 66, False)
    arrays = [np.asarray(s.tokens, dtype=np.int64) if len(s.tokens) > 1 else None for s in seqs]
    same = build_plan(seqs, starts, pad_seqs=4, pad_tokens=8, token_arrays=arrays)
    for name in ("token_ids", "tok_seq", "tok_pos", "seq_slot", "seq_start", "seq_qlen", "cu_q", "want_rows"):
        assert np.array_equal(getattr(plan, name), getattr(same, name)), name
    with pytest.raises(ValueError, match="outside its 1 tokens"):
        build_plan([SequenceStep(0, [5], [1])], [0])
    assert build_plan([SequenceStep(0, [5], [0]), SequenceStep(1, [6], [])], [3, 4]).all_decode
