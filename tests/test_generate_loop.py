"""The generation loop's decisions, with a scripted engine and sampler (no GPU)."""
import pytest

from airframe_b200.cache import IndexPool
from airframe_b200.engine.generate import GenerationLoop, RequestError
from airframe_b200.sampling import SamplingParams


class FakeCache:
    def __init__(self, pages, slots):
        self.total_pages, self.n_slots = pages, slots


class FakeEngine:
    """Keeps slots and lengths; 'logits' are just the slots of the step."""

    def __init__(self, pages=64, slots=8, max_context=32, vocab=100):
        self.cache = FakeCache(pages, slots)
        self.pool = IndexPool(slots, "slot")
        self.max_context, self.vocab_size = max_context, vocab
        self.lens, self.steps = {}, []

    def take_slot(self):
        s = self.pool.take()
        self.lens[s] = 0
        return s

    def free_slot(self, s):
        self.pool.give_back(s)
        del self.lens[s]

    def step(self, entries, borrow=False):
        starting = [self.lens[e.slot] == 0 for e in entries]
        assert all(starting) or not any(starting)
        if not all(starting):
            assert all(len(e.tokens) == 1 for e in entries)
        for e in entries:
            self.lens[e.slot] += len(e.tokens)
            assert self.lens[e.slot] <= self.max_context
            assert e.want == [len(e.tokens) - 1]
        self.steps.append([(e.slot, list(e.tokens)) for e in entries])
        return [e.slot for e in entries]


class ScriptSampler:
    """Request i emits script[i][k] as its k-th token."""

    def __init__(self, script):
        self.script = script

    def new_state(self, params, index):
        return {"index": index, "k": 0}

    def sample(self, logits, states, params):
        out = []
        for st in states:
            out.append(self.script[st["index"]][st["k"]])
            st["k"] += 1
        return out


P = lambda **kw: SamplingParams(temperature=0.0, repetition_penalty=1.0, **kw)


def test_unequal_prompts_stop_tokens_and_early_ends():
    eng = FakeEngine()
    script = {0: [5, 6, 9, 1], 1: [9], 2: [5, 5, 5, 5, 5, 5]}
    loop = GenerationLoop(eng, ScriptSampler(script), stop_token_ids=[9])
    seen = []
    out = loop.generate([[1, 2, 3], [4], [7, 7, 7, 7, 7]], P(max_tokens=4), on_token=lambda i, t: seen.append((i, t)))
    assert out == [[5, 6], [], [5, 5, 5, 5]]                     # the stop token is not emitted
    assert loop.finish_reasons == ["stop", "stop", "length"]
    assert eng.steps[0] == [(0, [1, 2, 3]), (1, [4]), (2, [7, 7, 7, 7, 7])]   # all prompts in one step
    assert eng.steps[1] == [(0, [5]), (2, [5])]                  # request 1 has left
    assert eng.steps[2] == [(0, [6]), (2, [5])]
    assert eng.steps[3] == [(2, [5])]                            # request 0 ended earlier
    assert len(eng.steps) == 4                                   # the last token is not fed
    assert eng.pool.n_held == 0
    assert seen == [(0, 5), (2, 5), (0, 6), (2, 5), (2, 5), (2, 5)]


def test_ignore_eos_and_explicit_stops():
    eng = FakeEngine()
    loop = GenerationLoop(eng, ScriptSampler({0: [9, 4, 8, 8]}), stop_token_ids=[9])
    assert loop.generate([[1]], P(max_tokens=4, ignore_eos=True, stop_token_ids=[8])) == [[9, 4]]
    assert loop.finish_reasons == ["stop"]


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(slots=2)
    script = {i: [i + 10] * 3 for i in range(5)}
    loop = GenerationLoop(eng, ScriptSampler(script))
    out = loop.generate([[1]] * 5, P(max_tokens=2))
    assert out == [[i + 10] * 2 for i in range(5)]
    assert loop.batches_run == [[0, 1], [2, 3], [4]]
    assert [s for step in eng.steps for s, _ in step if True][:2] == [0, 1]
    assert {s for step in eng.steps for s, _ in step} == {0, 1}   # only two slots ever used
    assert eng.pool.n_held == 0


def test_batches_respect_the_page_budget():
    eng = FakeEngine(pages=3, slots=8, max_context=200)
    loop = GenerationLoop(eng, ScriptSampler({i: [1] * 80 for i in range(4)}))
    # a request of 60 + 9 tokens holds 2 pages, one of 10 + 9 holds 1
    assert loop.plan_batches([[0] * 60, [0] * 10, [0] * 10, [0] * 60], P(max_tokens=10)) == [[0, 1], [2, 3]]
    with pytest.raises(RequestError, match="cache pages"):
        loop.plan_batches([[0] * 190], P(max_tokens=10))
    loop2 = GenerationLoop(eng, ScriptSampler({}), max_batch=1)
    assert loop2.plan_batches([[0], [0]], P(max_tokens=1)) == [[0], [1]]


def test_context_limit_ends_a_sequence():
    eng = FakeEngine(max_context=6)
    loop = GenerationLoop(eng, ScriptSampler({0: [3] * 10}))
    out = loop.generate([[1, 2, 3, 4]], P(max_tokens=10))
    assert out == [[3, 3, 3]] and loop.finish_reasons == ["context"]
    assert eng.pool.n_held == 0


def test_bad_requests_and_zero_tokens():
    eng = FakeEngine(max_context=4)
    loop = GenerationLoop(eng, ScriptSampler({}))
    with pytest.raises(RequestError, match="empty"):
        loop.generate([[]], P())
    with pytest.raises(RequestError, match="context holds"):
        loop.generate([[1] * 5], P())
    with pytest.raises(RequestError, match="outside the vocabulary"):
        loop.generate([[100]], P())
    with pytest.raises(ValueError, match="top_p"):
        loop.generate([[1]], SamplingParams(top_p=0.0))
    assert loop.generate([[1]], P(max_tokens=0)) == [[]] and eng.steps == []


def test_slots_come_back_when_a_step_fails():
    class Failing(FakeEngine):
        def step(self, entries, borrow=False):
            if len(self.steps) == 1:
                raise RuntimeError("boom")
            return super().step(entries)
    eng = Failing()
    loop = GenerationLoop(eng, ScriptSampler({0: [1] * 5, 1: [1] * 5}))
    with pytest.raises(RuntimeError, match="boom"):
        loop.generate([[1], [2]], P(max_tokens=5))
    assert eng.pool.n_held == 0
