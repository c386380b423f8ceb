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


# ---------------------------------------------------------------- the device one step ahead of the host

class AheadEngine(FakeEngine):
    """An engine whose decode steps can take their tokens from 'the device'."""
    use_graphs = True

    def decode_rows(self, slots, tokens_dev, borrow=True):
        live = [(r, s) for r, s in enumerate(slots) if s is not None]
        assert live and len(slots) == len(tokens_dev)
        for r, s in live:
            assert self.lens[s] > 0
            self.lens[s] += 1
            assert self.lens[s] <= self.max_context
        self.steps.append([(s, [tokens_dev[r]]) for r, s in live])
        return list(slots)


class Pending:
    def __init__(self, tokens):
        self.device = tokens
        self.read = False

    def result(self):
        self.read = True
        return self.device


class AheadSampler(ScriptSampler):
    def sample_async(self, logits, states, params):
        out = []
        for st in states:
            if st is None:
                out.append(0)
                continue
            seq = self.script[st["index"]]
            out.append(seq[st["k"]] if st["k"] < len(seq) else 0)
            st["k"] += 1
        return Pending(out)


SCRIPTS = [
    ({0: [5, 6, 9, 1], 1: [9], 2: [5, 5, 5, 5, 5, 5]}, [[1, 2, 3], [4], [7, 7, 7, 7, 7]], dict(max_tokens=4)),
    ({0: [9], 1: [9]}, [[1], [2]], dict(max_tokens=3)),
    ({0: [1, 2, 3, 4, 5, 6, 7, 8], 1: [1, 9]}, [[1] * 28, [2]], dict(max_tokens=8)),       # request 0 meets the context limit
    ({0: [4], 1: [4, 4], 2: [4, 4, 9]}, [[1], [2], [3]], dict(max_tokens=1)),
    ({i: [i + 10] * 3 for i in range(5)}, [[1]] * 5, dict(max_tokens=2)),
]


@pytest.mark.parametrize("script,prompts,kw", SCRIPTS)
def test_a_step_ahead_gives_the_same_tokens_and_reasons(script, prompts, kw):
    runs = []
    for ahead in (False, True):
        eng = AheadEngine(slots=3)
        loop = GenerationLoop(eng, AheadSampler({k: list(v) for k, v in script.items()}), stop_token_ids=[9])
        loop.pipelined = ahead
        seen = {}
        out = loop.generate(prompts, P(**kw), on_token=lambda i, t: seen.setdefault(i, []).append(t))
        assert eng.pool.n_held == 0
        runs.append((out, loop.finish_reasons, seen, eng.steps, loop.batches_run))
    assert runs[0][0] == runs[1][0] and runs[0][1] == runs[1][1] and runs[0][2] == runs[1][2]
    assert runs[0][4] == runs[1][4]
    # one step ahead, a sequence is fed at most one token more than in step: the stop token it ended on
    fed = [sum(len(t) for step in r[3] for _, t in step) for r in runs]
    n_stops = sum(1 for reason in runs[0][1] if reason == "stop")
    assert fed[0] <= fed[1] <= fed[0] + n_stops


def test_a_step_ahead_feeds_nothing_after_the_last_allowed_token():
    eng = AheadEngine()
    loop = GenerationLoop(eng, AheadSampler({0: [3, 3, 3, 3], 1: [4, 9, 4, 4]}), stop_token_ids=[9])
    assert loop.generate([[1, 1], [2]], P(max_tokens=3)) == [[3, 3, 3], [4]]
    assert loop.finish_reasons == ["length", "stop"]
    # prompts; both rows; both rows (request 1's stop token is in flight); request 0 alone is never fed its third token
    assert eng.steps == [[(0, [1, 1]), (1, [2])], [(0, [3]), (1, [4])], [(0, [3]), (1, [9])]]


def test_a_repetition_penalty_keeps_the_loop_in_step():
    eng = AheadEngine()
    loop = GenerationLoop(eng, AheadSampler({0: [3, 9]}), stop_token_ids=[9])
    out = loop.generate([[1]], SamplingParams(temperature=0.0, repetition_penalty=1.3, max_tokens=4))
    assert out == [[3]] and eng.steps == [[(0, [1])], [(0, [3])]]


# ---------------------------------------------------------------- the control hook

def test_logits_processor_allows_forces_stops_and_blocks():
    from airframe_b200.engine.generate import STOP, Blocked
    script = {0: [10, 11, 12, 13, 14], 1: [20, 21, 22, 23, 24], 2: [30, 31, 32, 33, 34]}
    eng = FakeEngine()
    loop = GenerationLoop(eng, ScriptSampler(script), stop_token_ids=[99])
    seen = []

    def control(index, step, row, tokens):
        seen.append((index, step, row, list(tokens)))
        if index == 0 and step == 1:
            return 77                      # ForceToken: 77 goes out instead of the sampler's 11
        if index == 1 and step == 2:
            return STOP                    # EarlyExit after two tokens
        if index == 2 and step == 1:
            return 99                      # a forced stop token ends the sequence like a sampled one
        return None                        # Allow

    params = SamplingParams(max_tokens=4, temperature=0.0)
    out = loop.generate([[1, 2], [3], [4, 5, 6]], params, logits_processor=control)
    assert out == [[10, 77, 12, 13], [20, 21], [30]]
    assert loop.finish_reasons == ["length", "control", "stop"]
    # the hook sees, per live sequence and step, its own row of logits and its tokens so far
    assert (0, 0, 0, [1, 2]) in seen and (0, 2, 0, [1, 2, 10, 77]) in seen and (1, 2, 1, [3, 20, 21]) in seen
    assert not any(i == 1 and st == 3 for i, st, _, _ in seen)
    # the forced token is what the next step is fed
    assert (0, [77]) in [x for stp in eng.steps for x in stp]
    assert eng.pool.n_held == 0

    def block(index, step, row, tokens):
        if step == 1:
            raise Blocked("policy says no")
        return None

    with pytest.raises(Blocked, match="policy"):
        loop.generate([[1, 2]], params, logits_processor=block)
    assert eng.pool.n_held == 0            # the slots came back although the call ended in an error
    with pytest.raises(RequestError, match="logits processor returned"):
        loop.generate([[1, 2]], params, logits_processor=lambda i, s, r, t: 1000)
    assert eng.pool.n_held == 0


def test_a_processor_keeps_the_loop_in_lock_step():
    """With a processor the loop never uses decode_rows (the host must see every token first)."""
    class AheadEngine(FakeEngine):
        use_graphs = True

        def decode_rows(self, slots, tokens):
            raise AssertionError("queued a step ahead although a processor was given")

    class S(ScriptSampler):
        def sample_async(self, *a):
            raise AssertionError("sampled ahead although a processor was given")

    loop = GenerationLoop(AheadEngine(), S({0: [5, 6, 7]}))
    out = loop.generate([[1]], SamplingParams(max_tokens=3, temperature=0.0, repetition_penalty=1.0),
                        logits_processor=lambda i, s, r, t: None)
    assert out == [[5, 6, 7]]
