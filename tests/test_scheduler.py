"""The scheduler's decisions, on a fake engine (no GPU): a real cache manager on the host,
and a next token that is a function of everything the request was fed, so that a wrong,
missing or repeated token in any step changes all later tokens."""

import random

import pytest

from mini_llm_b200.cache import CacheManager
from mini_llm_b200.engine.scheduler import Request, Scheduler
from mini_llm_b200.parts.spec import PagedKV

VOCAB = 1000


def next_token(history):
    value = 17
    for token in history:
        value = (value * 31 + token + 7) % 1000003
    return value % VOCAB


def expected_tokens(prompt, n):
    history, out = list(prompt), []
    for _ in range(n):
        out.append(next_token(history))
        history.append(out[-1])
    return out


class FakeEngine:
    def __init__(self, n_pages=64, page_size=4, max_requests=4, max_positions=64):
        self.cache = CacheManager([PagedKV(1, 16)], page_size, n_pages, max_requests, max_positions)
        self.max_positions = max_positions
        self.fed = {}
        self.batches = []
        self.fail_next = False
        self._sampled = []

    def open_request(self):
        slot = self.cache.open()
        if slot is not None:
            self.fed[slot] = []
        return slot

    def close_request(self, slot):
        self.cache.close(slot)
        del self.fed[slot]

    def step(self, entries, sampling=None):
        if self.fail_next:
            self.fail_next = False
            raise RuntimeError("device fault (injected)")
        assert len({e.slot for e in entries}) == len(entries)
        needed = sum(self.cache.pages_needed(e.slot, len(e.tokens))[0] for e in entries)
        assert needed <= self.cache.pages_free()[0], "the scheduler built a batch that does not fit the pages"
        self._sampled = []
        wanted = 0
        for e in entries:
            assert self.cache.reserve(e.slot, len(e.tokens))
            self.cache.commit(e.slot, len(e.tokens))
            self.fed[e.slot].extend(e.tokens)
            for place in e.want:
                assert place == len(e.tokens) - 1
                self._sampled.append(next_token(self.fed[e.slot]))
                wanted += 1
        assert sampling is None or len(sampling) == wanted
        self.sampling = sampling
        self.batches.append([(e.slot, len(e.tokens), bool(e.want)) for e in entries])
        self.cache.check()

    def sampled_tokens(self):
        return self._sampled


def prompt(seed, n):
    rng = random.Random(seed)
    return [rng.randrange(VOCAB) for _ in range(n)]


def test_one_request_in_portions_then_decoding():
    engine = FakeEngine()
    s = Scheduler(engine, max_tokens_per_step=8, max_prefill_chunk=5)
    r = Request(prompt(1, 13), max_new_tokens=4)
    s.submit(r)
    s.run()
    assert [b[0][1] for b in engine.batches] == [5, 5, 3, 1, 1, 1]
    assert [b[0][2] for b in engine.batches] == [False, False, True, True, True, True]
    assert r.generated == expected_tokens(r.tokens, 4) and r.finish_reason == "length"
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == 4
    stats = s.stats()
    assert (stats["steps"], stats["tokens"], stats["prefills"], stats["prefill_tokens"], stats["decode_tokens"]) == \
        (6, 4, 1, 13, 3)


def test_finish_reasons_in_the_references_order():
    engine = FakeEngine(max_positions=16)
    s = Scheduler(engine)
    p = prompt(2, 10)
    eos = expected_tokens(p, 3)[2]
    stop = Request(p, max_new_tokens=3, eos_token_id=eos)          # eos arrives with the length limit: "stop" wins
    context = Request(prompt(3, 12), max_new_tokens=50)
    length = Request(prompt(4, 3), max_new_tokens=1)
    seen = []
    stop.emit = lambda token, reason: seen.append((token, reason))
    for r in (stop, context, length):
        s.submit(r)
    s.run()
    assert stop.finish_reason == "stop" and len(stop.generated) == 3
    assert seen == [(t, None) for t in stop.generated[:2]] + [(eos, "stop")]
    assert context.finish_reason == "context" and len(context.tokens) + len(context.generated) == 16
    assert length.finish_reason == "length" and len(length.generated) == 1
    assert length.generated == expected_tokens(length.tokens, 1)


def test_token_budget_decodes_first_then_portions_in_arrival_order():
    engine = FakeEngine(max_requests=4)
    s = Scheduler(engine, max_tokens_per_step=7)
    requests = [Request(prompt(10 + i, n), max_new_tokens=12) for i, n in enumerate((1, 9, 24, 40))]
    for r in requests:
        s.submit(r)
    s.run()
    for batch in engine.batches:
        assert sum(n for _, n, _ in batch) <= 7
        kinds = [n == 1 and want for _, n, want in batch]
        assert kinds == sorted(kinds, reverse=True) or all(n == 1 for _, n, _ in batch[:kinds.count(True)])
    assert engine.batches[0] == [(0, 1, True), (1, 6, False)]            # 1-token prompt, then 6 of the second
    assert engine.batches[1] == [(0, 1, True), (1, 3, True), (2, 3, False)]
    assert any(len(b) == 4 for b in engine.batches)                      # four live at once
    for r in requests:
        assert r.generated == expected_tokens(r.tokens, 12), "batching changed a request's tokens"


def test_no_slot_means_waiting_and_arrival_order_is_kept():
    engine = FakeEngine(max_requests=2)
    s = Scheduler(engine, max_tokens_per_step=64)
    a, b, c = (Request(prompt(20 + i, 5), max_new_tokens=n) for i, n in enumerate((2, 6, 3)))
    for r in (a, b, c):
        s.submit(r)
    s.step()
    assert len(s.running) == 2 and list(s.waiting) == [c]
    s.step()                                    # a ends here
    assert a.finish_reason == "length" and list(s.waiting) == [c]
    s.step()                                    # its slot goes to c
    assert not s.waiting and {r.request is c for r in s.running} == {True, False}
    s.run()
    assert c.generated == expected_tokens(c.tokens, 3) and b.generated == expected_tokens(b.tokens, 6)


def test_no_pages_means_waiting_and_nothing_overtakes():
    engine = FakeEngine(n_pages=8, page_size=4, max_requests=4)           # 32 tokens of cache
    s = Scheduler(engine, max_tokens_per_step=64)
    big = Request(prompt(30, 20), max_new_tokens=2)                       # 5 pages (+1 for the decoded tokens)
    second = Request(prompt(31, 16), max_new_tokens=2)                    # 4 pages: does not fit beside big
    small = Request(prompt(32, 2), max_new_tokens=2)                      # would fit, but must not overtake
    for r in (big, second, small):
        s.submit(r)
    s.step()
    assert [r.request for r in s.running] == [big]                        # second waits for its whole prompt's pages
    assert engine.batches[0] == [(0, 20, True)] and list(s.waiting) == [second, small]
    s.run()
    assert s.stats()["preemptions"] == 0
    for r in (big, second, small):
        assert r.generated == expected_tokens(r.tokens, 2)


def test_pages_run_out_while_decoding_the_last_admitted_is_preempted_and_recomputed():
    engine = FakeEngine(n_pages=6, page_size=4, max_requests=3)           # 24 tokens
    s = Scheduler(engine, max_tokens_per_step=64)
    first = Request(prompt(40, 7), max_new_tokens=12)                     # 2 pages now, grows to 5
    last = Request(prompt(41, 8), max_new_tokens=9)                       # 2 pages now, grows to 5
    s.submit(first)
    s.submit(last)
    s.run()
    assert s.stats()["preemptions"] >= 1 and last.preemptions >= 1 and first.preemptions == 0
    assert first.generated == expected_tokens(first.tokens, 12)
    assert last.generated == expected_tokens(last.tokens, 9), "recomputation changed the request's tokens"
    recompute = [b for b in engine.batches if any(n > 1 and want for _, n, want in b)]
    assert recompute[0] == [(0, 7, True), (1, 8, True)]                   # both prompts in one batch
    again = recompute[1][0][1]                                            # the preempted request, recomputed as a prompt
    assert 8 < again <= 8 + 9 and len(recompute) >= 2
    assert engine.cache.pages_in_use() == [0]


def test_a_request_that_cannot_fit_alone_fails_and_the_others_go_on():
    engine = FakeEngine(n_pages=4, page_size=4, max_requests=2, max_positions=64)      # 16 tokens
    s = Scheduler(engine, max_tokens_per_step=64)
    messages = []
    too_big = Request(prompt(50, 30), max_new_tokens=2, fail=messages.append)
    grows = Request(prompt(51, 14), max_new_tokens=8)                     # fits at first, then outgrows the cache
    fine = Request(prompt(52, 5), max_new_tokens=3)
    for r in (too_big, grows, fine):
        s.submit(r)
    s.run(max_steps=100)
    assert too_big.error and "out of pages" in too_big.error and messages == [too_big.error]
    assert grows.error and "out of pages" in grows.error and len(grows.generated) >= 2
    assert fine.generated == expected_tokens(fine.tokens, 3) and fine.error is None
    assert engine.cache.pages_in_use() == [0] and not s.running and not s.waiting


def test_cancel_before_and_during():
    engine = FakeEngine(max_requests=2)
    s = Scheduler(engine, max_tokens_per_step=64)
    a, b, c = (Request(prompt(60 + i, 6), max_new_tokens=10) for i in range(3))
    for r in (a, b, c):
        s.submit(r)
    c.cancel()
    s.step()
    s.step()
    a.cancel()
    s.step()
    assert all(slot != 0 or False for slot, _, _ in engine.batches[-1]) or len(engine.batches[-1]) == 1
    assert len(engine.batches[-1]) == 1                                   # a left before the step ran
    s.run()
    assert b.generated == expected_tokens(b.tokens, 10) and len(a.generated) == 2 and c.generated == []
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == 2


def test_engine_error_fails_the_running_requests_only():
    engine = FakeEngine(max_requests=2)
    s = Scheduler(engine, max_tokens_per_step=64)
    failed = []
    a, b, c = (Request(prompt(70 + i, 4), max_new_tokens=5, fail=failed.append) for i in range(3))
    for r in (a, b, c):
        s.submit(r)
    s.step()
    engine.fail_next = True
    s.step()
    assert a.error == b.error == "device fault (injected)" and len(failed) == 2
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == 2
    s.run()
    assert c.error is None and c.generated == expected_tokens(c.tokens, 5)


def test_a_raising_callback_drops_only_its_request():
    engine = FakeEngine()
    s = Scheduler(engine)

    def broken(token, reason):
        raise ConnectionError("consumer is gone")

    a = Request(prompt(80, 4), max_new_tokens=5, emit=broken)
    b = Request(prompt(81, 4), max_new_tokens=5)
    s.submit(a)
    s.submit(b)
    s.run()
    assert a.finish_reason == "stop" and len(a.generated) == 1
    assert b.generated == expected_tokens(b.tokens, 5)
    assert engine.cache.pages_in_use() == [0]


def test_bad_prompts_are_refused_at_once():
    engine = FakeEngine(max_positions=16)
    s = Scheduler(engine)
    empty, long = Request([]), Request(prompt(90, 16))
    s.submit(empty)
    s.submit(long)
    assert empty.error == "empty prompt" and "16" in long.error and not s.waiting
    # ids that are no tokens fail their own request, before any batch is built; a negative id
    # is never a request's to give (the engine reads one as "the token sampled last")
    engine.vocab_size = VOCAB
    good, beyond, negative, text = Request(prompt(91, 5)), Request([1, VOCAB]), Request([-1]), Request([3, "x"])
    for request in (good, beyond, negative, text):
        s.submit(request)
    assert good.error is None and list(s.waiting) == [good]
    assert str(VOCAB) in beyond.error and "-1" in negative.error and "'x'" in text.error
    s.run()
    assert len(good.generated) > 0 or good.finish_reason is not None
    with pytest.raises(ValueError):
        Scheduler(engine, max_tokens_per_step=0)


def test_sampling_parameters_follow_the_request_not_the_batch():
    engine = FakeEngine()
    s = Scheduler(engine, max_tokens_per_step=64)
    a = Request(prompt(95, 3), max_new_tokens=3, temperature=0.8, top_p=0.9, seed=11)
    b = Request(prompt(96, 3), max_new_tokens=2, temperature=0.0, seed=12)
    s.submit(a)
    s.submit(b)
    s.step()
    assert [(p.temperature, p.top_p, p.seed, p.counter) for p in engine.sampling] == [(0.8, 0.9, 11, 0), (0.0, 1.0, 12, 0)]
    s.step()
    assert [(p.seed, p.counter) for p in engine.sampling] == [(11, 1), (12, 1)]
    s.step()
    assert [(p.seed, p.counter) for p in engine.sampling] == [(11, 2)]


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_end_clean_and_batching_never_changes_tokens(seed):
    rng = random.Random(seed)
    engine = FakeEngine(n_pages=rng.choice([10, 14, 24]), page_size=4, max_requests=rng.choice([2, 3, 5]),
                        max_positions=40)
    s = Scheduler(engine, max_tokens_per_step=rng.choice([5, 9, 32]), max_prefill_chunk=rng.choice([None, 3, 8]))
    requests = [Request(prompt(seed * 100 + i, rng.randrange(1, 24)), max_new_tokens=rng.randrange(1, 12))
                for i in range(14)]
    pending = list(requests)
    for _ in range(2000):
        if pending and rng.random() < 0.3:
            s.submit(pending.pop(0))
        if not s.step() and not pending:
            break
        engine.cache.check()
    assert not pending and not s.running and not s.waiting
    for r in requests:
        assert r.error is None and r.finish_reason in ("length", "context")
        assert r.generated == expected_tokens(r.tokens, len(r.generated))
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == engine.cache.max_requests


# ---- run-ahead: a step is launched before the tokens of the step before are read -------------

class RunAheadEngine(FakeEngine):
    """A fake engine that resolves PREVIOUS from what the slot sampled last, keeps the last two
    steps' tokens and notes the order of launches and reads."""

    def __init__(self, **kwargs):
        super().__init__(**kwargs)
        self.kept = {}
        self.history = [[], []]
        self.calls = []

    def open_request(self):
        slot = super().open_request()
        self.kept.pop(slot, None)
        return slot

    def step(self, entries, sampling=None):
        from mini_llm_b200.engine.engine import PREVIOUS, StepEntry
        resolved = []
        for e in entries:
            tokens = list(e.tokens)
            if tokens[0] == PREVIOUS:
                assert e.slot in self.kept, "PREVIOUS for a slot that has sampled nothing"
                tokens[0] = self.kept[e.slot]
            assert PREVIOUS not in tokens
            resolved.append(StepEntry(e.slot, tokens, e.want))
        super().step(resolved, sampling)
        cursor = 0
        for e in resolved:
            if e.want:
                self.kept[e.slot] = self._sampled[cursor]
                cursor += 1
        self.history = [list(self._sampled), self.history[0]]
        self.calls.append("step")

    def sampled_tokens(self, ago=0):
        self.calls.append(f"read{ago}")
        return self.history[ago]


def test_run_ahead_launches_the_next_step_before_it_reads_the_last():
    engine = RunAheadEngine()
    s = Scheduler(engine, max_tokens_per_step=64, run_ahead=True)
    a, b = Request(prompt(100, 5), max_new_tokens=6), Request(prompt(101, 9), max_new_tokens=4)
    s.submit(a)
    s.submit(b)
    s.run()
    assert a.generated == expected_tokens(a.tokens, 6) and b.generated == expected_tokens(b.tokens, 4)
    assert a.finish_reason == b.finish_reason == "length"
    # prompt step, then five decode steps each launched before the step before is read, then the last read
    assert engine.calls == ["step"] + ["step", "read1"] * 5 + ["read0"]
    assert engine.batches[3] == [(0, 1, True), (1, 1, True)] and engine.batches[4] == [(0, 1, True)]   # b's 4th token was its last
    assert [(p.seed, p.counter) for p in engine.sampling] == [(0, 5)]
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == 4


def test_run_ahead_finds_the_stop_token_one_step_late_and_drops_the_extra_token():
    engine = RunAheadEngine()
    s = Scheduler(engine, max_tokens_per_step=64, run_ahead=True)
    p = prompt(110, 6)
    eos = expected_tokens(p, 3)[2]
    seen = []
    stops = Request(p, max_new_tokens=10, eos_token_id=eos, emit=lambda token, reason: seen.append((token, reason)))
    other = Request(prompt(111, 4), max_new_tokens=8)
    late = Request(prompt(112, 7), max_new_tokens=3)
    s.submit(stops)
    s.submit(other)
    for _ in range(3):
        s.step()
    s.submit(late)                         # takes the slot the stopped request gives back
    s.run()
    assert stops.finish_reason == "stop" and stops.generated == expected_tokens(p, 3)
    assert seen[-1] == (eos, "stop") and len(seen) == 3
    assert other.generated == expected_tokens(other.tokens, 8)
    assert late.generated == expected_tokens(late.tokens, 3)
    assert sum(1 for b in engine.batches for slot, n, want in b if slot == 0 and n == 1) >= 3   # one step more than it needed
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == 4


def test_run_ahead_reads_first_when_pages_are_short_so_that_preemption_knows_every_token():
    engine = RunAheadEngine(n_pages=6, page_size=4, max_requests=3)
    s = Scheduler(engine, max_tokens_per_step=64, run_ahead=True)
    first = Request(prompt(40, 7), max_new_tokens=12)
    last = Request(prompt(41, 8), max_new_tokens=9)
    s.submit(first)
    s.submit(last)
    s.run()
    assert s.stats()["preemptions"] >= 1 and last.preemptions >= 1 and first.preemptions == 0
    assert first.generated == expected_tokens(first.tokens, 12)
    assert last.generated == expected_tokens(last.tokens, 9)
    assert "read0" in engine.calls[:-1]
    assert engine.cache.pages_in_use() == [0]


@pytest.mark.parametrize("seed", range(6))
def test_run_ahead_random_workloads_give_the_same_tokens(seed):
    rng = random.Random(1000 + seed)
    engine = RunAheadEngine(n_pages=rng.choice([10, 14, 24]), page_size=4, max_requests=rng.choice([2, 3, 5]),
                            max_positions=40)
    s = Scheduler(engine, max_tokens_per_step=rng.choice([5, 9, 32]), max_prefill_chunk=rng.choice([None, 3, 8]),
                  run_ahead=True)
    requests = []
    for i in range(14):
        p = prompt(seed * 100 + i, rng.randrange(1, 24))
        limit = rng.randrange(1, 12)
        eos = expected_tokens(p, limit)[rng.randrange(limit)] if rng.random() < 0.4 else None
        requests.append(Request(p, max_new_tokens=limit, eos_token_id=eos))
    pending = list(requests)
    for _ in range(2000):
        if pending and rng.random() < 0.3:
            s.submit(pending.pop(0))
        if not s.step() and not pending:
            break
        engine.cache.check()
    assert not pending and not s.running and not s.waiting and s._flight is None
    for r in requests:
        assert r.error is None and r.finish_reason in ("length", "context", "stop")
        assert r.generated == expected_tokens(r.tokens, len(r.generated))
        if r.finish_reason == "stop":
            assert r.generated[-1] == r.eos_token_id and r.eos_token_id not in r.generated[:-1]
        elif r.eos_token_id is not None:
            assert r.eos_token_id not in r.generated
    assert engine.cache.pages_in_use() == [0] and engine.cache.free_slots == engine.cache.max_requests
