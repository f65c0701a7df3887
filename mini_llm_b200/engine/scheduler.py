"""Continuous batching above the step function.

The reference's scheduler (pytorch/src/mini_llm/scheduler.py) admits a waiting
request when a whole cache is free, prefills its whole prompt alone
(:156-183), then decodes all running requests together (:213-231), and ends a
request on "stop" (end-of-text token), "context" (prompt + generated reaches
the position limit) or "length" (:185-196), checked in that order on every
delivered token.  Its caches never run out.  Here the same loop runs on
pages and mixed batches:

* every iteration builds ONE batch under a token budget: first one token for
  every decoding request, then portions of prompts (continued ones, then new
  ones in arrival order), each at most ``max_prefill_chunk`` tokens;
* a request is admitted only if a slot is free and the pages of its next
  portion are; nothing is admitted past a request that does not fit (arrival
  order is kept);
* when pages run out for a DECODING request, the request admitted last is
  preempted: its pages and slot are given back and it returns to the front of
  the waiting queue with its tokens so far, to be recomputed as a prompt
  (recomputation is the one policy that works for any kind of mixer state);
* a request that cannot fit even alone fails with "out of pages".

Sampling uses (seed, number of tokens generated so far) per request, so a
request's tokens depend neither on its batch nor on preemption.

With ``run_ahead`` the scheduler launches a step before it has read the tokens
of the step before: a decoding request's entry names its token as ``PREVIOUS``
(the engine takes it on the device), and the host reads the earlier step's
tokens while the new step runs.  What is known without the tokens decides the
batch (lengths, "length" and "context" endings); a request that ends on its
end-of-text token is found one step late, its extra token is dropped.  When
pages are so short that a decoding request might have to be preempted, the
step in flight is read first, so that a preempted request always knows all of
its tokens.

The scheduler needs from its engine: ``open_request``, ``close_request``,
``step(entries, sampling)``, ``sampled_tokens()``, ``max_positions`` and
``cache`` (a ``CacheManager``).  Tests drive it with a fake engine, as the
reference does (pytorch/tests/batch_fakes.py:6-45).
"""

from __future__ import annotations

import collections
import operator
from dataclasses import dataclass, field
from typing import Callable

from .engine import PREVIOUS, SamplingParams, StepEntry


@dataclass(eq=False)
class Request:
    tokens: list                              # the prompt
    max_new_tokens: int | None = None
    eos_token_id: int | None = None
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0
    emit: Callable | None = None              # emit(token, finish_reason or None)
    fail: Callable | None = None              # fail(message)
    generated: list = field(default_factory=list, init=False)
    finish_reason: str | None = field(default=None, init=False)
    error: str | None = field(default=None, init=False)
    cancelled: bool = field(default=False, init=False)
    preemptions: int = field(default=0, init=False)

    def cancel(self) -> None:
        self.cancelled = True

    @property
    def done(self) -> bool:
        return self.finish_reason is not None or self.error is not None or self.cancelled


@dataclass(eq=False)
class _Running:
    request: Request
    slot: int
    pending: list               # tokens not yet run: the rest of the prompt (or of a recomputation), or the last sampled token
    order: int                  # admission counter: the largest was admitted last
    decoding: bool = False      # its prompt is in the cache and it has sampled its first token
    awaiting: bool = False      # a step that samples for it has been launched and not been read yet


class Scheduler:
    def __init__(self, engine, max_tokens_per_step: int = 2048, max_prefill_chunk: int | None = None,
                 max_batch: int | None = None, run_ahead: bool = False):
        if max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be at least 1")
        self.engine = engine
        self.budget = int(max_tokens_per_step)
        self.chunk = int(max_prefill_chunk) if max_prefill_chunk else self.budget
        self.max_batch = int(max_batch) if max_batch else None
        self.waiting: collections.deque = collections.deque()
        self.running: list[_Running] = []
        self._admitted = 0
        self.counters = collections.Counter()
        self.run_ahead = bool(run_ahead)
        self._flight = None               # (entries, owners, ids of the owners it samples for) of the launched step whose tokens are unread

    # ---- requests in ------------------------------------------------------------------------
    def submit(self, request: Request) -> None:
        limit = self.engine.max_positions
        vocab = getattr(self.engine, "vocab_size", None)
        # A prompt is checked here, so that a bad one fails alone: the engine checks a whole
        # batch and refuses all of it.  Ids below zero are never a request's to give (the
        # engine reads one of them as "what this request sampled last").
        try:
            request.tokens = [operator.index(t) for t in request.tokens]
            bad = next((t for t in request.tokens if t < 0 or (vocab is not None and t >= vocab)), None)
        except TypeError:
            bad = next(t for t in request.tokens if not hasattr(t, "__index__"))
        if not request.tokens:
            self._fail(request, "empty prompt")
        elif bad is not None:
            self._fail(request, f"token id {bad!r} is not an integer in the vocabulary"
                                + (f" [0, {vocab})" if vocab is not None else ""))
        elif len(request.tokens) >= limit:
            # The reference's servers trim such prompts from the left (pytorch/src/mini_llm/
            # api_common.py:38-41); the engine itself refuses them.
            self._fail(request, f"prompt of {len(request.tokens)} tokens leaves no room in {limit} positions")
        else:
            self.waiting.append(request)

    def stats(self) -> dict:
        c = self.counters
        return {"steps": c["steps"], "decode_steps": c["decode_steps"], "tokens": c["tokens"],
                "prefills": c["prefills"], "prefill_tokens": c["prefill_tokens"],
                "decode_tokens": c["decode_tokens"], "preemptions": c["preemptions"],
                "mean_batch_size": c["batch_entries"] / c["steps"] if c["steps"] else 0.0,
                "running": len(self.running), "waiting": len(self.waiting),
                "pages_in_use": self.engine.cache.pages_in_use(), "pages_free": self.engine.cache.pages_free()}

    # ---- one iteration ----------------------------------------------------------------------
    def step(self) -> bool:
        """Build and run one batch.  Returns False if there was nothing to do."""
        self._drop_cancelled()
        if self._flight is not None and self._pages_are_short():
            self._collect(0)                  # preemption may be needed: every token must be known
        try:
            entries, owners = self._build_batch()
        except Exception as error:
            self._flight = None
            self._fail_running(str(error))
            return True
        if not entries:
            if self._flight is not None:
                self._collect(0)
                return True
            return bool(self.running or self.waiting)
        sampling = []
        for running, entry in zip(owners, entries):
            if entry.want:
                r = running.request
                sampling.append(SamplingParams(r.temperature, r.top_p, r.seed, len(r.generated) + running.awaiting))
        try:
            self.engine.step(entries, sampling)
        except Exception as error:          # the engine is shared: every running request is affected
            self._flight = None
            self._fail_running(str(error))
            return True
        self.counters["steps"] += 1
        self.counters["batch_entries"] += len(entries)
        if any(len(e.tokens) == 1 and e.want for e in entries):
            self.counters["decode_steps"] += 1
        earlier, self._flight = self._flight, (entries, owners, {id(o) for o, e in zip(owners, entries) if e.want})
        for running, entry in zip(owners, entries):
            n = len(entry.tokens)
            self.counters["decode_tokens" if running.decoding else "prefill_tokens"] += n
            running.pending = running.pending[n:]
            if entry.want:
                if not running.decoding:
                    self.counters["prefills"] += 1
                running.decoding = True
                running.awaiting = True
                running.pending = [PREVIOUS]
        if earlier is not None:
            self._collect(1, earlier)         # the step before, while the new one runs
        if not self.run_ahead:
            self._collect(0)
        self.running = [r for r in self.running if not r.request.done]
        return True

    def _collect(self, ago: int, flight=None) -> None:
        """Read a launched step's tokens and deliver them."""
        if flight is None:
            flight, self._flight = self._flight, None
        entries, owners, _ = flight
        try:
            sampled = self.engine.sampled_tokens(ago) if self.run_ahead else self.engine.sampled_tokens()
        except Exception as error:
            self._flight = None
            self._fail_running(str(error))
            return
        cursor = 0
        for running, entry in zip(owners, entries):
            if entry.want:
                token = int(sampled[cursor])
                cursor += 1
                running.awaiting = self._in_flight(running)
                if not running.request.done:       # else: it ended a step ago; this token is dropped
                    self._deliver(running, token)
        self.running = [r for r in self.running if not r.request.done]

    def _in_flight(self, running) -> bool:
        return self._flight is not None and id(running) in self._flight[2]

    def _pages_are_short(self) -> bool:
        """Whether the decoding requests' next tokens need more pages than are free (lengths
        are known without the tokens: a launched step has already been committed)."""
        cache = self.engine.cache
        free = cache.pages_free()
        decoding = sum(1 for running in self.running if running.decoding)
        if all(f >= decoding for f in free):
            return False                      # one more token takes at most one page per group
        need = [0] * len(free)
        for running in self.running:
            if running.decoding:
                for g, count in enumerate(cache.pages_needed(running.slot, 1)):
                    need[g] += count
        return any(n > f for n, f in zip(need, free))

    def run(self, max_steps: int | None = None) -> int:
        """Iterate until nothing runs or waits; returns the number of iterations."""
        steps = 0
        while (self.running or self.waiting or self._flight) and (max_steps is None or steps < max_steps):
            self.step()
            steps += 1
        return steps

    # ---- building the batch -----------------------------------------------------------------
    def _build_batch(self):
        cache = self.engine.cache
        spare = [0] * len(cache.groups)
        entries, owners = [], []
        budget = self.budget

        def take(running, n, want, needed=None):
            if needed is None:
                needed = cache.pages_needed(running.slot, n)
            for g, count in enumerate(needed):
                spare[g] += count
            entries.append(StepEntry(running.slot, running.pending[:n], [n - 1] if want else []))
            owners.append(running)

        # 1. one token for every decoding request; preempt from the back while pages are short
        for running in [r for r in self.running if r.decoding]:
            if running not in self.running:
                continue                      # preempted below
            while (needed := cache.room_for(running.slot, 1, spare)) is None:
                victim = max(self.running, key=lambda r: r.order)
                if victim is running and len(self.running) == 1:
                    self._close(running)
                    self._fail(running.request, "out of pages: the request does not fit the cache even alone")
                    break
                if victim in owners:          # its entry of this step is withdrawn
                    index = owners.index(victim)
                    for g, count in enumerate(cache.pages_needed(victim.slot, len(entries[index].tokens))):
                        spare[g] -= count
                    budget += len(entries[index].tokens)
                    del owners[index], entries[index]
                self._preempt(victim)
                if victim is running:
                    break
            if running.awaiting and self._ends_on_count(running.request, 1):
                continue                      # the token on its way is its last
            if running in self.running and not running.request.done and budget > 0:
                take(running, 1, True, needed)
                budget -= 1

        # 2. portions of prompts: continued ones first, then new requests in arrival order
        for running in self.running:
            if budget <= 0:
                break
            if running.decoding or running in owners or not running.pending:
                continue
            n = min(len(running.pending), self.chunk, budget)
            while n > 0 and not cache.can_reserve(running.slot, n, spare):
                n = self._largest_fit(running.slot, n, spare)
            if n <= 0:
                if not entries and len(self.running) == 1 and not self._could_ever_fit(running, 1):
                    self._close(running)
                    self._fail(running.request, "out of pages: the request does not fit the cache even alone")
                continue
            take(running, n, n == len(running.pending))
            budget -= n
        # A new request is admitted only if the pages of its WHOLE prompt (and of its first
        # new token) are free beyond what this step takes and what the prompts still being
        # prefilled will take: a request admitted on less would soon be preempted again.
        promised = [0] * len(cache.groups)
        for running in self.running:
            if not running.decoding:
                rest = len(running.pending) - (len(entries[owners.index(running)].tokens) if running in owners else 0)
                whole = cache.pages_needed(running.slot, min(len(running.pending) + 1, self.engine.max_positions -
                                                             cache.length(running.slot)))
                now = cache.pages_needed(running.slot, len(running.pending) - rest)
                for g in range(len(promised)):
                    promised[g] += whole[g] - now[g]
        while budget > 0 and self.waiting and (self.max_batch is None or len(self.running) < self.max_batch):
            request = self.waiting[0]
            if request.cancelled:
                self.waiting.popleft()
                continue
            slot = self.engine.open_request()
            if slot is None:
                break                         # no slot: wait for a running request to end
            pending = list(request.tokens) + list(request.generated)
            whole = min(len(pending) + 1, self.engine.max_positions)
            if not cache.can_reserve(slot, whole, [a + b for a, b in zip(spare, promised)]):
                self.engine.close_request(slot)
                if not self.running:
                    self.waiting.popleft()
                    self._fail(request, "out of pages: the request does not fit the cache even alone")
                    continue
                break                         # no pages: wait; nothing overtakes this request
            n = min(len(pending), self.chunk, budget)
            self.waiting.popleft()
            running = _Running(request, slot, pending, self._admitted)
            self._admitted += 1
            self.running.append(running)
            needed_whole = cache.pages_needed(slot, whole)
            take(running, n, n == len(pending))
            needed_now = cache.pages_needed(slot, n)
            for g in range(len(promised)):
                promised[g] += needed_whole[g] - needed_now[g]
            budget -= n
        return entries, owners

    def _largest_fit(self, slot, n, spare) -> int:
        """The largest portion <= n whose pages are free (0 if not even one token fits)."""
        cache = self.engine.cache
        lo, hi = 0, n
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if cache.can_reserve(slot, mid, spare):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _could_ever_fit(self, running, n) -> bool:
        cache = self.engine.cache
        needed = cache.pages_needed(running.slot, n)
        held = cache.pages_held(running.slot)
        return all(not g.paged or needed[g.index] + held[g.index] <= g.pool.n_pages for g in cache.groups)

    # ---- requests out -----------------------------------------------------------------------
    def _ends_on_count(self, request: Request, more: int) -> bool:
        """Whether ``more`` further tokens end the request on "context" or "length"."""
        count = len(request.generated) + more
        return (len(request.tokens) + count >= self.engine.max_positions or
                (request.max_new_tokens is not None and count >= request.max_new_tokens))

    def _finish_reason(self, request: Request, token: int) -> str | None:
        if request.eos_token_id is not None and token == request.eos_token_id:
            return "stop"
        if len(request.tokens) + len(request.generated) >= self.engine.max_positions:
            return "context"
        if request.max_new_tokens is not None and len(request.generated) >= request.max_new_tokens:
            return "length"
        return None

    def _deliver(self, running: _Running, token: int) -> None:
        request = running.request
        request.generated.append(token)
        if not self.run_ahead:
            running.pending = [token]
        running.decoding = True
        self.counters["tokens"] += 1
        reason = self._finish_reason(request, token)
        if request.emit is not None:
            try:
                request.emit(token, reason)
            except Exception:
                # the consumer is gone: that ends this request only (scheduler.py:202-208)
                reason = reason or "stop"
        if reason is not None:
            request.finish_reason = reason
            self._close(running)

    def _close(self, running: _Running) -> None:
        self.engine.close_request(running.slot)
        if running in self.running:
            self.running.remove(running)

    def _preempt(self, running: _Running) -> None:
        self._close(running)
        running.request.preemptions += 1
        self.counters["preemptions"] += 1
        self.waiting.appendleft(running.request)

    def _drop_cancelled(self) -> None:
        for running in [r for r in self.running if r.request.cancelled]:
            self._close(running)

    def _fail(self, request: Request, message: str) -> None:
        request.error = message
        if request.fail is not None:
            try:
                request.fail(message)
            except Exception:
                pass

    def _fail_running(self, message: str) -> None:
        for running in list(self.running):
            self._close(running)
            self._fail(running.request, message)

    def fail_everything(self, message: str) -> None:
        self._flight = None
        self._fail_running(message)
        while self.waiting:
            self._fail(self.waiting.popleft(), message)
