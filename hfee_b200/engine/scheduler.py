"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

It follows ``Runner`` in hostfog/hfee internal/llm/runner.go: requests wait until a
slot is free (:155-163), every step feeds one token of each decoding request first
and then prompt portions while the budget lasts (:232-261), a request whose logits
came back is sampled (:263-280), end tokens stop it without being emitted
(:288-291), ``num_predict`` and a full context end it with ``length`` (:309-310,
:248-251).  The reference reserves a whole context per slot, so it can never run
out of cache; here pages can run out, and then the request admitted last is
preempted: its pages are freed and it goes back to the *front* of the waiting queue
with what it generated so far appended to its prompt, to be recomputed when pages
are free again.  A request that does not fit the cache even alone ends with
``length``.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

from ..sampling.options import SamplingOptions
from ..sampling.sampler import fresh_seed
from .batch import StepEntry


DEVICE_TOKEN = -1      # placeholder for a token that was sampled on the device and not read back yet


class FinishReason:
    STOP = "stop"          # an end token was sampled (or a stop string matched)
    LENGTH = "length"      # num_predict reached, the context is full, or the cache cannot hold it
    ABORT = "abort"        # cancelled by the caller


@dataclass
class RequestStats:
    """The counters of ``llm.Stats`` (internal/llm/runner.go:15-21)."""
    prompt_tokens: int = 0
    prompt_seconds: float = 0.0
    eval_tokens: int = 0
    eval_seconds: float = 0.0
    done_reason: str = ""
    preemptions: int = 0


@dataclass
class Request:
    id: Any
    prompt: List[int]
    options: SamplingOptions
    output: List[int] = field(default_factory=list)
    feed: List[int] = field(default_factory=list)       # tokens still to run
    slot: Optional[int] = None
    seed: int = 0
    draws: int = 0
    ring_loaded: bool = False          # the device-side ring of recent tokens holds this request's history
    decoding: bool = False                               # the prompt has been read (evalStart set)
    finished: Optional[str] = None
    order: int = -1                                      # admission sequence number
    stats: RequestStats = field(default_factory=RequestStats)
    started: float = 0.0
    eval_started: float = 0.0

    @property
    def history(self) -> List[int]:
        return self.prompt + self.output


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    wants_logits: bool


class Scheduler:
    def __init__(self, cache: Any, max_batch_tokens: int, prefill_chunk: Optional[int] = None,
                 eos_token_ids: Sequence[int] = (), clock=time.perf_counter):
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.prefill_chunk = prefill_chunk or max_batch_tokens
        self.eos = frozenset(eos_token_ids)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.clock = clock
        self._admissions = 0
        self.preemptions = 0
        self._done: List[Request] = []

    # ------------------------------------------------------------------ intake
    def add(self, request: Request) -> None:
        """Queue a request.  Like runner.go:95-97 a prompt that does not leave room for
        one new token in the context is refused."""
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(request.prompt) >= self.cache.max_context:
            raise ValueError(f"prompt is {len(request.prompt)} tokens but the context window is "
                             f"{self.cache.max_context}")
        request.feed = list(request.prompt)
        request.seed = request.options.seed if request.options.seed >= 0 else fresh_seed()
        request.stats.prompt_tokens = len(request.prompt)
        self.waiting.append(request)

    def abort(self, request: Request) -> None:
        """Cancel a request wherever it is (runner.go:244-247: a cancelled context ends the
        request before its next pass).  What it holds goes back at once; tokens that were sampled
        on the device and not read back yet are dropped from its output."""
        if request.finished:
            return
        self.cut(request, len(request.output), FinishReason.ABORT)

    def finish(self, request: Request, reason: str) -> None:
        """End a running request from outside."""
        if not request.finished:
            self._finish(request, reason)

    def cut(self, request: Request, keep: int, reason: str) -> None:
        """End ``request`` with ``reason`` keeping its first ``keep`` output tokens (a stop string
        began behind them, runner.go:306-308).  Placeholders of tokens not read back yet go in any
        case; like the reference, tokens that were sampled still count in ``eval_tokens``."""
        out = request.output
        while out and out[-1] == DEVICE_TOKEN:
            out.pop()
            request.stats.eval_tokens -= 1
        del out[keep:]
        request.feed = []
        if request.finished:
            request.finished = request.stats.done_reason = reason
        else:
            self._finish(request, reason)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    def pop_finished(self) -> List[Request]:
        """Requests that finished (in ``plan`` or ``update``) since the last call."""
        done, self._done = self._done, []
        return done

    # ------------------------------------------------------------------ planning
    def plan(self) -> List[PlannedEntry]:
        """Decide what the next step runs.  May admit, preempt or finish requests."""
        self._admit()
        while True:
            entries, short = self._build()
            if short is None:
                return entries
            self._relieve(short)

    def _pages_for(self, tokens: int) -> int:
        return -(-tokens // self.cache.page_size)

    def _admit(self) -> None:
        promised = 0
        while self.waiting and self.cache.free_slots() > 0:
            req = self.waiting[0]
            first = min(len(req.feed), self.prefill_chunk, self.max_batch_tokens)
            if self._pages_for(first) + promised > self.cache.free_pages() and self.running:
                break          # wait for pages; with nothing running, _build shrinks the portion instead
            self.waiting.popleft()
            if req.stats.preemptions and not req.decoding:
                req.feed = req.prompt + req.output        # recompute everything it has so far
            req.slot = self.cache.open()
            req.order = self._admissions
            self._admissions += 1
            if not req.started:
                req.started = self.clock()
            self.running.append(req)
            promised += self._pages_for(first)

    def _build(self) -> Tuple[List[PlannedEntry], Optional[Request]]:
        """One pass over the running requests, decoding ones first.  Returns the entries
        and, if a request that must run cannot get pages, that request."""
        budget = self.max_batch_tokens
        free = self.cache.free_pages()
        entries: List[PlannedEntry] = []
        for decoding in (True, False):
            for req in list(self.running):
                if req.decoding != decoding or req.finished:
                    continue
                length = self.cache.length[req.slot]
                if length >= self.cache.max_context:            # runner.go:248-251
                    self._finish(req, FinishReason.LENGTH)
                    continue
                if budget == 0:
                    continue
                n = min(len(req.feed), budget, self.cache.max_context - length)
                if not decoding:
                    n = min(n, self.prefill_chunk)
                need = self.cache.pages_needed(req.slot, length + n)
                if need > free:
                    if decoding:
                        return entries, req
                    # a prompt portion: take what the free pages hold, down to nothing
                    room = (self._pages_for(length) + free) * self.cache.page_size - length
                    n = min(n, max(room, 0))
                    if n == 0:
                        if entries:
                            continue                             # others progress; wait for pages
                        return entries, req
                    need = self.cache.pages_needed(req.slot, length + n)
                free -= need
                budget -= n
                entries.append(PlannedEntry(req, req.feed[:n], wants_logits=(n == len(req.feed))))
        return entries, None

    def _relieve(self, short: Request) -> None:
        """``short`` cannot get the pages it needs.  Preempt the request admitted last; if
        ``short`` is the only one holding anything, it cannot fit the cache at all."""
        others = [r for r in self.running if r is not short]
        if not others:
            self._finish(short, FinishReason.LENGTH)
            return
        victim = max(self.running, key=lambda r: r.order)
        self._preempt(victim)

    def _preempt(self, req: Request) -> None:
        self.cache.close(req.slot)
        self.running.remove(req)
        req.slot = None
        req.feed = req.prompt + req.output          # recompute everything when re-admitted (rebuilt at admission,
        req.decoding = False                        # when placeholders in the output have been resolved)
        req.ring_loaded = False
        req.stats.preemptions += 1
        self.preemptions += 1
        self.waiting.appendleft(req)

    # ------------------------------------------------------------------ results
    def update(self, entries: Sequence[PlannedEntry], sampled: Sequence[int]) -> None:
        """Account for a step that ran ``entries``; ``sampled`` holds one token for each
        entry with ``wants_logits``, in order."""
        it = iter(sampled)
        now = self.clock()
        for e in entries:
            req = e.request
            req.feed = req.feed[len(e.tokens):]
            if not e.wants_logits:
                continue
            tok = int(next(it))
            if not req.decoding:                                # runner.go:273-277
                req.decoding = True
                if not req.eval_started:
                    req.stats.prompt_seconds = now - req.started
                    req.eval_started = now
            req.draws += 1
            if tok in self.eos:                                 # runner.go:288-291: not emitted, not counted
                self._finish(req, FinishReason.STOP)
                continue
            req.output.append(tok)
            req.stats.eval_tokens += 1
            if 0 <= req.options.num_predict <= req.stats.eval_tokens:      # runner.go:309-310
                self._finish(req, FinishReason.LENGTH)
            else:
                req.feed = [tok]

    # ------------------------------------------------------------------ results, one step late
    def update_provisional(self, entries: Sequence[PlannedEntry]) -> List[Tuple[Request, int]]:
        """Account for a step that was launched but whose sampled tokens stay on the device for
        now: each request whose logits were computed gets the placeholder ``DEVICE_TOKEN`` as its
        new output and next input.  Returns (request, output index) pairs in the order of the
        step's logits rows, for :meth:`resolve`."""
        pending: List[Tuple[Request, int]] = []
        now = self.clock()
        for e in entries:
            req = e.request
            req.feed = req.feed[len(e.tokens):]
            if not e.wants_logits:
                continue
            if not req.decoding:
                req.decoding = True
                if not req.eval_started:
                    req.stats.prompt_seconds = now - req.started
                    req.eval_started = now
            req.draws += 1
            req.output.append(DEVICE_TOKEN)
            req.stats.eval_tokens += 1
            pending.append((req, len(req.output) - 1))
            if 0 <= req.options.num_predict <= req.stats.eval_tokens:
                self._finish(req, FinishReason.LENGTH)
            else:
                req.feed = [DEVICE_TOKEN]
        return pending

    def resolve(self, pending: Sequence[Tuple[Request, int]], tokens: Sequence[int]) -> None:
        """Fill in the tokens of an earlier :meth:`update_provisional`.  An end token found now
        ends its request at that point: it and whatever was provisionally produced after it are
        dropped (the reference does not emit or count the end token, runner.go:288-291)."""
        for (req, idx), tok in zip(pending, tokens):
            if idx >= len(req.output):
                continue                                  # cut off by an end token, a stop string or a cancel
            tok = int(tok)
            if tok in self.eos:
                dropped = len(req.output) - idx
                del req.output[idx:]
                req.stats.eval_tokens -= dropped
                req.feed = []
                if req.finished:
                    req.finished = req.stats.done_reason = FinishReason.STOP
                else:
                    self._finish(req, FinishReason.STOP)
            else:
                req.output[idx] = tok

    def _finish(self, req: Request, reason: str) -> None:
        if req in self.waiting:
            self.waiting.remove(req)
        if req.slot is not None:
            self.cache.close(req.slot)
            req.slot = None
        if req in self.running:
            self.running.remove(req)
        req.finished = req.stats.done_reason = reason
        if req.eval_started:
            req.stats.eval_seconds = self.clock() - req.eval_started
        self._done.append(req)
