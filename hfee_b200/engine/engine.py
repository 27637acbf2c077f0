"""The Python entry point: ``Engine(model_dir).generate(prompts, options)``.

It stands where the reference has ``Runner.Generate`` behind its server
(hostfog/hfee internal/llm/runner.go:93-141): prompts in, tokens (and text, if the
model folder has a tokenizer) out, with the counters of ``llm.Stats``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

import torch

from ..config import EngineConfig
from ..kernels import ops
from ..sampling import BatchSampler, SamplingOptions
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import DEVICE_TOKEN, FinishReason, Request, RequestStats, Scheduler
from .text import TextStream, TokenizerAdapter


@dataclass
class GenerationResult:
    token_ids: List[int]
    text: Optional[str]
    stats: RequestStats


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ[name])
    except (KeyError, ValueError):
        return default


class Engine:
    """A model, its cache, a scheduler and a sampler.

    ``generate`` takes token-id prompts (lists of ints) or, when the model folder
    holds a ``tokenizer.json`` and the ``tokenizers`` package is importable, text.
    Engine settings are an :class:`EngineConfig` or its fields as keywords; like the
    reference's server (internal/server/server.go:46-57) ``HFEE_NUM_PARALLEL`` and
    ``HFEE_NUM_CTX`` give the defaults of ``max_requests`` and ``max_context``."""

    def __init__(self, model_dir: str, engine: Optional[EngineConfig] = None, tokenizer: Any = None,
                 **settings: Any):
        if engine is None:
            settings.setdefault("max_requests", max(1, _env_int("HFEE_NUM_PARALLEL", 4)))
            settings.setdefault("max_context", max(256, _env_int("HFEE_NUM_CTX", 4096)))
            engine = EngineConfig(**settings)
        elif settings:
            raise TypeError("pass either an EngineConfig or keyword settings, not both")
        self.model_dir = model_dir
        self.runner = ModelRunner(model_dir, engine)
        self.config = engine
        spec = self.runner.spec
        # like runner.go:72 the usable context is capped by what the model was trained for
        self.max_context = min(engine.max_context, spec.max_positions)
        self.runner.cache.max_context = min(self.runner.cache.max_context, self.max_context)
        self.sampler = BatchSampler(self.runner.device, engine.max_requests)
        self.eos_token_ids = tuple(spec.eos_token_ids)
        # text in and out: the folder's tokenizer.json, or any object with encode() and decode()
        # (and optionally piece(id) -> bytes) handed in
        tokenizer = tokenizer if tokenizer is not None else _load_tokenizer(model_dir)
        self.tokenizer = TokenizerAdapter(tokenizer) if tokenizer is not None else None
        self.pipeline = True          # overlap host work with the GPU where the sampling options allow it
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._next_id = 0

    # ------------------------------------------------------------------ text
    def encode(self, text: str) -> List[int]:
        if self.tokenizer is None:
            raise RuntimeError(f"{self.model_dir} has no tokenizer.json (or the tokenizers package is missing): "
                               "pass token ids")
        ids = self.tokenizer.encode(text)
        bos = self.runner.spec.bos_token_id
        return ([bos] if bos is not None else []) + ids        # Encode(prompt, addSpecial=true), runner.go:94

    def decode(self, ids: Sequence[int]) -> Optional[str]:
        return None if self.tokenizer is None else self.tokenizer.decode(ids)

    # ------------------------------------------------------------------ generation
    def new_scheduler(self) -> Scheduler:
        return Scheduler(self.runner.cache, self.config.max_batch_tokens, self.config.prefill_chunk,
                         self.eos_token_ids)

    def generate(self, prompts: Union[Sequence[int], str, Sequence[Union[Sequence[int], str]]],
                 options: Union[SamplingOptions, Sequence[SamplingOptions], None] = None,
                 on_token: Optional[Callable[[int, int], Optional[bool]]] = None,
                 on_text: Optional[Callable[[int, str], Optional[bool]]] = None,
                 cancel: Optional[Any] = None) -> List[GenerationResult]:
        """Continue every prompt; returns one result per prompt, in order.

        ``on_token(prompt_index, token_id)`` is called for each new token and, with a tokenizer,
        ``on_text(prompt_index, text)`` for each piece of text that may be shown: whole characters
        only, nothing that may still become a stop string, never the stop string itself
        (internal/llm/text.go:16-78); with stop strings a token is reported once all its text has
        been.  A callback that returns ``False`` cancels its request, and so does adding the
        prompt's index to ``cancel`` (any object with ``in``, e.g. a set another thread fills): the
        request ends before the next step with ``done_reason == "abort"`` and what it held is
        free again (runner.go:244-247).  A request stopped by a stop string keeps the tokens in
        front of it (runner.go:296-308)."""
        if isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int)):
            prompts = [prompts]
        if options is None:
            options = SamplingOptions()
        if isinstance(options, SamplingOptions):
            options = [options] * len(prompts)
        if len(options) != len(prompts):
            raise ValueError("one SamplingOptions per prompt (or one for all) is needed")
        if self.tokenizer is None and any(o.stop for o in options):
            raise ValueError(f"stop strings need text, and {self.model_dir} has no tokenizer")
        sched = self.new_scheduler()
        requests = []
        for i, (p, o) in enumerate(zip(prompts, options)):
            ids = self.encode(p) if isinstance(p, str) else [int(t) for t in p]
            req = Request(id=i, prompt=ids, options=o)
            sched.add(req)
            requests.append(req)
        n = len(requests)
        streams = [TextStream(self.tokenizer, o.stop) if self.tokenizer is not None else None for o in options]
        seen = [0] * n          # output tokens already turned into text
        emitted = [0] * n       # output tokens already given to on_token
        closed = [False] * n    # the request has ended and everything of it was delivered
        cancelled = cancel if cancel is not None else set()

        def tell(i: int, upto: int) -> None:
            r = requests[i]
            while emitted[i] < min(upto, len(r.output)):
                tok = r.output[emitted[i]]
                emitted[i] += 1
                if on_token is not None and on_token(i, tok) is False:
                    cancelled.add(i)

        def deliver() -> None:
            """Look at every token that has become known since the last call."""
            for i, r in enumerate(requests):
                if closed[i]:
                    continue
                st = streams[i]
                while seen[i] < len(r.output) and r.output[seen[i]] != DEVICE_TOKEN:
                    tok = r.output[seen[i]]
                    seen[i] += 1
                    if st is None:
                        continue
                    text, hit = st.push(tok)
                    if text and on_text is not None and on_text(i, text) is False:
                        cancelled.add(i)
                    if hit:
                        sched.cut(r, st.whole_tokens, FinishReason.STOP)
                        break
                held_back = st is not None and bool(st.stopper.stops)
                tell(i, st.whole_tokens if held_back else seen[i])
                if r.finished and seen[i] >= len(r.output):
                    if st is not None and r.finished != FinishReason.ABORT:
                        rest = st.finish()
                        if rest and on_text is not None:
                            on_text(i, rest)
                        if st.hit:                      # found in what the last characters completed
                            sched.cut(r, st.whole_tokens, FinishReason.STOP)
                    tell(i, len(r.output))
                    closed[i] = True

        def drop_cancelled() -> None:
            for i, r in enumerate(requests):
                if not r.finished and i in cancelled:
                    sched.abort(r)

        # When every request samples on the device, steps are pipelined: the sampled tokens stay
        # on the device for the next step and the host reads them one step late, so planning and
        # launching overlap the GPU's work.  A stop string or a cancel found late cuts the request
        # where it belongs; the step that was already launched for it changes nothing that is kept.
        on_device = all(o.device_only for o in options) or all(
            o.device_chain and self.sampler.chain_takes(self.runner.vocab) for o in options)
        if self.pipeline and on_device:
            inflight = None
            while not sched.idle or inflight is not None:
                drop_cancelled()
                launched = self.launch_step(sched) if not sched.idle else None
                if inflight is not None:
                    pending, handle = inflight
                    if handle is not None:
                        tokens = self.sampler.fetch(handle)
                        self.d2h_bytes += 4 * len(tokens)
                        sched.resolve(pending, tokens)
                inflight = launched
                deliver()
                sched.pop_finished()
        else:
            while not sched.idle:
                drop_cancelled()
                self.run_step(sched)
                deliver()
                sched.pop_finished()
        deliver()
        ops.check_status()
        return [GenerationResult(list(r.output), streams[i].text if streams[i] is not None else None, r.stats)
                for i, r in enumerate(requests)]

    def launch_step(self, sched: Scheduler):
        """Plan and launch one step without waiting for its result.  Returns (pending, handle) for
        ``Scheduler.resolve`` / ``BatchSampler.fetch``, or None if nothing could run."""
        plan = sched.plan()
        if not plan:
            return None
        entries = [StepEntry(e.request.slot, e.tokens, (len(e.tokens) - 1,) if e.wants_logits else ())
                   for e in plan]
        logits = self.runner.step(entries)
        step = self.runner.last_step
        self.h2d_bytes += step.h2d_bytes
        handle = None
        if logits is not None:
            who = [e.request for e in plan if e.wants_logits]
            for r in who:                     # a request's first draw since it was admitted: its recent tokens go to the device
                if r.options.penalises and not r.ring_loaded:
                    self.sampler.load_history(r.slot, r.prompt + r.output)
                    r.ring_loaded = True
            handle = self.sampler.launch(logits, [r.options for r in who], [r.seed for r in who],
                                         [r.draws for r in who], step.logit_slots, self.runner.feedback)
        return sched.update_provisional(plan), handle

    def run_step(self, sched: Scheduler) -> int:
        """Plan, run and account for one step; returns the number of tokens it ran."""
        plan = sched.plan()
        if not plan:
            return 0
        entries = [StepEntry(e.request.slot, e.tokens, (len(e.tokens) - 1,) if e.wants_logits else ())
                   for e in plan]
        logits = self.runner.step(entries)
        self.h2d_bytes += self.runner.last_step.h2d_bytes
        sampled: List[int] = []
        if logits is not None:
            who = [e.request for e in plan if e.wants_logits]
            sampled = self.sampler.sample(logits, [r.options for r in who], [r.seed for r in who],
                                          [r.draws for r in who], [r.history for r in who])
            self.d2h_bytes += 4 * len(sampled)
        sched.update(plan, sampled)
        return sum(len(e.tokens) for e in plan)


def _load_tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.isfile(path):
        return None
    try:
        from tokenizers import Tokenizer
    except ImportError:
        return None
    return Tokenizer.from_file(path)
