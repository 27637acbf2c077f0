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

    def __init__(self, model_dir: str, engine: Optional[EngineConfig] = None, **settings: Any):
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
        self.tokenizer = _load_tokenizer(model_dir)
        self.pipeline = True          # overlap host work with the GPU where the sampling options allow it
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._next_id = 0

    # ------------------------------------------------------------------ text
    def encode(self, text: str) -> List[int]:
        if self.tokenizer is None:
            raise RuntimeError(f"{self.model_dir} has no tokenizer.json (or the tokenizers package is missing): "
                               "pass token ids")
        ids = self.tokenizer.encode(text, add_special_tokens=False).ids
        bos = self.runner.spec.bos_token_id
        return ([bos] if bos is not None else []) + ids        # Encode(prompt, addSpecial=true), runner.go:94

    def decode(self, ids: Sequence[int]) -> Optional[str]:
        return None if self.tokenizer is None else self.tokenizer.decode(list(ids))

    # ------------------------------------------------------------------ generation
    def new_scheduler(self) -> Scheduler:
        return Scheduler(self.runner.cache, self.config.max_batch_tokens, self.config.prefill_chunk,
                         self.eos_token_ids)

    def generate(self, prompts: Union[Sequence[int], str, Sequence[Union[Sequence[int], str]]],
                 options: Union[SamplingOptions, Sequence[SamplingOptions], None] = None,
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Continue every prompt; returns one result per prompt, in order.
        ``on_token(prompt_index, token_id)`` is called for each new token as it is sampled."""
        if isinstance(prompts, str) or (len(prompts) > 0 and isinstance(prompts[0], int)):
            prompts = [prompts]
        if options is None:
            options = SamplingOptions()
        if isinstance(options, SamplingOptions):
            options = [options] * len(prompts)
        if len(options) != len(prompts):
            raise ValueError("one SamplingOptions per prompt (or one for all) is needed")
        sched = self.new_scheduler()
        requests = []
        for i, (p, o) in enumerate(zip(prompts, options)):
            ids = self.encode(p) if isinstance(p, str) else [int(t) for t in p]
            req = Request(id=i, prompt=ids, options=o)
            sched.add(req)
            requests.append(req)
        emitted = [0] * len(requests)
        cut = {}                     # request index -> text cut at its stop string

        def emit() -> None:
            if on_token is None:
                return
            for i, r in enumerate(requests):
                while emitted[i] < len(r.output) and r.output[emitted[i]] != DEVICE_TOKEN:
                    on_token(i, r.output[emitted[i]])
                    emitted[i] += 1

        # When every request samples on the device and nothing needs text, steps are pipelined:
        # the sampled tokens stay on the device for the next step and the host reads them one step
        # late, so planning and launching overlap the GPU's work.
        on_device = all(o.device_only for o in options) or all(o.device_chain for o in options)
        if self.pipeline and on_device and not any(o.stop for o in options):
            inflight = None
            while not sched.idle or inflight is not None:
                launched = self.launch_step(sched) if not sched.idle else None
                if inflight is not None:
                    pending, handle = inflight
                    if handle is not None:
                        tokens = self.sampler.fetch(handle)
                        self.d2h_bytes += 4 * len(tokens)
                        sched.resolve(pending, tokens)
                inflight = launched
                emit()
                sched.pop_finished()
            ops.check_status()
            return [GenerationResult(list(r.output), self.decode(r.output), r.stats) for r in requests]

        while not sched.idle:
            self.run_step(sched)
            for i, r in enumerate(requests):       # stop strings (text.go:41-78), when text is available
                if r.options.stop and self.tokenizer is not None and not r.finished and r.output:
                    text = self.decode(r.output)
                    hits = [text.find(s) for s in r.options.stop if s and s in text]
                    if hits:
                        cut[i] = text[:min(hits)]
                        sched.finish(r, FinishReason.STOP)
            emit()
            sched.pop_finished()
        ops.check_status()
        return [GenerationResult(list(r.output), cut.get(i, self.decode(r.output)), r.stats)
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
