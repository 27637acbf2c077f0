"""The step function: runs one batch of (request, next tokens) entries through the
model from the cache and returns the logits at the wanted places.

Counterpart of ``Model.Forward([]Batch)`` in hostfog/hfee
internal/llm/forward.go:51-142, where entries may be portions of prompts beside
single decoded tokens; here over a paged cache and returning logits at any wanted
token, not only the last.
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence

import torch

from ..cache import CacheManager, OutOfPages
from ..config import EngineConfig, resolve_model_dir
from ..parts import DecoderModel, Runtime
from ..weights import Checkpoint
from .batch import Step, StepBuffers, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
# A decode step is a chain of short kernels, and an SM changes its split between shared memory and L1
# only when it is empty: the kernels of such a step all ask for one split (percent of the shared-memory
# maximum).  Measured, benchmark model, ms per step against the driver's per-kernel choice: 58 % at
# batch 2 / 4 / 8 / 16: 0.752 / 0.806 / 0.833 / 1.043 against 0.761 / 0.818 / 0.861 / 1.064 (more
# shared memory than that starves the kernels that stream weights through L1: 100 % at batch 8 takes
# 1.135, at batch 16 1.46).  From 17 requests on the products run on tcgen05 with rings of 200 KB and the
# attention wants three CTAs of 76 KB per SM: 100 % at batch 17 / 20 / 24 / 40 / 48 / 64: 1.096 / 1.154 /
# 1.270 / 1.488 / 1.606 / 1.78 against 1.144 / 1.279 / 1.333 / 1.575 / 1.654 / 1.85 at 58 % (batch 32 and 36
# are within 1 % either way).  A prompt of 2,048 tokens: 4.29 ms at 58 % against 4.35.
STEP_CARVEOUT, DECODE_CARVEOUT_MANY, DECODE_MANY_REQUESTS = 58, 100, 17
# Steps of up to this many tokens are replayed from CUDA graphs once their shape has been seen twice: the
# host needs about 2 ms to launch a pass of a 16-layer model whatever its size, the GPU less than that
# below about 1,000 tokens.  At most GRAPH_LIMIT graphs are kept.
GRAPH_MAX_TOKENS, GRAPH_LIMIT = 1024, 64
DEVICE_TOKEN = -1        # as a single-token entry: "the token the device sampled last for this request"


class ModelRunner:
    """A loaded model with its cache: ``open()`` / ``step()`` / ``close()`` per request."""

    def __init__(self, model_dir: str, engine: Optional[EngineConfig] = None):
        self.engine = engine or EngineConfig()
        e = self.engine
        self.arch, self.config = resolve_model_dir(model_dir)
        self.spec = self.arch.build_spec(self.config)
        self.device = torch.device(e.device)
        self.rt = Runtime(_DTYPES[e.dtype], self.device, e.max_batch_tokens, e.max_requests, e.page_size)
        checkpoint = Checkpoint(model_dir)
        self.model = DecoderModel(self.spec, checkpoint, self.rt)
        checkpoint.files.close()
        self.cache = CacheManager(self.model.cache_needs(), e.page_size, e.num_pages, e.max_requests,
                                  e.max_context, self.rt.dtype, self.device)
        self.buffers = StepBuffers(e.max_batch_tokens, e.max_requests, self.device)
        self.vocab = self.spec.vocab
        # the token last sampled on the device for each request slot; a step may name it with
        # the token id DEVICE_TOKEN instead of a value the host has not read back yet
        self.feedback = torch.zeros(e.max_requests, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        # decode-only steps are captured in a CUDA graph per batch size: first sight runs
        # eagerly (and makes every scratch buffer), second sight captures, later ones replay
        self._graphs = {}
        self._graph_seen = set()
        self.graph_replays = 0

    # ------------------------------------------------------------------ requests
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Append each entry's tokens to its request and return float32 logits
        [sum(len(e.want)), vocab] on the device in the order of the entries and of
        ``want`` (None if nothing is wanted).  Raises :class:`OutOfPages`, before
        anything ran, if the cache cannot hold the new tokens."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        cache = self.cache
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            lo, hi = min(e.tokens), max(e.tokens)
            if lo == DEVICE_TOKEN and len(e.tokens) == 1:
                lo = 0
            if lo < 0 or hi >= self.vocab:
                raise ValueError(f"token id {lo if lo < 0 else hi} is outside the vocabulary of {self.vocab}")
            if cache.length[e.slot] + len(e.tokens) > cache.max_context:
                raise ValueError(f"slot {e.slot}: {cache.length[e.slot] + len(e.tokens)} tokens exceed the "
                                 f"context limit of {cache.max_context}")
        # all or nothing: check every group's free pages against the whole step's demand
        for g in cache.paged:
            need = sum(cache._missing(g, e.slot, cache.length[e.slot] + len(e.tokens)) for e in entries)
            if need > g.pool.free_pages:
                raise OutOfPages(f"step needs {need} pages, {g.pool.free_pages} are free")
        for e in entries:
            cache.reserve(e.slot, cache.length[e.slot] + len(e.tokens))
        cache.sync()
        step = Step(entries, cache.length, self.buffers)
        step.feedback = self.feedback
        if self.device.type == "cuda":
            # in effect until the next step: what runs between steps (sampling) belongs to the chain too
            from ..kernels import ops
            ops.set_carveout(DECODE_CARVEOUT_MANY if step.decode_only and step.r >= DECODE_MANY_REQUESTS
                             else STEP_CARVEOUT)
        key = self._graph_key(step, entries)
        if key is not None:
            logits = self._graphed_forward(step, key)
        else:
            logits = self.model.forward(step, cache.views())
        for e in entries:
            cache.commit(e.slot, cache.length[e.slot] + len(e.tokens))
        self.steps_run += 1
        self.last_step = step
        return logits

    def _graph_key(self, step: Step, entries: Sequence[StepEntry]):
        """What a captured step can be replayed for, or None for a step that runs eagerly.  Everything
        the kernels of a graph-safe model read of a step lies in device buffers whose addresses depend
        only on the numbers of tokens, requests and wanted rows; what the launches themselves depend on
        (grids, the choice of kernels) follows from the token count of each request.  Decode-only steps
        that want every request's logits are keyed by their batch size; other steps of at most
        GRAPH_MAX_TOKENS tokens (prompt portions under a token budget, alone or beside decoded tokens,
        which the host cannot launch as fast as the GPU runs them) by the counts in batch order."""
        if not (self.engine.use_cuda_graphs and self.model.graph_safe and self.device.type == "cuda"):
            return None
        if step.decode_only and all(tuple(e.want) == (0,) for e in entries):
            return step.r
        if step.n <= GRAPH_MAX_TOKENS:
            return (tuple(len(e.tokens) for e in entries), step.n_logits)
        return None

    def _graphed_forward(self, step: Step, key) -> torch.Tensor:
        """A step through a CUDA graph.  The step's integers
        live at the same device addresses for every step of that key and are copied in before the
        replay, block tables likewise; launch parameters that depend on context lengths are planned
        for the longest context the engine allows."""
        from ..kernels import ops
        step.planning_context = self.cache.max_context
        hit = self._graphs.get(key)
        if hit is None:
            if key not in self._graph_seen:
                self._graph_seen.add(key)
                return self.model.forward(step, self.cache.views())
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph):
                out = self.model.forward(step, self.cache.views())
            while len(self._graphs) >= GRAPH_LIMIT:          # oldest first
                self._graphs.pop(next(iter(self._graphs)))
            hit = self._graphs[key] = (graph, out, ops.launch_count() - before)
        graph, out, kernels = hit
        graph.replay()
        ops.count_launches(kernels)
        self.graph_replays += 1
        return out
