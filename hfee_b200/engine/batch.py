"""One step's batch: (request, its next tokens) entries flattened for the device.

Counterpart of the flattening at the top of ``Model.Forward`` in hostfog/hfee
internal/llm/forward.go:55-64: token i belongs to a request and sits at position
(tokens already cached) + (its index in the entry).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepEntry:
    """``tokens`` are appended to the request in ``slot``; ``want`` lists the indices
    among these tokens whose logits are asked for (may be empty)."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepBuffers:
    """Device and pinned host staging for the integers a step needs, laid out
    compactly: token ids, positions, slot per token, logit rows, then per request
    cu_tokens, slot, context before and after."""

    RING = 4

    def __init__(self, max_tokens: int, max_requests: int, device):
        self.max_tokens, self.max_requests = max_tokens, max_requests
        self.capacity = 5 * max_tokens + 4 * max_requests + 8
        self.device = torch.device(device)
        self.dev = torch.zeros(self.capacity, dtype=torch.int32, device=self.device)
        pin = self.device.type == "cuda"
        self.host = [torch.zeros(self.capacity, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.turn = 0

    def upload(self, packed: np.ndarray) -> int:
        """Copy ``packed`` (int32) to the start of the device buffer; returns the bytes copied."""
        i = self.turn
        self.turn = (i + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        n = packed.size
        self.host[i][:n] = torch.from_numpy(packed)
        self.dev[:n].copy_(self.host[i][:n], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev
        return n * 4


class Step:
    """What the parts see of a step.

    Device int32 tensors: ``token_ids[n]``, ``positions[n]``, ``slot_of_token[n]``,
    ``logit_rows[n_logits]`` (flat token indices), ``logit_slots[n_logits]``, ``cu_tokens[r+1]``, ``slots[r]``,
    ``context_before[r]``, ``context_after[r]``.  Host: ``requests`` = list of
    (slot, first position, token count) in batch order; ``memo`` for work that parts
    share within the step (rotary tables); ``max_context`` = longest context after
    the step; ``decode_only`` = every entry is a single token.
    """

    def __init__(self, entries: Sequence[StepEntry], lengths: Sequence[int], buffers: StepBuffers):
        n = sum(len(e.tokens) for e in entries)
        r = len(entries)
        m = sum(len(e.want) for e in entries)
        if n > buffers.max_tokens:
            raise ValueError(f"step of {n} tokens exceeds the batch limit of {buffers.max_tokens}")
        if r > buffers.max_requests:
            raise ValueError(f"step of {r} requests exceeds the limit of {buffers.max_requests}")
        packed = np.empty(3 * n + 2 * m + 4 * r + 1, dtype=np.int32)
        tok, pos, slot = packed[0:n], packed[n:2 * n], packed[2 * n:3 * n]
        rows, row_slots = packed[3 * n:3 * n + m], packed[3 * n + m:3 * n + 2 * m]
        o = 3 * n + 2 * m
        cu, slots = packed[o:o + r + 1], packed[o + r + 1:o + 2 * r + 1]
        before, after = packed[o + 2 * r + 1:o + 3 * r + 1], packed[o + 3 * r + 1:o + 4 * r + 1]
        self.requests: List[Tuple[int, int, int]] = []
        at = w = 0
        cu[0] = 0
        for j, e in enumerate(entries):
            k = len(e.tokens)
            start = lengths[e.slot]
            tok[at:at + k] = np.asarray(e.tokens, dtype=np.int64)
            pos[at:at + k] = np.arange(start, start + k)
            slot[at:at + k] = e.slot
            for idx in e.want:
                if not 0 <= idx < k:
                    raise ValueError(f"entry {j}: wanted index {idx} is outside its {k} tokens")
                rows[w] = at + idx
                row_slots[w] = e.slot
                w += 1
            self.requests.append((e.slot, start, k))
            at += k
            cu[j + 1] = at
            slots[j], before[j], after[j] = e.slot, start, start + k
        self.n, self.r, self.n_logits = n, r, m
        self.h2d_bytes = buffers.upload(packed)
        d = buffers.dev
        self.token_ids, self.positions, self.slot_of_token = d[0:n], d[n:2 * n], d[2 * n:3 * n]
        self.logit_rows = d[3 * n:3 * n + m]
        self.logit_slots = d[3 * n + m:3 * n + 2 * m]       # request slot of each wanted row
        self.feedback = None        # int32 per slot: tokens sampled on the device (set by the runner)
        self.cu_tokens, self.slots = d[o:o + r + 1], d[o + r + 1:o + 2 * r + 1]
        self.context_before, self.context_after = d[o + 2 * r + 1:o + 3 * r + 1], d[o + 3 * r + 1:o + 4 * r + 1]
        self.max_context = max((s + k for _, s, k in self.requests), default=0)
        self.planning_context = self.max_context      # what launch heuristics (key splits) plan for
        self.max_new = max((k for _, _, k in self.requests), default=0)
        self.decode_only = all(k == 1 for _, _, k in self.requests)
        self.logits_capacity = max(buffers.max_requests, 1 << max(0, (m - 1)).bit_length())
        self.memo: Dict[Any, Any] = {}
