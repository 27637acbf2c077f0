"""Choosing the next token from logits.

The chain of hostfog/hfee internal/llm/sampler.go:54-130: repeat penalty over the
recent history, argmax if the temperature is <= 0, else the top-k logits in
descending order, probabilities ``exp((l - l_max)/T)`` in float64, top-p and min-p
cuts, and a draw ``r = U * total`` that walks the kept candidates.  The uniform
number U comes from a counter-based generator keyed by (seed, draw index), so a
request's draws do not depend on what else is in the batch or on preemption.

Greedy and plain temperature sampling run in a device kernel over the whole batch.  The
whole chain runs on the device too when every row's top-k is at most 64 and its penalty looks
at no more than 256 recent tokens (the reference's defaults are 40 and 64): the recent tokens
of each request are kept in a ring on the device, so generation stays pipelined.  Other options
take the same logits through the host chain.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .options import SamplingOptions

_MASK = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def uniform(seed: int, stream: int, counter: int) -> float:
    """Uniform in [0, 1) from (seed, stream, counter); the same function as
    ``hfee_uniform`` in csrc/common.cuh."""
    h = _mix64(_mix64(_mix64(seed & _MASK) ^ (stream & _MASK)) ^ (counter & _MASK))
    return (h >> 11) * (1.0 / 9007199254740992.0)


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(7), "little")


def apply_repeat_penalty(logits: np.ndarray, history: Sequence[int], opts: SamplingOptions) -> None:
    """In place, sampler.go:57-74: each distinct recent id once; positive logits are
    divided by the penalty, the others multiplied."""
    if not opts.penalises:
        return
    recent = history
    if opts.repeat_last_n > 0 and len(recent) > opts.repeat_last_n:
        recent = recent[len(recent) - opts.repeat_last_n:]
    for tok in set(int(t) for t in recent):
        if tok >= logits.shape[0]:
            continue
        if logits[tok] > 0:
            logits[tok] /= np.float32(opts.repeat_penalty)
        else:
            logits[tok] *= np.float32(opts.repeat_penalty)


def sample_host(logits: np.ndarray, history: Sequence[int], opts: SamplingOptions, u: float) -> int:
    """The whole chain on the host for one row of float32 logits."""
    logits = np.array(logits, dtype=np.float32, copy=True)
    apply_repeat_penalty(logits, history, opts)
    if opts.temperature <= 0:
        return int(np.argmax(logits))               # first maximum, sampler.go:77-83
    k = opts.top_k if 0 < opts.top_k <= logits.shape[0] else logits.shape[0]
    # descending logits, equal logits by ascending id (the reference's sort leaves ties in no
    # particular order; the device kernels use this one)
    if k < logits.shape[0]:
        kth = np.partition(logits, logits.shape[0] - k)[logits.shape[0] - k]      # the k-th largest value
        idx = np.nonzero(logits >= kth)[0]
        idx = idx[np.argsort(-logits[idx], kind="stable")][:k]
    else:
        idx = np.argsort(-logits, kind="stable")
    cand = logits[idx]
    probs = np.exp(((cand - cand[0]) / np.float32(opts.temperature)).astype(np.float64))
    probs /= probs.sum()
    keep = len(probs)
    if 0 < opts.top_p < 1:
        cum = np.cumsum(probs)
        hit = np.nonzero(cum >= float(np.float32(opts.top_p)))[0]
        if hit.size:
            keep = int(hit[0]) + 1
    if opts.min_p > 0:
        below = np.nonzero(probs[1:keep] < float(np.float32(opts.min_p)) * probs[0])[0]
        if below.size:
            keep = int(below[0]) + 1
    total = float(probs[:keep].sum())
    r = u * total
    for i in range(keep):
        r -= probs[i]
        if r <= 0:
            return int(idx[i])
    return int(idx[keep - 1])


class BatchSampler:
    """Samples one token for each row of a step's logits."""

    def __init__(self, device, max_rows: int):
        self.device = torch.device(device)
        self.max_rows = max_rows
        pin = self.device.type == "cuda"
        self.out = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.temp = torch.zeros(max_rows, dtype=torch.float32, device=self.device)
        self.unif = torch.zeros(max_rows, dtype=torch.float64, device=self.device)
        self.out_host = torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin)
        # two sets of result buffers so that a step's choice can be read back while the next is made
        self.outs = [torch.zeros(max_rows, dtype=torch.int32, device=self.device) for _ in range(2)]
        self.out_hosts = [torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.turn = 0
        self.argmax_scratch = torch.zeros(max_rows * ops.ARGMAX_CHUNKS * 2, dtype=torch.float32, device=self.device)
        # the device chain: per-row parameters (two pinned copies used in turn), candidates, history rings
        self.params = torch.zeros(max_rows, 8, dtype=torch.float64, device=self.device)
        self.params_host = [torch.zeros(max_rows, 8, dtype=torch.float64, pin_memory=pin) for _ in range(2)]
        self.temp_host = [torch.zeros(max_rows, dtype=torch.float32, pin_memory=pin) for _ in range(2)]
        self.unif_host = [torch.zeros(max_rows, dtype=torch.float64, pin_memory=pin) for _ in range(2)]
        self.chain_scratch: Optional[torch.Tensor] = None
        self.use_device_chain = True          # False: truncating or penalising options always go through the host chain
        self.history = torch.zeros(max_rows, ops.CHAIN_HISTORY, dtype=torch.int32, device=self.device)
        self.history_len = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        # the same for the unpipelined path, where the host rewrites the rings before every draw
        self.row_history = torch.zeros(max_rows, ops.CHAIN_HISTORY, dtype=torch.int32, device=self.device)
        self.row_history_len = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.rows = torch.arange(max_rows, dtype=torch.int32, device=self.device)
        # pinned staging for the rings of requests that start (or come back after a preemption)
        self.ring_host = [torch.zeros(ops.CHAIN_HISTORY + 1, dtype=torch.int32, pin_memory=pin) for _ in range(4)]
        self.ring_events = [None] * 4
        self.ring_turn = 0

    @staticmethod
    def _chain_params(o: SamplingOptions, u: float) -> List[float]:
        """A row of parameters for the device chain; top-p, min-p and the penalty rounded to float32 as
        the reference holds them."""
        return [max(o.temperature, 0.0), o.top_k, float(np.float32(o.top_p)), float(np.float32(o.min_p)),
                float(np.float32(o.repeat_penalty)) if o.penalises else 1.0, o.repeat_last_n if o.penalises else 0, u, 0.0]

    def _chain_scratch(self, vocab: int) -> torch.Tensor:
        need = ops.chain_scratch_floats(self.max_rows, vocab)
        if self.chain_scratch is None or self.chain_scratch.numel() < need:
            self.chain_scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        return self.chain_scratch

    def chain_takes(self, vocab: int) -> bool:
        """Whether the device chain can run over a vocabulary of this size."""
        return self.use_device_chain and vocab <= ops.CHAIN_MAX_VOCAB

    def load_history(self, slot: int, tokens: Sequence[int]) -> None:
        """Start the ring of recent tokens of the request in ``slot`` from its tokens so far.  The
        tokens and their count go through pinned staging rows used in turn, so the host does not
        wait for the GPU (this runs in the steps that are meant to run ahead of it)."""
        tail = np.asarray(tokens[-ops.CHAIN_HISTORY:], dtype=np.int32)
        i = self.ring_turn
        self.ring_turn = (i + 1) % len(self.ring_host)
        if self.ring_events[i] is not None:
            self.ring_events[i].synchronize()            # that staging row's last upload is done
        host = self.ring_host[i]
        host[:len(tail)] = torch.from_numpy(tail)
        host[ops.CHAIN_HISTORY] = len(tail)
        self.history[slot].copy_(host[:ops.CHAIN_HISTORY], non_blocking=True)
        self.history_len[slot:slot + 1].copy_(host[ops.CHAIN_HISTORY:], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.ring_events[i] = ev

    def sample(self, logits: torch.Tensor, options: Sequence[SamplingOptions], seeds: Sequence[int],
               draws: Sequence[int], histories: Sequence[Sequence[int]]) -> List[int]:
        """``logits`` [m, vocab] float32 on the device; per row its options, seed, index of
        this draw and token history (prompt + output).  Returns m token ids (host)."""
        m = logits.shape[0]
        assert m == len(options) <= self.max_rows
        us = [uniform(seeds[i], 0, draws[i]) if options[i].temperature > 0 else 0.0 for i in range(m)]
        if (self.chain_takes(logits.shape[1]) and self.device.type == "cuda" and not all(o.device_only for o in options)
                and all(o.device_chain for o in options)):
            # the whole chain on the device; the host knows every row's history here, so the rings of
            # recent tokens are simply written anew (rows stand in for request slots)
            cap = ops.CHAIN_HISTORY
            tails = [[int(t) for t in h[-cap:]] if o.penalises else [] for h, o in zip(histories, options)]
            ring = torch.zeros(m, cap, dtype=torch.int32)
            for i, t in enumerate(tails):
                if t:
                    ring[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
            self.row_history[:m].copy_(ring)
            self.row_history_len[:m].copy_(torch.tensor([len(t) for t in tails], dtype=torch.int32))
            self.params[:m].copy_(torch.tensor([self._chain_params(o, u) for o, u in zip(options, us)], dtype=torch.float64))
            ops.sample_chain(logits, self.params[:m], self.out[:m], self._chain_scratch(logits.shape[1]), self.rows[:m], None,
                             self.row_history, self.row_history_len, penalise=any(o.penalises for o in options))
            self.out_host[:m].copy_(self.out[:m])
            return [int(t) for t in self.out_host[:m]]
        if all(o.temperature <= 0 for o in options) and all(o.device_only for o in options):
            ops.argmax(logits, self.out[:m], self.argmax_scratch)
        else:
            self.temp[:m].copy_(torch.tensor([o.temperature if o.device_only else 0.0 for o in options],
                                             dtype=torch.float32))
            self.unif[:m].copy_(torch.tensor(us, dtype=torch.float64))
            ops.sample(logits, self.out[:m], self.temp[:m], self.unif[:m])
        self.out_host[:m].copy_(self.out[:m])          # device -> host, synchronises
        tokens = [int(t) for t in self.out_host[:m]]
        for i, o in enumerate(options):
            if not o.device_only:
                row = logits[i].cpu().numpy()
                tokens[i] = sample_host(row, histories[i], o, us[i])
        return tokens

    # -- pipelined use: launch now, read the result one step later -------------------------------
    def launch(self, logits: torch.Tensor, options: Sequence[SamplingOptions], seeds: Sequence[int],
               draws: Sequence[int], slots: torch.Tensor, feedback: torch.Tensor):
        """Start choosing a token for each row on the device (options must all be ``device_only``
        or all ``device_chain``): the choices go to ``feedback[slots[r]]`` for the next step and, asynchronously, to pinned
        host memory.  Returns a handle for :meth:`fetch`."""
        m = logits.shape[0]
        assert m == len(options) <= self.max_rows
        simple = all(o.device_only for o in options)
        assert simple or all(o.device_chain for o in options)
        b = self.turn
        self.turn ^= 1
        out = self.outs[b][:m]
        if not simple:
            host = self.params_host[b]
            host.numpy()[:m] = [self._chain_params(o, uniform(seeds[i], 0, draws[i]) if o.temperature > 0 else 0.0)
                                for i, o in enumerate(options)]
            self.params[:m].copy_(host[:m], non_blocking=True)
            ops.sample_chain(logits, self.params[:m], out, self._chain_scratch(logits.shape[1]), slots, feedback, self.history,
                             self.history_len, penalise=any(o.penalises for o in options))
        elif all(o.temperature <= 0 for o in options):
            ops.argmax(logits, out, self.argmax_scratch, slots, feedback)
        else:
            us = [uniform(seeds[i], 0, draws[i]) if options[i].temperature > 0 else 0.0 for i in range(m)]
            self.temp_host[b][:m] = torch.tensor([o.temperature for o in options], dtype=torch.float32)
            self.unif_host[b][:m] = torch.tensor(us, dtype=torch.float64)
            self.temp[:m].copy_(self.temp_host[b][:m], non_blocking=True)        # pinned: the host does not wait
            self.unif[:m].copy_(self.unif_host[b][:m], non_blocking=True)
            ops.sample(logits, out, self.temp[:m], self.unif[:m], slots, feedback)
        self.out_hosts[b][:m].copy_(out, non_blocking=True)
        event = torch.cuda.Event() if self.device.type == "cuda" else None
        if event is not None:
            event.record()
        return b, m, event

    def fetch(self, handle) -> List[int]:
        """The tokens of a :meth:`launch` (waits for that step, not for later ones)."""
        b, m, event = handle
        if event is not None:
            event.synchronize()
        return self.out_hosts[b][:m].tolist()
