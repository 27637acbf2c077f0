"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Any

import torch

from .base import Block, register_part
from .norm import LazyNormed


class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` on the float32 residual
    stream (hostfog/hfee internal/llm/forward.go:82-114).  Built by the model with
    its four parts already constructed."""
    needs = ("mixer", "ffn", "mixer_norm", "ffn_norm")
    graph_safe = True

    def __init__(self, spec, tensors, rt, parts):
        super().__init__(spec, tensors, rt, parts)
        self.mixer, self.feed_forward = parts["mixer"], parts["ffn"]
        self.mixer_norm, self.ffn_norm = parts["mixer_norm"], parts["ffn_norm"]
        self.width = int(spec.width)

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        xn = self.rt.scratch("block_normed", (self.rt.max_tokens, self.width))[:step.n]
        self.mixer.forward(self._normed(self.mixer, self.mixer_norm, residual, xn), residual, step, cache, writes_cache)
        self.feed_forward.forward(self._normed(self.feed_forward, self.ffn_norm, residual, xn), residual, step)

    @staticmethod
    def _normed(consumer, norm, residual, buffer):
        """The consumer's input: a lazily normed one if it says it can take it (and may fuse the
        norm into its first product), else the normed tensor."""
        lazy = LazyNormed(norm, residual, buffer)
        return lazy if getattr(consumer, "accepts_lazy_input", False) else lazy.tensor()


register_part("block", "pre_norm", PreNormBlock)
