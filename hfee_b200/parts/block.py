"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Any

import torch

from .base import Part, register_part


class PreNormBlock(Part):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))`` on the float32 residual
    stream (hostfog/hfee internal/llm/forward.go:82-114).  Built by the model with
    its four parts already constructed."""
    category = "block"

    def __init__(self, spec, tensors, rt, mixer=None, feed_forward=None, mixer_norm=None, ffn_norm=None):
        super().__init__(spec, tensors, rt)
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.width = int(spec.width)

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        xn = self.rt.scratch("block_normed", (self.rt.max_tokens, self.width))[:step.n]
        self.mixer_norm.forward(residual, xn)
        self.mixer.forward(xn, residual, step, cache, writes_cache)
        self.ffn_norm.forward(residual, xn)
        self.feed_forward.forward(xn, residual, step)


register_part("block", "pre_norm", PreNormBlock)
