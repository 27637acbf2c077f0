"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Any

import torch

from ..kernels import ops
from .base import Block, register_part
from .norm import LazyNormed


def residual_dtype_is_not_compute(rt) -> bool:
    """The fused tail kernel is a bfloat16 kernel (the residual stream is float32 in both dtypes)."""
    return rt.dtype != torch.bfloat16


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
        mixer_in = self._normed(self.mixer, self.mixer_norm, residual, xn)
        if self._tail_in_one_kernel(step):
            # a decode step of a few tokens: the mixer's output projection, the second norm and the
            # feed-forward run as one kernel that streams all three weight matrices without a break
            heads_out = self.mixer.forward(mixer_in, residual, step, cache, writes_cache, project=False)
            weight, eps, add_unit = self.ffn_norm.fused_params()
            ffn = self.feed_forward
            ops.tag("tail")
            ops.decode_tail(heads_out, self.mixer.output_weight, residual, weight, eps, add_unit, ffn.w_gate_up,
                            ffn.w_down, ffn.hidden_scratch(step.n))
            return
        self.mixer.forward(mixer_in, residual, step, cache, writes_cache)
        self.feed_forward.forward(self._normed(self.feed_forward, self.ffn_norm, residual, xn), residual, step)

    def _tail_in_one_kernel(self, step: Any) -> bool:
        """True when the fused kernel takes this step: the parts are the kinds whose weights it reads
        (a mixer that ends in a linear projection, a gated feed-forward with its rows interleaved in
        fours, a norm that can hand out its parameters) and the sizes fit."""
        mixer, ffn = self.mixer, self.feed_forward
        w_o = getattr(mixer, "output_weight", None)
        if w_o is None or getattr(ffn, "granule", None) != ops.SWIGLU_GRANULE or not hasattr(ffn, "hidden_scratch"):
            return False
        if getattr(self.ffn_norm, "fused_params", None) is None or residual_dtype_is_not_compute(self.rt):
            return False
        if step.n < ops.DECODE_TAIL_MIN_TOKENS:      # one or two tokens: the products that norm their input themselves are faster
            return False
        return ops.decode_tail_takes(step.n, self.width, w_o.shape[1], ffn.inner, self.rt.dtype)

    @staticmethod
    def _normed(consumer, norm, residual, buffer):
        """The consumer's input: a lazily normed one if it says it can take it (and may fuse the
        norm into its first product), else the normed tensor."""
        lazy = LazyNormed(norm, residual, buffer)
        return lazy if getattr(consumer, "accepts_lazy_input", False) else lazy.tensor()


register_part("block", "pre_norm", PreNormBlock)
