"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` added to the residual
stream (hostfog/hfee internal/llm/forward.go:110-114, internal/ggml/ops.go:160-165)."""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class SwiGLUFeedForward(Part):
    """spec: ``width``, ``inner`` (intermediate size)."""
    category = "feed_forward"

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"gate": TensorNeed((spec.inner, spec.width)), "up": TensorNeed((spec.inner, spec.width)),
                "down": TensorNeed((spec.width, spec.inner))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.inner = int(spec.inner)
        # one fused projection: rows [gate | up]
        self.w_gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.w_down = tensors["down"]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step: Any) -> None:
        n, rt = step.n, self.rt
        gu = rt.scratch("ffn_gate_up", (rt.max_tokens, 2 * self.inner))[:n]
        ops.linear(xn, self.w_gate_up, gu)
        h = rt.scratch("ffn_hidden", (rt.max_tokens, self.inner))[:n]
        ops.swiglu(gu, h)
        ops.linear(h, self.w_down, residual, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
