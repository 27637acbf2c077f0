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
    graph_safe = True
    accepts_lazy_input = True        # the input norm may be fused into the gate/up projection

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"gate": TensorNeed((spec.inner, spec.width)), "up": TensorNeed((spec.inner, spec.width)),
                "down": TensorNeed((spec.width, spec.inner))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.inner = int(spec.inner)
        # one fused projection.  bfloat16: rows in groups of 4 gate rows then 4 up rows, so a
        # kernel that owns 8 consecutive rows can apply SwiGLU in its epilogue; else [gate | up].
        gate, up = tensors["gate"], tensors["up"]
        g = ops.SWIGLU_GRANULE
        if gate.dtype == torch.bfloat16 and self.inner % g == 0:
            self.granule = g
            w = torch.stack([gate.reshape(self.inner // g, g, -1), up.reshape(self.inner // g, g, -1)], dim=1)
            self.w_gate_up = w.reshape(2 * self.inner, -1).contiguous()
        else:
            self.granule = self.inner
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors["down"]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step: Any) -> None:
        n, rt = step.n, self.rt
        gu = rt.scratch("ffn_gate_up", (rt.max_tokens, 2 * self.inner))[:n]
        h = rt.scratch("ffn_hidden", (rt.max_tokens, self.inner))[:n]
        ops.tag("gate_up")
        ops.linear_swiglu_normed(xn, self.w_gate_up, h, self.granule, gu)
        ops.tag("down")
        ops.linear(h, self.w_down, residual, accumulate=True)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
