"""Rotary position encoding part.

``invFreq[i] = 1 / theta^(2i/rope_dim)``, optionally divided per frequency
(hostfog/hfee internal/llm/model.go:150-158); the angle ``pos * invFreq[i]`` and its
sine and cosine are evaluated in float64 (internal/llm/forward.go:185-186) once per
step for the step's positions and shared by every layer with equal parameters.
"""
from __future__ import annotations

from typing import Any, List, Optional

import torch

from ..config.llama import RopeScaling
from ..config.spec import PartSpec
from ..kernels import ops
from .base import Part, register_part


def inverse_frequencies(rope_dim: int, theta: float, scaling: Optional[RopeScaling]) -> List[float]:
    inv = [1.0 / (theta ** (2.0 * i / rope_dim)) for i in range(rope_dim // 2)]
    return scaling.apply(inv) if scaling is not None else inv


class Rotary(Part):
    """spec: ``head_dim``, ``rope_dim`` (<= head_dim, even), ``theta``, ``scaling``
    (a RopeScaling or None) and ``pairing``: ``"half"`` rotates (i, i+rope_dim/2),
    ``"interleaved"`` rotates (2i, 2i+1) as internal/llm/forward.go:187-190 does."""
    category = "position"
    graph_safe = True

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.rope_dim = int(spec.get("rope_dim", spec.head_dim))
        if self.rope_dim % 2 or not 0 < self.rope_dim <= spec.head_dim:
            raise ValueError(f"rope_dim {self.rope_dim} must be even and within head_dim {spec.head_dim}")
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {spec.pairing!r}")
        self.interleaved = spec.pairing == "interleaved"
        scaling = spec.get("scaling")
        self.inv_freq_host = inverse_frequencies(self.rope_dim, float(spec.theta), scaling)
        self.inv_freq = torch.tensor(self.inv_freq_host, dtype=torch.float64, device=rt.device)
        self._key = ("rotary", spec)
        self._table = rt.scratch(f"rope_table_{abs(hash(spec)) & 0xffffffff:x}",
                                 (rt.max_tokens, self.rope_dim // 2, 2), torch.float32)

    def table(self, step: Any) -> torch.Tensor:
        """(cos, sin) for each token of the step, [n, rope_dim/2, 2] float32."""
        t = step.memo.get(self._key)
        if t is None:
            t = self._table[:step.n]
            ops.tag("rope")
            ops.rope_table(step.positions, self.inv_freq, t)
            step.memo[self._key] = t
        return t


class NoPosition(Part):
    """No position encoding: queries and keys are cached as projected."""
    category = "position"
    graph_safe = True
    rope_dim = 0
    interleaved = False

    def table(self, step: Any) -> None:
        return None


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
