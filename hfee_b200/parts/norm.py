"""RMS norm part.  Formula of hostfog/hfee internal/ggml/ops.go:125-134:
``dst = x * 1/sqrt(mean(x^2) + eps) * weight`` per row, with the sum in float32
here (float64 in the reference)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class RMSNorm(Part):
    """spec: ``width``, ``eps``, ``add_unit`` (scale by 1+w instead of w; default False)."""
    category = "norm"

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((spec.width,), role="scale")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.weight = tensors["weight"]
        self.eps = float(spec.eps)
        self.add_unit = bool(spec.get("add_unit", False))

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, out, self.eps, rows=rows, add_unit=self.add_unit)


register_part("norm", "rms_norm", RMSNorm)
