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
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"weight": TensorNeed((spec.width,), role="scale")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.weight = tensors["weight"]
        self.eps = float(spec.eps)
        self.add_unit = bool(spec.get("add_unit", False))

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        before = ops.tag("norm")
        ops.rmsnorm(x, self.weight, out, self.eps, rows=rows, add_unit=self.add_unit)
        ops.tag(before)


    def fused_params(self):
        """(weight, eps, add_unit): what a kernel needs to apply this norm itself."""
        return self.weight, self.eps, self.add_unit


class LazyNormed:
    """The normed input of a mixer, feed-forward or head that has not been computed yet.

    A part that can fuse the norm into its first matrix product hands this object to
    ``ops.linear_normed``; any other use calls :meth:`tensor`, which runs the norm once into
    ``buffer`` and returns it.  ``rows`` gathers source rows (the head norms only the rows whose
    logits are wanted)."""

    def __init__(self, norm, source: torch.Tensor, buffer: torch.Tensor, rows: Optional[torch.Tensor] = None):
        self.norm, self.source, self.buffer, self.rows = norm, source, buffer, rows
        self.n = buffer.shape[0]
        self.out_dtype = buffer.dtype
        self._done = False

    def fused_params(self):
        f = getattr(self.norm, "fused_params", None)
        return f() if f is not None else None

    def tensor(self) -> torch.Tensor:
        if not self._done:
            self.norm.forward(self.source, self.buffer, rows=self.rows)
            self._done = True
        return self.buffer


register_part("norm", "rms_norm", RMSNorm)
