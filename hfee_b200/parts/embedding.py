"""Token embedding and the output head."""
from __future__ import annotations

from typing import Any, Dict

import torch

from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Part, register_part


class TokenEmbedding(Part):
    """``x[i,:] = table[token_i,:]``, unscaled (hostfog/hfee internal/llm/forward.go:75-77).
    spec: ``vocab``, ``width``."""
    category = "embedding"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {"table": TensorNeed((spec.vocab, spec.width), role="table")}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.table = tensors["table"]

    def forward(self, step: Any, residual: torch.Tensor) -> None:
        ops.tag("embed")
        ops.embed(self.table, step.token_ids, residual, step.slot_of_token, getattr(step, "feedback", None))


class LinearHead(Part):
    """``logits = x . W^T`` in float32 (internal/llm/forward.go:132-141).  spec: ``vocab``,
    ``width``, ``tied`` (use the embedding table as W, internal/llm/model.go:118-121)."""
    category = "head"
    graph_safe = True

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        # tied: the checkpoint need not hold a head; if it does, that tensor is used, as the
        # reference uses output.weight whenever the file has one (internal/llm/model.go:118-121)
        return {"weight": TensorNeed((spec.vocab, spec.width), optional=bool(spec.get("tied", False)))}

    def __init__(self, spec, tensors, rt, embedding: TokenEmbedding = None):
        super().__init__(spec, tensors, rt)
        if "weight" in tensors:
            self.weight = tensors["weight"]
        elif spec.get("tied", False):
            if embedding is None:
                raise ValueError("a tied head needs the embedding part")
            self.weight = embedding.table
        else:
            raise ValueError("the head has no weight and is not tied to the embedding")

    accepts_lazy_input = True        # the final norm may be fused into the product

    def forward(self, xn, logits: torch.Tensor) -> None:
        if isinstance(xn, torch.Tensor):
            ops.tag("head")
            ops.linear(xn, self.weight, logits)
        else:
            ops.tag("head")
            ops.linear_normed(xn, self.weight, logits)


register_part("embedding", "token", TokenEmbedding)
register_part("head", "linear", LinearHead)
