"""A decoder assembled from a :class:`~hfee_b200.config.ModelSpec`.

Builds every part the spec names, hands each the tensors it asked for (looked up
by the checkpoint names the architecture mapped them to), and runs the layers in
the order the spec's schedule lists.  The sequence of calls mirrors
hostfog/hfee internal/llm/forward.go:75-141: embedding, layers, final norm on the
rows whose logits are wanted, head.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ..config.spec import LayerSpec, ModelSpec, PartSpec, check_schedule
from ..weights.loader import Checkpoint, TensorNeed
from .base import Runtime, build_part, part_class
from .norm import LazyNormed


def _named(needs: Mapping[str, TensorNeed], prefix: str, names: Mapping[str, str], where: str) -> Dict[str, Tuple[str, TensorNeed]]:
    out = {}
    for key, need in needs.items():
        local = f"{prefix}.{key}"
        if local not in names:
            if need.optional:       # an architecture that never stores an optional tensor gives it no name
                continue
            raise ValueError(f"{where}: the architecture gives no checkpoint name for tensor {local!r}")
        out[local] = (names[local], need)
    return out


def _collect(spec: ModelSpec) -> Tuple[Dict[str, Tuple[str, TensorNeed]], List[Dict[str, Tuple[str, TensorNeed]]]]:
    """(model-level, per-layer) maps: local key -> (checkpoint name, need)."""
    top: Dict[str, Tuple[str, TensorNeed]] = {}
    top.update(_named(part_class("embedding", spec.embedding.kind).tensor_needs(spec.embedding), "embedding", spec.names, "model"))
    top.update(_named(part_class("norm", spec.final_norm.kind).tensor_needs(spec.final_norm), "final_norm", spec.names, "model"))
    top.update(_named(part_class("head", spec.head.kind).tensor_needs(spec.head), "head", spec.names, "model"))
    layers = []
    for i, layer in enumerate(spec.layers):
        m: Dict[str, Tuple[str, TensorNeed]] = {}
        for prefix, (cat, ps) in layer.parts.items():
            m.update(_named(part_class(cat, ps.kind).tensor_needs(ps), prefix, layer.names, f"layer {i}"))
        layers.append(m)
    return top, layers


def model_tensor_needs(spec: ModelSpec) -> Dict[str, TensorNeed]:
    """Checkpoint name -> need, for every tensor any part of the model asks for."""
    top, layers = _collect(spec)
    out: Dict[str, TensorNeed] = {}
    for m in [top] + layers:
        for name, need in m.values():
            if name in out and out[name] != need:
                raise ValueError(f"tensor {name} is asked for twice with different shapes or roles")
            out[name] = need
    return out


class DecoderModel:
    def __init__(self, spec: ModelSpec, checkpoint: Checkpoint, rt: Runtime):
        check_schedule(spec.layers, spec.schedule)
        self.spec, self.rt = spec, rt
        checkpoint.check(model_tensor_needs(spec), spec.ignorable)
        top, layers = _collect(spec)

        def fetch(m: Mapping[str, Tuple[str, TensorNeed]], prefix: str) -> Dict[str, torch.Tensor]:
            out = {}
            for local, (name, need) in m.items():
                if local.startswith(prefix + ".") and checkpoint.has(name):
                    out[local[len(prefix) + 1:]] = checkpoint.fetch(name, need, rt.dtype, rt.device)
            return out

        self.embedding = build_part("embedding", spec.embedding, fetch(top, "embedding"), rt)
        self.final_norm = build_part("norm", spec.final_norm, fetch(top, "final_norm"), rt)
        self.head = part_class("head", spec.head.kind)(spec.head, fetch(top, "head"), rt, embedding=self.embedding)
        self.blocks = []
        for layer, m in zip(spec.layers, layers):
            parts = {prefix: build_part(cat, ps, fetch(m, prefix), rt) for prefix, (cat, ps) in layer.parts.items()}
            self.blocks.append(part_class("block", layer.block.kind)(layer.block, {}, rt, parts=parts))
        self.width, self.vocab = spec.width, spec.vocab
        # decode steps may be captured in CUDA graphs only if every part of the schedule allows it
        self.graph_safe = (self.embedding.graph_safe and self.final_norm.graph_safe and self.head.graph_safe
                           and all(self.blocks[run.layer].all_graph_safe for run in spec.schedule))

    def cache_needs(self) -> Dict[int, Any]:
        """cache id -> what the writing run's mixer needs (PagedKV, FixedState or None)."""
        out: Dict[int, Any] = {}
        for run in self.spec.schedule:
            need = self.blocks[run.layer].cache_need()
            if run.writes_cache:
                out[run.cache] = need
            elif out.get(run.cache) != need:
                raise ValueError(f"layer {run.layer} reads cache {run.cache}, whose layout {out.get(run.cache)} "
                                 f"differs from what it needs ({need})")
        return out

    def forward(self, step: Any, caches: Mapping[int, Any]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every scheduled layer; returns float32 logits
        [len(step.logit_rows), vocab] (None if no logits are wanted)."""
        if self.rt.device.type != "cuda":
            return self._forward(step, caches)
        from ..kernels import ops
        with ops.stream_held():          # one stream for the whole pass, looked up once
            return self._forward(step, caches)

    def _forward(self, step: Any, caches: Mapping[int, Any]) -> Optional[torch.Tensor]:
        rt = self.rt
        residual = rt.scratch("residual", (rt.max_tokens, self.width), torch.float32)[:step.n]
        self.embedding.forward(step, residual)
        for run in self.spec.schedule:
            self.blocks[run.layer].forward(residual, step, caches.get(run.cache), run.writes_cache)
        m = step.n_logits
        if m == 0:
            return None
        xn = rt.scratch("head_normed", (rt.max_tokens, self.width))[:m]
        lazy = LazyNormed(self.final_norm, residual, xn, rows=step.logit_rows)
        logits = rt.scratch("logits", (step.logits_capacity, self.vocab), torch.float32)[:m]
        self.head.forward(lazy if getattr(self.head, "accepts_lazy_input", False) else lazy.tensor(), logits)
        return logits
