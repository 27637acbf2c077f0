"""Interfaces of the parts a model is assembled from, and the registry of kinds.

A part is built from a :class:`~hfee_b200.config.PartSpec` (its sizes and
constants), the tensors it asked for and a :class:`Runtime`.  No part knows which
model it is in: tensor names are mapped by the architecture, the cache is handed in
per call, and the batch is described by the step object alone.

Categories and what each must provide:

``norm``          ``forward(x_f32[n,w], out[n,w], rows=None)``
``position``      ``table(step)`` -> per-step device data for the mixer (or None)
``mixer``         ``cache_need()`` and ``forward(xn[n,w], residual_f32[n,w], step, cache, writes_cache)``
                  (adds its output into ``residual``)
``feed_forward``  ``forward(xn[n,w], residual_f32[n,w], step)`` (adds into ``residual``)
``block``         ``forward(residual_f32[n,w], step, cache, writes_cache)``, arranging the above; it is
                  built with ``parts={key: part}`` for the keys its layer spec names
``embedding``     ``forward(step, residual_f32[n,w])``
``head``          ``forward(xn[m,w], logits_f32[m,vocab])``

Every part class has ``tensor_needs(spec) -> {local key: TensorNeed}`` and the flag
``graph_safe``: True says that ``forward`` launches the same kernels on the same buffers for every
decode-only step of a given batch size and takes everything that changes from step to step (slots,
positions, lengths, block tables) from device memory, so such a step may be captured in a CUDA
graph and replayed.  A part that reads the step's host-side lists leaves it False, and a model
with such a part always runs eagerly.
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Tuple, Type

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorNeed

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block", "embedding", "head")
_PARTS: Dict[Tuple[str, str], Type["Part"]] = {}


def register_part(category: str, kind: str, cls: Type["Part"]) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    _PARTS[(category, kind)] = cls


def part_class(category: str, kind: str) -> Type["Part"]:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise ValueError(f"no {category} of kind {kind!r} is registered (known: {known})") from None


class Runtime:
    """What parts share at run time: compute dtype, device, batch limits and named
    scratch buffers that live as long as the engine (stable addresses, so steps can
    be captured in CUDA graphs)."""

    def __init__(self, dtype: torch.dtype, device, max_tokens: int, max_requests: int, page_size: int):
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_tokens = max_tokens
        self.max_requests = max_requests
        self.page_size = page_size
        self._scratch: Dict[str, torch.Tensor] = {}

    def scratch(self, key: str, shape: Tuple[int, ...], dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The buffer named ``key``, made on first use.  Parts that use the same key,
        shape and dtype share it (activations of different layers never live at once)."""
        dtype = dtype or self.dtype
        t = self._scratch.get(key)
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            if t is not None:
                key = f"{key}#{'x'.join(map(str, shape))}#{dtype}"
                t = self._scratch.get(key)
            if t is None:
                t = torch.empty(shape, dtype=dtype, device=self.device)
                self._scratch[key] = t
        return t

    def scratch_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._scratch.values())


class Part:
    category: str = ""
    graph_safe: bool = False

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        return {}

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt


class Mixer(Part):
    category = "mixer"

    def cache_need(self):
        """A :class:`~hfee_b200.cache.PagedKV`, a :class:`~hfee_b200.cache.FixedState` or None."""
        return None

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        raise NotImplementedError


class Block(Part):
    """Arrangement of a layer's parts.  ``needs`` lists the keys it asks of ``LayerSpec.parts``;
    the model builds those parts and hands them over as ``parts``."""
    category = "block"
    needs: Tuple[str, ...] = ()

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], rt: Runtime, parts: Mapping[str, Part]):
        super().__init__(spec, tensors, rt)
        missing = [k for k in self.needs if k not in parts]
        if missing:
            raise ValueError(f"block {spec.kind!r} needs the parts {list(self.needs)}; the layer gives no {missing}")
        self.parts = dict(parts)

    def cache_need(self):
        """What the layer caches per request: its mixer's need, if it has a part called ``mixer``."""
        mixer = self.parts.get("mixer")
        return mixer.cache_need() if mixer is not None else None

    @property
    def all_graph_safe(self) -> bool:
        return bool(self.graph_safe) and all(p.graph_safe for p in self.parts.values())

    def forward(self, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        raise NotImplementedError


def build_part(category: str, spec: PartSpec, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> Part:
    return part_class(category, spec.kind)(spec, tensors, rt)
