"""Data that describes a model as an arrangement of parts.

A model is a :class:`ModelSpec`: the embedding, a list of :class:`LayerSpec`
(each naming its mixer, feed-forward, norms and block arrangement by *kind* with
the sizes and constants as parameters), the order in which layers run
(:class:`RunSpec` list) and the head.  Nothing here knows an architecture; an
architecture is a function from its typed config to a ``ModelSpec``
(``hfee_b200.config.registry``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence, Tuple


class PartSpec:
    """``kind`` plus free-form parameters, e.g. ``PartSpec("rms_norm", width=64, eps=1e-5)``.

    Immutable and hashable so equal specs can share per-step work (one rotary
    table for every layer that uses the same rotary parameters)."""

    __slots__ = ("kind", "_params", "_key")

    def __init__(self, kind: str, **params: Any):
        object.__setattr__(self, "kind", kind)
        object.__setattr__(self, "_params", dict(params))
        object.__setattr__(self, "_key", (kind, _freeze(params)))

    def __setattr__(self, *_):
        raise AttributeError("PartSpec is immutable")

    def __getattr__(self, name: str) -> Any:
        try:
            return object.__getattribute__(self, "_params")[name]
        except KeyError:
            raise AttributeError(f"{self.kind} spec has no parameter {name!r}") from None

    def get(self, name: str, default: Any = None) -> Any:
        return self._params.get(name, default)

    @property
    def params(self) -> Mapping[str, Any]:
        return dict(self._params)

    def replace(self, **changes: Any) -> "PartSpec":
        p = dict(self._params)
        p.update(changes)
        return PartSpec(self.kind, **p)

    def __hash__(self) -> int:
        return hash(self._key)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, PartSpec) and self._key == other._key

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v!r}" for k, v in self._params.items())
        return f"PartSpec({self.kind!r}, {inner})"


def _freeze(v: Any) -> Any:
    if isinstance(v, PartSpec):
        return v._key
    if isinstance(v, Mapping):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    return v


@dataclass(frozen=True)
class LayerSpec:
    """One layer: its block arrangement, the parts the block is made of, and where the parts'
    tensors are in the file.

    ``parts`` maps a key of the block's choosing (``"mixer"``, ``"ffn"``, ``"mixer_norm"`` ...) to
    (category, spec); the block kind says which keys it asks for.  ``names`` maps a part-local
    tensor key (``"mixer.q"``, ``"ffn.down"``, ``"mixer_norm.weight"`` ...: the part's key, a dot,
    the tensor's key within the part) to the tensor's name in the checkpoint."""
    block: PartSpec
    parts: Mapping[str, Tuple[str, PartSpec]]
    names: Mapping[str, str] = field(default_factory=dict)

    @classmethod
    def pre_norm(cls, block: PartSpec, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 ffn_norm: PartSpec, names: Optional[Mapping[str, str]] = None) -> "LayerSpec":
        """The four parts of a block with a norm in front of its mixer and of its feed-forward."""
        return cls(block, {"mixer": ("mixer", mixer), "ffn": ("feed_forward", feed_forward),
                           "mixer_norm": ("norm", mixer_norm), "ffn_norm": ("norm", ffn_norm)}, dict(names or {}))


@dataclass(frozen=True)
class RunSpec:
    """One entry of the execution order.

    ``layer`` indexes ``ModelSpec.layers`` (the same layer may be named by
    several entries: its weights are shared).  ``cache`` is the id of the cache
    this run uses; runs with the same id share one cache, and only a run with
    ``writes_cache`` stores into it, so a later run can read what an earlier
    layer cached."""
    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    width: int
    vocab: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    names: Mapping[str, str] = field(default_factory=dict)   # "embedding.table", "final_norm.weight", "head.weight"
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    max_positions: int = 2048
    # name patterns (fnmatch) of tensors that files of this architecture may carry without any part
    # asking for them; they are skipped with a warning instead of failing the load
    ignorable: Tuple[str, ...] = ()

    @staticmethod
    def sequential(n_layers: int) -> Tuple[RunSpec, ...]:
        """Every layer once, in order, each with a cache of its own."""
        return tuple(RunSpec(layer=i, cache=i) for i in range(n_layers))


def check_schedule(layers: Sequence[LayerSpec], schedule: Sequence[RunSpec]) -> None:
    seen_writer = set()
    for i, run in enumerate(schedule):
        if not 0 <= run.layer < len(layers):
            raise ValueError(f"schedule[{i}] names layer {run.layer}, but the model has {len(layers)} layers")
        if run.writes_cache:
            if run.cache in seen_writer:
                raise ValueError(f"schedule[{i}]: cache {run.cache} already has a writer; "
                                 "a second run over the same cache must set writes_cache=False")
            seen_writer.add(run.cache)
        elif run.cache not in seen_writer:
            raise ValueError(f"schedule[{i}] reads cache {run.cache} before any run has written it")
