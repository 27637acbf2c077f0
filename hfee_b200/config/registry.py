"""One registry from an architecture's name (``architectures[0]`` of config.json)
to its typed config class and the function that lays it out as parts.

The reference keeps a map from the GGUF architecture string to a model variant
and refuses unknown names with ``unsupported model architecture``
(hostfog/hfee internal/llm/model.go:51-56,77-81); this is that map for model
folders.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

from .llama import ConfigError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]
    # optional: (config.json content, {tensor name: shape}) -> config.json content with the sizes it left
    # out taken from the checkpoint's tensors
    fill_from_tensors: Optional[Callable[[Mapping[str, Any], Mapping[str, Tuple[int, ...]]], Mapping[str, Any]]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable[[Mapping[str, Any]], Any],
                          build_spec: Callable[[Any], ModelSpec], fill_from_tensors=None) -> None:
    """Make ``name`` loadable: ``config_from_dict`` turns config.json into a typed
    config, ``build_spec`` turns that config into a :class:`ModelSpec`; ``fill_from_tensors``
    (optional) completes a config.json from the shapes of the checkpoint's tensors."""
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_spec, fill_from_tensors)


def architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES)) or "none"
        raise ConfigError(f"unsupported model architecture {name!r} (registered: {known})") from None


def known_architectures() -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_ARCHITECTURES))


def read_config_json(model_dir: str) -> Mapping[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in this model folder")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None


def resolve(config_json: Mapping[str, Any], tensor_shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> Tuple[Architecture, Any]:
    """(architecture entry, typed config) for the content of a config.json.  ``tensor_shapes``
    (checkpoint tensor name -> shape), when the caller has a checkpoint at hand, lets an
    architecture take a size that config.json leaves out from the tensors themselves."""
    archs = config_json.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: missing key 'architectures'")
    arch = architecture(str(archs[0]))
    if tensor_shapes is not None and arch.fill_from_tensors is not None:
        config_json = arch.fill_from_tensors(config_json, tensor_shapes)
    return arch, arch.config_from_dict(config_json)


def resolve_model_dir(model_dir: str) -> Tuple[Architecture, Any]:
    """:func:`resolve` for a model folder, with the shapes of its checkpoint's tensors if it has one."""
    shapes = None
    try:
        from ..weights.safetensors_io import TensorFiles
        files = TensorFiles(model_dir)
        shapes = {n: tuple(files.info(n).shape) for n in files.names()}
        files.close()
    except Exception:          # no readable checkpoint: the configuration alone decides (and says what it lacks)
        shapes = None
    return resolve(read_config_json(model_dir), shapes)


def _ensure_builtin() -> None:
    # models register themselves on import; imported lazily to avoid a cycle
    from .. import models  # noqa: F401
