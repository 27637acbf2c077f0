"""Random weights: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor is drawn from a generator seeded by (seed, tensor name), so its values
do not depend on the order or the set of tensors written.  Matrices and tables are
N(0, 0.02), norm scales 1 + N(0, 0.02), integer tables zeros.  The reference has no
such mode (it only reads GGUF files, hostfog/hfee internal/llm/model.go:58-71).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping

import torch

from .loader import TensorNeed
from .safetensors_io import write_file

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") >> 1


def random_tensors(needs: Mapping[str, TensorNeed], seed: int, dtype: torch.dtype = torch.float32,
                   std: float = 0.02) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for name, need in needs.items():
        if need.role == "index":
            out[name] = torch.zeros(need.shape, dtype=torch.int32)
            continue
        g = torch.Generator().manual_seed(_tensor_seed(seed, name))
        t = torch.randn(need.shape, generator=g, dtype=torch.float32) * std
        if need.role == "scale":
            t += 1.0
        out[name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, config_json: Mapping[str, Any], seed: int, dtype: str = "float32",
                       std: float = 0.02) -> str:
    """Write ``config.json`` and ``model.safetensors`` for the architecture that
    ``config_json`` names, with every tensor its parts ask for drawn at random."""
    from ..config.registry import resolve
    from ..parts.model import model_tensor_needs

    if dtype not in _STORE:
        raise ValueError(f"dtype must be one of {sorted(_STORE)}, got {dtype!r}")
    arch, cfg = resolve(config_json)
    needs = {n: need for n, need in model_tensor_needs(arch.build_spec(cfg)).items() if not need.optional}
    os.makedirs(model_dir, exist_ok=True)
    out = dict(config_json)
    out["torch_dtype"] = dtype
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(out, f, indent=1)
    write_file(os.path.join(model_dir, "model.safetensors"), random_tensors(needs, seed, _STORE[dtype], std),
               metadata={"format": "pt", "seed": str(seed)})
    return model_dir
