"""Weights by tensor name, checked against what the model's parts ask for.

The reference looks tensors up by name and reports the first one missing
(``model is missing tensor X``, hostfog/hfee internal/llm/model.go:163-174) or of
the wrong rank (model.go:188-191).  Here every part declares the tensors it needs
(:class:`TensorNeed`); the whole list is compared with the file once and ONE error
names everything missing, unexpected and mis-shaped.
"""
from __future__ import annotations

import fnmatch
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from .safetensors_io import TensorFiles


class WeightError(ValueError):
    """The checkpoint does not hold the tensors the model needs.

    ``missing``, ``unexpected`` and ``wrong_shape`` list the tensor names."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: List[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  unusable dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {d}" for n, d in self.wrong_dtype))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorNeed:
    """What a part asks of the checkpoint for one tensor.

    ``role`` decides the dtype it is kept in and how random weights draw it:
    ``matrix``/``table`` (GEMM operands and embedding tables: the compute dtype,
    N(0, 0.02)), ``scale`` (norm weights: float32, 1 + N(0, 0.02)), ``vector``
    (float32, N(0, 0.02)), ``index`` (integer tables: int32, zeros)."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


_FLOATS = (torch.float32, torch.float16, torch.bfloat16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_tensors(needs: Mapping[str, TensorNeed], have: Mapping[str, Tuple[torch.dtype, Tuple[int, ...]]],
                  ignorable: Sequence[str] = ()) -> List[str]:
    """Compare what the parts ask for with what the files hold; raises ONE :class:`WeightError`
    for everything missing, unexpected, mis-shaped or of an unusable dtype.  Tensors nobody asked
    for whose names match one of the ``ignorable`` patterns (buffers that exporters store beside the
    weights, named by the architecture) are returned instead of counted as unexpected."""
    missing = [n for n, need in needs.items() if n not in have and not need.optional]
    extra = [n for n in have if n not in needs]
    ignored = [n for n in extra if any(fnmatch.fnmatchcase(n, pat) for pat in ignorable)]
    unexpected = [n for n in extra if n not in set(ignored)]
    wrong_shape = []
    wrong_dtype = []
    for n, need in needs.items():
        if n not in have:
            continue
        dtype, shape = have[n]
        if tuple(shape) != tuple(need.shape):
            wrong_shape.append((n, tuple(shape), tuple(need.shape)))
        ok = _INTS if need.role == "index" else _FLOATS
        if dtype not in ok:
            wrong_dtype.append((n, str(dtype)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(sorted(missing), sorted(unexpected), sorted(wrong_shape), sorted(wrong_dtype))
    return sorted(ignored)


def kept_dtype(need: TensorNeed, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device: GEMM operands and tables in the
    compute dtype; integer tables as int32; norm scales and other vectors, and
    anything the part marks ``keep32``, in float32."""
    if need.role == "index":
        return torch.int32
    if need.role in ("matrix", "table"):
        return compute
    return torch.float32


class Checkpoint:
    """Named tensors of a model folder, validated against the parts' needs."""

    def __init__(self, model_dir: str):
        self.files = TensorFiles(model_dir)

    def check(self, needs: Mapping[str, TensorNeed], ignorable: Sequence[str] = ()) -> None:
        have = {n: (self.files.info(n).dtype, self.files.info(n).shape) for n in self.files.names()}
        ignored = check_tensors(needs, have, ignorable)
        if ignored:
            shown = ", ".join(ignored[:4]) + (", ..." if len(ignored) > 4 else "")
            warnings.warn(f"{len(ignored)} tensors of the checkpoint are not used by the model and were skipped: {shown}")

    def has(self, name: str) -> bool:
        return name in self.files

    def fetch(self, name: str, need: TensorNeed, compute: torch.dtype, device) -> torch.Tensor:
        t = self.files.tensor(name)
        return t.to(device=device, dtype=kept_dtype(need, t.dtype, compute)).contiguous()

    def raw(self, name: str) -> torch.Tensor:
        return self.files.tensor(name)
