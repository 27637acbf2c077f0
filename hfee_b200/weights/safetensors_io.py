"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw
little-endian tensor bytes.  It stands where hostfog/hfee has its GGUF reader
(internal/gguf/gguf.go:39-115): a name -> (type, dims, bytes) table over a
memory-mapped file.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class WeightFormatError(ValueError):
    """The file is not a readable safetensors file."""


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    file: str
    begin: int          # absolute byte offsets in ``file``
    end: int


def _read_header(path: str) -> Tuple[Dict[str, dict], int]:
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise WeightFormatError(f"{path}: truncated (no header length)")
        (n,) = struct.unpack("<Q", head)
        if n <= 0 or 8 + n > size:
            raise WeightFormatError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise WeightFormatError(f"{path}: header is not JSON ({e})") from None
    return header, 8 + n


def index_file(path: str) -> Dict[str, TensorInfo]:
    header, base = _read_header(path)
    size = os.path.getsize(path)
    out: Dict[str, TensorInfo] = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _DTYPES:
            raise WeightFormatError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
        dtype = _DTYPES[meta["dtype"]]
        shape = tuple(int(s) for s in meta["shape"])
        lo, hi = (int(x) for x in meta["data_offsets"])
        count = 1
        for s in shape:
            count *= s
        if hi - lo != count * dtype.itemsize or base + hi > size or lo < 0:
            raise WeightFormatError(f"{path}: tensor {name}: byte range [{lo},{hi}) does not match "
                                    f"shape {list(shape)} of {meta['dtype']} or leaves the file")
        out[name] = TensorInfo(name, dtype, shape, path, base + lo, base + hi)
    return out


class TensorFiles:
    """All tensors of a model folder by name (``model.safetensors``, or the shards
    listed in ``model.safetensors.index.json``), memory-mapped on demand."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        files: List[str]
        if os.path.isfile(index_path):
            with open(index_path) as f:
                files = sorted(set(json.load(f)["weight_map"].values()))
            files = [os.path.join(model_dir, x) for x in files]
        elif os.path.isfile(single):
            files = [single]
        else:
            raise WeightFormatError(f"{model_dir}: no model.safetensors in this model folder")
        self.infos: Dict[str, TensorInfo] = {}
        for path in files:
            for name, info in index_file(path).items():
                if name in self.infos:
                    raise WeightFormatError(f"tensor {name} appears in both {self.infos[name].file} and {path}")
                self.infos[name] = info
        self._maps: Dict[str, mmap.mmap] = {}

    def names(self) -> Iterable[str]:
        return self.infos.keys()

    def __contains__(self, name: str) -> bool:
        return name in self.infos

    def info(self, name: str) -> TensorInfo:
        return self.infos[name]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (copy before writing to it)."""
        info = self.infos[name]
        mm = self._maps.get(info.file)
        if mm is None:
            with open(info.file, "rb") as f:
                mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
            self._maps[info.file] = mm
        count = 1
        for s in info.shape:
            count *= s
        if count == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        t = torch.frombuffer(mm, dtype=info.dtype, count=count, offset=info.begin)
        return t.reshape(info.shape)

    def close(self) -> None:
        self._maps.clear()


def write_file(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) as one safetensors file."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightFormatError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
