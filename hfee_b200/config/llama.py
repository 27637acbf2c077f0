"""Typed configuration of the dense Llama decoder, read from its config.json keys.

Counterpart of ``llm.Config`` and the metadata reading in hostfog/hfee's
internal/llm/model.go:13-26,83-100 (there from GGUF ``llama.*`` keys, here from
the Hugging Face style ``config.json`` of a model folder).  Defaults follow the
reference: ``num_key_value_heads`` = heads (model.go:98), ``head_dim`` =
hidden/heads (model.go:99), eps 1e-5 (model.go:91), rope base 10000
(model.go:92), trained context 2048 (model.go:90).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the engine cannot run."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of kind ``llama3``: low frequencies are slowed by
    ``factor``, high ones kept, the band between blended.  The reference only
    consumes the resulting per-frequency divisors (``rope_freqs.weight``,
    internal/llm/model.go:151-157)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def apply(self, inv_freq: List[float]) -> List[float]:
        lo_wavelen = self.original_max_position_embeddings / self.low_freq_factor
        hi_wavelen = self.original_max_position_embeddings / self.high_freq_factor
        out = []
        for w in inv_freq:
            wavelen = 2.0 * math.pi / w
            if wavelen < hi_wavelen:
                out.append(w)
            elif wavelen > lo_wavelen:
                out.append(w / self.factor)
            else:
                s = (self.original_max_position_embeddings / wavelen - self.low_freq_factor) / (
                    self.high_freq_factor - self.low_freq_factor)
                out.append((1.0 - s) * w / self.factor + s * w)
        return out


def _need(d: Mapping[str, Any], key: str) -> Any:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing key {key!r}")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str) -> int:
    v = _need(d, key)
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    rope_pairing: str                  # "half": pairs (i, i+d/2); "interleaved": pairs (2i, 2i+1)
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]
    torch_dtype: str

    architecture = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        hidden = _pos_int(d, "hidden_size")
        layers = _pos_int(d, "num_hidden_layers")
        heads = _pos_int(d, "num_attention_heads")
        kv = d.get("num_key_value_heads")
        kv = heads if kv is None else _pos_int(d, "num_key_value_heads")
        hd = d.get("head_dim")
        if hd is None:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and head_dim is not given")
            hd = hidden // heads
        else:
            hd = _pos_int(d, "head_dim")
        if heads % kv:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv}")
        if hd % 2:
            raise ConfigError(f"config.json: head_dim {hd} must be even for rotary embedding")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"config.json: {key}=true is not supported by the Llama decoder")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (silu only)")

        scaling = None
        rs = d.get("rope_scaling")
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind == "llama3":
                try:
                    scaling = RopeScaling(float(rs["factor"]), float(rs["low_freq_factor"]),
                                          float(rs["high_freq_factor"]),
                                          int(rs["original_max_position_embeddings"]))
                except KeyError as e:
                    raise ConfigError(f"config.json: rope_scaling is missing {e.args[0]!r}") from None
                if scaling.high_freq_factor <= scaling.low_freq_factor:
                    raise ConfigError("config.json: rope_scaling.high_freq_factor must exceed low_freq_factor")
            elif kind not in (None, "default"):
                raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported (llama3 only)")

        pairing = d.get("rope_pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ConfigError(f"config.json: rope_pairing must be 'half' or 'interleaved', got {pairing!r}")

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(e) for e in eos)

        return cls(
            hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv, head_dim=hd,
            intermediate_size=_pos_int(d, "intermediate_size"),
            vocab_size=_pos_int(d, "vocab_size"),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=scaling, rope_pairing=pairing,
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=d.get("bos_token_id"), eos_token_ids=eos_ids,
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
        )

    def to_dict(self) -> dict:
        """The config.json that :meth:`from_dict` reads back to an equal config."""
        d = {
            "architectures": [self.architecture], "model_type": "llama",
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "rope_scaling": None, "rope_pairing": self.rope_pairing,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu",
            "attention_bias": False, "mlp_bias": False,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": list(self.eos_token_ids) if self.eos_token_ids else None,
            "torch_dtype": self.torch_dtype,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            d["rope_scaling"] = {"rope_type": "llama3", "factor": s.factor,
                                 "low_freq_factor": s.low_freq_factor,
                                 "high_freq_factor": s.high_freq_factor,
                                 "original_max_position_embeddings": s.original_max_position_embeddings}
        return d
