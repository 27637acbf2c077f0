"""Plain, slow Llama decoder used as the oracle of the test-suite.

It rests on the formulas of hostfog/hfee's Go sources (cited per function as
``path:line`` inside that project); the reference is Go and cannot be compiled
or imported here, so nothing in this file was checked against a run of it.

Whole sequences only, no cache, one function for each part, numpy float64
throughout (the reference mixes float32 and float64; float64 everywhere is the
stricter truth).  It shares no code with the ``hfee_b200`` package: it has its
own safetensors reader, its own config reading and its own RoPE tables.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# --------------------------------------------------------------------------
# model folder reading (independent of hfee_b200.weights)
# --------------------------------------------------------------------------
_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I32": np.int32,
       "I64": np.int64, "U8": np.uint8}


def read_safetensors(path):
    """name -> float64/int ndarray.  BF16 is widened by a 16-bit shift, as
    internal/ggml/dequant.go:63-67 does for GGUF BF16."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            arr = np.frombuffer(raw, dtype=np.dtype(_NP[meta["dtype"]]).newbyteorder("<"))
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float64)
        out[name] = arr.reshape(meta["shape"])
    return out


def to_bf16_grid(a):
    """Round float values to the nearest bfloat16 (ties to even), returned as float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(f.shape)


class PlainConfig:
    """The keys of config.json that the plain model needs, with the reference's
    defaults (internal/llm/model.go:83-100)."""

    def __init__(self, d):
        self.dim = int(d["hidden_size"])
        self.layers = int(d["num_hidden_layers"])
        self.heads = int(d["num_attention_heads"])
        self.kv_heads = int(d.get("num_key_value_heads") or self.heads)          # model.go:98
        self.head_dim = int(d.get("head_dim") or self.dim // self.heads)          # model.go:99
        self.hidden = int(d["intermediate_size"])
        self.eps = float(d.get("rms_norm_eps", 1e-5))                             # model.go:91
        self.rope_base = float(d.get("rope_theta", 10000.0))                      # model.go:92
        self.rope_scaling = d.get("rope_scaling")
        self.tied = bool(d.get("tie_word_embeddings", False))
        self.vocab = int(d["vocab_size"])
        self.pairing = d.get("rope_pairing", "half")
        self.window = d.get("sliding_window")


def load_model_dir(path, round_to_bf16=False):
    with open(os.path.join(path, "config.json")) as f:
        cfg = PlainConfig(json.load(f))
    w = read_safetensors(os.path.join(path, "model.safetensors"))
    if round_to_bf16:
        w = {k: (to_bf16_grid(v) if v.ndim == 2 else v) for k, v in w.items()}
    return cfg, w


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embed(table, tokens):
    """x[i,:] = E[token_i,:], unscaled (internal/llm/forward.go:75-77)."""
    return np.stack([table[int(t)] for t in tokens]).astype(np.float64)


def rms_norm(x, weight, eps):
    """dst = x * 1/sqrt(mean(x^2)+eps) * w, row by row (internal/ggml/ops.go:125-134)."""
    out = np.empty_like(x)
    for i in range(x.shape[0]):
        ss = float(np.sum(x[i] * x[i]))
        scale = 1.0 / math.sqrt(ss / x.shape[1] + eps)
        out[i] = x[i] * scale * weight
    return out


def linear(x, w):
    """out[t, r] = W[r, :] . x[t, :] (internal/ggml/ops.go:54-70)."""
    return x @ w.T


def rope_inv_freq(head_dim, base, scaling=None):
    """invFreq[i] = 1 / base^(2i/d) (internal/llm/model.go:150-158); the
    per-frequency divisor that model.go:155-157 reads from ``rope_freqs.weight``
    is computed here from the llama3 rope_scaling keys of config.json."""
    inv = np.array([1.0 / (base ** (2.0 * i / head_dim)) for i in range(head_dim // 2)])
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv
    assert kind == "llama3", kind
    f = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = inv.copy()
    for i, w in enumerate(inv):
        wavelen = 2.0 * math.pi / w
        if wavelen < orig / hi:
            continue
        if wavelen > orig / lo:
            out[i] = w / f
        else:
            s = (orig / wavelen - lo) / (hi - lo)
            out[i] = (1.0 - s) * w / f + s * w
    return out


def rope(x, heads, head_dim, positions, inv_freq, pairing):
    """Rotate each head of each row (internal/llm/forward.go:181-196): pair
    (2i, 2i+1) when interleaved, (i, i+d/2) when half-split."""
    out = x.copy().reshape(x.shape[0], heads, head_dim)
    src = x.reshape(x.shape[0], heads, head_dim)
    half = head_dim // 2
    for t, pos in enumerate(positions):
        for i in range(half):
            ang = float(pos) * inv_freq[i]
            s, c = math.sin(ang), math.cos(ang)
            a, b = (i, i + half) if pairing == "half" else (2 * i, 2 * i + 1)
            x0, x1 = src[t, :, a], src[t, :, b]
            out[t, :, a] = x0 * c - x1 * s
            out[t, :, b] = x0 * s + x1 * c
    return out.reshape(x.shape)


def softmax(s):
    """internal/ggml/ops.go:136-150."""
    e = np.exp(s - np.max(s))
    return e / np.sum(e)


def attention(q, k, v, heads, kv_heads, head_dim, window=None):
    """Causal grouped-query attention over one whole sequence
    (internal/llm/forward.go:146-178): token i sees keys 0..i (or the last
    ``window`` of them), q head h uses kv head h // (heads/kv_heads), scores are
    scaled by 1/sqrt(head_dim) after the dot."""
    n = q.shape[0]
    group = heads // kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    qh = q.reshape(n, heads, head_dim)
    kh = k.reshape(n, kv_heads, head_dim)
    vh = v.reshape(n, kv_heads, head_dim)
    out = np.zeros((n, heads, head_dim))
    for i in range(n):
        lo = 0 if window is None else max(0, i + 1 - int(window))
        for h in range(heads):
            g = h // group
            scores = (kh[lo:i + 1, g, :] @ qh[i, h, :]) * scale
            p = softmax(scores)
            out[i, h, :] = p @ vh[lo:i + 1, g, :]
    return out.reshape(n, heads * head_dim)


def swiglu(gate, up):
    """g / (1 + exp(-g)) * u (internal/ggml/ops.go:160-165)."""
    return gate / (1.0 + np.exp(-gate)) * up


def feed_forward(x, w_gate, w_up, w_down):
    """internal/llm/forward.go:110-113."""
    return linear(swiglu(linear(x, w_gate), linear(x, w_up)), w_down)


def block(x, positions, w, prefix, cfg, inv_freq):
    """One pre-norm decoder layer (internal/llm/forward.go:79-115)."""
    p = prefix
    xb = rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
    q = linear(xb, w[p + "self_attn.q_proj.weight"])
    k = linear(xb, w[p + "self_attn.k_proj.weight"])
    v = linear(xb, w[p + "self_attn.v_proj.weight"])
    q = rope(q, cfg.heads, cfg.head_dim, positions, inv_freq, cfg.pairing)
    k = rope(k, cfg.kv_heads, cfg.head_dim, positions, inv_freq, cfg.pairing)
    att = attention(q, k, v, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.window)
    x = x + linear(att, w[p + "self_attn.o_proj.weight"])
    xb = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps)
    x = x + feed_forward(xb, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                         w[p + "mlp.down_proj.weight"])
    return x


def forward(cfg, w, tokens):
    """Logits [len(tokens), vocab] of one whole sequence starting at position 0
    (internal/llm/forward.go:51-142, with the logits of every row, not just the last)."""
    positions = list(range(len(tokens)))
    inv_freq = rope_inv_freq(cfg.head_dim, cfg.rope_base, cfg.rope_scaling)
    x = embed(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg.layers):
        x = block(x, positions, w, f"model.layers.{l}.", cfg, inv_freq)
    x = rms_norm(x, w["model.norm.weight"], cfg.eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]  # model.go:118-121
    return linear(x, head)


def greedy_generate(cfg, w, prompt, steps):
    """Argmax continuation, first maximum wins (internal/llm/sampler.go:76-84)."""
    toks = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(np.argmax(forward(cfg, w, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
