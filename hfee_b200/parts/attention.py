"""Causal grouped-query attention over the paged cache.

Per hostfog/hfee internal/llm/forward.go:83-107: q/k/v projections of the normed
input, position encoding of q and k, k and v stored in the cache at the token's
position *before* attending, attention of every token over its own request's cache
up to its position, output projection added to the residual stream.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch

from ..cache.needs import PagedKV
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.loader import TensorNeed
from .base import Mixer, build_part, register_part


class PagedAttention(Mixer):
    """spec: ``width``, ``heads``, ``kv_heads``, ``head_dim``, ``position`` (a PartSpec),
    ``window`` (None = all keys, else the last ``window`` positions), ``scale``
    (None = head_dim**-0.5, internal/llm/forward.go:149)."""

    accepts_lazy_input = True        # the input norm may be fused into the q/k/v projection

    @property
    def graph_safe(self) -> bool:    # every launch reads the batch from device buffers; the position part decides
        return bool(self.position.graph_safe)

    @staticmethod
    def tensor_needs(spec: PartSpec) -> Dict[str, TensorNeed]:
        q, kv = spec.heads * spec.head_dim, spec.kv_heads * spec.head_dim
        return {"q": TensorNeed((q, spec.width)), "k": TensorNeed((kv, spec.width)),
                "v": TensorNeed((kv, spec.width)), "o": TensorNeed((spec.width, q))}

    def __init__(self, spec, tensors, rt):
        super().__init__(spec, tensors, rt)
        self.heads, self.kv_heads, self.head_dim = int(spec.heads), int(spec.kv_heads), int(spec.head_dim)
        if self.heads % self.kv_heads:
            raise ValueError(f"heads {self.heads} must be a multiple of kv_heads {self.kv_heads}")
        self.window = spec.get("window")
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part("position", spec.position, {}, rt)
        # one fused projection: rows [q heads | k heads | v heads]
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.w_o = tensors["o"]
        self.q_cols = self.heads * self.head_dim
        self.qkv_cols = (self.heads + 2 * self.kv_heads) * self.head_dim
        # partial results of a decode step whose keys are split among CTAs
        self.split_scratch = rt.scratch("attn_partials", (rt.max_requests * self.heads * ops.MAX_SPLITS *
                                                          (self.head_dim + 2),), torch.float32)

    def cache_need(self) -> PagedKV:
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, step: Any, cache: Any, writes_cache: bool) -> None:
        n, rt = step.n, self.rt
        cs = self.position.table(step)
        q = rt.scratch("attn_q", (rt.max_tokens, self.q_cols))[:n]
        # a run that reads the cache another run filled needs the queries only
        w = self.w_qkv if writes_cache else self.w_qkv[:self.q_cols]
        qkv = rt.scratch("attn_qkv", (rt.max_tokens, self.qkv_cols))[:n, :w.shape[0]]
        k_pool, v_pool = (cache.k, cache.v) if writes_cache else (None, None)
        decode = ops.decode_rope_fusable(step, qkv.dtype, self.heads, self.kv_heads, self.head_dim,
                                         self.position.rope_dim, qkv, self.split_scratch)
        fused_qkv = not decode and ops.qkv_rope_fusable(rt.dtype, n, w, self.head_dim, self.position.rope_dim, cs, q)
        ops.tag("qkv")
        if fused_qkv:            # a prompt portion: rotation and cache write happen in the product's epilogue
            ops.linear_rope_cache(xn if isinstance(xn, torch.Tensor) else xn.tensor(), w, cs, step.positions,
                                  step.slot_of_token, q, k_pool, v_pool, cache.block_table, cache.page_size,
                                  self.heads, self.kv_heads, self.head_dim, self.position.interleaved)
        else:
            ops.linear_normed(xn, w, qkv)
        att = rt.scratch("attn_out", (rt.max_tokens, self.q_cols))[:n]
        if decode:
            # a decode step: rotation and cache write happen inside the attention kernel
            ops.tag("attention")
            ops.paged_attention_rope(qkv, cs, self.position.rope_dim, self.position.interleaved, writes_cache,
                                     cache.k, cache.v, cache.block_table, cache.page_size, att, self.heads,
                                     self.kv_heads, self.head_dim, self.scale, int(self.window or 0), step,
                                     self.split_scratch)
            ops.tag("o")
            ops.linear(att, self.w_o, residual, accumulate=True)
            return
        if not fused_qkv:
            ops.tag("rope")
            ops.rope_cache_write(qkv, cs, step.positions, step.slot_of_token, q, k_pool, v_pool, cache.block_table,
                             cache.page_size, self.heads, self.kv_heads, self.head_dim, self.position.rope_dim,
                             self.position.interleaved)
        ops.tag("attention")
        ops.paged_attention(q, cache.k, cache.v, cache.block_table, cache.page_size, step.positions,
                            step.slot_of_token, att, self.heads, self.kv_heads, self.head_dim, self.scale,
                            int(self.window or 0), step=step, scratch=self.split_scratch)
        ops.tag("o")
        ops.linear(att, self.w_o, residual, accumulate=True)


register_part("mixer", "attention", PagedAttention)
