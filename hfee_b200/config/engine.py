"""Engine-wide settings (not part of a model's config.json).

The reference takes these from the environment: ``HFEE_NUM_PARALLEL`` (default 4)
and ``HFEE_NUM_CTX`` (default 4096) in hostfog/hfee internal/server/server.go:46-57,
and a fixed per-pass token budget of 256 in internal/llm/runner.go:11.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class EngineConfig:
    dtype: str = "bfloat16"            # "bfloat16" | "float32"
    page_size: int = 64                # tokens per cache page
    max_requests: int = 4              # live requests (HFEE_NUM_PARALLEL)
    max_context: int = 4096            # tokens one request may hold (HFEE_NUM_CTX)
    max_cache_tokens: Optional[int] = None   # pool size in tokens; default max_requests*max_context
    max_batch_tokens: int = 2048       # token budget of one step (runner.go batchSize)
    prefill_chunk: Optional[int] = None      # largest prompt portion per request and step
    use_cuda_graphs: bool = True
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype in ("bf16", "bfloat16"):
            self.dtype = "bfloat16"
        elif self.dtype in ("fp32", "float32", "float"):
            self.dtype = "float32"
        else:
            raise ValueError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.page_size < 16 or self.page_size & (self.page_size - 1):
            raise ValueError(f"page_size must be a power of two of at least 16, got {self.page_size}")
        if self.max_requests <= 0 or self.max_context <= 0 or self.max_batch_tokens <= 0:
            raise ValueError("max_requests, max_context and max_batch_tokens must be positive")
        if self.max_cache_tokens is None:
            self.max_cache_tokens = self.max_requests * self.pages_for(self.max_context) * self.page_size
        if self.prefill_chunk is None:
            self.prefill_chunk = self.max_batch_tokens

    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    @property
    def num_pages(self) -> int:
        return self.max_cache_tokens // self.page_size
