"""Sampling options with the names, meanings and defaults of hostfog/hfee's
``llm.Options`` / ``DefaultOptions()`` (internal/llm/sampler.go:10-34)."""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import List, Optional


@dataclass
class SamplingOptions:
    temperature: float = 0.8        # <= 0: greedy (sampler.go:76)
    top_k: int = 40                 # <= 0: all tokens (sampler.go:133-136)
    top_p: float = 0.9              # active for 0 < p < 1 (sampler.go:98)
    min_p: float = 0.0              # active when > 0 (sampler.go:109)
    repeat_penalty: float = 1.1     # 1: off (sampler.go:57)
    repeat_last_n: int = 64         # < 0: whole history, 0: off (sampler.go:57-61)
    seed: int = -1                  # < 0: a fresh random seed per request (sampler.go:41-45)
    num_predict: int = -1           # most new tokens, < 0: until the context is full (runner.go:309)
    stop: List[str] = field(default_factory=list)   # stop strings; need a tokenizer (text.go:41-78)

    @classmethod
    def greedy(cls, num_predict: int = -1) -> "SamplingOptions":
        """Pure argmax: temperature 0 and no repeat penalty."""
        return cls(temperature=0.0, repeat_penalty=1.0, num_predict=num_predict)

    def with_(self, **changes) -> "SamplingOptions":
        return replace(self, **changes)

    @property
    def penalises(self) -> bool:
        return self.repeat_penalty != 1 and self.repeat_last_n != 0

    @property
    def device_only(self) -> bool:
        """True when the device kernel covers the whole chain: greedy or plain
        temperature sampling over all tokens, without penalty or truncation."""
        if self.penalises:
            return False
        if self.temperature <= 0:
            return True
        return self.top_k <= 0 and not (0 < self.top_p < 1) and not self.min_p > 0

    @property
    def device_chain(self) -> bool:
        """True when the device kernels for the whole chain take these options: a top-k of at most
        64 (greedy is k = 1) and a repeat penalty over at most the last 256 tokens."""
        if self.penalises and not 0 < self.repeat_last_n <= 256:
            return False
        if self.temperature <= 0:
            return True
        return 0 < self.top_k <= 64
