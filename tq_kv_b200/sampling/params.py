"""Generation parameters, with the reference's names and defaults
(src/engine.rs:29-49: max_tokens 512, temperature 0.7, top_p 0.9, top_k 40,
repeat_penalty 1.1, seed 0)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence


@dataclass
class GenerationParams:
    max_tokens: int = 512
    temperature: float = 0.7          # <= 0 selects arg-max (src/engine.rs:353-354)
    top_p: float = 0.9                # >= 1 switches top-p off
    top_k: int = 40                   # 0 switches top-k off
    repeat_penalty: float = 1.1       # 1 switches the penalty off (src/engine.rs:403)
    seed: int = 0
    stop_token_ids: Optional[Sequence[int]] = None   # None: the model's end-of-sequence ids

    def validate(self) -> None:
        if self.max_tokens < 0:
            raise ValueError("max_tokens must be >= 0")
        if not self.repeat_penalty > 0:
            raise ValueError("repeat_penalty must be > 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0 < self.top_p:
            raise ValueError("top_p must be > 0")

    @classmethod
    def greedy(cls, max_tokens: int = 512, **kw) -> "GenerationParams":
        return cls(max_tokens=max_tokens, temperature=0.0, top_p=1.0, top_k=0, repeat_penalty=1.0, **kw)
