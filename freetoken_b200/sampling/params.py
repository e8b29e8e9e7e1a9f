"""Per-request sampling options.

Names, meanings and defaults follow the reference's ``SamplingParams``
(python/freetoken/core.py:18-31): ``temperature`` 0.0, ``top_k`` -1 (off),
``top_p`` 1.0, ``ignore_eos`` False, ``max_tokens`` 1024, ``stop_strs`` [] (a
request stops when one of them shows in the text of its newest tokens; needs a
tokenizer; python/freetoken/scheduler/scheduler.py:420-434); a request is greedy
when ``(temperature <= 0 or top_k == 1) and top_p == 1``.  ``stop_token_ids``
does the same by token id, tokenizer or not.  ``seed`` is an
addition: the reference seeds once per process
(python/freetoken/engine/engine.py:303); here every request has a random
stream of its own, so its tokens do not depend on what else is in the batch.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    ignore_eos: bool = False
    max_tokens: int = 1024
    stop_strs: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None

    @property
    def is_greedy(self) -> bool:
        return (self.temperature <= 0.0 or self.top_k == 1) and self.top_p == 1.0
