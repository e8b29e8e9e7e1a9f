"""Generated tokens against the plain implementation, token by token.

For every generated token the plain model runs the whole sequence so far
(prompt + the tokens generated before it) and chooses for itself: argmax, or
``softmax(logits / T)`` and an inverse-CDF draw with the request's uniform
number (python/freetoken/engine/sample.py:24-50,58-79).  The generated token
must be that choice.  Two correct implementations in bfloat16 may differ where
the choice hangs by less than their rounding: two top logits closer than
``GREEDY_TIE``, a draw closer than ``CDF_TIE`` to the boundary between two
tokens, or a router whose k-th and (k+1)-th scores lie within ``ROUTE_TIE`` at
the position that chose the token.  Such positions are counted and must stay
few; float32 gets no such allowance beyond ``1e-5``.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

GREEDY_TIE = {"float32": 1e-4, "bfloat16": 5e-2}
CDF_TIE = {"float32": 1e-5, "bfloat16": 1e-3}
ROUTE_TIE = 5e-3


def draw(logits: torch.Tensor, temperature: float, u: float):
    """Inverse-CDF draw in float64; returns (token, distance of the draw to the
    nearest boundary of the chosen token's interval)."""
    p = torch.softmax(logits.double() / max(temperature, 1e-6), dim=-1)
    cdf = p.cumsum(0)
    u = float(torch.tensor(min(max(u, 0.0), 0.99999994), dtype=torch.float32))
    target = u * float(cdf[-1])
    token = int((cdf > target).nonzero()[0])
    below = float(cdf[token - 1]) if token > 0 else 0.0
    return token, min(target - below, float(cdf[token]) - target), cdf, target


def check_generation(plain, prompt: Sequence[int], generated: Sequence[int], dtype: str,
                     temperature: float = 0.0, uniforms: Optional[Sequence[float]] = None) -> int:
    """Assert that ``generated`` is what the plain model generates from ``prompt``;
    returns how many positions were decided by a tie (always 0 in float32 unless a
    draw fell within 1e-5 of a boundary)."""
    seq: List[int] = list(prompt)
    ties = 0
    for i, token in enumerate(generated):
        logits = plain.forward(seq)[-1]
        route_margin = min((float(m[-1]) for _, m in plain.routing), default=1.0)
        if temperature <= 0.0:
            want = int(torch.argmax(logits))
            top2 = logits.topk(2).values
            tie = float(top2[0] - logits[token]) < GREEDY_TIE[dtype]
        else:
            want, _, cdf, target = draw(logits, temperature, uniforms[i])
            below = float(cdf[token - 1]) if token > 0 else 0.0
            # how far the draw lies outside the generated token's interval
            outside = max(below - target, target - float(cdf[token]), 0.0)
            tie = outside < CDF_TIE[dtype]
        if token != want:
            if not tie and not (dtype == "bfloat16" and route_margin < ROUTE_TIE):
                raise AssertionError(
                    f"[{dtype}] generated token {i} is {token}, the plain model chooses {want} "
                    f"(prompt of {len(prompt)} tokens, temperature {temperature})")
            ties += 1
        seq.append(int(token))
    return ties
