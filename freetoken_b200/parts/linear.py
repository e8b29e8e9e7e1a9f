"""Matrix products ``y = x @ W^T`` for the parts, by compute dtype.

* float32 compute: the CUDA-core kernel of ``gemm_simt.cu`` - true 32-bit
  arithmetic with a fixed summation order (no tensor cores, no TF32), weights
  read as stored (float32 or bfloat16, upcast exactly in registers).
* bfloat16 compute, bfloat16 result: a library product (cuBLAS through
  ``torch.matmul``), as the reference does for its dense projections
  (python/freetoken/layers/linear.py:31-32).  Few rows (decode) go through the
  weight-streaming kernel of ``skinny_gemm.cu`` instead.
* bfloat16 compute, float32 result (logits, router logits): our kernels, so the
  result leaves the float32 accumulator unrounded.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = x @ weight^T``; ``weight`` is ``[N, K]``; ``out`` preallocated."""
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        rows = x.shape[0]
        takes = ops.skinny_gemm_takes(x, weight, out)
        if takes and (rows <= SKINNY_ROWS or out.dtype != torch.bfloat16):
            ops.skinny_gemm(x, weight, out, rows_per_pass=ops.pass_rows(rows))
            return out
        if out.dtype == torch.bfloat16:
            torch.matmul(x, weight.t(), out=out)
            return out
    ops.gemm_rows(x, weight, out)
    return out


# Up to this many rows the weight-streaming kernel reads the weights once;
# above it the library's tiled product wins.
SKINNY_ROWS = 32


def libraries(compute: torch.dtype) -> list:
    return ["gemm_simt"] if compute == torch.float32 else ["gemm_simt", "skinny_gemm"]
