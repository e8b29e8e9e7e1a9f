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
        if takes and rows <= SKINNY_ROWS:
            ops.skinny_gemm(x, weight, out, rows_per_pass=ops.pass_rows(rows))
            return out
        if out.dtype == torch.bfloat16:
            torch.matmul(x, weight.t(), out=out)
            return out
        if out.dtype == torch.float32 and library_f32_out(x, weight, out):
            return out
        if takes:
            ops.skinny_gemm(x, weight, out, rows_per_pass=32)
            return out
    ops.gemm_rows(x, weight, out)
    return out


_F32_OUT = {"ok": None}


def library_f32_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """bfloat16 x bfloat16 -> float32 through the library product, where this
    PyTorch offers it (``torch.mm(..., out_dtype=)``); the result is the
    float32 accumulator, not a rounded bfloat16."""
    if _F32_OUT["ok"] is False:
        return False
    try:
        torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        _F32_OUT["ok"] = True
        return True
    except (TypeError, RuntimeError):
        _F32_OUT["ok"] = False
        return False


# Up to this many rows the weight-streaming kernel reads the weights once;
# above it the library's tiled product wins.
SKINNY_ROWS = 32


def libraries(compute: torch.dtype) -> list:
    return ["gemm_simt"] if compute == torch.float32 else ["gemm_simt", "skinny_gemm"]
