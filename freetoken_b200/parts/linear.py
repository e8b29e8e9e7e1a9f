"""Matrix products ``y = x @ W^T`` for the parts, by compute dtype.

* float32 compute: the CUDA-core kernel of ``gemm_simt.cu`` - true 32-bit
  arithmetic with a fixed summation order (no tensor cores, no TF32), weights
  read as stored (float32 or bfloat16, upcast exactly in registers).
* bfloat16 compute, bfloat16 result: a library product (cuBLAS through
  ``torch.matmul``), as the reference does for its dense projections
  (python/freetoken/layers/linear.py:31-32).  Few rows (decode) go through the
  weight-streaming kernel of ``skinny_gemm.cu`` instead.
* bfloat16 compute, float32 result (logits of many rows, the router's logits
  of a long step): the library product with a float32 result where this
  PyTorch offers one (``torch.mm(..., out_dtype=float32)``), else the
  weight-streaming kernel; either way the result is the float32 accumulator,
  never a rounded bfloat16.
"""

from __future__ import annotations


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


def library_offers_f32_out(device) -> bool:
    """Whether ``torch.mm`` takes ``out_dtype`` (asked once, on a tiny product).
    Only "this PyTorch has no such argument" counts as no; any other error is
    a real one and is raised."""
    if _F32_OUT["ok"] is None:
        a = torch.zeros((16, 16), dtype=torch.bfloat16, device=device)
        try:
            torch.mm(a, a.t(), out_dtype=torch.float32)
            _F32_OUT["ok"] = True
        except (TypeError, NotImplementedError):
            _F32_OUT["ok"] = False
    return _F32_OUT["ok"]


def library_f32_out(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> bool:
    """bfloat16 x bfloat16 -> float32 through the library product, where this
    PyTorch offers it; the result is the float32 accumulator, not a rounded
    bfloat16.  False: the caller takes one of our kernels instead."""
    if not library_offers_f32_out(x.device):
        return False
    torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
    return True


# Up to this many rows the weight-streaming kernel reads the weights once;
# above it the library's tiled product wins.
SKINNY_ROWS = 32


def libraries(compute: torch.dtype) -> list:
    return ["gemm_simt"] if compute == torch.float32 else ["gemm_simt", "skinny_gemm"]
