"""One kernel on one small, real-width workload: time it, print its roofline share.

    python -m freetoken_b200.kernel_bench --kernel expert_gemv [--reps 20]

Used by hand and as the program profiled under ``ncu`` (the summaries under
``profiles/`` name the command).  Workloads hold well under 2 GB on the device
and are larger than the L2 cache; the input that is streamed is rotated between
repetitions so that no repetition finds it in L2.

Kernels: ``expert_gemv`` (decode experts, weight-streaming mma.sync kernel),
``lm_head`` (the same kernel, dense, float32 result), ``moe_gemm_tc`` (prefill
experts on tcgen05/TMEM with TMA, 64 rows per expert; ``_busy``: 512 rows per expert), ``attn_decode`` (64 rows x 2,048 keys; ``_32k``: 8 rows x 32,768 keys), ``attn_prefill`` (mma.sync), ``attn_prefill_tc`` (tcgen05/TMEM, TMA-fed; ``_8k``: a
8,192-token prompt),
``router`` (float32 router logits + top-k for a decode batch); ``*_flashinfer``: the same
attention shapes through FlashInfer's trtllm-gen kernels (the reference's backend on
this GPU), as a comparison point; ``peak_copy`` / ``peak_gemm``: a 1 GiB device copy and an
8192^3 library bf16 product, the two roofline denominators measured in place; ``peak_read``:
a 4 GiB read-only stream, the tighter ceiling of a decode step.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Callable, Dict, Tuple

import torch

from .benchmark import load_peaks
from .csrc import ops
from .parts.base import Workspace

H, I, D, NQ, NKV = 3072, 1536, 128, 48, 8
DEV = "cuda:0"


def _routes(experts: int, tokens: int, k: int, seed: int = 0):
    """Sorted routes of ``tokens`` tokens choosing ``k`` of ``experts`` uniformly."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(tokens)]).to(torch.int32)
    flat = ids.view(-1)
    order = torch.sort(flat.long(), stable=True).indices.to(torch.int32)
    counts = torch.bincount(flat.long(), minlength=experts)
    offsets = torch.zeros(experts + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    busy = (counts > 0).nonzero().flatten().to(torch.int32)
    active = torch.zeros(experts + 1, dtype=torch.int32)
    active[:busy.numel()] = busy
    active[experts] = busy.numel()
    dev = lambda t: t.to(DEV)
    return dev(order), dev((order // k).to(torch.int32)), dev(offsets), dev(active), int(busy.numel())


def expert_gemv(sets: int = 2):
    """Decode, batch 8: 64 routes over 48 experts, gate_up + GLU then down."""
    E, T, k = 48, 8, 8
    w1 = [torch.randn(E, 2 * I, H, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
    w2 = [torch.randn(E, H, I, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    route, token, offsets, active, busy = _routes(E, T, k)
    R = T * k
    mid = torch.empty(R, I, device=DEV, dtype=torch.bfloat16)
    parts = torch.empty(R, H, device=DEV, dtype=torch.bfloat16)
    rw = torch.rand(R, device=DEV)

    def run(i):
        ops.skinny_gemm(x, w1[i % sets], mid, group_offsets=offsets, active=active, a_rows=token, rows=R, glu=True)
        ops.skinny_gemm(mid, w2[i % sets], parts, group_offsets=offsets, active=active, c_rows=route,
                        row_scale=rw, rows=R)
    return run, busy * 3 * I * H * 2, 0.0, "hbm"


def lm_head(sets: int = 2):
    V, T = 200064, 8
    w = [torch.randn(V, H, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(T, V, device=DEV)
    return (lambda i: ops.skinny_gemm(x, w[i % sets], out)), V * H * 2, 0.0, "hbm"


def _moe_gemm_tc(E: int, T: int, sets: int):
    k = 8
    w1 = [torch.randn(E, 2 * I, H, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
    w2 = [torch.randn(E, H, I, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    route, token, offsets, active, busy = _routes(E, T, k)
    R = T * k
    ws = Workspace(DEV)
    mid = torch.empty(R, I, device=DEV, dtype=torch.bfloat16)
    parts = torch.empty(R, H, device=DEV, dtype=torch.bfloat16)
    rw = torch.rand(R, device=DEV)

    def run(i):     # gather + tile list + both products, as a step runs them
        ops.moe_experts_tc(x, w1[i % sets], w2[i % sets], mid, parts, offsets, active, route, token, rw, R,
                           "silu", 1.702, 7.0, ws)
    return run, busy * 3 * I * H * 2, 2.0 * R * 3 * I * H


def moe_gemm_tc(sets: int = 1):
    """Prefill: 512 tokens x 8 routes over 64 experts (64 rows each), 1.8 GB of weights."""
    run, nbytes, flops = _moe_gemm_tc(64, 512, sets)
    return run, nbytes, flops, "hbm"


def moe_gemm_tc_busy(sets: int = 1):
    """Prefill with busy experts: 4,096 tokens x 8 routes over 64 experts (512 rows each)."""
    run, nbytes, flops = _moe_gemm_tc(64, 4096, sets)
    return run, nbytes, flops, "flops"


def _kv(batch: int, ctx: int, sets: int):
    P = 64
    width = ctx // P
    pages = batch * width + 1
    kv = [torch.randn(2, pages, NKV, P, D, device=DEV, dtype=torch.bfloat16) for _ in range(sets)]
    table = (torch.randperm(pages - 1)[: batch * width] + 1).to(torch.int32).view(batch, width).to(DEV)
    return kv, table


def attn_decode(sets: int = 2, B: int = 64, ctx: int = 2048):
    kv, table = _kv(B, ctx, sets)
    q = torch.randn(B, NQ * D, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=DEV)
    seg = torch.arange(B, dtype=torch.int32, device=DEV)
    ws = Workspace(DEV)

    def run(i):
        ops.attn_decode(q, out, kv[i % sets], None, B, pos, seg, table, NQ, NKV, D, D ** -0.5, None, ctx, ws)
    return run, B * ctx * 2 * NKV * D * 2, 4.0 * B * NQ * D * ctx, "hbm"


def attn_decode_32k():
    """8 decode rows with 32,768-token contexts (1.07 GB of K/V)."""
    return attn_decode(sets=1, B=8, ctx=32768)


def attn_prefill(sets: int = 1, tc: bool = False, T: int = 2048):
    kv, table = _kv(1, T, sets)
    q = torch.randn(T, NQ * D, device=DEV, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    tiles = list(range(0, T, 64))

    lists = (i32([0] * len(tiles)), i32(tiles), i32([0, T]), i32([0]))

    def run(i):
        if tc:
            ops.attn_prefill_tc(q, out, kv[0], *lists, table, NQ, NKV, D, D ** -0.5)
        else:
            ops.attn_prefill(q, out, kv[0], *lists, table, NQ, NKV, D, D ** -0.5, None)
    return run, 0, 4.0 * NQ * D * (T * (T + 1) / 2), "tensor"


def attn_prefill_tc():
    """One 2,048-token prompt, 48 heads of 128: tcgen05/TMEM with TMA-fed pages."""
    return attn_prefill(tc=True)


def attn_prefill_tc_8k():
    return attn_prefill(tc=True, T=8192)


def attn_prefill_8k():
    return attn_prefill(T=8192)


# ---- the same shapes through FlashInfer's trtllm-gen kernels (sm_100a cubins shipped
# with the flashinfer_cubin package): the reference's attention backend on this GPU
# (python/freetoken/attention/trtllm.py:62-100).  A comparison point only: nothing of
# the engine calls them.
def _flashinfer():
    try:
        import flashinfer
        return flashinfer
    except Exception as exc:           # not installed, or its launcher cannot be built here
        raise SystemExit(json.dumps({"unavailable": f"flashinfer does not import: {exc!r}"}))


def attn_decode_flashinfer(B: int = 64, ctx: int = 2048):
    fi = _flashinfer()
    kv, table = _kv(B, ctx, 2)
    q = torch.randn(B, NQ, D, device=DEV, dtype=torch.bfloat16)
    seq = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    work = torch.zeros(256 << 20, dtype=torch.uint8, device=DEV)

    def run(i):
        fi.decode.trtllm_batch_decode_with_kv_cache(q, (kv[i % 2][0], kv[i % 2][1]), work, table, seq, ctx,
                                                    bmm1_scale=D ** -0.5, bmm2_scale=1.0)
    return run, B * ctx * 2 * NKV * D * 2, 4.0 * B * NQ * D * ctx, "hbm"


def attn_decode_32k_flashinfer():
    return attn_decode_flashinfer(8, 32768)


def attn_prefill_flashinfer(T: int = 2048):
    fi = _flashinfer()
    kv, table = _kv(1, T, 1)
    q = torch.randn(T, NQ, D, device=DEV, dtype=torch.bfloat16)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    seq, cu = i32([T]), i32([0, T])
    work = torch.zeros(256 << 20, dtype=torch.uint8, device=DEV)

    def run(i):
        fi.prefill.trtllm_batch_context_with_kv_cache(q, (kv[0][0], kv[0][1]), work, table, seq, T, T,
                                                      D ** -0.5, 1.0, 1, cu, cu)
    return run, 0, 4.0 * NQ * D * (T * (T + 1) / 2), "tensor"


def attn_prefill_8k_flashinfer():
    return attn_prefill_flashinfer(8192)


# ---- the two denominators, measured the way the fallback figures were: a device-to-device
# copy (read + write bytes over time) and a large library bf16 product
def peak_copy():
    n = 1 << 30
    a = torch.empty(n, dtype=torch.uint8, device=DEV)
    b = torch.empty(n, dtype=torch.uint8, device=DEV)
    return (lambda i: b.copy_(a)), 2 * n, 0.0, "hbm"


def peak_read(gib: int = 4):
    """A read-only stream over 4 GiB (our own load-only kernel): the ceiling of a step that
    reads weights and cache and writes almost nothing."""
    a = torch.empty(gib << 30, dtype=torch.uint8, device=DEV)
    a.view(torch.int32).random_(0, 1 << 20)
    partial = torch.empty(8 * ops.sm_count(DEV), dtype=torch.int32, device=DEV)
    return (lambda i: ops.read_sum(a, partial)), gib << 30, 0.0, "hbm"


def peak_gemm():
    n = 8192
    a = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(n, n, device=DEV, dtype=torch.bfloat16)
    c = torch.empty(n, n, device=DEV, dtype=torch.bfloat16)
    return (lambda i: torch.matmul(a, b, out=c)), 0, 2.0 * n ** 3, "tensor"


def router(sets: int = 8):
    E, T, k = 256, 8, 8
    w = [torch.randn(E, H, device=DEV) * 0.02 for _ in range(sets)]
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    logits = torch.empty(T, E, device=DEV)
    ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, k, device=DEV)

    def run(i):
        ops.router_logits(x, w[i % sets], logits)
        ops.router_select(logits, None, ids, wts, k, False, True, 1.0)
    return run, E * H * 4, 0.0, "hbm"


KERNELS: Dict[str, Callable[[], Tuple[Callable[[int], None], int, float, str]]] = {
    "expert_gemv": expert_gemv, "lm_head": lm_head, "moe_gemm_tc": moe_gemm_tc, "moe_gemm_tc_busy": moe_gemm_tc_busy,
    "attn_decode": attn_decode, "attn_decode_32k": attn_decode_32k, "attn_prefill": attn_prefill, "attn_prefill_tc": attn_prefill_tc,
    "attn_prefill_8k": attn_prefill_8k, "attn_prefill_tc_8k": attn_prefill_tc_8k, "router": router,
    "peak_copy": peak_copy, "peak_read": peak_read, "peak_gemm": peak_gemm,
    "attn_decode_flashinfer": attn_decode_flashinfer, "attn_decode_32k_flashinfer": attn_decode_32k_flashinfer,
    "attn_prefill_flashinfer": attn_prefill_flashinfer, "attn_prefill_8k_flashinfer": attn_prefill_8k_flashinfer,
}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="kernel_bench")
    p.add_argument("--kernel", required=True, choices=sorted(KERNELS))
    p.add_argument("--reps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    a = p.parse_args(argv)
    run, nbytes, flops, bound = KERNELS[a.kernel]()
    for i in range(a.warmup):
        run(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(a.reps):
        run(a.warmup + i)
    end.record()
    torch.cuda.synchronize()
    ops.check_tc_status(DEV)
    ms = start.elapsed_time(end) / a.reps
    peaks = load_peaks()
    out = {"kernel": a.kernel, "ms": ms, "bytes": nbytes, "flops": flops, "peaks": peaks["source"]}
    if nbytes:
        out["GB/s"] = nbytes / ms / 1e6
        out["hbm_frac"] = out["GB/s"] / peaks["hbm_gbs"]
    if flops:
        out["TFLOP/s"] = flops / ms / 1e9
        out["tensor_frac"] = out["TFLOP/s"] / peaks["bf16_tflops"]
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
