"""Python faces of the CUDA launchers.

Each function checks what the kernel assumes (device, dtype, contiguity,
sizes), then calls the ``extern "C"`` launcher on the current CUDA stream.  A
non-zero return code raises :class:`KernelError`; nothing here computes on the
CPU or through a library in a kernel's place.
"""

from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from . import build

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

_C = {"p": ctypes.c_void_p, "i": ctypes.c_int, "q": ctypes.c_longlong, "f": ctypes.c_float}


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported a launch error."""


_ERRORS = {-101: "unsupported element type", -102: "unsupported shape or size",
           -103: "size beyond the kernel's limit"}


def code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels") from None


_bound = {}

# How many of this package's kernels were launched since the counter was last
# reset; a launcher that starts two kernels counts as two.
LAUNCHES = 0
_KERNELS_PER_CALL = {"ft_moe_sort": 2, "ft_attn_decode": 2}


def reset_launch_count() -> None:
    global LAUNCHES
    LAUNCHES = 0


def launch_count() -> int:
    return LAUNCHES


def _fn(lib: str, name: str, sig: str):
    key = (lib, name)
    f = _bound.get(key)
    if f is None:
        f = getattr(build.load(lib), name)
        f.argtypes = [_C[c] for c in sig.split()] + [ctypes.c_void_p]
        f.restype = ctypes.c_int
        _bound[key] = f
    return f


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, name: str) -> None:
    global LAUNCHES
    LAUNCHES += _KERNELS_PER_CALL.get("ft_" + name, 1)
    if rc != 0:
        what = _ERRORS.get(rc, f"CUDA error {rc}")
        raise KernelError(f"{name}: {what}")


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


# ------------------------------------------------------------------ rows
def embed_gather(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[t,:] = float(table[ids[t],:])"""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    _need(residual, "residual", torch.float32)
    T, H = residual.shape
    if table.shape[1] != H or ids.numel() != T:
        raise KernelError("embed_gather: shapes do not match")
    f = _fn("elementwise", "ft_embed_gather", "p p i p i i i")
    _check(f(_ptr(ids), _ptr(table), code(table.dtype), _ptr(residual), T, H, table.shape[0],
             _stream()), "embed_gather")


def patch_tokens(ids: torch.Tensor, rows: torch.Tensor, src: torch.Tensor, src_index: torch.Tensor,
                 vocab: int) -> None:
    """ids[rows[i]] = src[src_index[i]] (all int32, on the device)."""
    for name, t in (("ids", ids), ("rows", rows), ("src", src), ("src_index", src_index)):
        _need(t, name, torch.int32)
    if rows.numel() != src_index.numel():
        raise KernelError("patch_tokens: rows and src_index differ in length")
    f = _fn("elementwise", "ft_patch_tokens", "p p p p i i")
    _check(f(_ptr(ids), _ptr(rows), _ptr(src), _ptr(src_index), rows.numel(), vocab, _stream()),
           "patch_tokens")


def rmsnorm(delta: Optional[torch.Tensor], residual: torch.Tensor, weight: torch.Tensor,
            out: torch.Tensor, eps: float, plus_one: bool) -> None:
    """residual += delta (if given); out = residual * rsqrt(mean(residual^2)+eps) * (weight [+1]).

    ``delta`` may be ``[T, k, H]``: k partial rows per token, added in order."""
    _need(residual, "residual", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    T, H = residual.shape
    k = 1
    if delta is not None:
        _need(delta, "delta", out.dtype)
        if delta.dim() == 3:
            k = delta.shape[1]
        if delta.shape[0] != T or delta.shape[-1] != H or delta.dim() not in (2, 3):
            raise KernelError("rmsnorm: delta must be [T, H] or [T, k, H]")
    if out.shape != residual.shape or weight.numel() != H:
        raise KernelError("rmsnorm: shapes do not match")
    f = _fn("elementwise", "ft_rmsnorm", "p p p p i i i f i i")
    _check(f(_ptr(delta), _ptr(residual), _ptr(weight), _ptr(out), code(out.dtype), T, H,
             float(eps), int(plus_one), k, _stream()), "rmsnorm")


def qk_rope_store(qkv: torch.Tensor, q_out: torch.Tensor, kv_pages: Optional[torch.Tensor],
                  q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                  cos_sin: Optional[torch.Tensor], token_pos: torch.Tensor,
                  token_seg: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                  num_kv_heads: int, head_dim: int, rotary_dim: int, norm_mode: int,
                  plus_one: bool, interleaved: bool, eps: float) -> None:
    """QK norm (0 none, 1 per layer, 2 per head), partial rotary, K/V page store.

    ``kv_pages`` is ``[2, pages, kv_heads, page_size, head_dim]`` or ``None``
    for a stop that reads another stop's cache."""
    _need(qkv, "qkv", contiguous=False)
    _need(q_out, "q_out", qkv.dtype)
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width or qkv.stride(1) != 1:
        raise KernelError("qk_rope_store: qkv rows must be [q | k | v] with unit stride")
    for name, t in (("token_pos", token_pos), ("token_seg", token_seg), ("block_table", block_table)):
        _need(t, name, torch.int32)
    page_stride = kv_stride = 0
    P = 1
    if kv_pages is not None:
        _need(kv_pages, "kv_pages", qkv.dtype)
        if kv_pages.dim() != 5 or kv_pages.shape[0] != 2 or kv_pages.shape[2] != num_kv_heads \
                or kv_pages.shape[4] != head_dim:
            raise KernelError("qk_rope_store: kv_pages must be [2, pages, kv_heads, page, head_dim]")
        P = kv_pages.shape[3]
        page_stride, kv_stride = kv_pages.stride(1), kv_pages.stride(0)
    if norm_mode:
        want = (num_heads * head_dim, num_kv_heads * head_dim) if norm_mode == 1 else (head_dim, head_dim)
        _need(q_weight, "q_weight", torch.float32)
        _need(k_weight, "k_weight", torch.float32)
        if q_weight.numel() != want[0] or k_weight.numel() != want[1]:
            raise KernelError("qk_rope_store: norm weights have the wrong length")
    if rotary_dim:
        _need(cos_sin, "cos_sin", torch.float32)
        if cos_sin.shape[1] != rotary_dim:
            raise KernelError("qk_rope_store: cos_sin table width differs from rotary_dim")
    f = _fn("elementwise", "ft_qk_rope_store",
            "p p p p p p p p p q q q i i i i i i i i i f i i")
    _check(f(_ptr(qkv), _ptr(q_out), _ptr(kv_pages), _ptr(q_weight), _ptr(k_weight),
             _ptr(cos_sin) if rotary_dim else None, _ptr(token_pos), _ptr(token_seg),
             _ptr(block_table), qkv.stride(0), page_stride, kv_stride, num_heads, num_kv_heads,
             head_dim, rotary_dim, P, block_table.shape[1], norm_mode, int(plus_one),
             int(interleaved), float(eps), code(qkv.dtype), T, _stream()), "qk_rope_store")


def combine(parts: torch.Tensor, out: torch.Tensor, k: int) -> None:
    """out[t,:] = sum_j parts[t*k+j,:] (float32 sum, ascending j)"""
    _need(parts, "parts")
    _need(out, "out", parts.dtype)
    T, H = out.shape
    if parts.shape[0] != T * k or parts.shape[1] != H:
        raise KernelError("combine: shapes do not match")
    f = _fn("elementwise", "ft_combine", "p p i i i i")
    _check(f(_ptr(parts), _ptr(out), code(out.dtype), T, k, H, _stream()), "combine")


def read_sum(src: torch.Tensor, partial: torch.Tensor) -> None:
    """Stream ``src`` once (loads only) and leave a checksum per block in ``partial``
    (int32, one word per block: the grid): the measure of the GPU's read bandwidth."""
    _need(src, "src")
    _need(partial, "partial", torch.int32)
    nbytes = src.numel() * src.element_size()
    f = _fn("elementwise", "ft_read_sum", "p q p i")
    _check(f(_ptr(src), nbytes, _ptr(partial), partial.numel(), _stream()), "read_sum")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, dst: torch.Tensor) -> None:
    _need(src, "src")
    _need(rows, "rows", torch.int32)
    _need(dst, "dst", src.dtype)
    n, H = dst.shape
    if src.shape[1] != H or rows.numel() != n:
        raise KernelError("gather_rows: shapes do not match")
    f = _fn("elementwise", "ft_gather_rows", "p p p i i i")
    _check(f(_ptr(src), _ptr(rows), _ptr(dst), code(src.dtype), n, H, _stream()), "gather_rows")


# ------------------------------------------------------------------ gemm
def gemm_rows(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, *,
              group_offsets: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None,
              c_rows: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
              rows: Optional[int] = None, glu: bool = False, act: str = "silu",
              act_alpha: float = 1.702, act_limit: float = 7.0) -> None:
    """c = a @ w^T on CUDA cores in float32 (dense, or grouped by expert).

    ``w`` is ``[N_w, K]`` or ``[G, N_w, K]``; with ``glu`` the N outputs are
    ``act(w[:N] a) * (w[N:] a)``.  ``rows`` is the number of (sorted) rows when
    ``a_rows`` / ``c_rows`` redirect them."""
    _need(a, "a", contiguous=False)
    _need(w, "w")
    _need(c, "c", contiguous=False)
    if w.dim() == 2:
        G, NW, K = 1, w.shape[0], w.shape[1]
    else:
        G, NW, K = w.shape
    N = NW // 2 if glu else NW
    M = rows if rows is not None else a.shape[0]
    if a.shape[1] != K or c.shape[1] != N or a.stride(1) != 1 or c.stride(1) != 1:
        raise KernelError("gemm_rows: shapes do not match")
    if (w.dim() == 3) != (group_offsets is not None):
        raise KernelError("gemm_rows: group_offsets must be given exactly for grouped ([G, N, K]) weights")
    for name, t in (("group_offsets", group_offsets), ("a_rows", a_rows), ("c_rows", c_rows)):
        if t is not None:
            _need(t, name, torch.int32)
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32)
    f = _fn("gemm_simt", "ft_gemm_rows", "p i q p i q p i q p p p p i i i i i i f f")
    _check(f(_ptr(a), code(a.dtype), a.stride(0), _ptr(w), code(w.dtype), NW * K, _ptr(c),
             code(c.dtype), c.stride(0), _ptr(group_offsets), _ptr(a_rows), _ptr(c_rows),
             _ptr(row_scale), M, N, K, G, int(glu), 0 if act == "silu" else 1, float(act_alpha),
             float(act_limit), _stream()), "gemm_rows")


def skinny_gemm_takes(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> bool:
    """Whether the weight-streaming tensor-core kernel takes these operands."""
    K = w.shape[-1]
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and c.dtype in (torch.bfloat16, torch.float32)
            and K % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1 and c.stride(1) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def skinny_gemm(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, *,
                group_offsets: Optional[torch.Tensor] = None,
                active: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None,
                c_rows: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
                rows: Optional[int] = None, glu: bool = False, act: str = "silu",
                act_alpha: float = 1.702, act_limit: float = 7.0, rows_per_pass: int = 8) -> None:
    """c = a @ w^T for few rows, streaming bfloat16 weights once through
    mma.sync; same conventions as :func:`gemm_rows`."""
    _need(a, "a", torch.bfloat16, contiguous=False)
    _need(w, "w", torch.bfloat16)
    _need(c, "c", contiguous=False)
    if w.dim() == 2:
        G, NW, K = 1, w.shape[0], w.shape[1]
    else:
        G, NW, K = w.shape
    N = NW // 2 if glu else NW
    M = rows if rows is not None else a.shape[0]
    if a.shape[1] != K or c.shape[1] != N:
        raise KernelError("skinny_gemm: shapes do not match")
    if not skinny_gemm_takes(a, w, c):
        raise KernelError("skinny_gemm: needs bfloat16 operands, K % 8 == 0 and 16-byte aligned rows")
    if (w.dim() == 3) != (group_offsets is not None):
        raise KernelError("skinny_gemm: group_offsets must be given exactly for grouped ([G, N, K]) weights")
    if rows_per_pass not in (8, 16, 32):
        raise KernelError("skinny_gemm: rows_per_pass must be 8, 16 or 32")
    if active is not None:
        _need(active, "active", torch.int32)
        if active.numel() < G + 1:
            raise KernelError("skinny_gemm: the active list needs G + 1 entries")
    f = _fn("skinny_gemm", "ft_skinny_gemm", "p q p q p i q p p p p p i i i i i i f f i")
    _check(f(_ptr(a), a.stride(0), _ptr(w), NW * K, _ptr(c), code(c.dtype), c.stride(0),
             _ptr(group_offsets), _ptr(active), _ptr(a_rows), _ptr(c_rows), _ptr(row_scale), M, N, K, G,
             int(glu), 0 if act == "silu" else 1, float(act_alpha), float(act_limit),
             rows_per_pass, _stream()), "skinny_gemm")


# ------------------------------------------------ grouped GEMM on tcgen05
_TC_MAPS = {}
_TC_STATUS = {}


def tc_status(device) -> torch.Tensor:
    """The device word in which a tcgen05 kernel records a wait that ran out."""
    idx = torch.device(device).index or 0
    if idx not in _TC_STATUS:
        _TC_STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _TC_STATUS[idx]


def _status_table() -> Dict[int, tuple]:
    """``{code: (kernel, role)}`` read from the ``X(name, code, "kernel", "role")``
    lines of ``status_codes.h``, the header the kernels take the numbers from."""
    global _STATUS_TABLE
    if _STATUS_TABLE is None:
        import re
        text = open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "status_codes.h")).read()
        _STATUS_TABLE = {int(c): (kernel, role) for _, c, kernel, role in
                         re.findall(r'X\((\w+),\s*(\d+),\s*"([^"]+)",\s*"([^"]+)"\)', text)}
    return _STATUS_TABLE


_STATUS_TABLE: Optional[Dict[int, tuple]] = None


def status_message(code_: int) -> str:
    kernel, role = _status_table().get(int(code_), ("a kernel", "a role"))
    return f"{kernel}: {role} waited on a barrier beyond its limit and gave up (code {int(code_)})"


def raise_for_status(code_: int, device) -> None:
    """Turn a status code that was read from the device into a :class:`KernelError`
    and clear the device word, so that the next check reports new failures only."""
    if code_:
        tc_status(device).zero_()
        raise KernelError(status_message(code_))


def check_tc_status(device) -> None:
    """Raise if a kernel gave up a bounded wait since the last check (synchronises)."""
    idx = torch.device(device).index or 0
    if idx in _TC_STATUS:
        raise_for_status(int(_TC_STATUS[idx].item()), device)


def wait_selftest(device, limit_ns: int, arrive: bool) -> None:
    """Launch one block whose first thread waits up to ``limit_ns`` on a barrier
    that is arrived at only if ``arrive``: the bounded wait every tcgen05 / TMA
    kernel here uses, made to run out on purpose (nothing hangs: the wait ends
    by its own limit and the kernel returns)."""
    f = _fn("moe_gemm_tc", "ft_wait_selftest", "p q i")
    with torch.cuda.device(torch.device(device)):
        _check(f(_ptr(tc_status(device)), int(limit_ns), int(bool(arrive)), _stream()), "wait_selftest")


def _tc_map(t: torch.Tensor, rows: int, K: int, row_stride: int, groups: int, box_rows: int):
    key = (t.data_ptr(), rows, K, row_stride, groups, box_rows)
    m = _TC_MAPS.get(key)
    if m is None:
        if len(_TC_MAPS) > 4096:
            _TC_MAPS.clear()
        m = ctypes.create_string_buffer(128)
        f = getattr(build.load("moe_gemm_tc"), "ft_tc_make_map")
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong,
                      ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int]
        f.restype = ctypes.c_int
        rc = f(ctypes.cast(m, ctypes.c_void_p), t.data_ptr(), groups, rows, K, row_stride, box_rows)
        if rc != 0:
            raise KernelError(f"moe_gemm_tc: cannot build a tensor map (code {rc})")
        _TC_MAPS[key] = m
    return m


def moe_gemm_tc_takes(x: torch.Tensor, w: torch.Tensor, c: torch.Tensor) -> bool:
    K = w.shape[-1]
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and c.dtype == torch.bfloat16
            and w.dim() == 3 and w.is_contiguous() and K % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and c.stride(1) == 1)


# From this many sorted rows per expert (on average) gate_up + GLU runs token-major: the
# tokens are the MMA's M operand, gate and up rows one N operand of 256 (measured with 256
# experts of real width against the weight-major form: 767 against 758 us at 64 rows per
# expert, level at 96, 905 against 919 at 128, 1,115 against 1,191 at 192, 1,343 against
# 1,480 at 256).  The down projection is token-major at every load.
TC_GLU_TOKEN_MAJOR_FROM_ROWS = int(os.environ.get("FREETOKEN_TC_GLU_TOKEN_MAJOR_FROM_ROWS", "112"))
TC_TOKENS_PER_TILE = 128


def moe_tile_map(group_offsets: torch.Tensor, active: torch.Tensor, rows: int, groups: int,
                 workspace) -> torch.Tensor:
    """The tile list of the tcgen05 grouped GEMM: one int32 quadruple per (busy expert,
    tile of up to 128 sorted rows): expert, first row, rows the MMA covers, end of the
    expert's rows.  An expert's rows are dealt out evenly over its tiles."""
    for name, t in (("group_offsets", group_offsets), ("active", active)):
        _need(t, name, torch.int32)
    bound = -(-rows // TC_TOKENS_PER_TILE) + min(groups, rows)
    tile_info = workspace.get("moe.tile_info", (bound, 4), torch.int32)
    f = _fn("moe_gemm_tc", "ft_moe_tile_map", "p p p i i i")
    _check(f(_ptr(group_offsets), _ptr(active), _ptr(tile_info), rows, groups, TC_TOKENS_PER_TILE, _stream()),
           "moe_tile_map")
    return tile_info


def moe_gemm_tc(x: torch.Tensor, w: torch.Tensor, c: torch.Tensor, *, tile_map: torch.Tensor,
                c_rows: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
                rows: int, glu: bool = False, token_major: bool = True, act: str = "silu",
                act_alpha: float = 1.702, act_limit: float = 7.0) -> None:
    """Grouped expert GEMM on tcgen05/TMEM fed by TMA.  ``x`` holds the sorted
    rows ``[>= rows, K]`` (already gathered), ``w`` is ``[G, N_w, K]``; same
    output conventions as :func:`gemm_rows`.  ``tile_map`` comes from :func:`moe_tile_map`.
    ``token_major``: up to 128 tokens are the MMA's M operand and 256 weight rows its N
    operand (with ``glu``: 128 gate rows and the 128 up rows of the same features), a thread
    of the epilogue owns a token and stores 16 features at a time; otherwise (``glu`` only)
    the weights are the M operand, gate and up two accumulators, and a tile is as narrow
    as the tokens it holds."""
    if not moe_gemm_tc_takes(x, w, c):
        raise KernelError("moe_gemm_tc: needs bfloat16 operands, K % 8 == 0 and 16-byte aligned rows")
    if not glu and not token_major:
        raise KernelError("moe_gemm_tc: the weight-major form exists with GLU only")
    G, NW, K = w.shape
    N = NW // 2 if glu else NW
    if x.shape[1] != K or c.shape[1] != N:
        raise KernelError("moe_gemm_tc: shapes do not match")
    form = (1 if token_major else 0) if glu else 2
    map_w = _tc_map(w, NW, K, K, G, 128)
    # the token rows through boxes of 64 and 128 rows: a tile takes the smaller if it holds it
    key = ("x2", x.data_ptr(), x.shape[0], K, x.stride(0))
    maps_x = _TC_MAPS.get(key)
    if maps_x is None:
        joined = b"".join(bytes(_tc_map(x, x.shape[0], K, x.stride(0), 0, box)) for box in (64, 128))
        maps_x = _TC_MAPS[key] = ctypes.create_string_buffer(joined, 256)
    status = tc_status(x.device)
    f = _fn("moe_gemm_tc", "ft_moe_gemm_tc", "p p p q p p p p i i i i i i i f f")
    _check(f(ctypes.cast(map_w, ctypes.c_void_p), ctypes.cast(maps_x, ctypes.c_void_p), _ptr(c),
             c.stride(0), _ptr(tile_map), _ptr(c_rows), _ptr(row_scale), _ptr(status), rows, N, K, G,
             TC_TOKENS_PER_TILE, form, 0 if act == "silu" else 1, float(act_alpha), float(act_limit),
             _stream()), "moe_gemm_tc")


def moe_experts_tc(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, mid: torch.Tensor,
                   parts: torch.Tensor, group_offsets: torch.Tensor, active: torch.Tensor,
                   sorted_route: torch.Tensor, sorted_token: torch.Tensor, route_weight: torch.Tensor,
                   rows: int, act: str, act_alpha: float, act_limit: float, workspace) -> None:
    """Both expert products of a step on the tcgen05 grouped GEMM:
    ``mid[sorted row] = act(Wgate x) * (Wup x)`` over the routes sorted by expert,
    then ``parts[route] = route_weight[route] * (Wdown mid)``.  ``x`` is ``[T, H]``,
    ``sorted_token`` / ``sorted_route`` give the token and the route of every sorted
    row, ``group_offsets`` / ``active`` come from :func:`moe_sort`."""
    G = w_gate_up.shape[0]
    xs = workspace.get("moe.sorted_x", (rows, x.shape[1]), x.dtype)
    gather_rows(x, sorted_token, xs)
    tiles = moe_tile_map(group_offsets, active, rows, G, workspace)
    busy_experts = -(-rows // max(1, G)) >= TC_GLU_TOKEN_MAJOR_FROM_ROWS
    moe_gemm_tc(xs, w_gate_up, mid, tile_map=tiles, rows=rows, glu=True, token_major=busy_experts, act=act,
                act_alpha=act_alpha, act_limit=act_limit)
    moe_gemm_tc(mid, w_down, parts, tile_map=tiles, c_rows=sorted_route, row_scale=route_weight, rows=rows)


def pass_rows(rows: int) -> int:
    """Tokens per pass of the skinny kernel for ``rows`` rows (per group)."""
    return 8 if rows <= 8 else (16 if rows <= 16 else 32)


# ------------------------------------------------------------- attention
def attn_paged_simt(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor,
                    token_pos: torch.Tensor, token_seg: torch.Tensor, block_table: torch.Tensor,
                    num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                    window: Optional[int], rows: Optional[torch.Tensor] = None) -> None:
    """Generic paged attention; ``rows`` limits it to those token rows."""
    _need(q, "q")
    _need(out, "out", q.dtype)
    _need(kv_pages, "kv_pages", q.dtype)
    for name, t in (("token_pos", token_pos), ("token_seg", token_seg), ("block_table", block_table)):
        _need(t, name, torch.int32)
    T = q.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if q.shape[1] != num_heads * head_dim or out.shape != q.shape:
        raise KernelError("attn_paged_simt: q/out must be [T, heads*head_dim]")
    f = _fn("attention_simt", "ft_attn_paged_simt", "p p p p p p p q q i i i i i i f i i")
    _check(f(_ptr(q), _ptr(out), _ptr(kv_pages), _ptr(token_pos), _ptr(token_seg),
             _ptr(block_table), _ptr(rows), kv_pages.stride(1), kv_pages.stride(0), num_heads, num_kv_heads,
             head_dim, kv_pages.shape[3], block_table.shape[1], int(window or 0), float(scale),
             code(q.dtype), T, _stream()), "attn_paged_simt")


DECODE_HEAD_DIMS = (32, 64, 128)
_SM_COUNT = {}


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def attn_decode_takes(q: torch.Tensor, head_dim: int) -> bool:
    return q.dtype == torch.bfloat16 and head_dim in DECODE_HEAD_DIMS


# Decode attention with K/V tiles fetched by TMA where the shapes allow it
# (FREETOKEN_DECODE_TMA=0: always the cp.async kernel).
DECODE_TMA = os.environ.get("FREETOKEN_DECODE_TMA", "1") not in ("", "0")
# ... and up to eight splits merged inside that kernel by a thread-block cluster
# (FREETOKEN_DECODE_CLUSTER=0: partials in global memory and the merge kernel).
DECODE_CLUSTER = os.environ.get("FREETOKEN_DECODE_CLUSTER", "1") not in ("", "0")


CLUSTER_SPLITS = 8     # splits the TMA-fed decode kernel merges by itself (a thread-block cluster)
MERGE_COST = 24        # what the separate merge kernel costs, in 64-key tiles of a CTA's work


def decode_splits(n_rows: int, num_kv_heads: int, group: int, max_kv_len: int, sms: int,
                  cluster_merge: bool = False):
    """``(splits, keys per split)``, whole 64-key tiles per split.

    Two CTAs of the decode kernel fit an SM and a launch takes as long as its
    rounds of CTAs: rounds x (tiles per split + a CTA's fixed cost, about three
    tiles' worth: query load, pipeline fill, partial write).  The split count with
    the least such time is taken, the smaller one on a tie - not just "enough
    CTAs to fill the SMs", which leaves a second round nearly empty at some
    sizes.  With ``cluster_merge`` up to :data:`CLUSTER_SPLITS` splits are merged
    inside the kernel; more need the merge kernel, whose launch is counted."""
    base = max(1, n_rows * num_kv_heads * (-(-group // 16)))
    tiles = max(1, -(-max_kv_len // 64))
    slots = 2 * sms
    best, best_cost = 1, None
    for want in range(1, min(tiles, 64) + 1):
        per = -(-tiles // want)
        splits = -(-tiles // per)
        if splits != want:
            continue                      # the same split as a smaller request
        rounds = -(-base * splits // slots)
        cost = rounds * (per + 3)
        if cluster_merge and splits > CLUSTER_SPLITS:
            cost += MERGE_COST
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    per = -(-tiles // best)
    return -(-tiles // per), per * 64


def attn_decode(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor,
                rows: Optional[torch.Tensor], n_rows: int, token_pos: torch.Tensor,
                token_seg: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                max_kv_len: int, workspace) -> None:
    """Split-KV tensor-core attention for single-token rows (bfloat16)."""
    _need(q, "q", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(kv_pages, "kv_pages", torch.bfloat16)
    if not attn_decode_takes(q, head_dim):
        raise KernelError(f"attn_decode: head_dim {head_dim} not in {DECODE_HEAD_DIMS}")
    for name, t in (("token_pos", token_pos), ("token_seg", token_seg), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if rows is not None:
        _need(rows, "rows", torch.int32)
    tma = DECODE_TMA and head_dim in (64, 128) and kv_pages.shape[3] % 64 == 0 \
        and kv_pages.stride(4) == 1 and kv_pages.stride(3) == head_dim
    splits, split_keys = decode_splits(n_rows, num_kv_heads, num_heads // num_kv_heads, max_kv_len,
                                       sm_count(q.device), cluster_merge=tma and DECODE_CLUSTER)
    part_o = part_ml = None
    if splits > 1 and not (tma and DECODE_CLUSTER and splits <= CLUSTER_SPLITS):
        part_o = workspace.get("attn.part_o", (n_rows, num_heads, splits, head_dim), torch.float32)
        part_ml = workspace.get("attn.part_ml", (n_rows, num_heads, splits, 2), torch.float32)
    if tma:
        # K and V tiles by TMA: a tile lies inside one page
        lib = build.load("attention_prefill_tc")

        def make_kv(dst):
            mk = lib.ft_attn_tc_kv_map
            mk.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_longlong] * 7
            mk.restype = ctypes.c_int
            return mk(dst, kv_pages.data_ptr(), kv_pages.shape[1], kv_pages.shape[2], kv_pages.shape[3],
                      head_dim, kv_pages.stride(2), kv_pages.stride(1), kv_pages.stride(0))
        map_kv = _attn_tc_map("kv", (kv_pages.data_ptr(),) + tuple(kv_pages.shape) + tuple(kv_pages.stride()),
                              make_kv)
        f = _fn("attention_decode_tma", "ft_attn_decode_tma", "p p p p p p p p p p i i i i i i i i i f")
        _check(f(ctypes.cast(map_kv, ctypes.c_void_p), _ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml),
                 _ptr(rows), _ptr(token_pos), _ptr(token_seg), _ptr(block_table), _ptr(tc_status(q.device)),
                 num_heads, num_kv_heads, head_dim, kv_pages.shape[3], block_table.shape[1],
                 int(window or 0), n_rows, splits, split_keys, float(scale), _stream()), "attn_decode_tma")
        if part_o is not None:
            fm = _fn("attention_decode", "ft_attn_merge", "p p p p i i i i")
            _check(fm(_ptr(part_o), _ptr(part_ml), _ptr(out), _ptr(rows), n_rows, num_heads, head_dim,
                      splits, _stream()), "attn_merge")
        return
    f = _fn("attention_decode", "ft_attn_decode", "p p p p p p p p p q q i i i i i i i i i f")
    _check(f(_ptr(q), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(kv_pages), _ptr(rows),
             _ptr(token_pos), _ptr(token_seg), _ptr(block_table), kv_pages.stride(1),
             kv_pages.stride(0), num_heads, num_kv_heads, head_dim, kv_pages.shape[3],
             block_table.shape[1], int(window or 0), n_rows, splits, split_keys, float(scale),
             _stream()), "attn_decode")


def attn_prefill(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor,
                 tile_seg: torch.Tensor, tile_q0: torch.Tensor, seg_q_start: torch.Tensor,
                 seg_pos0: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                 num_kv_heads: int, head_dim: int, scale: float, window: Optional[int]) -> None:
    """Tensor-core causal attention for the query tiles (64 tokens) listed in
    ``tile_seg`` / ``tile_q0`` (bfloat16; head sizes of :data:`DECODE_HEAD_DIMS`)."""
    _need(q, "q", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(kv_pages, "kv_pages", torch.bfloat16)
    if not attn_decode_takes(q, head_dim):
        raise KernelError(f"attn_prefill: head_dim {head_dim} not in {DECODE_HEAD_DIMS}")
    for name, t in (("tile_seg", tile_seg), ("tile_q0", tile_q0), ("seg_q_start", seg_q_start),
                    ("seg_pos0", seg_pos0), ("block_table", block_table)):
        _need(t, name, torch.int32)
    f = _fn("attention_prefill", "ft_attn_prefill", "p p p p p p p p q q i i i i i i i f")
    _check(f(_ptr(q), _ptr(out), _ptr(kv_pages), _ptr(tile_seg), _ptr(tile_q0), _ptr(seg_q_start),
             _ptr(seg_pos0), _ptr(block_table), kv_pages.stride(1), kv_pages.stride(0), num_heads,
             num_kv_heads, head_dim, kv_pages.shape[3], block_table.shape[1], int(window or 0),
             tile_seg.numel(), float(scale), _stream()), "attn_prefill")


# A step whose prompt portions score at least this many query-key pairs uses the
# tcgen05 kernel (tiles of 128 queries, a pipeline of about 20 us to fill);
# smaller ones keep the 64-query mma.sync tiles.  Measured crossover on a B200
# at 48 heads of 128: between 256 and 512 fresh tokens, or 64 tokens on a
# 4,096-token prefix.
PREFILL_TC_MIN_SCORES = int(os.environ.get("FREETOKEN_PREFILL_TC_MIN_SCORES", "100000"))
_ATTN_TC_MAPS: Dict[tuple, ctypes.Array] = {}


def _attn_tc_map(kind: str, key: tuple, make) -> ctypes.Array:
    m = _ATTN_TC_MAPS.get((kind,) + key)
    if m is None:
        if len(_ATTN_TC_MAPS) > 4096:
            _ATTN_TC_MAPS.clear()
        m = ctypes.create_string_buffer(128)
        rc = make(ctypes.cast(m, ctypes.c_void_p))
        if rc != 0:
            raise KernelError(f"attn_prefill_tc: cannot build the {kind} tensor map (code {rc})")
        _ATTN_TC_MAPS[(kind,) + key] = m
    return m


def attn_prefill_tc_takes(q: torch.Tensor, kv_pages: torch.Tensor, head_dim: int,
                          window: Optional[int]) -> bool:
    """bfloat16, head size 64 or 128, pages of a multiple of 64 tokens, all keys visible."""
    return (q.dtype == torch.bfloat16 and kv_pages.dtype == torch.bfloat16 and head_dim in (64, 128)
            and window is None and kv_pages.shape[3] % 64 == 0 and q.stride(1) == 1
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and kv_pages.data_ptr() % 16 == 0
            and kv_pages.stride(4) == 1 and kv_pages.stride(3) == head_dim)


def attn_prefill_tc(q: torch.Tensor, out: torch.Tensor, kv_pages: torch.Tensor,
                    tile_seg: torch.Tensor, tile_q0: torch.Tensor, seg_q_start: torch.Tensor,
                    seg_pos0: torch.Tensor, block_table: torch.Tensor, num_heads: int,
                    num_kv_heads: int, head_dim: int, scale: float) -> None:
    """Causal attention on tcgen05/TMEM with K and V pages fetched by TMA, for the
    query tiles (64 tokens; the kernel pairs them) in ``tile_seg`` / ``tile_q0``."""
    _need(q, "q", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    if not attn_prefill_tc_takes(q, kv_pages, head_dim, None) or not out.is_contiguous():
        raise KernelError("attn_prefill_tc: refuses these tensors (bfloat16, head_dim 64/128, page % 64 == 0)")
    for name, t in (("tile_seg", tile_seg), ("tile_q0", tile_q0), ("seg_q_start", seg_q_start),
                    ("seg_pos0", seg_pos0), ("block_table", block_table)):
        _need(t, name, torch.int32)
    lib = build.load("attention_prefill_tc")
    T, cols = q.shape

    def make_q(box_rows):
        def make(dst):
            f = lib.ft_attn_tc_q_map
            f.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_longlong] * 3 + [ctypes.c_int]
            f.restype = ctypes.c_int
            return f(dst, q.data_ptr(), T, cols, q.stride(0), box_rows)
        return make

    def make_kv(dst):
        f = lib.ft_attn_tc_kv_map
        f.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_longlong] * 7
        f.restype = ctypes.c_int
        return f(dst, kv_pages.data_ptr(), kv_pages.shape[1], kv_pages.shape[2], kv_pages.shape[3],
                 head_dim, kv_pages.stride(2), kv_pages.stride(1), kv_pages.stride(0))

    map_q = _attn_tc_map("q", (q.data_ptr(), T, cols, q.stride(0)), make_q(128))
    map_q2 = _attn_tc_map("q2", (q.data_ptr(), T, cols, q.stride(0)), make_q(64))
    map_kv = _attn_tc_map("kv", (kv_pages.data_ptr(),) + tuple(kv_pages.shape) + tuple(kv_pages.stride()),
                          make_kv)
    status = tc_status(q.device)
    f = _fn("attention_prefill_tc", "ft_attn_prefill_tc", "p p p p p p p p p p i i i i i i f")
    _check(f(ctypes.cast(map_q, ctypes.c_void_p), ctypes.cast(map_q2, ctypes.c_void_p),
             ctypes.cast(map_kv, ctypes.c_void_p), _ptr(out),
             _ptr(tile_seg), _ptr(tile_q0), _ptr(seg_q_start), _ptr(seg_pos0), _ptr(block_table),
             _ptr(status), num_heads, num_kv_heads, head_dim, kv_pages.shape[3], block_table.shape[1],
             tile_seg.numel(), float(scale), _stream()), "attn_prefill_tc")


# ---------------------------------------------------------------- router
def router_select(logits: torch.Tensor, bias: Optional[torch.Tensor], ids: torch.Tensor,
                  weights: torch.Tensor, k: int, softmax_scoring: bool, renormalize: bool,
                  scale: float, terms: int = 1) -> None:
    """Top-k of the scored router logits.  With ``terms`` > 1 a row of ``logits``
    holds that many partial logits per expert (``[T, terms * E]``), summed in
    order in float32 before scoring."""
    _need(logits, "logits", torch.float32)
    _need(ids, "ids", torch.int32)
    _need(weights, "weights", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    T, E = logits.shape[0], logits.shape[1] // terms
    if logits.shape[1] != E * terms or not logits.is_contiguous():
        raise KernelError(f"router_select: logits {tuple(logits.shape)} do not hold {terms} terms per expert")
    f = _fn("moe_route", "ft_router_select", "p p p p i i i i i f i")
    _check(f(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(weights), T, E, k, int(softmax_scoring),
             int(renormalize), float(scale), int(terms), _stream()), "router_select")


ROUTE_SMALL_MAX_T = 8


def route_small_takes(T: int, E: int, k: int) -> bool:
    """A handful of tokens: selection and route sort fit one block."""
    return T <= ROUTE_SMALL_MAX_T and k <= 32 and (T * 2 * E + T * k + 2 * E) * 4 <= 160 * 1024


def route_small(logits: torch.Tensor, bias: Optional[torch.Tensor], ids: torch.Tensor,
                weights: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor,
                sorted_route: torch.Tensor, sorted_token: torch.Tensor, active: torch.Tensor, k: int,
                softmax_scoring: bool, renormalize: bool, scale: float, terms: int = 1) -> None:
    """:func:`router_select` and :func:`moe_sort` in one launch (same results)."""
    _need(logits, "logits", torch.float32)
    _need(weights, "weights", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    for name, t in (("ids", ids), ("counts", counts), ("offsets", offsets),
                    ("sorted_route", sorted_route), ("sorted_token", sorted_token), ("active", active)):
        _need(t, name, torch.int32)
    T, E = logits.shape[0], logits.shape[1] // terms
    R = T * k
    if logits.shape[1] != E * terms or not route_small_takes(T, E, k):
        raise KernelError(f"route_small: refuses {T} tokens, {E} experts, top-{k}")
    if counts.numel() < E or offsets.numel() < E + 1 or sorted_route.numel() < R \
            or sorted_token.numel() < R or active.numel() < E + 1 or ids.numel() < R or weights.numel() < R:
        raise KernelError("route_small: output buffers are too small")
    f = _fn("moe_route", "ft_route_small", "p p p p p p p p p i i i i i f i")
    _check(f(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(weights), _ptr(counts), _ptr(offsets),
             _ptr(sorted_route), _ptr(sorted_token), _ptr(active), T, E, k, int(softmax_scoring),
             int(renormalize), float(scale), int(terms), _stream()), "route_small")


def router_logits_takes(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.dtype == torch.float32)


def router_logits(x: torch.Tensor, w: torch.Tensor, logits: torch.Tensor) -> None:
    """logits = x @ w^T in float32 for few tokens (a warp per expert row and 8 tokens)."""
    _need(x, "x", contiguous=False)
    _need(w, "w", torch.float32)
    _need(logits, "logits", torch.float32)
    T, H = x.shape
    E = w.shape[0]
    if w.shape[1] != H or logits.shape != (T, E) or x.stride(1) != 1:
        raise KernelError("router_logits: shapes do not match")
    f = _fn("moe_route", "ft_router_logits", "p i q p p i i i")
    _check(f(_ptr(x), code(x.dtype), x.stride(0), _ptr(w), _ptr(logits), T, E, H, _stream()),
           "router_logits")


def moe_sort(ids: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor,
             sorted_route: torch.Tensor, sorted_token: torch.Tensor, active: torch.Tensor,
             num_experts: int, k: int, scratch: Optional[torch.Tensor] = None) -> None:
    """Stable counting sort of the ``T*k`` routes by expert; ``active`` gets the
    experts that have routes (ascending) and, at index ``num_experts``, their number.
    With ``scratch`` (int32, :func:`moe_sort_scratch` elements) the routes are
    sorted in chunks, which is faster from a few thousand routes on."""
    for name, t in (("ids", ids), ("counts", counts), ("offsets", offsets),
                    ("sorted_route", sorted_route), ("sorted_token", sorted_token),
                    ("active", active)):
        _need(t, name, torch.int32)
    R = ids.numel()
    if counts.numel() < num_experts or offsets.numel() < num_experts + 1 \
            or sorted_route.numel() < R or sorted_token.numel() < R \
            or active.numel() < num_experts + 1:
        raise KernelError("moe_sort: output buffers are too small")
    if scratch is not None:
        _need(scratch, "scratch", torch.int32)
        if scratch.numel() < moe_sort_scratch(R, num_experts):
            raise KernelError("moe_sort: the scratch buffer is too small")
    f = _fn("moe_route", "ft_moe_sort", "p p p p p p p i i i")
    _check(f(_ptr(ids), _ptr(counts), _ptr(offsets), _ptr(sorted_route), _ptr(sorted_token),
             _ptr(active), _ptr(scratch), R, num_experts, k, _stream()), "moe_sort")
    if scratch is not None:
        global LAUNCHES
        LAUNCHES += 1      # three kernels instead of two


MOE_SORT_CHUNKED_FROM = 2048   # routes from which the chunked sort is used


def moe_sort_scratch(routes: int, num_experts: int) -> int:
    """int32 elements of scratch the chunked sort needs."""
    return -(-routes // 256) * num_experts


# -------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], uniform: Optional[torch.Tensor], out: torch.Tensor,
           probs: Optional[torch.Tensor]) -> None:
    """Per row: argmax when its temperature <= 0 (or none given), else a
    temperature / top-k / top-p inverse-CDF draw with the row's uniform."""
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32)
    rows, V = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
        _need(uniform, "uniform", torch.float32)
        _need(probs, "probs", torch.float32)
        if probs.numel() < rows * V:
            raise KernelError("sample: probs scratch is too small")
    if top_k is not None:
        _need(top_k, "top_k", torch.int32)
    if top_p is not None:
        _need(top_p, "top_p", torch.float32)
    f = _fn("sampling", "ft_sample", "p p p p p p p i i")
    _check(f(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(uniform), _ptr(out),
             _ptr(probs), rows, V, _stream()), "sample")
