"""ft_sample_static, the sampler entry point that allocates nothing.

Some hosts of the sampling kernel cannot obtain device memory when they call it
(a fixed memory budget, an allocator they must not touch, a plain C program
without PyTorch's caching allocator).  For them the library carries its own
scratch array; this test calls that entry point through its exported C symbol,
the way such a host would, and checks it against the ordinary entry point, whose
scratch the caller brings.  It runs last so that a failure here cannot hide
another test's result.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 1 << 20
TOO_LARGE = -103


def _symbol():
    from freetoken_b200.csrc import build
    fn = build.load("sampling").ft_sample_static
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def _case(rows, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(rows, vocab, generator=g) * 2).cuda()
    temps = torch.tensor([0.0, 0.8, 1.0, 0.6, 1.2][:rows], device="cuda")
    top_k = torch.tensor([0, 0, 7, 0, 50][:rows], dtype=torch.int32, device="cuda")
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.7, 0.9][:rows], device="cuda")
    u = torch.rand(rows, generator=g).cuda()
    return logits, temps, top_k, top_p, u


def test_static_sampler_matches_the_allocating_one_twice_in_a_row():
    from freetoken_b200.csrc import ops
    fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes: the second finds the first one's
    # leftovers in the shared scratch and must not be disturbed by them
    for rows, vocab, seed in ((5, 200064, 1), (4, 1000, 2)):
        logits, temps, top_k, top_p, u = _case(rows, vocab, seed)
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        ops.sample(logits, temps, top_k, top_p, u, want, torch.empty(rows * vocab, device="cuda"))
        got = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        rc = fn(logits.data_ptr(), temps.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                u.data_ptr(), got.data_ptr(), rows, vocab, stream)
        assert rc == 0
        torch.cuda.synchronize()
        # same kernel, same arithmetic: the chosen tokens are identical
        assert got.tolist() == want.tolist()
    # all-greedy call without temperature, filters or uniforms
    logits = _case(3, 777, 3)[0]
    got = torch.empty(3, dtype=torch.int32, device="cuda")
    assert fn(logits.data_ptr(), None, None, None, None, got.data_ptr(), 3, 777, stream) == 0
    torch.cuda.synchronize()
    assert got.tolist() == logits.argmax(-1).tolist()


def test_static_sampler_refuses_more_than_its_scratch_holds():
    fn = _symbol()
    rows, vocab = 6, 200064                      # 6 * 200064 > 2^20
    assert rows * vocab > STATIC_FLOATS
    logits = torch.zeros(rows, vocab, device="cuda")
    out = torch.full((rows,), -5, dtype=torch.int32, device="cuda")
    rc = fn(logits.data_ptr(), None, None, None, None, out.data_ptr(), rows, vocab,
            torch.cuda.current_stream().cuda_stream)
    assert rc == TOO_LARGE
    torch.cuda.synchronize()
    assert (out == -5).all()                     # nothing was launched
