"""Golden values from the reference's own Triton kernels, run once on a GPU.

    python tests/golden/make_kernel_golden.py --reference <path to TaoLe-si/FreeToken>

Runs, on small fixed inputs and one launch each, the kernels the plain
implementation's formulas are read from:

* ``apply_rope_with_cos_sin_cache_inplace`` (python/freetoken/kernel/triton/rope.py:28-140),
  NeoX and interleaved pairing, partial rotation;
* ``fused_add_rmsnorm`` / ``gemma_fused_add_rmsnorm`` / ``rmsnorm`` with a 3-D
  per-head input (python/freetoken/kernel/triton/norm.py:42-186);
* ``silu_and_mul`` / ``swigluoai_and_mul`` (python/freetoken/kernel/triton/activation.py:67-170);
* ``paged_attention`` (python/freetoken/kernel/triton/attention.py:45-145,883-949) on
  a paged cache with shuffled slots, a prefix in the cache and grouped heads;
* ``fused_experts_impl`` (python/freetoken/moe/fused.py:233-337): block-aligned
  grouped GEMM, activation, down projection with the route weight, k-way sum.

Only these modules are loaded.  The package's ``__init__`` files are NOT
executed (they import native extensions and packages that are absent here):
the script puts empty package shells into ``sys.modules`` whose ``__path__``
points into the reference, so that the modules' own ``from freetoken...``
imports resolve to the reference's files, and gives the shells the three
helpers (``div_ceil``, ``init_logger``, ``BaseMoeBackend``) the loaded modules
ask of them.  A module that does not import is recorded as
``unavailable: <error>`` in the output's metadata.

Inputs and outputs go to ``triton_kernels.safetensors`` beside this script;
``tests/test_plain_model.py`` compares the plain implementation with it.
"""

import argparse
import importlib
import json
import logging
import os
import struct
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
_CODES = {torch.float32: "F32", torch.bfloat16: "BF16", torch.int32: "I32", torch.int64: "I64"}


def write_safetensors(path, tensors, metadata):
    header, blobs, offset = {"__metadata__": metadata}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _CODES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)


def shells(reference):
    """Package shells for ``freetoken`` and the sub-packages the loaded modules name."""
    root = os.path.join(reference, "python", "freetoken")

    def shell(name, *rel):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(root, *rel)]
        sys.modules[name] = m
        return m

    shell("freetoken")
    kernel = shell("freetoken.kernel", "kernel")
    shell("freetoken.kernel.triton", "kernel", "triton")
    utils = shell("freetoken.utils", "utils")
    moe = shell("freetoken.moe", "moe")
    layers = shell("freetoken.layers", "layers")
    utils.div_ceil = lambda a, b: -(-a // b)

    class _Logger(logging.LoggerAdapter):
        def __getattr__(self, name):                     # warning_rank0 and the like
            if name.endswith("_rank0"):
                return getattr(self.logger, name[:-6])
            raise AttributeError(name)
    utils.init_logger = lambda name: _Logger(logging.getLogger(name), {})
    moe.BaseMoeBackend = object
    return kernel, layers


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--reference", required=True, help="checkout of TaoLe-si/FreeToken")
    p.add_argument("--out", default=os.path.join(HERE, "triton_kernels.safetensors"))
    a = p.parse_args()
    dev = "cuda:0"
    kernel, layers = shells(a.reference)
    g = torch.Generator().manual_seed(1234)
    rnd = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale)
    out, meta = {}, {"reference": "TaoLe-si/FreeToken", "device": torch.cuda.get_device_name(0)}

    def guarded(name, fn):
        try:
            fn()
            meta[name] = "ok"
        except Exception as exc:                      # recorded, not hidden
            meta[name] = f"unavailable: {type(exc).__name__}: {str(exc)[:200]}"
        print(name, meta[name], flush=True)

    # ---- rotary -----------------------------------------------------------------
    def rope():
        mod = importlib.import_module("freetoken.kernel.triton.rope")
        T, hq, hk, d, R = 6, 3, 1, 64, 32
        inv = 1.0 / (5e6 ** (torch.arange(0, R, 2, dtype=torch.float) / R))
        freqs = torch.arange(50, dtype=torch.float)[:, None] * inv[None, :]
        table = torch.cat((freqs.cos(), freqs.sin()), -1).contiguous()
        pos = torch.tensor([0, 1, 7, 30, 31, 49])
        q, k = rnd(T, hq * d), rnd(T, hk * d)
        out.update({"rope.table": table, "rope.positions": pos, "rope.q": q, "rope.k": k})
        for tag, neox in (("neox", True), ("interleaved", False)):
            qq, kk = q.clone().to(dev), k.clone().to(dev)
            mod.apply_rope_with_cos_sin_cache_inplace(pos.to(dev), qq, kk, d, table.to(dev), is_neox=neox)
            out[f"rope.q_{tag}"], out[f"rope.k_{tag}"] = qq.cpu(), kk.cpu()
    guarded("rope", rope)

    # ---- norms --------------------------------------------------------------------
    def norm():
        mod = importlib.import_module("freetoken.kernel.triton.norm")
        T, H, eps = 5, 96, 1e-5
        x, res, w = rnd(T, H), rnd(T, H), rnd(H, scale=0.3)
        out.update({"norm.x": x, "norm.residual": res, "norm.w": w, "norm.eps": torch.tensor([eps])})
        for tag, fn in (("plain", mod.fused_add_rmsnorm), ("gemma", mod.gemma_fused_add_rmsnorm)):
            xx, rr = x.clone().to(dev), res.clone().to(dev)
            fn(xx, rr, (w + (1.0 if tag == "plain" else 0.0)).to(dev), eps)
            out[f"norm.{tag}_out"], out[f"norm.{tag}_residual"] = xx.cpu(), rr.cpu()
        # per-head QK norm: a 3-D input normed over its last axis with a [d] weight
        xh, wh = rnd(T, 3, 64), rnd(64, scale=0.3)
        out.update({"norm.heads_x": xh, "norm.heads_w": wh})
        out["norm.heads_gemma_out"] = mod.gemma_rmsnorm(xh.to(dev), wh.to(dev), eps).cpu()
        out["norm.heads_plain_out"] = mod.rmsnorm(xh.to(dev), (wh + 1.0).to(dev), eps).cpu()
    guarded("norm", norm)

    # ---- gated activations ------------------------------------------------------------
    def activation():
        mod = importlib.import_module("freetoken.kernel.triton.activation")
        x = rnd(4, 2 * 40, scale=3.0)
        x[0, 0], x[0, 40], x[1, 41] = 9.5, 11.0, -12.0          # beyond the clamp limit
        out["act.x"] = x
        out["act.silu"] = mod.silu_and_mul(x.to(dev)).cpu()
        out["act.swigluoai"] = mod.swigluoai_and_mul(x.to(dev), alpha=1.702, limit=7.0).cpu()
        layers.silu_and_mul, layers.gelu_and_mul = mod.silu_and_mul, mod.gelu_and_mul
        layers.gelu_tanh_and_mul = mod.gelu_tanh_and_mul
    guarded("activation", activation)

    # ---- paged attention -----------------------------------------------------------------
    def attention():
        mod = importlib.import_module("freetoken.kernel.triton.attention")
        nq, nkv, d = 4, 2, 64
        lens = [(9, 5), (0, 7)]                      # (keys already cached, new tokens)
        total = [p + n for p, n in lens]
        slots = torch.randperm(40, generator=g)[: sum(total)]
        k_cache, v_cache = rnd(40, nkv, d), rnd(40, nkv, d)
        indptr = torch.tensor([0, total[0], total[0] + total[1]], dtype=torch.int32)
        q = rnd(sum(n for _, n in lens), nq, d)
        q_to_req = torch.tensor([0] * lens[0][1] + [1] * lens[1][1], dtype=torch.int32)
        q_pos = torch.tensor(list(range(9, 14)) + list(range(0, 7)), dtype=torch.int32)
        scale = d ** -0.5
        o = mod.paged_attention(q.to(dev), k_cache.to(dev), v_cache.to(dev), indptr.to(dev),
                                slots.to(torch.int32).to(dev), q_to_req.to(dev), q_pos.to(dev), scale)
        out.update({"attn.q": q, "attn.k_cache": k_cache, "attn.v_cache": v_cache, "attn.indptr": indptr,
                    "attn.indices": slots.to(torch.int32), "attn.q_to_req": q_to_req, "attn.q_pos": q_pos,
                    "attn.out": o.cpu()})
    guarded("attention", attention)

    # ---- routed experts ----------------------------------------------------------------------
    def experts():
        kernel.moe_impl = importlib.import_module("freetoken.kernel.moe_impl")
        kernel.fused_moe_kernel_triton = kernel.moe_impl.fused_moe_kernel_triton
        kernel.moe_sum_reduce_triton = kernel.moe_impl.moe_sum_reduce_triton
        fused = importlib.import_module("freetoken.moe.fused")
        T, H, E, I, k = 6, 64, 4, 32, 2
        x = rnd(T, H).to(torch.bfloat16)
        w1 = rnd(E, 2 * I, H, scale=0.2).to(torch.bfloat16)
        w2 = rnd(E, H, I, scale=0.2).to(torch.bfloat16)
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
        wts = torch.rand(T, k, generator=g)
        y = fused.fused_experts_impl(x.clone().to(dev), w1.to(dev), w2.to(dev), wts.to(dev), ids.to(dev),
                                     activation="silu")
        out.update({"moe.x": x, "moe.w1": w1, "moe.w2": w2, "moe.ids": ids, "moe.weights": wts, "moe.out": y.cpu()})
    guarded("experts", experts)

    write_safetensors(a.out, out, meta)
    print("wrote", a.out, os.path.getsize(a.out), "bytes")


if __name__ == "__main__":
    main()
