"""Golden values from the two pieces of the reference that run on a CPU.

    python tests/golden/make_golden.py --reference <path to TaoLe-si/FreeToken> 

The reference's model code cannot run here as a whole (its norm, rotary,
attention and expert ops need a GPU through FlashInfer / Triton, its package
import needs the absent ``flashlib`` wheel, and its ``minimax_m3`` module
computes a different variant of the decoder).  Two pieces do run once
``flashlib`` is replaced by an empty stand-in module: the router's ``_route``
(python/freetoken/models/minimax_m3/moe.py:71-81) and the rotary cos/sin table
(python/freetoken/layers/rotary.py:40-59).  This script runs them on fixed
inputs and writes the inputs and outputs to ``router_rope.json`` beside it;
``tests/test_plain_model.py`` compares the plain implementation with that file.
"""

import argparse
import json
import os
import sys
import types

import torch


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--reference", required=True, help="checkout of TaoLe-si/FreeToken")
    a = p.parse_args()
    sys.path.insert(0, os.path.join(a.reference, "python"))
    # empty stand-ins for the absent package; nothing of it is called below
    import enum
    flashlib, kernels, slot = (types.ModuleType(n) for n in
                               ("flashlib", "flashlib.kernels", "flashlib.kernels.slot_cache"))
    flashlib.__path__, kernels.__path__ = [], []
    slot.N_STATS, slot.Stat, slot.lru_ensure = 0, enum.IntEnum("Stat", {"NONE": 0}), None
    flashlib.kernels, kernels.slot_cache = kernels, slot
    sys.modules.update({"flashlib": flashlib, "flashlib.kernels": kernels,
                        "flashlib.kernels.slot_cache": slot})
    os.environ["FREETOKEN_M3_SPARSE"] = "0"
    os.environ["FREETOKEN_M3_ATTN_MXFP8"] = "0"
    os.environ["FREETOKEN_M3_MLP_MXFP8"] = "0"

    from freetoken.layers.rotary import RotaryEmbedding
    from freetoken.models.minimax_m3.moe import MiniMaxM3SparseMoeBlock

    g = torch.Generator().manual_seed(0)
    E, H, T, k = 8, 32, 6, 3
    gate = torch.randn(E, H, generator=g) * 0.2
    bias = torch.randn(E, generator=g) * 0.05
    x = torch.randn(T, H, generator=g)

    # the method needs these attributes only
    block = types.SimpleNamespace(top_k=k, norm_topk_prob=True, routed_scaling_factor=2.0,
                                  e_score_correction_bias=bias,
                                  gate=types.SimpleNamespace(weight=gate))
    w, ids = MiniMaxM3SparseMoeBlock._route(block, x)

    rope = RotaryEmbedding(64, 32, 40, 5e6)   # head 64 (the module refuses other sizes), rotary 32
    table = rope._cos_sin_cache

    out = {
        "router": {"gate": gate.tolist(), "bias": bias.tolist(), "x": x.tolist(), "top_k": k,
                   "scale": 2.0, "weights": w.tolist(), "ids": ids.tolist()},
        "rope": {"rotary_dim": 32, "theta": 5e6, "positions": 40, "cos_sin": table.tolist()},
    }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "router_rope.json")
    with open(path, "w") as f:
        json.dump(out, f)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
