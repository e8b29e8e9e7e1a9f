"""Where a step's device time goes: per-kernel durations of decode or prefill steps.

    python -m freetoken_b200.step_profile --layers 4 --batch 8            # decode steps
    python -m freetoken_b200.step_profile --layers 4 --mode prefill       # one 2,048-token prompt

Builds the benchmark model (real layer widths, random weights, ``--layers``
layers), runs warm-up steps, then records five steps with the PyTorch profiler
(CUPTI kernel timestamps; decode steps are CUDA-graph replays) and prints, per
kernel, the device time per step, the launches per step and the share.
"""

from __future__ import annotations

import argparse
import sys

import numpy as np
import torch
from torch.profiler import ProfilerActivity, profile

from .benchmark import BENCH_CONFIG, bench_random_options
from .engine import Engine, EngineArgs, StepEntry


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="step_profile")
    p.add_argument("--layers", type=int, default=4)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--mode", choices=["decode", "prefill"], default="decode")
    a = p.parse_args(argv)
    cfg = dict(BENCH_CONFIG)
    cfg["num_hidden_layers"] = a.layers
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], a.context + 256)
    engine = Engine.from_config(cfg, 0, EngineArgs(
        dtype="bfloat16", page_size=64, max_tokens=a.batch * (a.context + 128) + a.context + 64,
        max_running_requests=a.batch + 1), random_options=bench_random_options())
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    ids = [f"d{i}" for i in range(a.batch)]
    if a.mode == "decode":
        per = max(1, 8192 // a.context)
        for i in range(0, a.batch, per):
            engine.step([StepEntry(r, rng.integers(0, V, a.context).tolist(), []) for r in ids[i:i + per]])

        def one():
            engine.step([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in ids])
    else:
        def one():
            engine.step([StepEntry("p", rng.integers(0, V, a.context).tolist(), [a.context - 1])])
            engine.end_request("p")
    for _ in range(4):
        one()
    torch.cuda.synchronize()
    steps = 5
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(steps):
            one()
        torch.cuda.synchronize()
    rows = [(e.key, e.device_time_total / steps, e.count / steps) for e in prof.key_averages()
            if e.device_time_total > 0]
    total = sum(r[1] for r in rows)
    print(f"mode {a.mode}, layers {a.layers}, batch {a.batch}, context {a.context}: "
          f"{total:.1f} us of kernels per step")
    print(f"{'us/step':>10} {'share':>6} {'launches':>8} {'us each':>9}  kernel")
    for name, t, c in sorted(rows, key=lambda r: -r[1]):
        print(f"{t:10.1f} {100 * t / total:5.1f}% {c:8.1f} {t / c:9.1f}  {name[:90]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
