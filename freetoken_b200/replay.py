"""Trace replay: feed given token ids through a model step by step, write logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as ONE batch through :meth:`Engine.step` - the model,
cache and kernels that generation uses; this program has no forward pass, cache
or loader of its own and samples nothing.  For a step that wants logits it
writes ``OUT/<step>.f32`` (little-endian float32 ``[wanted, vocab]``, in the
order of the entries and of ``want``); after every step it prints ``done
<step>``.  Requests named in ``end`` give back what they hold after the step.

The reference has no such tool; its closest relative drives the scheduler's
page accounting without a model
(tests/scheduler/test_scheduler_chunked_prefill.py:49-77).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional



def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", "--model-path", required=True,
                   help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16: the kernels serving uses; float32: everything in true 32-bit")
    p.add_argument("--out", required=True, help="folder the logits files are written to")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to a page)")
    p.add_argument("--page-size", type=int, default=64, help="tokens per cache page")
    p.add_argument("--max-running-requests", type=int, default=4,
                   help="most requests live at a time")
    p.add_argument("--poison-freed-pages", action="store_true",
                   help="debugging: fill cache pages with NaN whenever they are free, so that a read of "
                        "stale data shows in the logits")
    return p


def main(argv: Optional[List[str]] = None) -> int:
    args = build_parser().parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    from .engine import Engine, EngineArgs, StepEntry

    page = args.page_size
    pages = -(-args.max_tokens // page)
    engine = Engine.from_folder(args.model, EngineArgs(
        dtype=args.dtype, page_size=page, num_pages=pages,
        max_running_requests=args.max_running_requests, max_seq_len=pages * page,
        poison_freed_pages=args.poison_freed_pages))
    import torch

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in step.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                torch.cuda.synchronize()
                engine.check_status()
                arr = logits.detach().cpu().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(args.out, f"{step['step']}.f32"))
        for rid in step.get("end", []):
            engine.end_request(rid)
        print(f"done {step['step']}", flush=True)
    engine.cache.check_integrity()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
