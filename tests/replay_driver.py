"""Ways of cutting requests into steps, and a driver that runs them.

A *schedule* is a list of steps; a step is ``(entries, ended)`` with entries
``(request id, first token index, number of tokens)``.  The driver feeds the
engine's step function (directly, or through ``bin/trace_run``) and collects,
per request, the logits at every position, to be compared with the plain
implementation's whole-sequence logits.
"""

from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

Step = Tuple[List[Tuple[str, int, int]], List[str]]


def whole(requests: Dict[str, List[int]]) -> List[Step]:
    """Each request alone and whole, one after the other."""
    return [([(rid, 0, len(toks))], [rid]) for rid, toks in requests.items()]


def decode_tail(requests: Dict[str, List[int]], tail: int = 32) -> List[Step]:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps: List[Step] = []
    for rid, toks in requests.items():
        n = len(toks)
        head = max(1, n - tail)
        steps.append(([(rid, 0, head)], []))
        for i in range(head, n):
            steps.append(([(rid, i, 1)], [rid] if i == n - 1 else []))
        if head == n:
            steps[-1] = (steps[-1][0], [rid])
    return steps


def portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (7, 2, 5, 3, 2, 11, 2, 4)) -> List[Step]:
    """Portions of changing size, down to two tokens."""
    steps: List[Step] = []
    for rid, toks in requests.items():
        i, j, n = 0, 0, len(toks)
        while i < n:
            size = min(sizes[j % len(sizes)], n - i)
            j += 1
            steps.append(([(rid, i, size)], [rid] if i + size == n else []))
            i += size
    return steps


def mixed(requests: Dict[str, List[int]], live: int = 4, prompt_part: float = 0.6,
          sizes: Sequence[int] = (5, 2, 9, 3, 6, 2)) -> List[Step]:
    """Up to ``live`` requests at a time; each first brings its "prompt" (the
    leading ``prompt_part`` of its tokens) in portions of changing size, then
    its remaining tokens one per step, beside whatever the others bring; a
    finished request ends and the next waiting one starts in its place."""
    waiting = list(requests)
    running: List[str] = []
    done_upto = {rid: 0 for rid in requests}
    prompt_len = {rid: max(1, int(len(t) * prompt_part)) for rid, t in requests.items()}
    steps: List[Step] = []
    turn = 0
    while waiting or running:
        while waiting and len(running) < live:
            running.append(waiting.pop(0))
        entries, ended = [], []
        for idx, rid in enumerate(list(running)):
            n = len(requests[rid])
            at = done_upto[rid]
            if at < prompt_len[rid]:
                # stagger: not every request brings tokens to every step
                if (turn + idx) % 3 == 2 and len(running) > 1:
                    continue
                size = min(sizes[(turn + idx) % len(sizes)], prompt_len[rid] - at)
            else:
                size = 1
            entries.append((rid, at, size))
            done_upto[rid] = at + size
            if at + size == n:
                ended.append(rid)
        for rid in ended:
            running.remove(rid)
        if entries:
            steps.append((entries, ended))
        turn += 1
    return steps


def peak_tokens(schedule: List[Step], page: int) -> int:
    """Most tokens live requests hold at any time, each rounded up to a page."""
    held: Dict[str, int] = {}
    peak = 0
    for entries, ended in schedule:
        for rid, first, n in entries:
            held[rid] = first + n
        peak = max(peak, sum(-(-v // page) * page for v in held.values()))
        for rid in ended:
            held.pop(rid, None)
    return peak


def run_engine(engine, requests: Dict[str, List[int]], schedule: List[Step], routing: Dict = None
               ) -> Dict[str, torch.Tensor]:
    """Drive ``engine.step``; logits of every position of every request.  With
    ``routing`` (a dict) the experts the engine chose are left there as
    ``routing[request] = int tensor [stops, positions, k]``."""
    from freetoken_b200.engine import StepEntry

    V = engine.vocab_size
    out = {rid: torch.full((len(t), V), float("nan")) for rid, t in requests.items()}
    for entries, ended in schedule:
        batch = [StepEntry(rid, requests[rid][first:first + n], list(range(n)))
                 for rid, first, n in entries]
        probe = {"router_ids": []} if routing is not None else None
        logits = engine.step(batch, probe=probe).float().cpu()
        row = 0
        for rid, first, n in entries:
            out[rid][first:first + n] = logits[row:row + n]
            if routing is not None:
                ids = torch.stack([x[row:row + n].cpu() for x in probe["router_ids"]])   # [stops, n, k]
                if rid not in routing:
                    routing[rid] = torch.full((ids.shape[0], len(requests[rid]), ids.shape[2]), -1,
                                              dtype=torch.int32)
                routing[rid][:, first:first + n] = ids
            row += n
        for rid in ended:
            engine.end_request(rid)
    engine.cache.check_integrity()
    return out


def run_trace_tool(model_dir: str, dtype: str, requests: Dict[str, List[int]], schedule: List[Step],
                   out_dir: str, max_tokens: int, page: int, vocab: int, env=None) -> Dict[str, torch.Tensor]:
    """The same through ``bin/trace_run`` as a child process."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lines = []
    for i, (entries, ended) in enumerate(schedule):
        lines.append(json.dumps({
            "step": i,
            "entries": [{"id": rid, "tokens": requests[rid][first:first + n], "want": list(range(n))}
                        for rid, first, n in entries],
            "end": ended}))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
         "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page)],
        input="\n".join(lines) + "\n", capture_output=True, text=True, env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-4000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(schedule))], proc.stdout[-2000:]
    out = {rid: torch.full((len(t), vocab), float("nan")) for rid, t in requests.items()}
    for i, (entries, _) in enumerate(schedule):
        arr = np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, vocab)
        row = 0
        for rid, first, n in entries:
            out[rid][first:first + n] = torch.from_numpy(arr[row:row + n].copy())
            row += n
    return out
