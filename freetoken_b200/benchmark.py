"""Throughput measurement: decode tokens/s, prefill tokens/s, roofline fractions.

Method, as far as the reference has one: decode speed is generated tokens over
elapsed time at a fixed batch (benchmarks/bench_decode_moe.py:304-372), device
time is taken with CUDA events after warm-up
(python/freetoken/benchmark/perf.py:10-51).  The workload here is synthetic:
random weights of the configured architecture and uniform random token ids.

One JSON line is printed.  ``value`` is decode tokens/s at the main batch
size, timed on the device around whole steps (step function + greedy
sampling); ``e2e`` is the same through ``LLM.run_step_overlapped``, the loop
``LLM.generate`` runs - plan, pinned-host to device copy of the step's inputs,
step, sample, device-to-host read of the tokens (of the step before: the next
step is launched first), bookkeeping.  Every step reads far more weight bytes than the L2 cache
holds, so no flush is needed between timed steps.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from typing import Any, Dict, List, Optional

# Layer sizes of the benchmark model (the 12-layer real-width configuration).
BENCH_CONFIG: Dict[str, Any] = dict(
    architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3",
    hidden_size=3072, num_hidden_layers=12, num_attention_heads=48, num_key_value_heads=8,
    head_dim=128, rotary_dim=64, rope_theta=5e6, max_position_embeddings=4096,
    rms_norm_eps=1e-6, use_gemma_norm=False, use_qk_norm=True, qk_norm_type="per_layer",
    num_local_experts=256, num_experts_per_tok=8, intermediate_size=1536,
    scoring_func="sigmoid", use_routing_bias=True, norm_topk_prob=True,
    routed_scaling_factor=1.0, hidden_act="silu", vocab_size=200064, tie_word_embeddings=False,
)
FAMILY_LAYERS = 62


def bench_random_options(router_bias_std: Optional[float] = None):
    """Scales of the benchmark's random weights.  With every matrix ~N(0, 0.02^2) the
    hidden states of a prompt's tokens are dominated by what the layers add (the
    attention of a random model averages over the prefix), the router sees almost the
    same vector at every position and from the second layer on about 60 of the 256
    experts get all tokens of a 2,048-token prompt - a prefill that reads a quarter of
    the weights a trained model's balanced routing reads.  Embedding rows of unit
    variance and residual-writing matrices scaled by 1/sqrt(2 * layers of the family),
    both usual initialisations, keep the token's own signal on top: every layer then
    routes like the first one (256 of 256 experts touched, the busiest with under twice
    the mean load)."""
    from .weights import RandomOptions
    return RandomOptions(embedding_std=1.0, residual_out_scale=(2.0 * FAMILY_LAYERS) ** -0.5,
                         router_bias_std=router_bias_std)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_peaks() -> Dict[str, Any]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.index = index
        self.proc: Optional[subprocess.Popen] = None
        self.lines: List[str] = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> Dict[str, Any]:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def step_bytes(cfg: Dict[str, Any], layers: int, batch: int, context: int,
               experts_touched: List[int]) -> int:
    """Bytes one decode step has to read: every weight it uses once, and the
    cache of the live requests (bfloat16)."""
    H, d = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    E, I, V = cfg["num_local_experts"], cfg["intermediate_size"], cfg["vocab_size"]
    dense = ((nq + 2 * nkv) * d * H + H * nq * d) * 2 + E * H * 4 + E * 4 + 2 * H * 4
    expert = 3 * I * H * 2
    kv = batch * context * 2 * nkv * d * 2
    total = layers * (dense + kv) + sum(experts_touched) * expert
    total += V * H * 2          # head
    total += batch * H * 2      # embedding rows
    return int(total)


def prefill_flops(cfg: Dict[str, Any], layers: int, tokens: int) -> float:
    H, d = cfg["hidden_size"], cfg["head_dim"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    E, I, V, k = (cfg["num_local_experts"], cfg["intermediate_size"], cfg["vocab_size"],
                  cfg["num_experts_per_tok"])
    per_token = 2 * ((nq + 2 * nkv) * d * H + H * nq * d + E * H + k * 3 * I * H)
    attn = 4 * nq * d * (tokens * (tokens + 1) / 2)
    return layers * (per_token * tokens + attn) + 2 * V * H


def measure_read_peak(timed, gib: int = 2) -> float:
    """GB/s of a load-only kernel over ``gib`` GiB (larger than L2), best of 3 runs of 5."""
    import torch

    from .csrc import ops
    buf = torch.empty(gib << 30, dtype=torch.uint8, device="cuda")
    buf.view(torch.int32).random_(0, 1 << 20)
    partial = torch.empty(8 * ops.sm_count(buf.device), dtype=torch.int32, device="cuda")
    for _ in range(3):
        ops.read_sum(buf, partial)
    best = min(timed(lambda: ops.read_sum(buf, partial), 5) for _ in range(3))
    del buf
    torch.cuda.empty_cache()
    return (gib << 30) / (best / 1e3) / 1e9


def equivalence(a) -> int:
    """The float32 path against the bfloat16 path at real width: same seed, same
    token ids, logits at 15 prompt positions and at 8 decoded tokens."""
    import numpy as np
    import torch

    from .engine import Engine, EngineArgs, StepEntry

    cfg = dict(BENCH_CONFIG)
    cfg["num_hidden_layers"] = a.layers or 2
    toks = np.random.default_rng(a.seed).integers(0, cfg["vocab_size"], 520).tolist()
    want = list(range(0, 512, 37)) + [511]
    logits = {}
    for dtype in ("float32", "bfloat16"):
        engine = Engine.from_config(cfg, a.seed, EngineArgs(dtype=dtype, page_size=64, max_tokens=1024,
                                                            max_running_requests=2),
                                    random_options=bench_random_options(a.router_bias_std))
        rows = [engine.step([StepEntry("a", toks[:512], want)]).float().cpu()]
        for t in toks[512:]:
            rows.append(engine.step([StepEntry("a", [t], [0])]).float().cpu())
        logits[dtype] = torch.cat(rows)
        del engine
        torch.cuda.empty_cache()
    f, b = logits["float32"], logits["bfloat16"]
    print(json.dumps({"equivalence": "float32 vs bfloat16", "layers": cfg["num_hidden_layers"],
                      "positions": f.shape[0], "logit_max_abs": f.abs().max().item(),
                      "max_abs_diff": (f - b).abs().max().item(), "mean_abs_diff": (f - b).abs().mean().item(),
                      "argmax_agree": (f.argmax(-1) == b.argmax(-1)).float().mean().item()}))
    return 0


def reference_unavailable() -> str:
    """Why the reference arm cannot run: tried against ``baseline/_ref``."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "freetoken")):
        return ("the reference is not installed under baseline/_ref (an offline install fails at its "
                "pinned dependencies apache-tvm-ffi==0.1.13.post3 and flashlib==0.3.0, which no local "
                "package source carries)")
    probe = subprocess.run([sys.executable, "-c", "import freetoken.llm"], capture_output=True, text=True,
                           env={**os.environ, "PYTHONPATH": ref})
    if probe.returncode != 0:
        last = (probe.stderr.strip().splitlines() or ["import failed"])[-1]
        return ("installed with --no-deps, but its public API does not import here: " + last +
                " (a hard dependency that is not installed)")
    return ("its MiniMax-M3 path serves NVFP4 experts through the expert offload cache only; there is "
            "no bfloat16 resident-weight configuration of this model to time")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="bench.py")
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=256)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--prefill-tokens", type=int, default=2048)
    p.add_argument("--prefill-requests", type=int, default=1,
                   help="prompts of --prefill-tokens tokens in the timed prefill step")
    p.add_argument("--points", default="1,64", help="further decode batch sizes")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--equivalence", action="store_true",
                   help="instead of timing: the same random model (--layers, default 2) in float32 and in "
                        "bfloat16 on one 512-token prompt and 8 decoded tokens; prints how far the logits differ")
    p.add_argument("--router-bias-std", type=float, default=None,
                   help="spread of the random score-correction bias (skews which experts are popular)")
    return p


def main(argv: Optional[List[str]] = None) -> int:
    a = build_parser().parse_args(argv)
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": reference_unavailable()}))
        return 0
    if a.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {a.gpus} is not supported (use --gpus 1)")
        return 2

    import numpy as np
    import torch

    if a.equivalence:
        return equivalence(a)

    from .csrc import ops
    from .engine import StepEntry
    from .llm import LLM
    from .sampling import SamplingParams

    cfg = dict(BENCH_CONFIG)
    layers = a.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    points = [int(x) for x in a.points.split(",") if x.strip()]
    batches = [a.batch] + [b for b in points if b != a.batch]
    max_batch = max(batches)
    page = 64
    room = a.context + a.steps + a.warmup + 2 * page
    pool_tokens = max_batch * (-(-room // page) * page) + a.prefill_requests * (-(-a.prefill_tokens // page) * page)
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], room + page)
    peaks = load_peaks()
    t0 = time.time()
    llm = LLM("", a.dtype, config=cfg, use_dummy_weight=True, seed=a.seed,
              dummy_weight_options=bench_random_options(a.router_bias_std),
              max_running_req=max_batch + a.prefill_requests, page_size=page, num_token_override=pool_tokens,
              max_extend_tokens=8192, max_seq_len_override=room + page)
    engine = llm.engine
    torch.cuda.synchronize()
    build_s = time.time() - t0
    V = cfg["vocab_size"]
    rng = np.random.default_rng(a.seed)
    greedy = SamplingParams(temperature=0.0)

    def timed(fn, reps: int) -> float:
        """Milliseconds per call, device time between two events."""
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps

    # ---- the read-only stream this GPU reaches, measured in place -----------
    # The driver's HBM peak is a copy (half reads, half writes); a decode step only reads.
    # Every HBM fraction below is given against both.
    read_gbs = measure_read_peak(timed)

    # ---- prefill: one prompt of --prefill-tokens tokens in one step -------
    def prefill_once():
        entries = []
        for i in range(a.prefill_requests):
            toks = rng.integers(0, V, a.prefill_tokens).tolist()
            entries.append(StepEntry(("prefill", i), toks, [len(toks) - 1]))
        logits = engine.step(entries)
        llm.sampler.sample(logits, [greedy] * a.prefill_requests, [0.0] * a.prefill_requests)
        for i in range(a.prefill_requests):
            engine.end_request(("prefill", i))

    for _ in range(3):
        prefill_once()
    with ClockSampler() as prefill_clocks:
        prefill_ms = timed(prefill_once, 5)
    pf = a.prefill_requests * prefill_flops(cfg, layers, a.prefill_tokens)
    # what bounds this step: a 2,048-token portion sends a few dozen rows to each of
    # the experts it touches, so their weights are read for a few rows each; hbm_frac is
    # the weight bytes of the step (experts counted from the router in an untimed probe
    # step, as for decode) over its time
    pf_probe: Dict[str, Any] = {}
    engine.step([StepEntry(("prefill", i), rng.integers(0, V, a.prefill_tokens).tolist(), [])
                 for i in range(a.prefill_requests)], probe=pf_probe)
    for i in range(a.prefill_requests):
        engine.end_request(("prefill", i))
    pf_touched = pf_probe.get("experts_touched", [cfg["num_local_experts"]] * layers)
    pf_bytes = step_bytes(cfg, layers, 1, a.prefill_tokens, pf_touched)
    prefill = {"value": a.prefill_requests * a.prefill_tokens / (prefill_ms / 1e3),
               "tokens": a.prefill_requests * a.prefill_tokens, "requests": a.prefill_requests,
               "ms": prefill_ms, "frac": pf / (prefill_ms / 1e3) / (peaks["bf16_tflops"] * 1e12),
               "hbm_frac": pf_bytes / (prefill_ms / 1e3) / (peaks["hbm_gbs"] * 1e9),
               "hbm_frac_of_read_peak": pf_bytes / (prefill_ms / 1e3) / (read_gbs * 1e9),
               "experts_touched_per_layer": sum(pf_touched) / max(1, len(pf_touched))}

    # ---- decode at each batch size -----------------------------------------
    def fill_contexts(batch: int) -> List[str]:
        """Contexts of ``--context`` tokens by real prefill, in steps of at most 8,192 tokens
        (several short requests per step, or a long one in portions)."""
        ids = [f"d{i}" for i in range(batch)]
        step_tokens = 8192
        if a.context <= step_tokens:
            per_step = max(1, step_tokens // a.context)
            for i in range(0, batch, per_step):
                group = ids[i:i + per_step]
                engine.step([StepEntry(r, rng.integers(0, V, a.context).tolist(), []) for r in group])
        else:
            for r in ids:
                for lo in range(0, a.context, step_tokens):
                    n = min(step_tokens, a.context - lo)
                    engine.step([StepEntry(r, rng.integers(0, V, n).tolist(), [])])
        return ids

    results: Dict[int, Dict[str, float]] = {}
    clocks_main: Dict[str, Any] = {}
    launches_main = 0
    touched_main: List[int] = []
    context_build: Dict[str, Any] = {}
    for batch in batches:
        torch.cuda.synchronize()
        t_fill = time.time()
        ids = fill_contexts(batch)
        torch.cuda.synchronize()
        if batch == a.batch:
            # wall time of building the contexts by real prefill (steps of at most 8,192 tokens)
            fill_s = time.time() - t_fill
            context_build = {"tokens": batch * a.context, "s": round(fill_s, 3),
                             "tokens_per_s": round(batch * a.context / fill_s)}
        params = [greedy] * batch
        zeros = [0.0] * batch

        def decode_once():
            toks = rng.integers(0, V, batch)
            logits = engine.step([StepEntry(r, [int(t)], [0]) for r, t in zip(ids, toks)])
            llm.sampler.sample(logits, params, zeros)

        for _ in range(max(3, a.warmup)):
            decode_once()
        probe: Dict[str, Any] = {}
        toks = rng.integers(0, V, batch)
        engine.step([StepEntry(r, [int(t)], [0]) for r, t in zip(ids, toks)], probe=probe)
        touched = probe.get("experts_touched", [])
        ops.reset_launch_count()
        ctx_before = engine.length(ids[0])
        with ClockSampler() as clocks:
            ms = timed(decode_once, a.steps)
        launches = ops.launch_count()
        # contexts grow by one token per step: bytes at the middle of the timed region
        ctx_now = (ctx_before + engine.length(ids[0])) // 2
        nbytes = step_bytes(cfg, layers, batch, ctx_now, touched)
        results[batch] = {"ms": ms, "tok_s": batch / (ms / 1e3), "bytes": nbytes,
                          "gbs": nbytes / (ms / 1e3) / 1e9}
        if batch == a.batch:
            clocks_main = clocks.summary()
            launches_main = launches
            touched_main = touched
        for r in ids:
            engine.end_request(r)

    # ---- end to end through the Python entry point -------------------------------
    sp = SamplingParams(temperature=0.0, ignore_eos=True, max_tokens=a.steps + a.warmup + 8)
    prompts = [rng.integers(0, V, a.context).tolist() for _ in range(a.batch)]
    from .engine.scheduler import Request
    from .sampling.sampler import RequestRng
    rngs = {}
    for i, p in enumerate(prompts):
        llm.scheduler.submit(Request(("e2e", i), p, sp))
        rngs[("e2e", i)] = RequestRng(i)
    while llm.scheduler.pending or llm.scheduler.prefilling:
        llm.run_step(rngs)
    # the loop generate() runs: a step is launched (its inputs copied from pinned host
    # memory) before the tokens of the step before it are read from pinned host memory
    for _ in range(max(3, a.warmup)):
        llm.run_step_overlapped(rngs)
    e2e_ms = timed(lambda: llm.run_step_overlapped(rngs), a.steps)
    llm.drain()
    h2d = engine.last_meta_ints * 4
    d2h = llm.d2h_bytes_last_step      # the sampled tokens and the kernels' status word
    for r in list(llm.scheduler.running):
        llm.scheduler.abort(r.id)

    main_r = results[a.batch]
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens; % of roofline",
        "value": main_r["tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": a.steps,
        "warmup": max(3, a.warmup), "ms_per_step": main_r["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if a.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights (unit-variance embedding, residual outputs / sqrt(2*62): balanced routing), uniform random token ids", "impl": "ours",
        "config": {
            "model": "MiniMax-M3 real width", "layers": layers, "layers_in_family": FAMILY_LAYERS,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "rotary_dim": cfg["rotary_dim"], "experts": cfg["num_local_experts"],
            "top_k": cfg["num_experts_per_tok"], "expert_intermediate": cfg["intermediate_size"],
            "vocab": V, "global_batch": a.batch, "seq_len": a.context, "page_size": page,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read per step)",
            "weights_gb": round(engine.weight_bytes / 1e9, 2),
        },
        "e2e": {"value": a.batch / (e2e_ms / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
        "gpu_launches": launches_main,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main_r["gbs"], "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": main_r["gbs"] / peaks["hbm_gbs"],
                     "peaks": peaks["source"], "read_peak": read_gbs,
                     "frac_of_read_peak": main_r["gbs"] / read_gbs, "bytes_per_step": main_r["bytes"],
                     "experts_touched_per_layer": (sum(touched_main) / max(1, len(touched_main)))},
        "points": {f"decode_b{b}": results[b]["tok_s"] for b in batches if b != a.batch},
        "points_roofline_frac": {f"decode_b{b}": results[b]["gbs"] / peaks["hbm_gbs"] for b in batches},
        "points_frac_of_read_peak": {f"decode_b{b}": results[b]["gbs"] / read_gbs for b in batches},
        "clocks": clocks_main,
        "prefill_clocks": prefill_clocks.summary(),
        "context_build": context_build,
        "setup_s": round(build_s, 1),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
