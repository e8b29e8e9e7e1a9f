"""Command line in the reference's manner: ``ft <command> [options]``.

The reference's ``ft`` dispatches sub-commands by name and answers
``--version`` (python/freetoken/cli.py:93-126); its engine options live on
``ft serve`` (python/freetoken/server/args.py:207-391).  This engine has no
server, so the commands are ``generate`` (offline generation from token ids),
``replay`` (trace replay), ``random-model`` (write a random-weights model
folder) and ``bench``; option names and meanings are the reference's where it
has them: ``--model-path/--model``, ``--dtype``, ``--max-running-requests``,
``--max-seq-len-override``, ``--memory-ratio``, ``--dummy-weight``,
``--max-prefill-length/--max-extend-length``, ``--num-pages`` / ``--num-tokens``,
``--page-size``, ``--cuda-graph-max-bs/--graph``; and of ``ft ctl generate``: ``--max-tokens``, ``--ignore-eos``.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional, Sequence

from .version import __version__

COMMANDS = ("generate", "replay", "random-model", "bench")


def _engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model-path", "--model", dest="model_path", required=True,
                   help="folder with config.json and safetensors weights")
    p.add_argument("--dtype", default="bfloat16", choices=["auto", "bfloat16", "float32"],
                   help="compute dtype; auto = bfloat16")
    p.add_argument("--max-running-requests", dest="max_running_req", type=int, default=4,
                   help="the maximum number of running requests")
    p.add_argument("--max-seq-len-override", type=int, default=None,
                   help="the maximum sequence length override")
    p.add_argument("--memory-ratio", type=float, default=0.9,
                   help="fraction of free GPU memory for weights + KV cache")
    p.add_argument("--dummy-weight", dest="use_dummy_weight", action="store_true",
                   help="use random weights (only config.json is read)")
    p.add_argument("--max-prefill-length", "--max-extend-length", dest="max_extend_tokens",
                   type=int, default=8192, help="token budget of one step (prompt portion size)")
    cap = p.add_mutually_exclusive_group()
    cap.add_argument("--num-pages", dest="num_page_override", type=int, default=None,
                     help="number of KV cache pages")
    cap.add_argument("--num-tokens", dest="num_token_override", type=int, default=None,
                     help="KV cache capacity in tokens")
    p.add_argument("--page-size", type=int, default=64, help="tokens per KV cache page")
    p.add_argument("--cuda-graph-max-bs", "--graph", dest="cuda_graph_max_bs", type=int, default=64,
                   help="the maximum batch size for CUDA graph capture of decode steps (0: off)")
    p.add_argument("--seed", type=int, default=0, help="seed of random weights and sampling")


def _print_help(out) -> None:
    out.write("usage: ft <command> [options]\n\ncommands:\n"
              "  generate      offline generation from token-id prompts\n"
              "  replay        feed given token ids step by step, write logits (trace replay)\n"
              "  random-model  write config.json + model.safetensors with random weights\n"
              "  bench         decode / prefill throughput of a random-weights model\n"
              "  --version     print the version\n")


def _run_generate(argv: Sequence[str]) -> int:
    p = argparse.ArgumentParser(prog="ft generate")
    _engine_options(p)
    p.add_argument("--prompt-ids", action="append", default=[],
                   help="comma-separated token ids; repeat for several prompts")
    p.add_argument("--prompt", action="append", default=[], help="text prompt (needs a tokenizer)")
    p.add_argument("--max-tokens", type=int, default=16)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--stop", action="append", default=[],
                   help="stop string (needs a tokenizer); repeat for several")
    p.add_argument("--stop-token-id", action="append", type=int, default=[],
                   help="token id that ends a request; repeat for several")
    a = p.parse_args(argv)
    from .llm import LLM
    from .sampling import SamplingParams

    prompts: List = [[int(t) for t in s.split(",") if t.strip()] for s in a.prompt_ids] + list(a.prompt)
    if not prompts:
        p.error("give at least one --prompt-ids or --prompt")
    llm = LLM(a.model_path, "bfloat16" if a.dtype == "auto" else a.dtype,
              max_running_req=a.max_running_req, page_size=a.page_size,
              num_page_override=a.num_page_override, num_token_override=a.num_token_override,
              max_extend_tokens=a.max_extend_tokens, max_seq_len_override=a.max_seq_len_override,
              memory_ratio=a.memory_ratio, use_dummy_weight=a.use_dummy_weight,
              cuda_graph_max_bs=a.cuda_graph_max_bs, seed=a.seed)
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                        ignore_eos=a.ignore_eos, max_tokens=a.max_tokens, seed=a.seed,
                        stop_strs=[x for x in a.stop if x], stop_token_ids=a.stop_token_id)
    try:
        results = llm.generate(prompts, sp)
    except ValueError as exc:           # e.g. text prompts or stop strings without a tokenizer
        print(f"ft generate: {exc}", file=sys.stderr)
        return 2
    for prompt, result in zip(prompts, results):
        print(json.dumps({"prompt": prompt, **result}))
    return 0


def _run_replay(argv: Sequence[str]) -> int:
    from .replay import main
    return main(list(argv))


def _run_random_model(argv: Sequence[str]) -> int:
    p = argparse.ArgumentParser(prog="ft random-model")
    p.add_argument("--config", required=True, help="config.json to build the model from")
    p.add_argument("--out", required=True, help="folder to write")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                   help="dtype of the stored matrices")
    p.add_argument("--norm-std", type=float, default=None)
    p.add_argument("--router-bias-std", type=float, default=None)
    p.add_argument("--matrix-std", type=float, default=None)
    a = p.parse_args(argv)
    import torch

    from .models import Model
    from .registry import architecture_of
    from .weights import RandomOptions, write_model_folder

    with open(a.config) as f:
        raw = json.load(f)
    arch = architecture_of(raw)
    model = Model(arch.build_plan(arch.read_config(raw)))
    write_model_folder(a.out, raw, model.tensor_specs(), a.seed,
                       torch.bfloat16 if a.dtype == "bfloat16" else torch.float32,
                       RandomOptions(a.matrix_std, a.norm_std, a.router_bias_std))
    print(f"wrote {a.out}")
    return 0


def _run_bench(argv: Sequence[str]) -> int:
    from .benchmark import main
    return main(list(argv))


def main(argv: Optional[Sequence[str]] = None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args:
        _print_help(sys.stderr)
        return 2
    if args[0] in ("-h", "--help"):
        _print_help(sys.stdout)
        return 0
    if args[0] in ("-V", "--version"):
        print(f"freetoken_b200 version {__version__}")
        return 0
    runner = {"generate": _run_generate, "replay": _run_replay,
              "random-model": _run_random_model, "bench": _run_bench}.get(args[0])
    if runner is None:
        print(f"unknown ft command: {args[0]}", file=sys.stderr)
        _print_help(sys.stderr)
        return 2
    return runner(args[1:])


if __name__ == "__main__":
    raise SystemExit(main())
