"""The Python entry point: ``LLM(model_path, dtype, **options).generate(...)``.

In the reference's manner (python/freetoken/llm/llm.py:30-43,105-142):
``LLM(model_path, dtype=torch.bfloat16, **kwargs)`` with the scheduler's option
names as keywords (``max_running_req``, ``page_size``, ``num_page_override``,
``max_extend_tokens``, ``max_seq_len_override``, ``memory_ratio``,
``use_dummy_weight``, ``cuda_graph_max_bs``; python/freetoken/engine/config.py:16-105,
python/freetoken/scheduler/config.py:14-43), and
``generate(prompts, sampling_params) -> [{"text", "token_ids"}, ...]`` where
prompts are token-id lists or, if the model folder has a tokenizer, strings.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from .csrc import ops
from .engine.engine import Engine, EngineArgs, StepEntry
from .engine.scheduler import PlannedEntry, Request, Scheduler
from .engine.status import StatusReporter
from .sampling.params import SamplingParams
from .sampling.sampler import RequestRng, Sampler


def _eos_ids(folder: Optional[str], config: Dict[str, Any]) -> List[int]:
    """EOS ids of config.json and generation_config.json
    (python/freetoken/utils/hf.py:44-72)."""
    ids: List[int] = []

    def add(value) -> None:
        if isinstance(value, int):
            ids.append(value)
        elif isinstance(value, (list, tuple)):
            ids.extend(int(v) for v in value)

    add(config.get("eos_token_id"))
    add((config.get("text_config") or {}).get("eos_token_id"))
    if folder:
        path = os.path.join(folder, "generation_config.json")
        if os.path.exists(path):
            with open(path) as f:
                add(json.load(f).get("eos_token_id"))
    return sorted(set(ids))


class _InFlight:
    """A launched step whose sampled tokens have not been read yet."""

    def __init__(self, plan: List[PlannedEntry], count: int, index_of: Dict[Any, int]):
        self.plan = plan
        self.count = count                  # entries that sample
        self.index_of = index_of            # request id -> place among the sampled tokens
        self.tokens_dev: Optional[torch.Tensor] = None
        self.tokens_host: Optional[torch.Tensor] = None
        self.status_host: Optional[torch.Tensor] = None     # the kernels' status word after this step
        self.event: Optional[torch.cuda.Event] = None


class LLM:
    def __init__(self, model_path: str, dtype: Union[torch.dtype, str] = torch.bfloat16, *,
                 max_running_req: int = 4, page_size: int = 64,
                 num_page_override: Optional[int] = None, num_token_override: Optional[int] = None,
                 max_extend_tokens: int = 8192, max_seq_len_override: Optional[int] = None,
                 memory_ratio: float = 0.9, use_dummy_weight: bool = False,
                 cuda_graph_max_bs: int = 64, seed: int = 0,
                 device: str = "cuda:0", config: Optional[Dict[str, Any]] = None,
                 dummy_weight_options=None, log_status=None, decode_log_interval: int = 40,
                 nvtx: bool = False):
        """``model_path``: a folder with ``config.json`` and safetensors files.
        With ``use_dummy_weight`` only ``config.json`` (or ``config``) is
        needed and weights are random from ``seed`` (scales from
        ``dummy_weight_options``, a :class:`freetoken_b200.weights.RandomOptions`).
        ``log_status``: a function that takes a line of text; it receives the scheduler's
        throughput lines (one per step with prompt tokens, one per
        ``decode_log_interval`` decode steps).  ``nvtx``: NVTX ranges around every part."""
        args = EngineArgs(dtype=dtype, device=device, page_size=page_size,
                          num_pages=num_page_override, max_tokens=num_token_override,
                          max_running_requests=max_running_req, max_seq_len=max_seq_len_override,
                          memory_ratio=memory_ratio, max_step_tokens=max_extend_tokens,
                          cuda_graph_max_bs=cuda_graph_max_bs, nvtx=nvtx)
        raw: Dict[str, Any]
        if config is not None:
            raw = dict(config)
        else:
            with open(os.path.join(model_path, "config.json")) as f:
                raw = json.load(f)
        if use_dummy_weight:
            if dummy_weight_options is not None:
                self.engine = Engine.from_config(raw, seed, args, random_options=dummy_weight_options)
            else:
                self.engine = Engine.from_config(raw, seed, args)
        else:
            self.engine = Engine.from_folder(model_path, args)
        self.model_path = model_path
        self.seed = seed
        self.eos_token_ids = _eos_ids(model_path if config is None else None, raw)
        self.scheduler = Scheduler(self.engine.cache, max_extend_tokens, self.eos_token_ids)
        self.sampler = Sampler(self.engine.device, self.engine.vocab_size)
        self.tokenizer = None
        self._counter = 0
        self._inflight: Optional[_InFlight] = None
        self._flip = 0
        self._tok_dev: List[Optional[torch.Tensor]] = [None, None]
        self._tok_host: List[Optional[torch.Tensor]] = [None, None]
        self._status_host = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.d2h_bytes_last_step = 0
        self.status = StatusReporter(log_status, decode_log_interval=decode_log_interval) if log_status else None

    # ---- text ------------------------------------------------------------
    def _tokenizer(self):
        if self.tokenizer is None:
            try:
                from transformers import AutoTokenizer
                self.tokenizer = AutoTokenizer.from_pretrained(self.model_path)
            except Exception as exc:  # no tokenizer files, or no tokenizer package
                raise ValueError(
                    "text prompts need a tokenizer in the model folder; pass token-id lists instead"
                ) from exc
        return self.tokenizer

    # ---- generation ----------------------------------------------------------
    def generate(self, prompts: Sequence[Union[str, List[int]]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams]]
                 ) -> List[Dict[str, Any]]:
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        requests: List[Request] = []
        rngs: Dict[Any, RequestRng] = {}
        if any(sp.stop_strs for sp in sampling_params):
            tok = self._tokenizer()             # raises if the folder has none
            self.scheduler.detokenize = tok.decode
        for prompt, sp in zip(prompts, sampling_params):
            ids = self._tokenizer().encode(prompt) if isinstance(prompt, str) else list(prompt)
            uid = self._counter
            self._counter += 1
            r = Request(uid, [int(t) for t in ids], sp)
            rngs[uid] = RequestRng(sp.seed if sp.seed is not None else self.seed * 1000003 + uid)
            requests.append(r)
            self.scheduler.submit(r)
        overlap = os.environ.get("FREETOKEN_DISABLE_OVERLAP_SCHEDULING", "0") in ("", "0")
        while self.scheduler.has_work() or self._inflight is not None:
            if overlap:
                self.run_step_overlapped(rngs)
            else:
                self.run_step(rngs)
        self.engine.check_status()
        self.scheduler.finished.clear()
        results = []
        for r in requests:
            out = list(r.output)
            if (r.finish_reason == "stop" and out and not r.params.ignore_eos
                    and out[-1] in self.eos_token_ids):
                # the EOS token itself is not part of the answer; a token that ended the
                # request through stop_token_ids or a stop string is
                # (python/freetoken/llm/llm.py:101-103)
                out = out[:-1]
            text = self.tokenizer.decode(out) if self.tokenizer is not None else ""
            results.append({"text": text, "token_ids": out, "finish_reason": r.finish_reason})
        return results

    def run_step(self, rngs: Dict[Any, RequestRng]) -> List[Request]:
        """Plan one step, run it, sample, read the tokens, record; returns
        finished requests."""
        done = self.drain()
        step = self._launch(rngs)
        if step is None:
            if not done:
                raise RuntimeError("the scheduler has work but could plan nothing: the page pool is too small")
            return done
        self._inflight = step
        return done + self.drain()

    def run_step_overlapped(self, rngs: Dict[Any, RequestRng]) -> List[Request]:
        """Launch the next step BEFORE reading the tokens of the one in flight:
        the host's planning, staging and bookkeeping of step N+1 run while the
        device works on step N, and the tokens step N sampled reach step N+1 on
        the device.  Returns the requests that finished in the step that was
        read (one step late).  A request that turns out to have stopped on an
        EOS has one token too many computed; the scheduler drops it.

        The reference overlaps the same way (python/freetoken/scheduler/scheduler.py:
        197-251, results drained one iteration late) and switches it off with the
        same variable, ``FREETOKEN_DISABLE_OVERLAP_SCHEDULING``."""
        step = self._launch(rngs)
        done = self.drain()
        if step is None and not done and self.scheduler.has_work():
            step = self._launch(rngs)       # everything waited for the drain (nothing was in flight)
            if step is None:
                raise RuntimeError("the scheduler has work but could plan nothing: the page pool is too small")
        self._inflight = step
        return done

    def _launch(self, rngs: Dict[Any, RequestRng]) -> Optional["_InFlight"]:
        """Plan a step and put it on the device: metadata copy, step, sampling
        and the copy of the sampled tokens to pinned memory, none waited for."""
        plan = self.scheduler.plan()
        if not plan:
            return None
        if self.status is not None:
            cache = self.engine.cache
            total, free = sum(cache.total_pages()), sum(cache.free_pages())
            self.status.report(plan, running=len(self.scheduler.running), queued=len(self.scheduler.pending),
                               pages_used=total - free, pages_total=total, page_size=cache.page_size)
        prev = self._inflight
        entries = []
        for e in plan:
            src = prev.index_of[e.request.id] if e.from_device else None
            entries.append(StepEntry(e.request.id, e.tokens, [len(e.tokens) - 1] if e.samples else [], src))
        logits = self.engine.step(entries, token_source=prev.tokens_dev if prev is not None else None)
        samplers = [e.request for e in plan if e.samples]
        step = _InFlight(plan, len(samplers), {r.id: i for i, r in enumerate(samplers)})
        if samplers:
            k = self._flip
            self._flip ^= 1
            rows = max(len(samplers), 64)
            if self._tok_dev[k] is None or self._tok_dev[k].numel() < rows:
                self._tok_dev[k] = torch.empty(rows, dtype=torch.int32, device=self.engine.device)
                self._tok_host[k] = torch.empty(rows, dtype=torch.int32).pin_memory()
            params = [r.params for r in samplers]
            uniforms = [0.0 if r.params.is_greedy else rngs[r.id].next_uniform() for r in samplers]
            step.tokens_dev = self.sampler.sample(logits, params, uniforms, out=self._tok_dev[k])
            step.tokens_host = self._tok_host[k]
            step.tokens_host[:len(samplers)].copy_(step.tokens_dev, non_blocking=True)
            # the word in which a kernel records a wait that ran out travels with the
            # tokens, so a failed step is noticed before its tokens are used (the
            # reference checks after every step too: engine/engine.py:922-925)
            step.status_host = self._status_host[k]
            step.status_host.copy_(ops.tc_status(self.engine.device), non_blocking=True)
            self.d2h_bytes_last_step = 4 * len(samplers) + 4
            step.event = torch.cuda.Event()
            step.event.record()
        return step

    def drain(self) -> List[Request]:
        """Wait for the step in flight (if any), read its tokens, record them."""
        step, self._inflight = self._inflight, None
        if step is None:
            return []
        sampled: List[int] = []
        if step.count:
            step.event.synchronize()
            ops.raise_for_status(int(step.status_host[0]), self.engine.device)
            sampled = step.tokens_host[:step.count].tolist()
        done = self.scheduler.complete(step.plan, sampled)
        self.engine._poison_freed()      # only in the page-poisoning debug mode
        return done
