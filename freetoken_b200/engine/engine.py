"""The engine: a model, its cache, and ONE step function.

``Engine.step(entries)`` takes a batch of ``(request, its next tokens, the
places whose logits are wanted)`` - portions of prompts beside single decoded
tokens, cut anywhere - runs exactly those tokens as one flat batch against the
cache earlier steps left, and returns float32 logits at the wanted places.
Everything above (scheduler, generation, trace replay, benchmark) drives this
one function.

The reference's step is ``Engine.forward_batch`` on a batch that is either all
prefill or all decode and returns sampled tokens
(python/freetoken/engine/engine.py:915-935, python/freetoken/core.py:112-116);
its scheduler builds positions, slot maps and attention metadata in pinned host
memory and copies them over (python/freetoken/scheduler/scheduler.py:877-908,
python/freetoken/attention/triton.py:218-269).  Here the batch is mixed, the
metadata is one packed int32 buffer (one host-to-device copy per step) and
logits are returned so that sampling stays a separate, testable step.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Hashable, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage, kv_bytes_per_token
from ..csrc import build, ops
from ..models.model import Model
from ..parts import linear
from ..parts.base import CacheView, Segment, StepContext, StepShape, Workspace
from ..registry import Architecture, architecture_of, read_model_config
from ..weights.loader import check_state, load_tensors
from ..weights.random_init import RandomOptions, random_state

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class StepEntry:
    """One request's share of a step."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among ``tokens`` whose logits are returned
    # When set, the entry's single token is not ``tokens[0]`` (a placeholder) but
    # element ``device_token`` of the ``token_source`` tensor given to the step:
    # a token sampled on the device that the host has not read yet.
    device_token: Optional[int] = None


@dataclass
class EngineArgs:
    """Runtime options (the reference's ``EngineConfig`` /``SchedulerConfig``,
    python/freetoken/engine/config.py:16-105, scheduler/config.py:14-43)."""

    dtype: Any = "bfloat16"
    device: str = "cuda:0"
    page_size: int = 64
    num_pages: Optional[int] = None          # pages per group; None: from max_tokens or free memory
    max_tokens: Optional[int] = None         # pool capacity in tokens (rounded up to pages)
    max_running_requests: int = 4
    max_seq_len: Optional[int] = None
    memory_ratio: float = 0.9
    max_step_tokens: int = 8192
    cuda_graph_max_bs: int = 64              # decode-only steps up to this batch are graph-replayed; 0: never
    poison_freed_pages: bool = False         # debugging: pages given back are filled with NaN
    nvtx: bool = False                       # NVTX ranges around every part of every layer (profiling)


def _align4(n: int) -> int:
    return (n + 3) & ~3


class Engine:
    def __init__(self, arch: Architecture, config: Any, tensors: Optional[Dict[str, torch.Tensor]],
                 args: EngineArgs, *, folder: Optional[str] = None, free_before: Optional[int] = None,
                 random_seed: Optional[int] = None, random_options: RandomOptions = RandomOptions(),
                 random_file_dtype: torch.dtype = torch.bfloat16):
        if not torch.cuda.is_available():
            raise RuntimeError("freetoken_b200 runs on a CUDA device only; no GPU is visible")
        self.args = args
        self.arch = arch
        self.config = config
        self.dtype: torch.dtype = DTYPES[args.dtype]
        self.device = torch.device(args.device)
        torch.cuda.set_device(self.device)
        if free_before is None:
            free_before = torch.cuda.mem_get_info(self.device)[0]
        self.plan = arch.build_plan(config)
        self.model = Model(self.plan, nvtx=args.nvtx)
        build.ensure_built(self.model.libraries(self.dtype))
        if self.dtype == torch.bfloat16:
            # asked once, here, so that no step (or graph capture) has to find out
            linear.library_offers_f32_out(self.device)
        specs = self.model.tensor_specs()
        if tensors is None and folder is not None:
            tensors = load_tensors(specs, folder, self.dtype, self.device, arch.rename_tensor,
                                   progress=None)
        elif tensors is None:
            tensors = random_state(specs, int(random_seed or 0), self.device, self.dtype,
                                   random_file_dtype, random_options)
        else:
            check_state(specs, tensors)
        self.tensors = tensors
        self.model.bind(tensors, self.dtype)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())

        needs = self.model.cache_needs()
        P = args.page_size
        max_pos = self.plan.max_position
        num_pages = args.num_pages
        if num_pages is None and args.max_tokens is not None:
            num_pages = -(-args.max_tokens // P)
        if num_pages is None:
            per_token = max(1, kv_bytes_per_token(needs, self.dtype))
            budget = int(args.memory_ratio * free_before) - self.weight_bytes - (4 << 30)
            num_pages = max(1, budget // (per_token * P))
            cap_len = args.max_seq_len or max_pos
            num_pages = min(num_pages, args.max_running_requests * (-(-cap_len // P)))
        self.max_seq_len = min(args.max_seq_len or max_pos, max_pos, num_pages * P)
        self.cache = CacheManager(needs, P, num_pages, args.max_running_requests, self.max_seq_len)
        self.storage = CacheStorage(self.cache, self.dtype, self.device)
        if args.poison_freed_pages:
            # every page but the sink starts out as unreadable as a freed one
            self.cache.record_freed = True
            for g, group in enumerate(self.cache.paged_groups):
                first = group.pool.first_page
                self.storage.poison(g, list(range(first, first + group.pool.num_pages)))
        self.workspace = Workspace(self.device)
        # parts whose kernels want step metadata of their own, one per plan key
        self._planners = self.model.step_planners()
        self._graphs_allowed = self.model.graph_capturable()
        self.cache_views: List[CacheView] = []
        for i, stop in enumerate(self.plan.schedule):
            owner = self.plan.cache_owner(i)
            view = CacheView(writes=(owner == i))
            if owner in self.cache.paged_index:
                view.kv_pages = self.storage.kv_of_stop(owner)
                view.block_table_index = self.cache.paged_index[owner][0]
            if owner in self.cache.state_index:
                view.state = self.storage.state_of_stop(owner)
            self.cache_views.append(view)
        self._pinned: List[torch.Tensor] = []
        self._pinned_events: List[torch.cuda.Event] = []
        self._pinned_turn = 0
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_generation = 0
        self._graphs: Dict[Tuple, "torch.cuda.CUDAGraph"] = {}
        self._graph_seen: Dict[Tuple, int] = {}
        self.graph_replays = 0
        self.steps = 0
        self.tokens_run = 0

    # ---- construction -----------------------------------------------------
    @classmethod
    def from_folder(cls, folder: str, args: Optional[EngineArgs] = None) -> "Engine":
        """A model folder: ``config.json`` picks the architecture, the
        safetensors files give the weights."""
        args = args or EngineArgs()
        arch, config = read_model_config(folder)
        return cls(arch, config, None, args, folder=folder)

    @classmethod
    def from_config(cls, config: Mapping[str, Any], seed: int, args: Optional[EngineArgs] = None,
                    random_options: RandomOptions = RandomOptions(),
                    file_dtype: torch.dtype = torch.bfloat16) -> "Engine":
        """Random weights created on the device from a config.json dictionary."""
        args = args or EngineArgs()
        arch = architecture_of(config)
        return cls(arch, arch.read_config(config), None, args, random_seed=seed,
                   random_options=random_options, random_file_dtype=file_dtype)

    # ---- requests ------------------------------------------------------------
    def has_request(self, request: Hashable) -> bool:
        return self.cache.has_request(request)

    def end_request(self, request: Hashable) -> None:
        """The request is finished: what it holds is given back."""
        if self.cache.has_request(request):
            self.cache.release(request)
            self._poison_freed()

    def _poison_freed(self) -> None:
        if self.args.poison_freed_pages:
            for group, pages in self.cache.take_freed():
                self.storage.poison(group, pages)

    def length(self, request: Hashable) -> int:
        return self.cache.length(request)

    @property
    def vocab_size(self) -> int:
        return self.plan.vocab_size

    # ---- the step --------------------------------------------------------------
    def _staging(self, count: int) -> torch.Tensor:
        turn = self._pinned_turn
        self._pinned_turn = (turn + 1) % 2
        while len(self._pinned) <= turn:
            self._pinned.append(torch.empty(0, dtype=torch.int32).pin_memory())
            self._pinned_events.append(torch.cuda.Event())
        self._pinned_events[turn].synchronize()
        if self._pinned[turn].numel() < count:
            self._pinned[turn] = torch.empty(max(count, 4096), dtype=torch.int32).pin_memory()
        if self._meta_dev is None or self._meta_dev.numel() < count:
            self._meta_dev = torch.empty(max(count, 4096), dtype=torch.int32, device=self.device)
            self._meta_generation += 1
        self._turn_used = turn
        return self._pinned[turn]

    def prepare(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None
                ) -> Tuple[StepContext, torch.Tensor, int, bool]:
        """Admit new requests, take pages for the step's tokens and stage the
        step's metadata on the device."""
        vocab = self.plan.vocab_size
        segments: List[Segment] = []
        seen = set()
        q = 0
        token_arrays: List[np.ndarray] = []
        for e in entries:
            arr = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
            n = arr.size
            if n == 0:
                raise ValueError(f"request {e.request!r} brings no tokens to the step")
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
            if arr.min() < 0 or arr.max() >= vocab:
                raise ValueError(f"request {e.request!r}: a token id is outside the vocabulary 0..{vocab - 1}")
            if e.device_token is not None:
                if n != 1 or token_source is None or not 0 <= e.device_token < token_source.numel():
                    raise ValueError(f"request {e.request!r}: a token on the device stands for exactly one "
                                     f"token and needs a token_source that holds it")
            token_arrays.append(arr.astype(np.int32))
        # New requests take a slot; every request takes the pages its tokens
        # need.  If that fails nothing of the step has run: requests that were
        # new give their slot and pages back, older ones keep pages they will
        # need anyway.
        fresh: List[Hashable] = []
        try:
            for e in entries:
                if not self.cache.has_request(e.request):
                    self.cache.admit(e.request)
                    fresh.append(e.request)
            for e, arr in zip(entries, token_arrays):
                self.cache.grow(e.request, self.cache.length(e.request) + arr.size)
        except Exception:
            for r in fresh:
                self.cache.release(r)
            raise
        for e, arr in zip(entries, token_arrays):
            segments.append(Segment(self.cache.slot(e.request), self.cache.length(e.request), arr.size, q))
            q += arr.size
        T, S = q, len(segments)
        N = sum(len(e.want) for e in entries)
        P = self.cache.page_size
        max_kv = max(s.pos0 + s.n for s in segments)
        max_q = max(s.n for s in segments)
        width = max(1, -(-max_kv // P))
        if max_q == 1:
            # decode-only steps keep their metadata layout (and with it a
            # captured graph) while contexts grow: the table width moves in
            # steps of 8 pages
            width = min(-(-width // 8) * 8, self.cache.max_pages_per_request)
        groups = self.cache.paged_groups

        # what the parts plan for their own kernels (row lists, tile lists)
        shape = StepShape(segments, T, P, width, max_q, max_kv)
        plans = {key: part.plan_step(shape) for key, part in self._planners.items()}

        # packed layout, every section 16-byte aligned
        off = {}
        cur = 0
        for name, size in (("token_ids", T), ("token_pos", T), ("token_seg", T), ("seg_slot", S),
                           ("seg_pos0", S), ("seg_q_start", S + 1), ("seg_kv_len", S),
                           ("logit_rows", N)):
            off[name] = cur
            cur = _align4(cur + size)
        for i, plan in enumerate(plans.values()):
            for name, array in plan.arrays.items():
                off[f"plan{i}.{name}"] = cur
                cur = _align4(cur + int(array.size))
        for g in range(len(groups)):
            off[f"table{g}"] = cur
            cur = _align4(cur + S * width)
        # after everything a captured graph reads, so that those offsets do not move
        patches = [(s.q_start, e.device_token) for e, s in zip(entries, segments)
                   if e.device_token is not None]
        for name in ("patch_rows", "patch_src"):
            off[name] = cur
            cur = _align4(cur + len(patches))
        host = self._staging(cur)
        h = host.numpy()
        rows: List[int] = []
        for i, (e, s) in enumerate(zip(entries, segments)):
            a, b = s.q_start, s.q_start + s.n
            h[off["token_ids"] + a: off["token_ids"] + b] = token_arrays[i]
            h[off["token_pos"] + a: off["token_pos"] + b] = np.arange(s.pos0, s.pos0 + s.n, dtype=np.int32)
            h[off["token_seg"] + a: off["token_seg"] + b] = i
            h[off["seg_slot"] + i] = s.slot
            h[off["seg_pos0"] + i] = s.pos0
            h[off["seg_q_start"] + i] = s.q_start
            h[off["seg_kv_len"] + i] = s.pos0 + s.n
            rows.extend(s.q_start + w for w in e.want)
            for g, group in enumerate(groups):
                base = off[f"table{g}"] + i * width
                h[base: base + width] = group.block_table[s.slot, :width]
        h[off["seg_q_start"] + S] = T
        if N:
            h[off["logit_rows"]: off["logit_rows"] + N] = np.asarray(rows, dtype=np.int32)
        for i, plan in enumerate(plans.values()):
            for name, array in plan.arrays.items():
                if array.size:
                    h[off[f"plan{i}.{name}"]: off[f"plan{i}.{name}"] + array.size] = array
        if patches:
            pp = np.asarray(patches, dtype=np.int32)
            h[off["patch_rows"]: off["patch_rows"] + len(patches)] = pp[:, 0]
            h[off["patch_src"]: off["patch_src"] + len(patches)] = pp[:, 1]
        dev = self._meta_dev
        self._last_meta_ints = cur
        dev[:cur].copy_(host[:cur], non_blocking=True)
        self._pinned_events[self._turn_used].record()

        def sec(name: str, size: int) -> torch.Tensor:
            return dev[off[name]: off[name] + size]

        if patches:
            ops.patch_tokens(sec("token_ids", T), sec("patch_rows", len(patches)), token_source,
                             sec("patch_src", len(patches)), vocab)

        for i, plan in enumerate(plans.values()):
            plan.tensors = {name: sec(f"plan{i}.{name}", int(array.size)) for name, array in plan.arrays.items()}
        ctx = StepContext(
            device=self.device, dtype=self.dtype, segments=segments, num_tokens=T,
            token_ids=sec("token_ids", T), token_pos=sec("token_pos", T),
            token_seg=sec("token_seg", T), seg_slot=sec("seg_slot", S), seg_pos0=sec("seg_pos0", S),
            seg_q_start=sec("seg_q_start", S + 1), seg_kv_len=sec("seg_kv_len", S),
            block_tables=[sec(f"table{g}", S * width).view(S, width) for g in range(len(groups))],
            workspace=self.workspace, page_size=P, max_q_len=max_q, max_kv_len=max_kv,
            max_positions=self.max_seq_len, plans=plans)
        in_order = N == T and rows == list(range(T))
        return ctx, sec("logit_rows", N), N, in_order

    def step(self, entries: Sequence[StepEntry], probe: Optional[Dict[str, Any]] = None,
             token_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch; returns float32 logits ``[wanted, vocab]`` on the
        device, in the order of the entries and of their ``want`` lists.
        ``token_source`` (int32, on the device) holds the tokens of entries
        that name a ``device_token``."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        ctx, logit_rows, N, in_order = self.prepare(entries, token_source)
        ctx.probe = probe
        self.last_meta_ints = self._last_meta_ints
        self.storage.clear_state(self.cache.take_fresh_slots())
        logits = self.workspace.get("engine.logits", (N, self.plan.vocab_size), torch.float32)
        if not self._replay_graph(ctx, logit_rows, logits, N, in_order, probe):
            self.model.forward(ctx, self.cache_views, logit_rows, logits, in_order)
        for e, seg in zip(entries, ctx.segments):
            self.cache.advance(e.request, seg.n)
        self._poison_freed()        # pages a window has passed
        self.steps += 1
        self.tokens_run += ctx.num_tokens
        return logits

    def _replay_graph(self, ctx: StepContext, logit_rows, logits, N: int, in_order: bool, probe) -> bool:
        """Decode-only steps with every row's logits wanted run as a captured
        CUDA graph (the reference captures its decode step per batch size,
        python/freetoken/engine/graph.py:127-198).  A key is run eagerly once
        (which also sizes every scratch buffer), captured at its second use
        and replayed from then on.  Returns whether the step ran as a graph."""
        T = ctx.num_tokens
        if (probe is not None or not ctx.decode_only or not in_order or N != T
                or T > self.args.cuda_graph_max_bs or self.dtype != torch.bfloat16
                or not self._graphs_allowed):
            return False
        key = (T, tuple(t.shape[1] for t in ctx.block_tables), self.workspace.generation,
               self._meta_generation)
        graph = self._graphs.get(key)
        if graph is None:
            seen = self._graph_seen.get(key, 0)
            self._graph_seen[key] = seen + 1
            if seen == 0:
                return False
            # drop graphs whose buffers were replaced
            for old in [k for k in self._graphs if k[2:] != key[2:]]:
                del self._graphs[old]
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(graph):
                self.model.forward(ctx, self.cache_views, logit_rows, logits, in_order)
            kernels = ops.launch_count() - before
            ops.LAUNCHES -= kernels          # recorded, not run
            self._graphs[key] = (graph, kernels)
            graph = self._graphs[key]
        graph[0].replay()
        ops.LAUNCHES += graph[1]
        self.graph_replays += 1
        return True

    def check_status(self) -> None:
        """Raise if a kernel recorded a failure (a bounded wait that ran out)
        since the last check.  Synchronises the device."""
        ops.check_tc_status(self.device)

    # ---- reporting ---------------------------------------------------------------
    def stats(self) -> Dict[str, Any]:
        return {
            "steps": self.steps,
            "tokens": self.tokens_run,
            "weight_bytes": self.weight_bytes,
            "cache_bytes": self.storage.bytes(),
            "workspace_bytes": self.workspace.bytes(),
            "pages_total": self.cache.total_pages(),
            "pages_free": self.cache.free_pages(),
            "live_requests": len(self.cache.live_requests()),
        }
