"""Loading a model's tensors from safetensors by name.

Given the :class:`TensorSpec` list of a built model and a folder, the loader
decides from the file headers alone whether the folder fits: every tensor that
is missing, every tensor nobody asked for and every tensor of the wrong shape
is collected into ONE :class:`WeightError` before a byte of data is read.  The
reference raises at the first offender instead: a shape/dtype assert per
tensor, ``Unexpected keys`` for leftovers, ``KeyError`` for a missing one
(python/freetoken/layers/base.py:39-53).

Assembly (q,k,v -> qkv; per-expert w1,w3,w2 -> stacked gate_up/down) happens
slice by slice straight into the destination device tensor, so no second host
copy of a stacked expert bank is ever made
(cf. python/freetoken/models/loader.py:265-289,363-429).
"""

from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import Checkpoint
from .spec import Cat, Name, Source, TensorSpec, device_dtype, leaves


class WeightError(RuntimeError):
    """The checkpoint does not fit the model; lists everything that is wrong."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]]):
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        lines = [f"weights in '{folder}' do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + _short_list(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + _short_list(unexpected))
        if wrong_shape:
            shown = [f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in wrong_shape]
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + _short_list(shown, sep="; "))
        super().__init__("\n".join(lines))


def _short_list(items: Sequence[str], limit: int = 12, sep: str = ", ") -> str:
    shown = sep.join(items[:limit])
    if len(items) > limit:
        shown += f"{sep}... and {len(items) - limit} more"
    return shown


def plan_loading(
    specs: Sequence[TensorSpec],
    available: Dict[str, Tuple[int, ...]],
    folder: str = "<memory>",
    ignorable: Callable[[str], bool] = lambda name: False,
) -> Dict[str, Source]:
    """Choose a source for every spec from tensor names and shapes alone.

    ``available`` maps checkpoint name -> stored shape.  Returns
    ``{spec.name: chosen source}`` or raises :class:`WeightError`.
    """
    chosen: Dict[str, Source] = {}
    used = set()
    missing: List[str] = []
    wrong: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]] = []
    for spec in specs:
        best: Optional[Source] = None
        best_present = -1
        for src in spec.all_sources():
            lv = leaves(src)
            present = sum(1 for leaf in lv if leaf.name in available)
            if present == len(lv):
                best, best_present = src, present
                break
            if present > best_present:
                best, best_present = src, present
        lv = leaves(best)
        absent = [leaf.name for leaf in lv if leaf.name not in available]
        if absent:
            if best_present == 0 and spec.optional:
                continue
            missing.extend(absent)
            used.update(leaf.name for leaf in lv)
            continue
        for leaf in lv:
            used.add(leaf.name)
            found = tuple(available[leaf.name])
            if found != tuple(leaf.shape):
                wrong.append((leaf.name, tuple(leaf.shape), found))
        chosen[spec.name] = best
    unexpected = sorted(n for n in available if n not in used and not ignorable(n))
    if missing or unexpected or wrong:
        raise WeightError(folder, sorted(set(missing)), unexpected, wrong)
    return chosen


def _fill(src: Source, dst: torch.Tensor, read: Callable[[str], torch.Tensor]) -> None:
    if isinstance(src, Name):
        dst.copy_(read(src.name))
        return
    if isinstance(src, Cat):
        start = 0
        for p in src.parts:
            size = p.shape[src.dim]
            _fill(p, dst.narrow(src.dim, start, size), read)
            start += size
        return
    for i, p in enumerate(src.parts):
        _fill(p, dst[i], read)


def load_tensors(
    specs: Sequence[TensorSpec],
    folder: str,
    compute_dtype: torch.dtype,
    device: torch.device | str,
    rename: Callable[[str], Optional[str]] = lambda name: name,
    progress: Optional[Callable[[str], None]] = None,
) -> Dict[str, torch.Tensor]:
    """Load every tensor in ``specs`` from ``folder`` onto ``device``.

    ``rename`` maps a checkpoint name to the name the specs use, or to
    ``None`` for tensors that do not belong to the text decoder (they are
    ignored rather than reported as unexpected).
    """
    with Checkpoint(folder) as ckpt:
        alias: Dict[str, str] = {}
        shapes: Dict[str, Tuple[int, ...]] = {}
        for raw_name, entry in ckpt.entries.items():
            name = rename(raw_name)
            if name is None:
                continue
            alias[name] = raw_name
            shapes[name] = entry.shape
        chosen = plan_loading(specs, shapes, folder)
        out: Dict[str, torch.Tensor] = {}
        for i, spec in enumerate(specs):
            src = chosen.get(spec.name)
            if src is None or not spec.keep:
                continue
            stored = ckpt.entries[alias[leaves(src)[0].name]].dtype
            dtype = device_dtype(spec.role, stored, compute_dtype)
            dst = torch.empty(tuple(spec.shape), dtype=dtype, device=device)
            _fill(src, dst, lambda n: ckpt.read(alias[n]))
            out[spec.name] = dst
            if progress is not None and (i % 16 == 0 or i == len(specs) - 1):
                progress(f"loaded {i + 1}/{len(specs)} tensors")
        return out


def check_state(specs: Sequence[TensorSpec], state: Dict[str, torch.Tensor]) -> None:
    """Validate an in-memory ``{model-side name: tensor}`` state against specs."""
    missing = [s.name for s in specs if s.name not in state and not s.optional]
    names = {s.name for s in specs}
    specs = [s for s in specs if s.keep]
    unexpected = sorted(n for n in state if n not in names)
    wrong = [
        (s.name, tuple(s.shape), tuple(state[s.name].shape))
        for s in specs
        if s.name in state and tuple(state[s.name].shape) != tuple(s.shape)
    ]
    if missing or unexpected or wrong:
        raise WeightError("<memory>", missing, unexpected, wrong)
