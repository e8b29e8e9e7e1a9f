"""One registry from an architecture's name to everything needed to serve it.

The reference maps ``hf_config.architectures[0]`` to a module, a model class, a
``parse_config`` and an ``iter_weights`` by name, imported lazily
(python/freetoken/models/register.py:11-143, python/freetoken/engine/config.py:88-92).
Here an :class:`Architecture` holds the typed configuration's reader, the
function that turns it into a :class:`ModelPlan`, and the checkpoint-name rule;
the model itself is always the generic :class:`freetoken_b200.models.Model`
built from the plan.  Adding an architecture is one ``register_architecture``
call; nothing else in the framework changes.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Sequence, Tuple

from .config.model_plan import ModelPlan


@dataclass(frozen=True)
class Architecture:
    name: str
    read_config: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed config
    build_plan: Callable[[Any], ModelPlan]
    config_to_dict: Callable[[Any], Dict[str, Any]]
    rename_tensor: Callable[[str], Optional[str]] = lambda name: name


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, aliases: Sequence[str] = ()) -> Architecture:
    for name in (arch.name, *aliases):
        _ARCHITECTURES[name] = arch
    return arch


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        known = ", ".join(sorted(_ARCHITECTURES))
        raise ValueError(f"Model architecture '{name}' is not supported (known: {known})") from None


def known_architectures() -> Tuple[str, ...]:
    _load_builtin()
    return tuple(sorted(_ARCHITECTURES))


def architecture_of(config: Mapping[str, Any]) -> Architecture:
    names = config.get("architectures") or []
    if not names:
        raise ValueError("config.json has no 'architectures' entry to choose the model by")
    return get_architecture(names[0])


def read_model_config(folder_or_file: str) -> Tuple[Architecture, Any]:
    """``(architecture, typed config)`` of a model folder (or config.json path)."""
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as f:
        raw = json.load(f)
    arch = architecture_of(raw)
    return arch, arch.read_config(raw)


_loaded = False


def _load_builtin() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    from .config import minimax_m3 as m3
    register_architecture(
        Architecture(
            name=m3.ARCHITECTURES[0],
            read_config=m3.MiniMaxM3Config.from_dict,
            build_plan=m3.build_plan,
            config_to_dict=lambda cfg: cfg.to_dict(),
            rename_tensor=m3.rename_checkpoint_tensor,
        ),
        aliases=m3.ARCHITECTURES[1:],
    )
