"""Random-weights mode: a model from a configuration and a seed.

The reference's ``--dummy-weight`` fills every float tensor with ``randn``
under one global seed and calls the output garbage
(python/freetoken/engine/engine.py:242-268,303).  Here every tensor has a
random stream of its own, keyed by ``(seed, tensor name)``, so values do not
depend on creation order, and scales are chosen so that logits are usable for
numerical tests: matrices ~N(0, 0.02^2), norm weights 1 (or 1 + N(0, s^2)),
router bias ~N(0, s^2).

Two uses: :func:`random_state` creates the tensors directly on a device (the
benchmark's 90 GB model never touches a disk); :func:`write_model_folder`
writes ``config.json`` and ``model.safetensors`` so that the loader is
exercised like with a real checkpoint.
"""

from __future__ import annotations

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Sequence

import torch

from .safetensors_io import write_safetensors
from .spec import TensorSpec, device_dtype, take_apart


@dataclass(frozen=True)
class RandomOptions:
    """Standard deviations by tensor tag; ``None`` keeps the part's own choice."""

    matrix_std: Optional[float] = None
    norm_std: Optional[float] = None
    router_bias_std: Optional[float] = None
    # Matrices that write into the residual stream (attention output, expert down
    # projection; tag "residual_out") are matrices too, times this factor: the
    # usual 1/sqrt(2 * layers) of residual networks.  Without it a deep random
    # model's hidden states are dominated by what the layers add, the tokens of a
    # prompt look alike to the router and a few experts get all of them - unlike a
    # trained model, whose routing is balanced.
    residual_out_scale: Optional[float] = None
    embedding_std: Optional[float] = None      # the token embedding (tag "embedding"); default: as matrices

    def std_for(self, spec: TensorSpec) -> float:
        if spec.tag == "residual_out":
            base = spec.init.std if self.matrix_std is None else self.matrix_std
            return base * (1.0 if self.residual_out_scale is None else self.residual_out_scale)
        if spec.tag == "embedding":
            if self.embedding_std is not None:
                return self.embedding_std
            return spec.init.std if self.matrix_std is None else self.matrix_std
        override = {
            "matrix": self.matrix_std,
            "norm": self.norm_std,
            "router_bias": self.router_bias_std,
        }.get(spec.tag)
        return spec.init.std if override is None else override


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 62) - 1)


_CHUNK_ELEMENTS = 1 << 27


def random_tensor(spec: TensorSpec, seed: int, device, dtype: torch.dtype,
                  options: RandomOptions = RandomOptions()) -> torch.Tensor:
    """``mean + std * N(0,1)`` drawn in float32, then rounded to ``dtype``."""
    device = torch.device(device)
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, spec.name))
    std = options.std_for(spec)
    out = torch.empty(tuple(spec.shape), dtype=dtype, device=device)
    if spec.role == "int32":
        out.zero_()
        return out
    flat = out.view(-1)
    n = flat.numel()
    for begin in range(0, n, _CHUNK_ELEMENTS):
        end = min(n, begin + _CHUNK_ELEMENTS)
        if std == 0.0:
            flat[begin:end] = spec.init.mean
            continue
        draw = torch.randn(end - begin, generator=gen, device=device, dtype=torch.float32)
        flat[begin:end] = (draw * std + spec.init.mean).to(dtype)
    return out


def random_state(specs: Sequence[TensorSpec], seed: int, device,
                 compute_dtype: torch.dtype, file_dtype: torch.dtype = torch.bfloat16,
                 options: RandomOptions = RandomOptions()) -> Dict[str, torch.Tensor]:
    """Model-side tensors on ``device`` with the dtypes the loader would give
    them for a folder written in ``file_dtype``."""
    state: Dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.optional:
            continue
        stored = _file_dtype(spec, file_dtype)
        dtype = device_dtype(spec.role, stored, compute_dtype)
        # Draw in the stored precision first so that both compute modes see
        # the same (representable) values.
        t = random_tensor(spec, seed, device, stored, options)
        state[spec.name] = t if t.dtype == dtype else t.to(dtype)
    return state


def _file_dtype(spec: TensorSpec, file_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int32":
        return torch.int32
    if spec.keep_float32_in_file:
        return torch.float32
    return file_dtype


def write_model_folder(folder: str, config: Mapping, specs: Sequence[TensorSpec], seed: int,
                       file_dtype: torch.dtype = torch.bfloat16,
                       options: RandomOptions = RandomOptions(),
                       fused_names: bool = False) -> None:
    """Write ``config.json`` and ``model.safetensors`` for a random model.

    Tensors are written under their checkpoint names (the first source of each
    spec: separate q/k/v, one tensor per expert and projection) unless
    ``fused_names`` asks for the model-side names.
    """
    os.makedirs(folder, exist_ok=True)
    tensors: Dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.optional:
            continue
        t = random_tensor(spec, seed, "cpu", _file_dtype(spec, file_dtype), options)
        if fused_names or not spec.sources:
            tensors[spec.name] = t
        else:
            take_apart(spec.sources[0], t, tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config), f, indent=1, sort_keys=True)
