"""Typed configuration of the MiniMax-M3 decoder, read from ``config.json``.

Field names are the architecture's own config.json keys as the reference reads
them (python/freetoken/models/minimax_m3/args.py:135-254,
python/freetoken/models/minimax_m3/config.py:61-198); defaults are the
reference readers' defaults, so a reference-style file parses to the same
values.  No size and no constant that config.json gives stands anywhere else
in the code: parts receive them as parameters through :func:`build_plan`.

Options the reference's ``minimax_m3`` module hard-wires and this decoder reads
instead: ``use_gemma_norm`` (args.py:208-210), ``qk_norm_type`` (args.py:207;
``per_layer`` is the sibling definition's form,
python/freetoken/models/minimax_m2/attention.py:45-47), ``scoring_func``
(args.py:199-202), ``norm_topk_prob`` (config.py:175), ``hidden_act``
(config.py:128-135).  Features of the reference's checkpoint that this decoder
does not have (block-sparse attention, shared expert, dense-MLP prefix,
quantized tensors, rope scaling) are refused with the offending key.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, fields
from typing import Any, Dict, Mapping, Tuple

from .model_plan import LayerSpec, ModelPlan, PartSpec, sequential_schedule

ARCHITECTURES: Tuple[str, ...] = (
    "MiniMaxM3ForCausalLM",
    "MiniMaxM3SparseForCausalLM",
    "MiniMaxM3SparseForConditionalGeneration",
)


class ConfigError(ValueError):
    """A config.json key is missing, malformed or asks for an unsupported feature."""


@dataclass(frozen=True)
class MiniMaxM3Config:
    # sizes
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    # position encoding
    rotary_dim: int
    rope_theta: float
    # norms
    rms_norm_eps: float
    use_gemma_norm: bool
    use_qk_norm: bool
    qk_norm_type: str
    # routed experts
    num_local_experts: int
    num_experts_per_tok: int
    intermediate_size: int
    scoring_func: str
    use_routing_bias: bool
    norm_topk_prob: bool
    routed_scaling_factor: float
    hidden_act: str
    swiglu_alpha: float
    swiglu_limit: float
    # head
    tie_word_embeddings: bool
    # bookkeeping
    architectures: Tuple[str, ...] = (ARCHITECTURES[0],)
    model_type: str = "minimax_m3"
    torch_dtype: str = "bfloat16"

    # ---- derived sizes -------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def sm_scale(self) -> float:
        # python/freetoken/attention/triton.py:163 -- head_dim ** -0.5
        return float(self.head_dim) ** -0.5

    # ---- reading ---------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "MiniMaxM3Config":
        top = dict(raw)
        text = dict(top.get("text_config") or top)  # config.py:42-43 unwraps text_config

        def need(key: str) -> Any:
            if key not in text or text[key] is None:
                raise ConfigError(f"config.json: required key '{key}' is missing")
            return text[key]

        def opt(key: str, default: Any) -> Any:
            value = text.get(key, default)
            return default if value is None else value

        hidden = int(need("hidden_size"))
        heads = int(need("num_attention_heads"))
        head_dim = int(opt("head_dim", hidden // heads))  # args.py:212-214
        rotary_dim = text.get("rotary_dim")
        if rotary_dim is None:  # args.py:215-217
            rotary_dim = int(head_dim * float(opt("partial_rotary_factor", 1.0)))
        theta = text.get("rope_theta")
        rope_params = text.get("rope_parameters") or {}
        if theta is None and isinstance(rope_params, Mapping):  # args.py:91-96
            theta = rope_params.get("rope_theta")
        theta = 10000.0 if theta is None else float(theta)

        scaling = text.get("rope_scaling") or rope_params or {}
        rope_type = scaling.get("rope_type", scaling.get("type", "default")) if scaling else "default"
        if rope_type not in (None, "default"):  # args.py:193-198
            raise ConfigError(f"config.json: 'rope_scaling' {scaling!r} is not supported (plain rope only)")

        _refuse_foreign_features(top, text)

        cfg = cls(
            hidden_size=hidden,
            num_hidden_layers=int(need("num_hidden_layers")),
            num_attention_heads=heads,
            num_key_value_heads=int(opt("num_key_value_heads", heads)),
            head_dim=head_dim,
            vocab_size=int(need("vocab_size")),
            max_position_embeddings=int(need("max_position_embeddings")),
            rotary_dim=int(rotary_dim),
            rope_theta=theta,
            rms_norm_eps=float(need("rms_norm_eps")),
            use_gemma_norm=bool(opt("use_gemma_norm", True)),
            use_qk_norm=bool(opt("use_qk_norm", True)),
            qk_norm_type=str(opt("qk_norm_type", "per_head")),
            num_local_experts=int(need("num_local_experts")),
            num_experts_per_tok=int(need("num_experts_per_tok")),
            intermediate_size=int(need("intermediate_size")),
            scoring_func=str(opt("scoring_func", "sigmoid")),
            use_routing_bias=bool(opt("use_routing_bias", False)),
            norm_topk_prob=bool(opt("norm_topk_prob", True)),
            routed_scaling_factor=float(opt("routed_scaling_factor", 1.0)),
            hidden_act=str(opt("hidden_act", "swigluoai")),
            swiglu_alpha=float(opt("swiglu_alpha", 1.702)),
            swiglu_limit=float(opt("swiglu_limit", 7.0)),
            tie_word_embeddings=bool(opt("tie_word_embeddings", False)),
            architectures=tuple(top.get("architectures") or (ARCHITECTURES[0],)),
            model_type=str(top.get("model_type", "minimax_m3")),
            torch_dtype=str(opt("torch_dtype", top.get("torch_dtype", "bfloat16"))),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "MiniMaxM3Config":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        out = asdict(self)
        out["architectures"] = list(self.architectures)
        return out

    def replace(self, **changes: Any) -> "MiniMaxM3Config":
        values = {f.name: getattr(self, f.name) for f in fields(self)}
        values.update(changes)
        cfg = MiniMaxM3Config(**values)
        cfg.validate()
        return cfg

    # ---- validation ----------------------------------------------------
    def validate(self) -> None:
        def bad(key: str, why: str) -> None:
            raise ConfigError(f"config.json: '{key}' = {getattr(self, key)!r} {why}")

        for key in (
            "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
            "head_dim", "vocab_size", "max_position_embeddings", "num_local_experts",
            "num_experts_per_tok", "intermediate_size",
        ):
            if getattr(self, key) <= 0:
                bad(key, "must be positive")
        if self.num_attention_heads % self.num_key_value_heads:
            bad("num_key_value_heads", f"does not divide num_attention_heads = {self.num_attention_heads}")
        if self.rotary_dim < 0 or self.rotary_dim > self.head_dim:
            bad("rotary_dim", f"must lie in 0..head_dim = {self.head_dim}")  # rotary.py:47
        if self.rotary_dim % 2:
            bad("rotary_dim", "must be even")  # rotary.py:48
        if self.num_experts_per_tok > self.num_local_experts:
            bad("num_experts_per_tok", f"exceeds num_local_experts = {self.num_local_experts}")
        if self.rms_norm_eps <= 0:
            bad("rms_norm_eps", "must be positive")
        if self.rope_theta <= 0:
            bad("rope_theta", "must be positive")
        if self.scoring_func not in ("sigmoid", "softmax"):
            bad("scoring_func", "is not one of 'sigmoid', 'softmax'")
        if self.qk_norm_type not in ("per_layer", "per_head"):
            bad("qk_norm_type", "is not one of 'per_layer', 'per_head'")
        if self.hidden_act not in ("silu", "swigluoai"):
            bad("hidden_act", "is not one of 'silu', 'swigluoai'")
        if self.routed_scaling_factor <= 0:
            bad("routed_scaling_factor", "must be positive")


def _refuse_foreign_features(top: Mapping[str, Any], text: Mapping[str, Any]) -> None:
    """Refuse keys that switch on parts this decoder does not have."""
    sparse = text.get("sparse_attention_config") or {}
    if sparse.get("use_sparse_attention"):  # args.py:99-122
        raise ConfigError("config.json: 'sparse_attention_config.use_sparse_attention' is not supported (dense attention only)")
    if "minimax_m3_sparse" in (text.get("layer_types") or []):
        raise ConfigError("config.json: 'layer_types' contains 'minimax_m3_sparse' (dense attention only)")
    if text.get("attention_output_gate"):  # args.py:204-206
        raise ConfigError("config.json: 'attention_output_gate' is not supported")
    if top.get("quantization_config") or text.get("quantization_config"):  # config.py:125-126
        raise ConfigError("config.json: 'quantization_config' is not supported (bfloat16 or float32 weights only)")
    if int(text.get("n_shared_experts") or 0) > 0:  # moe.py:63-69
        raise ConfigError("config.json: 'n_shared_experts' > 0 is not supported (no shared expert)")
    freq = text.get("moe_layer_freq")
    if freq is not None and not all(bool(f) for f in freq):  # args.py:125-132
        raise ConfigError("config.json: 'moe_layer_freq' has dense layers; every layer must be routed experts")
    mlp_types = text.get("mlp_layer_types")
    if mlp_types is not None and any(t != "sparse" for t in mlp_types):
        raise ConfigError("config.json: 'mlp_layer_types' has dense layers; every layer must be routed experts")
    if float(text.get("swiglu_beta", 1.0)) != 1.0:  # args.py:188-189
        raise ConfigError("config.json: 'swiglu_beta' other than 1.0 is not supported")


def build_plan(cfg: MiniMaxM3Config) -> ModelPlan:
    """Turn the typed configuration into the list of parts to build.

    Every layer is: RMSNorm -> GQA softmax attention (QK norm, partial NeoX
    rotary) -> RMSNorm -> sigmoid/softmax top-k routed SwiGLU experts, in the
    pre-norm residual arrangement of
    python/freetoken/models/minimax_m2/model.py:27-37.
    """
    def norm(scope: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps,
                                    "plus_one": cfg.use_gemma_norm, "scope": scope})

    qk_norm = cfg.qk_norm_type if cfg.use_qk_norm else "none"
    mixer = PartSpec("paged_attention", {
        "hidden_size": cfg.hidden_size,
        "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "sm_scale": cfg.sm_scale,
        "qk_norm": qk_norm,
        "qk_norm_eps": cfg.rms_norm_eps,
        "qk_norm_plus_one": cfg.use_gemma_norm,
        "sliding_window": None,
        "position": PartSpec("rotary_neox", {
            "head_dim": cfg.head_dim,
            "rotary_dim": cfg.rotary_dim,
            "theta": cfg.rope_theta,
            "max_position": cfg.max_position_embeddings,
        }),
        # tensor names: python/freetoken/models/minimax_m3/weight.py:182-196
        "scope": "self_attn",
        "checkpoint_names": {
            "qkv": "qkv_proj.weight", "o": "o_proj.weight",
            "q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight",
            "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
        },
    })
    ffn = PartSpec("routed_experts", {
        "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.intermediate_size,
        "num_experts": cfg.num_local_experts,
        "top_k": cfg.num_experts_per_tok,
        "scoring": cfg.scoring_func,
        "use_bias": cfg.use_routing_bias,
        "renormalize": cfg.norm_topk_prob,
        "scale": cfg.routed_scaling_factor,
        "activation": cfg.hidden_act,
        "act_alpha": cfg.swiglu_alpha,
        "act_limit": cfg.swiglu_limit,
        # tensor names: python/freetoken/models/minimax_m3/weight.py:30-54,209-222,
        # python/freetoken/layers/moe.py:83-92 (w1 = gate, w3 = up, w2 = down)
        "scope": "block_sparse_moe",
        "checkpoint_names": {
            "router": "gate.weight", "bias": "e_score_correction_bias",
            "gate_up": "experts.gate_up_proj", "down": "experts.down_proj",
            "gate": "experts.{e}.w1.weight", "up": "experts.{e}.w3.weight",
            "down_each": "experts.{e}.w2.weight",
        },
    })
    layers = tuple(
        LayerSpec(
            prefix=f"model.layers.{i}",
            block=PartSpec("prenorm", {}),
            mixer=mixer,
            feed_forward=ffn,
            mixer_norm=norm("input_layernorm"),
            feed_forward_norm=norm("post_attention_layernorm"),
        )
        for i in range(cfg.num_hidden_layers)
    )
    plan = ModelPlan(
        architecture=cfg.architectures[0],
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                               "hidden_size": cfg.hidden_size,
                                               "prefix": "model", "scope": "embed_tokens"}),
        layers=layers,
        schedule=sequential_schedule(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", {**norm("norm").params, "prefix": "model"}),
        head=PartSpec("lm_head", {
            "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
            "prefix": "", "scope": "lm_head",
            "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None}),
        max_position=cfg.max_position_embeddings,
    )
    plan.validate()
    return plan


# Tensors of a checkpoint that do not belong to the text decoder.
_IGNORED_PREFIXES = ("vision_tower.", "multi_modal_projector.", "visual.", "mtp.")


def rename_checkpoint_tensor(name: str):
    """Checkpoint tensor name -> model-side name, or ``None`` to ignore it.

    The checkpoint nests the decoder under ``language_model.``
    (python/freetoken/models/minimax_m3/weight.py:182-183,244-246), the sibling
    layout does not (python/freetoken/models/minimax_m2/weight.py:26-29); vision
    towers and calibration scales are skipped (minimax_m2/weight.py:70-76).
    """
    if name.startswith(_IGNORED_PREFIXES):
        return None
    if name.startswith("language_model."):
        name = name[len("language_model."):]
    if name.endswith((".k_scale", ".v_scale")) or (".self_attn." in name and name.endswith("_scale")):
        return None
    return name
