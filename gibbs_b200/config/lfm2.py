"""Typed configuration of the LFM2 architecture (``Lfm2ForCausalLM``) and its
plan: gated short-convolution layers and grouped-query attention layers with
per-head q/k RMSNorm, each followed by a SwiGLU feed-forward.

The keys, their fallbacks and the derived feed-forward width follow
MisterTK/gibbs ``arch/families/lfm2.json5:27-51``; the refusals follow
``arch/families/lfm2.json5:52-57``.  Unlike the reference, which decides a
layer's kind by the tensors present (``lfm2.json5:78-80``), the kinds are read
from ``layer_types`` / ``full_attn_idxs`` when config.json has them (and from
the tensor names otherwise), so that the loader can report a checkpoint that
disagrees with its configuration.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, asdict
from typing import Iterable, Optional

from .plan import ModelPlan, OrderEntry, PartSpec, prenorm_layer


class ConfigError(ValueError):
    pass


def _first(*vals):
    for v in vals:
        if v is not None:
            return v
    return None


@dataclass(frozen=True)
class Lfm2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    intermediate_size: int          # as written in config.json, before auto-adjust
    block_auto_adjust_ff_dim: bool
    block_ffn_dim_multiplier: float
    block_multiple_of: int
    norm_eps: float
    rope_theta: float
    conv_L_cache: int
    conv_bias: bool
    attention_bias: bool
    ffn_bias: bool
    tie_embedding: bool
    layer_types: tuple[str, ...]    # "conv" | "full_attention" per layer
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()

    # -- derived -------------------------------------------------------------
    @property
    def ffn_dim(self) -> int:
        """Feed-forward width (``lfm2.json5:36-40``): the written size, or when
        auto-adjust is on two thirds of it, scaled by the multiplier and
        rounded up to ``block_multiple_of`` if a multiplier is given."""
        if not self.block_auto_adjust_ff_dim:
            return self.intermediate_size
        ff23 = self.intermediate_size * 2 // 3
        if self.block_ffn_dim_multiplier > 0:
            m = self.block_multiple_of
            return m * math.ceil(int(self.block_ffn_dim_multiplier * ff23) / m)
        return ff23

    @property
    def attention_layers(self) -> tuple[int, ...]:
        return tuple(i for i, t in enumerate(self.layer_types) if t == "full_attention")

    @property
    def conv_layers(self) -> tuple[int, ...]:
        return tuple(i for i, t in enumerate(self.layer_types) if t == "conv")

    # -- parsing -------------------------------------------------------------
    @classmethod
    def from_dict(cls, cfg: dict, tensor_names: Optional[Iterable[str]] = None) -> "Lfm2Config":
        names = set(tensor_names) if tensor_names is not None else None

        def need(*keys):
            v = _first(*(cfg.get(k) for k in keys))
            if v is None:
                raise ConfigError(f"config.json has none of {list(keys)}")
            return v

        hidden = int(need("hidden_size"))
        layers = int(need("num_hidden_layers"))
        heads = int(need("num_attention_heads", "num_heads"))
        kv_heads = int(_first(cfg.get("num_key_value_heads"), heads))
        head_dim = int(_first(cfg.get("head_dim"), hidden // heads))
        rope_params = cfg.get("rope_parameters") or {}

        layer_types = cfg.get("layer_types")
        if layer_types is None and cfg.get("full_attn_idxs") is not None:
            idx = set(int(i) for i in cfg["full_attn_idxs"])
            bad = sorted(i for i in idx if not 0 <= i < layers)
            if bad:
                raise ConfigError(f"full_attn_idxs {bad} outside 0..{layers - 1}")
            layer_types = ["full_attention" if i in idx else "conv" for i in range(layers)]
        if layer_types is None:
            if names is None:
                raise ConfigError("config.json has neither layer_types nor full_attn_idxs, and no tensor names to decide by")
            layer_types = ["conv" if f"model.layers.{i}.conv.in_proj.weight" in names else "full_attention"
                           for i in range(layers)]
        layer_types = tuple(str(t) for t in layer_types)

        def has_any(suffix):
            return names is not None and any(n.endswith(suffix) for n in names)

        vocab = cfg.get("vocab_size")
        if vocab is None:
            raise ConfigError("config.json has no vocab_size")
        tie = _first(cfg.get("tie_embedding"), cfg.get("tie_word_embeddings"))
        if tie is None:
            tie = not (names is not None and "lm_head.weight" in names)
        eos = cfg.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))

        out = cls(
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=int(vocab),
            intermediate_size=int(_first(cfg.get("intermediate_size"), cfg.get("block_ff_dim"), 4 * hidden)),
            block_auto_adjust_ff_dim=cfg.get("block_auto_adjust_ff_dim") is True,
            block_ffn_dim_multiplier=float(_first(cfg.get("block_ffn_dim_multiplier"), 0)),
            block_multiple_of=int(_first(cfg.get("block_multiple_of"), 256)),
            norm_eps=float(_first(cfg.get("norm_eps"), cfg.get("rms_norm_eps"), 1e-5)),
            rope_theta=float(_first(cfg.get("rope_theta"), rope_params.get("rope_theta"), 10000)),
            conv_L_cache=int(need("conv_L_cache")),
            conv_bias=bool(_first(cfg.get("conv_bias"), has_any(".conv.conv.bias"))),
            attention_bias=bool(_first(cfg.get("attention_bias"), has_any(".self_attn.q_proj.bias"))),
            ffn_bias=bool(_first(cfg.get("ffn_bias"), has_any(".feed_forward.w1.bias"))),
            tie_embedding=bool(tie),
            layer_types=layer_types,
            max_position_embeddings=int(_first(cfg.get("max_position_embeddings"), 2048)),
            eos_token_ids=eos_ids,
        )
        out.check()
        return out

    def check(self) -> None:
        """Configurations that are refused, each with its reason."""
        if self.conv_L_cache < 2:
            raise ConfigError(f"LFM2 short-conv kernel (conv_L_cache) {self.conv_L_cache} must be >= 2")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim {self.head_dim} must be even for half-split rotary pairs")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(
                f"layer_types has {len(self.layer_types)} entries for {self.num_hidden_layers} layers")
        unknown = sorted(set(self.layer_types) - {"conv", "full_attention"})
        if unknown:
            raise ConfigError(f"unknown layer_types {unknown}; LFM2 knows 'conv' and 'full_attention'")
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "vocab_size", "block_multiple_of", "max_position_embeddings"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be positive, got {getattr(self, key)}")
        if self.ffn_dim <= 0:
            raise ConfigError(f"feed-forward width resolves to {self.ffn_dim}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm_eps must be positive, got {self.norm_eps}")

    def to_dict(self) -> dict:
        """config.json content that parses back to this configuration."""
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        eos = d.pop("eos_token_ids")
        if eos:
            d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        d["model_type"] = "lfm2"
        d["architectures"] = ["Lfm2ForCausalLM"]
        return d

    def dump(self) -> dict:
        """Resolved sizes, for ``--arch-dump``."""
        d = self.to_dict()
        d["ffn_dim (derived)"] = self.ffn_dim
        d["attention_layers (derived)"] = list(self.attention_layers)
        d["conv_layers (derived)"] = list(self.conv_layers)
        return d

    # -- plan ----------------------------------------------------------------
    def plan(self) -> ModelPlan:
        h, eps = self.hidden_size, self.norm_eps

        def norm(tensor, dim=h):
            return PartSpec("rmsnorm", {"dim": dim, "eps": eps}, {"weight": tensor})

        def with_bias(tensors: dict, stems: dict, on: bool) -> dict:
            if on:
                tensors = dict(tensors)
                tensors.update({local + ".bias": ckpt + ".bias" for local, ckpt in stems.items()})
            return tensors

        layers = []
        for i, kind in enumerate(self.layer_types):
            p = f"model.layers.{i}"
            if kind == "conv":
                stems = {"in_proj": f"{p}.conv.in_proj", "conv": f"{p}.conv.conv", "out_proj": f"{p}.conv.out_proj"}
                mixer = PartSpec(
                    "gated_short_conv",
                    {"hidden": h, "kernel": self.conv_L_cache, "bias": self.conv_bias},
                    with_bias({k + ".weight": v + ".weight" for k, v in stems.items()}, stems, self.conv_bias),
                )
            else:
                stems = {k: f"{p}.self_attn.{k}" for k in ("q_proj", "k_proj", "v_proj", "out_proj")}
                tensors = {k + ".weight": v + ".weight" for k, v in stems.items()}
                tensors["q_norm.weight"] = f"{p}.self_attn.q_layernorm.weight"
                tensors["k_norm.weight"] = f"{p}.self_attn.k_layernorm.weight"
                mixer = PartSpec(
                    "gqa_attention",
                    {
                        "hidden": h, "heads": self.num_attention_heads, "kv_heads": self.num_key_value_heads,
                        "head_dim": self.head_dim, "bias": self.attention_bias,
                        "qk_norm": True, "qk_norm_eps": eps, "scale": 1.0 / math.sqrt(self.head_dim),
                        "window": None,
                        "position": PartSpec("rope_half_split", {
                            "head_dim": self.head_dim, "rotary_dim": self.head_dim, "theta": self.rope_theta}),
                    },
                    with_bias(tensors, stems, self.attention_bias),
                )
            fstems = {k: f"{p}.feed_forward.{k}" for k in ("w1", "w3", "w2")}
            ffn = PartSpec(
                "swiglu", {"hidden": h, "inner": self.ffn_dim, "bias": self.ffn_bias},
                with_bias({"gate.weight": fstems["w1"] + ".weight", "up.weight": fstems["w3"] + ".weight",
                           "down.weight": fstems["w2"] + ".weight"},
                          {"gate": fstems["w1"], "up": fstems["w3"], "down": fstems["w2"]}, self.ffn_bias),
            )
            layers.append(prenorm_layer(norm(f"{p}.operator_norm.weight"), mixer, norm(f"{p}.ffn_norm.weight"), ffn))

        table = "model.embed_tokens.weight"
        plan = ModelPlan(
            architecture="Lfm2ForCausalLM",
            vocab_size=self.vocab_size,
            hidden_size=h,
            max_context=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"vocab": self.vocab_size, "dim": h}, {"weight": table}),
            layers=tuple(layers),
            order=tuple(OrderEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=norm("model.embedding_norm.weight"),
            head=PartSpec("lm_head", {"vocab": self.vocab_size, "dim": h},
                          {"weight": table if self.tie_embedding else "lm_head.weight"}),
        )
        plan.validate()
        return plan
