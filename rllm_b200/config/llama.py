"""Typed configuration of the Llama family, read from its own config.json keys.

Keys and defaults follow the reference's `ModelConfig`
(src/model/config.rs:332-378, 724-746, 966-968): `head_dim` defaults to
hidden_size / num_attention_heads; `rms_norm_eps` has the aliases `norm_eps`
and `layer_norm_epsilon`. Where the reference silently defaults a missing
`rope_theta` / eps to 0 we default to 10000 / 1e-5 instead. `sliding_window`
with `layer_types` (src/model/config.rs:553-558, 970-985) is honoured when
present, so one model may mix full and windowed attention layers.
`bos_token_id` and `eos_token_id` (a number or a list) are read where config.json has
them (`load_config` takes them from a generation_config.json beside it when config.json
has none); a model that names none has none. The reference hard-codes the Llama 3 ids in
its tokenizer wrapper (src/model/tokenizer.rs:64-65); here no id stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, ModelConfig, require_float, require_int

@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of config.json: the rule's name and its parameters. The names are those
    registered in `parts.rope_rules` (built in: "llama3", "linear"); the typed fields are the
    llama3 rule's, parameters of any other rule travel in `extra`."""
    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    extra: tuple = ()            # ((key, value), ...) of a registered rule's own keys

    @classmethod
    def from_dict(cls, raw: dict[str, Any] | None) -> "RopeScaling | None":
        from ..parts.rope_rules import check_rope_rule
        if raw is None:
            return None
        if not isinstance(raw, dict):
            raise ConfigError(f"rope_scaling must be an object or null, got {raw!r}")
        rtype = raw.get("rope_type", raw.get("type", "default"))
        if rtype == "default":
            return None
        params = {k: v for k, v in raw.items() if k not in ("rope_type", "type")}
        try:
            check_rope_rule(rtype, params)
        except ValueError as e:
            raise ConfigError(str(e)) from None
        if rtype == "linear":
            return cls(rope_type="linear", factor=float(params["factor"]))
        if rtype == "llama3":
            return cls("llama3", float(params["factor"]), float(params.get("low_freq_factor", 1.0)),
                       float(params.get("high_freq_factor", 4.0)), int(params["original_max_position_embeddings"]))
        try:
            return cls(rope_type=rtype, factor=float(params.get("factor", 1.0)), extra=tuple(sorted(params.items())))
        except TypeError:
            raise ConfigError(f"rope_scaling of rule {rtype!r}: parameters must be plain values") from None

    def to_dict(self) -> dict[str, Any]:
        if self.rope_type == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        if self.rope_type == "llama3":
            return {"rope_type": self.rope_type, "factor": self.factor,
                    "low_freq_factor": self.low_freq_factor,
                    "high_freq_factor": self.high_freq_factor,
                    "original_max_position_embeddings": self.original_max_position_embeddings}
        return {"rope_type": self.rope_type, **dict(self.extra)}


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    rope_scaling: RopeScaling | None = None
    attention_bias: bool = False
    sliding_window: int | None = None
    layer_types: tuple[str, ...] | None = None
    bos_token_id: int | None = None          # put in front of a text prompt
    eos_token_ids: tuple[int, ...] = ()      # a generation ends with any of these
    model_type: str = "llama"
    architectures: tuple[str, ...] = ("LlamaForCausalLM",)
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    # derived sizes
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> int | None:
        """The attention window of a layer, or None for all keys."""
        if not self.sliding_window:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "LlamaConfig":
        H = require_int(raw, "hidden_size")
        L = require_int(raw, "num_hidden_layers")
        nh = require_int(raw, "num_attention_heads")
        nkv = raw.get("num_key_value_heads")
        nkv = nh if nkv in (None, 0) else require_int(raw, "num_key_value_heads")
        hd = raw.get("head_dim")
        if hd in (None, 0):
            if H % nh:
                raise ConfigError(f"head_dim absent and hidden_size {H} is not a multiple of "
                                  f"num_attention_heads {nh}")
            hd = H // nh
        else:
            hd = require_int(raw, "head_dim")
        inter = require_int(raw, "intermediate_size")
        V = require_int(raw, "vocab_size")
        if nh % nkv:
            raise ConfigError(f"num_attention_heads {nh} is not a multiple of "
                              f"num_key_value_heads {nkv}")
        if hd % 2:
            raise ConfigError(f"head_dim {hd} must be even for rotary pairs")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported for Llama (silu only)")
        if raw.get("mlp_bias"):
            raise ConfigError("mlp_bias=true is not supported")
        sw = raw.get("sliding_window")
        if sw is not None:
            sw = require_int(raw, "sliding_window")
        lt = raw.get("layer_types")
        if lt is not None:
            if not isinstance(lt, (list, tuple)) or len(lt) != L:
                raise ConfigError(f"layer_types must list {L} entries, got {lt!r}")
            bad = [t for t in lt if t not in ("full_attention", "sliding_attention")]
            if bad:
                raise ConfigError(f"layer_types has unknown entries {sorted(set(bad))}")
            if "sliding_attention" in lt and not sw:
                raise ConfigError("layer_types names sliding_attention but sliding_window is unset")
            lt = tuple(lt)
        eps = require_float(raw, "rms_norm_eps", default=1e-5,
                            aliases=("norm_eps", "layer_norm_epsilon"))
        if eps <= 0:
            raise ConfigError(f"rms_norm_eps must be > 0, got {eps}")
        theta = require_float(raw, "rope_theta", default=10000.0)
        if theta <= 0:
            raise ConfigError(f"rope_theta must be > 0, got {theta}")
        bos, eos = raw.get("bos_token_id"), raw.get("eos_token_id")
        if eos is None:
            eos = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos = [eos]
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int) or not 0 <= bos < V):
            raise ConfigError(f"bos_token_id must be a token id below vocab_size {V}, got {bos!r}")
        if not isinstance(eos, (list, tuple)) or any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < V
                                                      for t in eos):
            raise ConfigError(f"eos_token_id must be a token id or a list of them below vocab_size {V}, got {eos!r}")
        known = {"bos_token_id", "eos_token_id", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                 "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings",
                 "rope_theta", "rms_norm_eps", "norm_eps", "layer_norm_epsilon",
                 "tie_word_embeddings", "rope_scaling", "attention_bias", "sliding_window",
                 "layer_types", "model_type", "architectures", "hidden_act", "mlp_bias"}
        return cls(
            hidden_size=H, num_hidden_layers=L, num_attention_heads=nh, num_key_value_heads=nkv,
            head_dim=hd, intermediate_size=inter, vocab_size=V,
            max_position_embeddings=require_int(raw, "max_position_embeddings", default=2048),
            rope_theta=theta, rms_norm_eps=eps,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            rope_scaling=RopeScaling.from_dict(raw.get("rope_scaling")),
            attention_bias=bool(raw.get("attention_bias", False)),
            sliding_window=sw, layer_types=lt, bos_token_id=bos, eos_token_ids=tuple(eos),
            model_type=raw.get("model_type", "llama"),
            architectures=tuple(raw.get("architectures") or ("LlamaForCausalLM",)),
            extra={k: v for k, v in raw.items() if k not in known},
        )

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architectures": list(self.architectures), "model_type": self.model_type,
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta, "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu",
            "attention_bias": self.attention_bias,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
        }
        if self.sliding_window:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        d["bos_token_id"] = self.bos_token_id
        d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0]
        return d
