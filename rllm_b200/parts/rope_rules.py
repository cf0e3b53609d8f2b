"""Rules that turn the plain rotary frequencies f_i = theta^(-2i/d) into a model's own, by name.

A rule is a function `(inverse frequencies as float64 list, the rule's parameters as a dict) ->
list` and, optionally, a check of the parameters that raises ValueError. The name is what a
config.json carries in `rope_scaling.rope_type`; the configuration reader accepts exactly the
registered names and the rotary part applies the rule, so another rule (another family's long
context scheme) is one `register_rope_rule` call, from anywhere.

Built in: "linear" (every frequency divided by `factor`) and "llama3", the three bands of the
reference's "yarn" kernel (src/gpu/cuda/shaders/rope.cu:233-251) with beta_fast =
high_freq_factor and beta_slow = low_freq_factor. The reference parses `rope_scaling` for Llama
(src/model/config.rs:724-746) but never applies it; here it is applied.
"""
from __future__ import annotations

import math
from typing import Callable

_RULES: dict[str, tuple[Callable, Callable | None]] = {}


def register_rope_rule(name: str, rule: Callable[[list[float], dict], list[float]],
                       check: Callable[[dict], None] | None = None) -> None:
    _RULES[name] = (rule, check)


def registered_rope_rules() -> list[str]:
    return sorted(_RULES)


def rope_rule(name: str) -> Callable[[list[float], dict], list[float]]:
    try:
        return _RULES[name][0]
    except KeyError:
        raise KeyError(f"no rotary frequency rule named {name!r}; registered: {registered_rope_rules()}") from None


def check_rope_rule(name: str, params: dict) -> None:
    """Raise ValueError if the rule's parameters are missing or out of range."""
    rule = _RULES.get(name)
    if rule is None:
        raise ValueError(f"rope_scaling.rope_type {name!r} is not supported (supported: "
                         f"{['default'] + registered_rope_rules()})")
    if rule[1] is not None:
        rule[1](params)


def _need(params: dict, key: str, kind=float):
    v = params.get(key)
    if v is None:
        raise ValueError(f"config.json lacks required key {key!r} (in rope_scaling)")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and not isinstance(v, int)):
        raise ValueError(f"config key {key!r} (in rope_scaling) must be a number, got {v!r}")
    return v


def _linear(freqs, p):
    return [f / float(p["factor"]) for f in freqs]


def _check_factor(p):
    if _need(p, "factor") <= 0:
        raise ValueError(f"rope_scaling.factor must be > 0, got {p['factor']}")


def _llama3(freqs, p):
    factor, low, high = float(p["factor"]), float(p.get("low_freq_factor", 1.0)), float(p.get("high_freq_factor", 4.0))
    orig = float(p["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / high:
            pass
        elif wavelen > orig / low:
            f = f / factor
        else:
            s = (orig / wavelen - low) / (high - low)
            f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def _check_llama3(p):
    _check_factor(p)
    low = p.get("low_freq_factor", 1.0)
    high = p.get("high_freq_factor", 4.0)
    if _need(p, "original_max_position_embeddings", int) < 1:
        raise ValueError("rope_scaling.original_max_position_embeddings must be >= 1")
    if high <= low:
        raise ValueError(f"rope_scaling: high_freq_factor must exceed low_freq_factor (got low={low}, high={high})")


register_rope_rule("linear", _linear, _check_factor)
register_rope_rule("llama3", _llama3, _check_llama3)
