"""What a model is put together from: parts with declared weights and cache needs.

A part (mixer, feed-forward, norm, position encoding, block, embedding, output
head) takes its sizes and constants as constructor arguments and never asks
which model it sits in. It declares

  * `params()`: the tensors it owns, each assembled from one or more checkpoint
    tensors (concatenated along dim 0), named relative to the part's prefix;
  * `cache_spec()`: what it needs per request from the cache manager (paged
    keys/values, all or a window of them; or a fixed-size state), or None;
  * `forward(...)` against a `StepContext`.

Part kinds are registered by name so that a configuration can choose them layer
by layer, and so that code outside the package can add a kind.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass(frozen=True)
class Source:
    """One tensor of the checkpoint. `init` tells the random-weights mode how to fill it:
    "normal" (N(0, std)), "norm" (1, or 1 + N(0, norm_std)), "zeros"."""
    name: str
    shape: tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class Param:
    """A tensor a part owns: `sources` concatenated along dim 0.
    role "matrix": stored in the run dtype (bfloat16 or float32);
    role "vector": kept as the checkpoint stores it (32-bit stays 32-bit; everything
    becomes float32 in the 32-bit run);
    role "table": integers, kept as int32."""
    attr: str
    sources: tuple[Source, ...]
    role: str = "matrix"

    @property
    def shape(self) -> tuple[int, ...]:
        first = self.sources[0].shape
        return (sum(s.shape[0] for s in self.sources),) + tuple(first[1:])


@dataclass(frozen=True)
class KVCacheSpec:
    """Paged keys and values: `window` None keeps every key, else only the last `window`."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state: name -> (shape, dtype). Zeroed when a request opens."""
    tensors: tuple[tuple[str, tuple[int, ...], torch.dtype], ...]


class Part:
    """Base of all parts. `prefix` (checkpoint name prefix, ending in '.') is set by
    whoever assembles the model."""
    prefix: str = ""
    # True when `forward` reads nothing of the step on the host (no `*_host` mirror of the
    # context, no device-to-host copy): only then can a decode step be captured in a CUDA graph
    graph_safe: bool = False

    def params(self) -> list[Param]:
        return []

    def children(self) -> list["Part"]:
        return []

    def cache_spec(self) -> KVCacheSpec | StateSpec | None:
        return None

    def finalize(self, device: torch.device, dtype: torch.dtype) -> None:
        """Called once after the weights are bound (build device tables here)."""

    def walk(self):
        yield self
        for c in self.children():
            yield from c.walk()


# ------------------------------------------------------------------ registry of part kinds

_KINDS: dict[tuple[str, str], Any] = {}
ROLES = ("mixer", "ffn", "norm", "position", "block")


def register_part(role: str, name: str, factory) -> None:
    """Make `factory(**kwargs) -> Part` available under (role, name)."""
    if role not in ROLES:
        raise ValueError(f"unknown part role {role!r}; roles: {ROLES}")
    _KINDS[(role, name)] = factory


def make_part(role: str, name: str, **kwargs) -> Part:
    try:
        factory = _KINDS[(role, name)]
    except KeyError:
        known = sorted(n for r, n in _KINDS if r == role)
        raise KeyError(f"no {role} part named {name!r}; registered: {known}") from None
    return factory(**kwargs)


def registered_parts(role: str) -> list[str]:
    return sorted(n for r, n in _KINDS if r == role)


@dataclass
class LayerCache:
    """What a mixer gets for its cache layer in one step.

    KV layers: `k`, `v` [pages, kv_heads, page_size, head_dim]; `slots` [T] (page*page_size +
    offset of each new token, -1 where the layer must not write); `block_table`
    [sequences, pages] (-1 where a page was given back). State layers: `state[name]`
    [slots, *shape]; the request's slot is `ctx.state_slots[seq]`."""
    spec: KVCacheSpec | StateSpec
    page_size: int = 0
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    slots: torch.Tensor | None = None
    block_table: torch.Tensor | None = None
    writes: bool = True
    state: dict[str, torch.Tensor] = field(default_factory=dict)
