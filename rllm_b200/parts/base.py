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
from typing import Any, Callable

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

    def cache_spec(self):
        """A spec of a registered cache kind (`KVCacheSpec`, `StateSpec`, or a class of one's own,
        see `register_cache_kind`), or None."""
        return None

    def finalize(self, device: torch.device, dtype: torch.dtype) -> None:
        """Called once after the weights are bound (build device tables here)."""

    def walk(self):
        yield self
        for c in self.children():
            yield from c.walk()


# ------------------------------------------------------------------ kinds of cache need

@dataclass(frozen=True)
class CacheKind:
    """How the cache manager serves one class of cache spec.

    `paged` kinds get pages: layers whose specs are equal form a group with a page pool and a block
    table of its own; `allocate(spec, num_pages, page_size, dtype, device)` returns one layer's
    tensors by name, each with the page as its first dimension. `window(spec)` is how many positions
    a query looks back (None: all; pages that lie wholly before it go back to the pool);
    `num_pages(spec, default)` the size of the group's pool; `page_bytes(spec, page_size, dtype)`
    what one page of one layer costs (for sizing the pool from free memory).
    Kinds that are not paged get a slot per live request:
    `allocate(spec, max_requests, None, dtype, device)` returns tensors with the slot first; a
    request's slot is zeroed when it opens."""
    paged: bool
    allocate: Callable[..., dict]
    window: Callable[[Any], int | None] = lambda spec: None
    num_pages: Callable[[Any, int], int] = lambda spec, default: default
    page_bytes: Callable[[Any, int, torch.dtype], int] = lambda spec, page_size, dtype: 0


_CACHE_KINDS: dict[type, CacheKind] = {}


def register_cache_kind(spec_cls: type, kind: CacheKind) -> None:
    """Tell the cache manager how to serve specs of class `spec_cls` (and its subclasses). A mixer
    with a cache need of a new shape (a compressed latent per token, one tensor per page, pools of
    another size) brings its spec class and this call; the manager itself stays as it is."""
    _CACHE_KINDS[spec_cls] = kind


def cache_kind_of(spec) -> CacheKind:
    for cls in type(spec).__mro__:
        if cls in _CACHE_KINDS:
            return _CACHE_KINDS[cls]
    raise TypeError(f"no cache kind is registered for {type(spec).__name__}; registered: "
                    f"{sorted(c.__name__ for c in _CACHE_KINDS)}")


def _kv_allocate(spec, num_pages, page_size, dtype, device):
    shape = (num_pages, spec.kv_heads, page_size, spec.head_dim)
    return {"k": torch.zeros(shape, dtype=dtype, device=device), "v": torch.zeros(shape, dtype=dtype, device=device)}


def _state_allocate(spec, max_requests, _page_size, _dtype, device):
    return {name: torch.zeros((max_requests,) + tuple(shape), dtype=dt, device=device)
            for name, shape, dt in spec.tensors}


register_cache_kind(KVCacheSpec, CacheKind(
    paged=True, allocate=_kv_allocate, window=lambda spec: spec.window,
    page_bytes=lambda spec, page_size, dtype: 2 * spec.kv_heads * spec.head_dim * page_size
    * torch.empty((), dtype=dtype).element_size()))
register_cache_kind(StateSpec, CacheKind(paged=False, allocate=_state_allocate))


# ------------------------------------------------------------------ registry of part kinds

_KINDS: dict[tuple[str, str], Any] = {}
ROLES = ("mixer", "ffn", "norm", "position", "block", "embedding", "head")


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

    Paged layers: `tensors[name]` with the page first (keys and values: `k`, `v`
    [pages, kv_heads, page_size, head_dim]); `slots` [T] (page*page_size + offset of each new
    token, -1 where the layer must not write); `block_table` [sequences, pages] (-1 where a page was
    given back). Slot layers: `state[name]` [slots, *shape]; the request's slot is
    `ctx.state_slots[seq]`."""
    spec: Any
    page_size: int = 0
    k: torch.Tensor | None = None
    v: torch.Tensor | None = None
    slots: torch.Tensor | None = None
    block_table: torch.Tensor | None = None
    writes: bool = True
    state: dict[str, torch.Tensor] = field(default_factory=dict)
    tensors: dict[str, torch.Tensor] = field(default_factory=dict)
