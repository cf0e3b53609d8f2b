"""From a model folder (or a configuration and a seed) to an `Engine`: configuration ->
registry -> parts -> weights -> cache pool -> step function. The counterpart of the
reference's `load_and_run_single_gpu` (src/engine/loader.rs:229-398)."""
from __future__ import annotations

import torch

from ..cache import CacheManager, pages_for
from ..config import config_from_dict, load_config
from ..kernels.backend import Backend
from ..weights import init_random_weights, load_weights
from .step import Engine

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {name!r}") from None


def default_num_pages(model, page_size: int, dtype: torch.dtype, device, weights_bytes: int = 0,
                      fraction: float = 0.75) -> int:
    """Pages that fit in `fraction` of the free device memory (the reference takes 75 % of
    what is left after the weights, src/model/config.rs:1195-1226, clamped there to
    [256, 8192] blocks; here only a floor is kept)."""
    free, _ = torch.cuda.mem_get_info(device)
    per_page = CacheManager.bytes_per_page(model.cache_specs(), page_size, dtype)
    if per_page == 0:
        return 0
    return max(16, int(free * fraction) // per_page)


def make_engine(model, dtype, device="cuda:0", page_size: int = 16, num_pages: int | None = None,
                max_tokens: int | None = None, max_requests: int = 256) -> Engine:
    """`model` must already hold its weights on `device`."""
    dtype = parse_dtype(dtype)
    backend = Backend(dtype, device)
    if num_pages is None:
        if max_tokens is not None:
            num_pages = pages_for(max_tokens, page_size)
        else:
            num_pages = default_num_pages(model, page_size, dtype, device)
    cache = CacheManager(model.cache_specs(), page_size, num_pages, max_requests, dtype, device)
    from ..kernels import profile
    if profile.enabled():
        # per-operation timing: every backend call bracketed by events, no graph replays
        return Engine(model, profile.OpProfile(backend), cache, use_graphs=False)
    return Engine(model, backend, cache)


def load_engine(model_dir: str, dtype="bfloat16", device="cuda:0", **kw) -> Engine:
    dtype = parse_dtype(dtype)
    arch, cfg = load_config(model_dir)
    model = arch.build(cfg)
    load_weights(model, model_dir, dtype, device)
    return make_engine(model, dtype, device, **kw)


def random_engine(config: dict, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02,
                  norm_std: float = 0.0, **kw) -> Engine:
    dtype = parse_dtype(dtype)
    arch, cfg = config_from_dict(config)
    model = arch.build(cfg)
    init_random_weights(model, seed, dtype, device, std, norm_std)
    return make_engine(model, dtype, device, **kw)
