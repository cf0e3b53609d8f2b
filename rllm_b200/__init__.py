"""rllm_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

From a model folder to generated tokens: typed configuration and registry, weights by
name, layers put together from parts, a paged cache manager, one step function for mixed
batches, a scheduler with sampling, and trace replay; hand-written CUDA kernels
underneath, with a true 32-bit path beside the bfloat16 one.
"""
from . import models as _models  # noqa: F401  (registers the architectures)
from .config import load_config, register_architecture, registered_architectures
from .parts import register_part

__version__ = "0.1.0"


def __getattr__(name):
    # heavier entry points are imported on first use
    if name in ("generate", "LLM", "SamplingParams"):
        from . import api
        return getattr(api, name)
    raise AttributeError(name)


__all__ = ["load_config", "register_architecture", "registered_architectures", "register_part",
           "generate", "LLM", "SamplingParams", "__version__"]
