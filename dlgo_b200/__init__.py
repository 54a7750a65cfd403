"""dlgo_b200: a small generation library for one GPU (NVIDIA B200, sm_100a).

From a model folder (config.json + model.safetensors) to generated tokens: a
typed configuration and an architecture registry, weights by tensor name, layers
put together from parts, a paged cache with a slot per sequence, one step
function for batches of unequal lengths, a generation loop with greedy and
temperature sampling, and hand-written CUDA kernels underneath.  The public
entry point mirrors computerex/dlgo's ``LoadLLM`` / ``Generate`` (dlgo.go:37-115).
"""
from .config import (ConfigError, LlamaConfig, load_config, register_architecture, registered_architectures)

__version__ = "0.1.0"
__all__ = ["ConfigError", "LLM", "LlamaConfig", "load_config", "load_llm", "register_architecture",
           "registered_architectures", "write_random_model"]


def __getattr__(name):
    if name in ("load_llm", "LLM", "ModelInfo", "BenchmarkResult"):
        from . import api
        return getattr(api, name)
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)
