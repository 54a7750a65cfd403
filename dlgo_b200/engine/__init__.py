"""Model assembly, the step function, CUDA graphs for decode, and the generation loop."""
from .generate import GenerateConfig, GenerateResult, GenerationError, GenerationLoop

__all__ = ["Engine", "StepError", "CausalLM", "GenerateConfig", "GenerateResult", "GenerationError",
           "GenerationLoop", "Runtime"]


def __getattr__(name):
    if name in ("Engine", "StepError"):
        from . import engine
        return getattr(engine, name)
    if name == "CausalLM":
        from .model import CausalLM
        return CausalLM
    if name == "Runtime":
        from .runtime import Runtime
        return Runtime
    raise AttributeError(name)
