"""mstar_b200: a single-GPU inference engine for dense Llama decoders on NVIDIA B200.

    from mstar_b200 import LLM, SamplingParams
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    if name == "GenerationResult":
        from .engine.llm import GenerationResult
        return GenerationResult
    raise AttributeError(f"module 'mstar_b200' has no attribute {name!r}")


__all__ = ["LLM", "SamplingParams", "GenerationResult", "__version__"]
