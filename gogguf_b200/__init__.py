"""gogguf_b200: a small, whole Qwen3 inference library for NVIDIA B200 (sm_100a).

    import gogguf_b200 as gg
    engine = gg.load("model_dir")                      # config.json + model.safetensors
    out = engine.new_context().generate([1, 2, 3], gg.GenerateParams(max_tokens=8))
"""
from . import config  # noqa: F401  (registers architectures)
from . import parts   # noqa: F401  (registers part kinds)
from .api import Context, Conversation, Engine, Greedy, LoadOptions, load, load_random, new_sampler
from .engine.generate import GenerateParams, GenerationResult, GenerationSession
from .engine.step import LayerTaps, StepEntry, StepError, StepOutcome
from .sampling.sampler import Sampler, SamplerConfig

__version__ = "0.1.0"
__all__ = ["Context", "Conversation", "Engine", "Greedy", "LoadOptions", "load", "load_random", "new_sampler", "GenerateParams",
           "GenerationResult", "GenerationSession", "Sampler", "SamplerConfig", "LayerTaps", "StepEntry", "StepError",
           "StepOutcome"]
