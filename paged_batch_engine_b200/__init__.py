"""A small, whole paged-batch inference engine for one GPU (B200, sm_100a): a model folder
to generated tokens, for the Qwen2.5 dense decoder.

    from paged_batch_engine_b200 import Engine, SamplingParams
"""
from .config import Qwen2Config, load_config, register_architecture
from .sampling.params import SamplingParams

__all__ = ["Engine", "GenerationResult", "generate", "ModelRunner", "SamplingParams", "Qwen2Config",
           "load_config", "register_architecture"]
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "GenerationResult", "generate"):
        from .engine import engine
        return getattr(engine, name)
    if name == "ModelRunner":
        from .engine.runner import ModelRunner
        return ModelRunner
    raise AttributeError(name)
