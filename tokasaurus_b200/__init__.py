"""tokasaurus_b200: a one-GPU inference engine for the dense Llama decoder on NVIDIA B200."""

from tokasaurus_b200.config import EngineConfig, LlamaConfig, register_architecture  # noqa: F401
from tokasaurus_b200.sampling.params import Request, RequestOutput, SamplingParams  # noqa: F401


def __getattr__(name):
    if name == "Engine":
        from tokasaurus_b200.engine.engine import Engine

        return Engine
    raise AttributeError(name)
