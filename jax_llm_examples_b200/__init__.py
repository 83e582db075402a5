"""A Llama 4 text inference engine for one B200: config.json + safetensors -> paged cache ->
one step function -> scheduler and sampling -> generated tokens.  CUDA kernels for sm_100a only."""

from .cache import CacheManager, OutOfPages, Retention
from .config import ConfigError, Llama4Config, known_architectures, preset, register_architecture, resolve
from .engine import Batch, Engine, EngineError, Generator, Request, Scheduler, StepEntry, decode_step, generate, prefill
from .loading import load_config, load_model, model_from_tensors, random_model
from .sampling import Sampler, SamplingParams
from .tokenizer import load_tokenizer
from .weights import WeightError, write_random_model

__all__ = [
    "Batch", "CacheManager", "ConfigError", "Engine", "EngineError", "Generator", "Llama4Config", "OutOfPages", "Request",
    "Retention", "Sampler", "SamplingParams", "Scheduler", "StepEntry", "WeightError", "decode_step", "generate",
    "known_architectures", "load_config", "load_model", "load_tokenizer", "model_from_tensors", "prefill", "preset", "random_model", "register_architecture",
    "resolve", "write_random_model",
]
