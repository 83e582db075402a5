"""From a model folder (or a configuration and a seed) to a model on the GPU.

The reference loads a converted orbax tree (llama4/main.py:54-56); here config.json names the
architecture, the registry gives its tensor list and builder, and tensors are read from
safetensors by name straight to the device.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from .config.base import load_config_json
from .config.registry import resolve
from .parts.base import Runtime
from .parts.decoder import DecoderModel
from .weights.loader import check_tensors, load_tensors
from .weights.random_init import random_tensor

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _built(model: DecoderModel) -> DecoderModel:
    """Building re-lays weights through temporaries as large as the largest tensor; they go back to the
    driver here, so that the cache pool and the steps' buffers do not compete with a full allocator cache."""
    if model.runtime.device.type == "cuda":
        torch.cuda.empty_cache()
    return model


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}") from None


def load_config(config_path: str | Path):
    """config.json (the file, or the folder that holds it) -> the typed configuration of its architecture
    (the reference's ``load_config``, llama4/llama4_jax/model.py:229-231)."""
    path = Path(config_path)
    cfg_json = load_config_json(path.parent if path.is_file() else path)
    return resolve(cfg_json).parse_config(cfg_json)


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16", device: str | torch.device = "cuda") -> DecoderModel:
    """config.json + model.safetensors -> model.  ``dtype``: bfloat16 (serving precision; stored
    32-bit tensors stay 32-bit) or float32 (everything in true 32-bit)."""
    dt = parse_dtype(dtype)
    cfg_json = load_config_json(model_dir)
    arch = resolve(cfg_json)
    cfg = arch.parse_config(cfg_json)
    tensors = load_tensors(model_dir, arch.tensor_specs(cfg), arch.canonical_name, dt, device)
    return _built(arch.build(cfg, tensors, Runtime(dt, torch.device(device))))


def random_model(config_json: Mapping[str, Any], seed: int, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda", std: float = 0.02, norm_noise: float = 0.0,
                 weight_dtype: torch.dtype = torch.bfloat16, draw_on: str = "device") -> DecoderModel:
    """A model with seeded random weights made directly on the device (no folder is written).

    NOT the tensors of ``write_random_model`` for the same seed, unless ``draw_on="cpu"``: a tensor's values
    depend on (seed, tensor name) AND on the generator that draws them, and by default each tensor is drawn by
    the device's generator (a large model is made without a host copy), while a folder is written from the
    CPU's.  With ``draw_on="cpu"`` every tensor is drawn on the CPU and copied over: the model that
    ``load_model`` gives for a folder written with the same configuration, seed, std and norm_noise."""
    if draw_on not in ("device", "cpu"):
        raise ValueError(f"draw_on must be 'device' or 'cpu', not {draw_on!r}")
    dt = parse_dtype(dtype)
    arch = resolve(config_json)
    cfg = arch.parse_config(config_json)
    specs = arch.tensor_specs(cfg)
    store = torch.float32 if dt == torch.float32 else weight_dtype

    class _Lazy(dict):
        """Makes each tensor when the builder takes it, so that only one is unfused at a time."""

        def pop(self, name, *a):
            return random_tensor(specs[name], seed, store, "cpu" if draw_on == "cpu" else device, std, norm_noise).to(device)

        def __contains__(self, name):
            return name in specs and not specs[name].optional

    return _built(arch.build(cfg, _Lazy(), Runtime(dt, torch.device(device))))


def model_from_tensors(config_json: Mapping[str, Any], tensors: Mapping[str, torch.Tensor],
                       dtype: str | torch.dtype = "bfloat16", device: str | torch.device = "cuda") -> DecoderModel:
    dt = parse_dtype(dtype)
    arch = resolve(config_json)
    cfg = arch.parse_config(config_json)
    check_tensors(tensors, arch.tensor_specs(cfg))
    conv = {n: (t.to(torch.float32) if dt == torch.float32 or t.dtype == torch.float32 else t.to(torch.bfloat16)).to(device)
            for n, t in tensors.items()}
    return _built(arch.build(cfg, conv, Runtime(dt, torch.device(device))))
