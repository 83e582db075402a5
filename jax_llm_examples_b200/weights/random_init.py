"""Random-weights mode: tensors, or a whole model folder, from a configuration and a seed.

The reference initialises one tensor per leaf from a split key (llama4/llama4_jax/model.py:
274-307: he_normal matrices, norm weights 1).  Here every tensor is drawn from its own
generator, seeded by (seed, tensor name), so that a tensor's values do not depend on which
other tensors exist or in which order they are made, and so that a large model can be made
tensor by tensor on the GPU without a host copy.  Matrices are N(0, std); norm weights are
1 + N(0, norm_noise).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Mapping

import torch

from .loader import TensorSpec


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device: str | torch.device,
                  std: float, norm_noise: float) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    n = 1
    for s in spec.shape:
        n *= s
    if n <= (1 << 28):
        t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device)
        if spec.init == "norm":
            return (1.0 + norm_noise * t).to(dtype)
        return (std * t).to(dtype)
    # large tensors: draw in the target precision, slab by slab, to bound the temporary
    out = torch.empty(spec.shape, dtype=dtype, device=device)
    flat = out.view(-1)
    step = 1 << 28
    for lo in range(0, n, step):
        hi = min(n, lo + step)
        t = torch.randn(hi - lo, generator=g, dtype=torch.float32, device=device)
        flat[lo:hi] = ((1.0 + norm_noise * t) if spec.init == "norm" else (std * t)).to(dtype)
    return out


def random_tensors(specs: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str | torch.device = "cpu", std: float = 0.02, norm_noise: float = 0.0) -> dict[str, torch.Tensor]:
    return {n: random_tensor(s, seed, dtype, device, std, norm_noise) for n, s in specs.items() if not s.optional}


def write_random_model(model_dir: str | Path, config_json: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, std: float = 0.02, norm_noise: float = 0.0) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` for the architecture that config_json names.  The
    tensors are drawn by the CPU's generator: ``random_model`` gives the same ones only with ``draw_on="cpu"``."""
    from safetensors.torch import save_file

    from ..config.registry import resolve

    arch = resolve(config_json)
    cfg = arch.parse_config(config_json)
    tensors = random_tensors(arch.tensor_specs(cfg), seed, dtype, "cpu", std, norm_noise)
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    (model_dir / "config.json").write_text(json.dumps(dict(config_json), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(model_dir / "model.safetensors"))
    return model_dir
