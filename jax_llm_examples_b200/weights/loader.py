"""Weights from safetensors, by tensor name.

The reference reads every tensor of the safetensors shards into a dictionary
(llama4/scripts/convert_weights.py:36-40), maps names with a regex table
(llama4/llama4_jax/chkpt_utils.py:161-196) and raises on an unknown, unexpected, duplicate or
missing tensor and on a wrong shape (chkpt_utils.py:85-159, 256-261, 274-275) one at a time.
Here the architecture declares the tensors it needs as :class:`TensorSpec` and all complaints
about a folder come in ONE :class:`WeightError` that lists missing tensors, unexpected
tensors and wrong shapes together.

Stored precision is kept: bfloat16 (and float16) tensors become bfloat16, tensors stored in
32-bit stay 32-bit, integer tables become int32.  ``dtype=torch.float32`` widens every
floating tensor to 32-bit (exactly) for the true 32-bit path.
"""

from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Callable, Mapping

import torch


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    init: str = "normal"  # "normal": N(0, std);  "norm": 1 + N(0, norm_noise)
    optional: bool = False


class WeightError(ValueError):
    """A model folder whose tensors do not fit the architecture; lists every problem."""

    def __init__(self, where: str, missing: list[str], unexpected: list[str], wrong: list[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"weights in {where} do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def _shard_files(model_dir: Path) -> list[Path]:
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        names = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        return [model_dir / n for n in names]
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [single]
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no model.safetensors in model folder {model_dir}")
    return files


def _keep_precision(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if t.dtype in (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8, torch.bool):
        return t.to(torch.int32)
    if dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    return t.to(torch.bfloat16)


def load_tensors(
    model_dir: str | Path,
    specs: Mapping[str, TensorSpec],
    canonical_name: Callable[[str], str | None] | None,
    dtype: torch.dtype,
    device: str | torch.device = "cpu",
) -> dict[str, torch.Tensor]:
    """Reads the folder's tensors into ``{spec name: tensor}`` on ``device``.

    ``canonical_name`` maps a name in the file to a spec name, or to None for tensors that
    belong to another part of the checkpoint (a vision tower) and are skipped.
    """
    from safetensors import safe_open

    model_dir = Path(model_dir)
    found: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong: list[str] = []
    for shard in _shard_files(model_dir):
        with safe_open(str(shard), framework="pt", device=str(device)) as f:
            for file_name in f.keys():
                name = canonical_name(file_name) if canonical_name else file_name
                if name is None:
                    continue
                if name not in specs:
                    unexpected.append(file_name)
                    continue
                if name in found:
                    unexpected.append(f"{file_name} (given twice)")
                    continue
                shape = tuple(f.get_slice(file_name).get_shape())
                if shape != tuple(specs[name].shape):
                    wrong.append(f"{file_name}: expected {list(specs[name].shape)}, found {list(shape)}")
                    found[name] = None  # type: ignore[assignment]
                    continue
                found[name] = _keep_precision(f.get_tensor(file_name), dtype)
    missing = [n for n, s in specs.items() if n not in found and not s.optional]
    if missing or unexpected or wrong:
        raise WeightError(str(model_dir), missing, sorted(unexpected), wrong)
    return found


def check_tensors(tensors: Mapping[str, torch.Tensor], specs: Mapping[str, TensorSpec], where: str = "memory") -> None:
    """The same three-way check for tensors that did not come from a file."""
    missing = [n for n, s in specs.items() if n not in tensors and not s.optional]
    unexpected = sorted(n for n in tensors if n not in specs)
    wrong = [
        f"{n}: expected {list(specs[n].shape)}, found {list(t.shape)}"
        for n, t in tensors.items()
        if n in specs and tuple(t.shape) != tuple(specs[n].shape)
    ]
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)
