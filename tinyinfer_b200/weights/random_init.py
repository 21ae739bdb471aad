"""Random-weights mode: a model folder (config.json + model.safetensors) from a configuration and
a seed, and a direct on-device fill for models too large to be worth writing to disk.

The reference has nothing like it (its parameters start as torch.empty,
tinyinfer/layers/linear.py:13). Matrices are N(0, std), norm weights 1 + N(0, 0.1), drawn by a
seeded CPU generator in the fixed order of ``expected_tensors()``; a bfloat16 folder holds the
rounded float32 draw, so both dtypes of one seed describe the same model.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict

import torch
from safetensors.torch import save_file

from ..config.registry import lookup_architecture
from .loader import apply_role


def _draw(ts, generator, std: float, device="cpu") -> torch.Tensor:
    if ts.role == "int":
        return torch.zeros(ts.shape, dtype=torch.int32, device=device)
    t = torch.randn(ts.shape, generator=generator, dtype=torch.float32, device=device)
    if ts.init == "ones_noise":
        return 1.0 + 0.1 * t
    return t * std


def random_tensors(config, seed: int, std: float = 0.02, device="cpu", store=torch.float32) -> Dict[str, torch.Tensor]:
    """name -> CPU tensor (``store`` type for floating point) for every tensor the architecture of
    ``config`` expects, drawn in float32 on ``device`` (the values depend on the device's generator)."""
    arch = lookup_architecture(config.architectures[0])
    shapes = arch.model_factory(config, torch.float32, "cpu").expected_tensors()
    gen = torch.Generator(device=device).manual_seed(int(seed))
    out = {}
    for name, ts in shapes.items():
        t = _draw(ts, gen, std, device=device)
        out[name] = (t.to(store) if t.is_floating_point() else t).contiguous().cpu()
    return out


def write_random_model(folder, config, seed: int, dtype: str = "float32", std: float = 0.02,
                       device="cpu") -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``. ``dtype`` is the storage
    type of the matrices ('float32' or 'bfloat16'); norm weights follow it too. ``device``: where the
    numbers are drawn; a CUDA device makes a folder of many gigabytes in seconds, with other values
    than the CPU's generator gives for the same seed."""
    if dtype not in ("float32", "bfloat16"):
        raise ValueError("dtype must be 'float32' or 'bfloat16'")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(config, seed, std, device=device, store=store)
    cfg = config.to_dict()
    cfg["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def fill_random_on_device(model, seed: int, std: float = 0.02) -> None:
    """Fills ``model`` with random weights drawn on its own device (benchmarks at sizes where a
    16 GB file would only cost time). The values differ from ``write_random_model``'s. Each tensor is
    drawn when the model asks for it and let go of once packed, so a model of 65 GB needs little more
    than its own size while it is filled."""
    expected = model.expected_tensors()
    order = {name: i for i, name in enumerate(expected)}

    class Drawn:
        def __getitem__(self, name):
            # a generator of its own per tensor: the values do not depend on the order of the asking
            gen = torch.Generator(device=model.device).manual_seed(int(seed) * 1000003 + order[name])
            ts = expected[name]
            return apply_role(_draw(ts, gen, std, device=model.device), ts.role, model.dtype)

    model.load_tensors(Drawn())
