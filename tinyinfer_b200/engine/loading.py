"""From a model folder to a loaded model: config.json picks the architecture, the registry gives
its classes, the loader fills the tensors."""
from __future__ import annotations

import torch

from .. import models  # noqa: F401  (registers the built-in architecture)
from ..config import load_config, parse_dtype
from ..weights import load_weights

TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("tinyinfer_b200 runs on a CUDA device only (sm_100a); there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is visible: tinyinfer_b200 needs a B200 (sm_100a)")
    return device


def load_model(folder, dtype="bfloat16", device="cuda:0"):
    """(model, typed configuration) of ``folder`` with weights on ``device``."""
    arch, config = load_config(folder)
    model = arch.model_factory(config, TORCH_DTYPES[parse_dtype(dtype)], torch.device(device))
    load_weights(model, folder)
    return model, config


def build_random_model(config, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02):
    """A model of ``config`` with random weights drawn on the device (no folder involved)."""
    from ..config import lookup_architecture
    from ..weights import fill_random_on_device
    arch = lookup_architecture(config.architectures[0])
    model = arch.model_factory(config, TORCH_DTYPES[parse_dtype(dtype)], torch.device(device))
    fill_random_on_device(model, seed, std)
    return model
