"""Safetensors loading by tensor name.

What the reference's loader does (tinyinfer/utils/loader.py:20-30 file discovery, :34-40 shape
check, :103-105 a tied model ignores a stored lm_head, :139-151 strict errors on missing and
unexpected names) is kept; what differs: every fault of a checkpoint (missing names, unexpected
names, wrong shapes) is gathered into ONE error, and the packing of q/k/v and gate/up is left to
the parts that own those tensors.

Dtypes: 'matrix' tensors are kept in the compute dtype (bfloat16 or float32); 'vector32'
tensors (norm weights, biases) are kept in float32 whatever the file or the compute dtype says,
so a tensor stored in 32 bits stays so; 'int' tensors become int32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Tuple

import torch
from safetensors import safe_open


class WeightError(RuntimeError):
    """A checkpoint does not fit the model. Carries the three lists the message shows."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"checkpoint {where} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): {self.missing}")
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): {self.unexpected}")
        if self.wrong_shape:
            lines.append("  wrong shapes ({}): {}".format(
                len(self.wrong_shape),
                [f"{n}: checkpoint {tuple(got)} vs model {tuple(want)}" for n, got, want in self.wrong_shape]))
        super().__init__("\n".join(lines))


@dataclass
class LoadReport:
    loaded: List[str] = field(default_factory=list)
    skipped_tied: List[str] = field(default_factory=list)
    bytes_on_device: int = 0


def checkpoint_files(folder) -> List[Path]:
    folder = Path(folder).expanduser()
    files = sorted(folder.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files found under {folder}")
    return files


def checkpoint_index(folder) -> Dict[str, Tuple[Path, Tuple[int, ...]]]:
    """name -> (file, shape) of every tensor of the folder, without reading the data."""
    index: Dict[str, Tuple[Path, Tuple[int, ...]]] = {}
    for file in checkpoint_files(folder):
        with safe_open(str(file), framework="pt", device="cpu") as f:
            for name in f.keys():
                index[name] = (file, tuple(f.get_slice(name).get_shape()))
    return index


def apply_role(t: torch.Tensor, role: str, dtype: torch.dtype) -> torch.Tensor:
    if role == "matrix":
        return t.to(dtype)
    if role == "vector32":
        return t.to(torch.float32)
    if role == "int":
        return t.to(torch.int32)
    raise ValueError(f"unknown tensor role {role!r}")


def load_weights(model, folder) -> LoadReport:
    """Fills ``model`` (a DecoderModel) from the safetensors files of ``folder``."""
    expected = model.expected_tensors()
    ignored = set(model.ignored_tensors())
    index = checkpoint_index(folder)
    missing = [n for n in expected if n not in index]
    unexpected = sorted(n for n in index if n not in expected and n not in ignored)
    wrong = [(n, index[n][1], expected[n].shape) for n in expected
             if n in index and tuple(index[n][1]) != tuple(expected[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where=str(folder))

    report = LoadReport(skipped_tied=sorted(n for n in index if n in ignored))
    reader = _TensorReader(index, expected, model.dtype, model.device, report)
    try:
        model.load_tensors(reader)
    finally:
        reader.close()
    return report


class _TensorReader:
    """``reader[name]``: the checkpoint's tensor of that name, role applied, on the device. Read when
    asked for and not kept, so that a model that packs tensors as it loads them never has the packed
    and the unpacked copy of more than one part on the device."""

    def __init__(self, index, expected, dtype, device, report: LoadReport):
        self.index, self.expected, self.dtype, self.device, self.report = index, expected, dtype, device, report
        self._open = {}

    def __getitem__(self, name: str) -> torch.Tensor:
        file = self.index[name][0]
        handle = self._open.get(file)
        if handle is None:
            handle = self._open[file] = safe_open(str(file), framework="pt", device="cpu").__enter__()
        t = apply_role(handle.get_tensor(name), self.expected[name].role, self.dtype).to(self.device)
        self.report.loaded.append(name)
        self.report.bytes_on_device += t.numel() * t.element_size()
        return t

    def close(self) -> None:
        for handle in self._open.values():
            handle.__exit__(None, None, None)
        self._open.clear()
