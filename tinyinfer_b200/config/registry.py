"""The one registry from an architecture's name (``config.json['architectures'][0]``) to its
typed configuration class and its model class.

The reference hard-codes its only model class (tinyinfer/engine/model_runner.py:218); here a new
architecture is one ``register_architecture`` call and no edit elsewhere.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Mapping, Optional


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type            # has from_dict(dict) -> config, to_dict(), model_spec()
    model_factory: Callable       # (config, dtype, device) -> model
    presets: Mapping[str, dict] = None   # name -> config.json keys of a size worth running with random weights


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, model_factory: Callable,
                          presets: Optional[Mapping[str, dict]] = None) -> None:
    """``presets``: named sizes of this architecture (config.json keys without 'architectures') that the
    command line and the benchmarks offer as ``--random-config NAME``."""
    for attr in ("from_dict", "to_dict", "model_spec"):
        if not hasattr(config_class, attr):
            raise TypeError(f"config class of {name!r} lacks {attr}()")
    _ARCHITECTURES[name] = Architecture(name, config_class, model_factory, dict(presets or {}))


def known_architectures():
    return sorted(_ARCHITECTURES)


def known_presets() -> Dict[str, str]:
    """preset name -> the architecture that offers it (the one registered last wins a shared name)."""
    from .. import models  # noqa: F401  (the built-in architecture registers itself on import)
    return {preset: arch.name for arch in _ARCHITECTURES.values() for preset in arch.presets}


def preset_config(preset: str, **overrides):
    """The typed configuration of a named size, whichever architecture registered it; ``overrides``
    replace config.json keys (num_hidden_layers=2 for a cut-down benchmark, say)."""
    owner = known_presets().get(preset)
    if owner is None:
        raise KeyError(f"unknown preset {preset!r}; known: {sorted(known_presets())}")
    arch = _ARCHITECTURES[owner]
    return arch.config_class.from_dict(dict(arch.presets[preset], architectures=[arch.name], **overrides))


def lookup_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise KeyError(f"unknown architecture {name!r}; known: {known_architectures()}") from None


def architecture_of(config_dict: dict) -> Architecture:
    names = config_dict.get("architectures")
    if not isinstance(names, (list, tuple)) or not names:
        raise ValueError("config.json has no 'architectures' list; known: "
                         f"{known_architectures()}")
    return lookup_architecture(names[0])


def load_config(folder):
    """(Architecture, typed configuration) of a model folder."""
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json under {folder}")
    data = json.loads(path.read_text())
    arch = architecture_of(data)
    return arch, arch.config_class.from_dict(data)
