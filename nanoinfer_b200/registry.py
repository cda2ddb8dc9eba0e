"""The one registry from an architecture's name (config.json's ``architectures[0]``) to its
configuration class and its model builder.

The reference's registry maps names to forward *strategies* (``Stage::spec``,
crates/core/src/stages/mod.rs:157-268, unknown name -> ``Error::UnknownStage``,
crates/core/src/error.rs:17); it knows one architecture only.  Here the registry maps
architectures, so that another one is added by one ``register_architecture`` call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Type

from .config.base import ConfigError, ModelConfig, architecture_name, read_config_json
from .models.spec import ModelSpec


@dataclass
class Architecture:
    name: str
    config_cls: Type[ModelConfig]
    build_spec: Callable[[ModelConfig], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


class UnknownArchitecture(ConfigError):
    pass


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          build_spec: Callable[[ModelConfig], ModelSpec]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise UnknownArchitecture(f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name]


def architectures():
    return sorted(_ARCHITECTURES)


def load_config(model_dir: str) -> ModelConfig:
    """Read ``model_dir/config.json`` into the typed configuration of its architecture.  A configuration
    that leaves sizes to the checkpoint's tensor shapes (``sizes_from_tensors``) is shown the header of
    ``model_dir/model.safetensors`` where that file exists."""
    import os

    raw = read_config_json(model_dir)
    arch = get_architecture(architecture_name(raw))
    cfg = arch.config_cls.from_dict(raw)
    path = os.path.join(model_dir, "model.safetensors")
    if hasattr(cfg, "sizes_from_tensors") and os.path.isfile(path):
        from .weights.safetensors_io import SafetensorsFile

        st = SafetensorsFile(path)
        try:
            cfg.sizes_from_tensors({name: tuple(st.info(name).shape) for name in st.names()})
        finally:
            st.close()
    return cfg


def _register_builtin() -> None:
    from .config.gpt2 import GPT2Config
    from .models.gpt2 import build_gpt2_spec

    register_architecture("GPT2LMHeadModel", GPT2Config, build_gpt2_spec)

    from .config.vadonex import VadonexConfig
    from .models.vadonex import build_vadonex_spec

    register_architecture("Vadonex", VadonexConfig, build_vadonex_spec)

    from .config.mulavik import MulavikConfig
    from .models.mulavik import build_mulavik_spec

    register_architecture("Mulavik", MulavikConfig, build_mulavik_spec)

    from .config.kemuzen import KemuzenConfig
    from .models.kemuzen import build_kemuzen_spec

    register_architecture("Kemuzen", KemuzenConfig, build_kemuzen_spec)

    from .config.nagilix import NagilixConfig
    from .models.nagilix import build_nagilix_spec

    register_architecture("Nagilix", NagilixConfig, build_nagilix_spec)


_register_builtin()
