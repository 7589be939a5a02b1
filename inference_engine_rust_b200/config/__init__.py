"""Typed configurations, the architecture registry and the architecture-neutral specs."""
from .registry import (ConfigError, architecture, architecture_name_of, config_from_dict,
                       known_architectures, load_config, read_config_json,
                       register_architecture, spec_of)
from .specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .mistral import MistralConfig  # registers "MistralForCausalLM"
from .vefulix import VefulixConfig  # registers "Vefulix"
from .sifasun import SifasunConfig  # registers "Sifasun"
from .kuvelix import KuvelixConfig  # registers "Kuvelix"
from .vufinex import VufinexConfig  # registers "Vufinex"
from .presets import PRESETS, preset

__all__ = [
    "ConfigError", "architecture", "architecture_name_of", "config_from_dict",
    "known_architectures", "load_config", "read_config_json", "register_architecture",
    "spec_of", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "MistralConfig", "VefulixConfig", "SifasunConfig", "KuvelixConfig", "VufinexConfig", "PRESETS", "preset",
]
