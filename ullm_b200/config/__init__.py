from .borosun import BorosunConfig, BorosunConfigError, borosun_model_spec
from .engine_config import EngineConfig
from .finosun import FinosunConfig, FinosunConfigError, finosun_model_spec
from .pidenex import PidenexConfig, PidenexConfigError, pidenex_model_spec
from .ludalix import LudalixConfig, LudalixConfigError, ludalix_model_spec
from .qwen3 import ConfigError, Qwen3Config, qwen3_model_spec
from .registry import (
    ARCHITECTURES,
    Architecture,
    load_model_spec,
    read_config_json,
    register_architecture,
    resolve_architecture,
)
from .specs import (
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
    TokenSideSpec,
)

register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_model_spec)
register_architecture("Ludalix", LudalixConfig.from_dict, ludalix_model_spec)
register_architecture("Borosun", BorosunConfig.from_dict, borosun_model_spec, reads_shapes=True)
register_architecture("Pidenex", PidenexConfig.from_dict, pidenex_model_spec)
register_architecture("Finosun", FinosunConfig.from_dict, finosun_model_spec)

__all__ = [
    "ARCHITECTURES", "Architecture", "BorosunConfig", "BorosunConfigError", "borosun_model_spec", "ConfigError", "EngineConfig", "FeedForwardSpec", "FinosunConfig", "FinosunConfigError", "finosun_model_spec", "LayerSpec",
    "LudalixConfig", "LudalixConfigError", "ludalix_model_spec", "PidenexConfig", "PidenexConfigError", "pidenex_model_spec", "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec", "Qwen3Config", "ScheduleEntry", "TokenSideSpec",
    "load_model_spec", "qwen3_model_spec", "read_config_json", "register_architecture",
    "resolve_architecture",
]
