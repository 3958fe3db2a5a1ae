from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .qwen3 import ConfigError, Qwen3Config, qwen3_model_spec
from .luvavik import LuvavikConfig, luvavik_model_spec
from .rogosun import RogosunConfig, rogosun_model_spec
from .vumezen import VumezenConfig, vumezen_model_spec
from .sepitar import SepitarConfig, sepitar_model_spec
from .registry import (Family, UnknownArchitecture, family_for, load_config, register_family, registered,
                       unregister_family)

register_family(Family(name="Qwen3ForCausalLM", model_type="qwen3", config_class=Qwen3Config,
                       model_spec=qwen3_model_spec), replace=True)

register_family(Family(name="Luvavik", model_type="luvavik", config_class=LuvavikConfig,
                       model_spec=luvavik_model_spec), replace=True)

register_family(Family(name="Rogosun", model_type="rogosun", config_class=RogosunConfig,
                       model_spec=rogosun_model_spec), replace=True)

register_family(Family(name="Vumezen", model_type="vumezen", config_class=VumezenConfig,
                       model_spec=vumezen_model_spec), replace=True)

register_family(Family(name="Sepitar", model_type="sepitar", config_class=SepitarConfig,
                       model_spec=sepitar_model_spec), replace=True)

__all__ = [
    "SepitarConfig", "sepitar_model_spec",
    "VumezenConfig", "vumezen_model_spec",
    "ConfigError", "Family", "LayerSpec", "LuvavikConfig", "ModelSpec", "PartSpec", "Qwen3Config", "luvavik_model_spec", "ScheduleEntry",
    "UnknownArchitecture", "default_schedule", "family_for", "load_config", "qwen3_model_spec",
    "register_family", "registered", "RogosunConfig", "rogosun_model_spec", "unregister_family",
]
