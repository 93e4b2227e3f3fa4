from oxr_inference_b200.config.model_config import ConfigError, Qwen3Config, load_model_config, read_config_json
from oxr_inference_b200.config.registry import ARCHITECTURES, Architecture, register_architecture, resolve_architecture
from oxr_inference_b200.config.settings import EngineSettings

__all__ = [
    "ARCHITECTURES", "Architecture", "ConfigError", "EngineSettings", "Qwen3Config", "load_model_config",
    "read_config_json", "register_architecture", "resolve_architecture",
]
