from .model_config import ConfigError, KesozenConfig, Qwen3Config, TofilornConfig, read_config_json, write_config_json
from .engine_options import EngineOptions

__all__ = ["ConfigError", "KesozenConfig", "Qwen3Config", "TofilornConfig", "EngineOptions", "read_config_json", "write_config_json"]
