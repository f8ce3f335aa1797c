from .model_config import ConfigError, ModelConfig, Qwen3Config, read_config_json  # noqa: F401
