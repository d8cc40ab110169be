from .base import ConfigError, KeyReader, load_config_json
from .falcon_h1 import AttentionConfig, FalconH1Config, Mamba2Config, Multipliers
from .registry import (Architecture, open_model_dir, register_architecture, registered_architectures,
                       resolve_architecture)
