from .model_config import (ConfigError, LlamaConfig, RopeScaling, config_from_json_dict, known_architectures,
                           load_config, register_config_class, save_config)
from .vabanex_config import VabanexConfig
from .lupusun_config import LupusunConfig
from .tokolorn_config import TokolornConfig
from .finolix_config import FinolixConfig
from .registry import MODEL_CONFIGS, get_config, register_config

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "VabanexConfig", "LupusunConfig", "TokolornConfig", "FinolixConfig", "config_from_json_dict", "known_architectures",
           "load_config", "register_config_class", "save_config", "MODEL_CONFIGS", "get_config", "register_config"]
