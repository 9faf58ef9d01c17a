from .base import (ConfigError, ModelConfig, architecture_of, config_from_dict, describe_model,
                   known_architectures, load_config, register_architecture)
from .kaketar import KaketarConfig
from .panolorn import PanolornConfig
from .pevolorn import PevolornConfig
from .qwen3 import Qwen3Config
from .tetodra import TetodraConfig
