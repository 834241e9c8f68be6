from .model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json
from .engine_config import EngineConfig
from .viresun_config import ViresunConfig
from .bivatar_config import BivatarConfig
from .lazolix_config import LazolixConfig
from .gezozen_config import GezozenConfig

__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "read_config_json", "EngineConfig", "ViresunConfig",
           "BivatarConfig", "LazolixConfig", "GezozenConfig"]
