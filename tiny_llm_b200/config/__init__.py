from .errors import ConfigError
from .registry import (config_class_for, config_from_dict, load_config, register_architecture,
                       registered_architectures)
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .llama import LlamaConfig
from .dunelix import DunelixConfig
from .zozenex import ZozenexConfig
from .fiponex import FiponexConfig
from .gevovik import GevovikConfig

__all__ = ["ConfigError", "LlamaConfig", "DunelixConfig", "ZozenexConfig", "FiponexConfig", "GevovikConfig", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec",
           "config_class_for", "config_from_dict", "load_config", "register_architecture",
           "registered_architectures"]
