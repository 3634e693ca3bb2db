from .base import (ConfigError, ModelConfig, config_from_dict, load_config, lookup_architecture,  # noqa: F401
                   register_architecture, registered_architectures)
from .falcon_h1 import FalconH1Config  # noqa: F401
