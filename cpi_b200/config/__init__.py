from .common import ConfigError, read_config_json
from .spec import PartSpec, LayerSpec, RunEntry, ModelSpec
from .registry import (Architecture, register_architecture, registered_architectures,
                       get_architecture, architecture_of, spec_from_model_dir)
