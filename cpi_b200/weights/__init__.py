from .safetensors_io import SafetensorsDir, SafetensorsError, write_safetensors
from .store import (WeightsError, TensorReq, WeightSource, SafetensorsSource, DictSource,
                    check_source, kept_dtype)
from .random_init import RandomSource, write_random_model
