from .binder import (WeightsError, check_weights, expected_tensors, load_weights, random_weights,  # noqa: F401
                     write_random_model)
from .safetensors_io import SafetensorsError, SafetensorsFile, open_checkpoint, write_safetensors  # noqa: F401
