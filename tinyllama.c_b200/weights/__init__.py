from .loader import (WeightError, build_model, check_tensors, load_model, random_tensors,  # noqa: F401
                     write_random_model)
from .safetensors_io import SafetensorsError, load_file, load_model_dir, save_file  # noqa: F401
