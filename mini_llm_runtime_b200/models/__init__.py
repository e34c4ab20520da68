from .decoder import DecoderModel
from .factory import (build_model, load_model, parse_dtype, random_model, write_random_model_dir)

__all__ = ["DecoderModel", "build_model", "load_model", "parse_dtype", "random_model",
           "write_random_model_dir"]
