"""A small, whole model library for one GPU (NVIDIA B200, sm_100a): from a request's tokens
to its next token for the Mistral / Llama-style dense decoder.

    from inference_engine_rust_b200 import LoadedModel
    model = LoadedModel.load("path/to/folder", dtype="bfloat16")
    session = model.session(max_tokens=8192)
    ids = session.generate([[1, 5, 9], [1, 7]], max_new_tokens=16)
"""
from .api import InferenceSession, LoadedModel, parse_dtype, write_random_model
from .config import (ConfigError, MistralConfig, ModelSpec, config_from_dict, known_architectures,
                     load_config, register_architecture, spec_of)
from .engine import Engine, GenerationResult, Model, StepError
from .sampling import Sampler, SamplingError, SamplingParams
from .weights import WeightError

__all__ = ["InferenceSession", "LoadedModel", "parse_dtype", "write_random_model", "ConfigError",
           "MistralConfig", "ModelSpec", "config_from_dict", "known_architectures", "load_config",
           "register_architecture", "spec_of", "Engine", "GenerationResult", "Model", "StepError",
           "Sampler", "SamplingError", "SamplingParams", "WeightError"]
