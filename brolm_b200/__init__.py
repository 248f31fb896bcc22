"""brolm_b200: a small, whole model library with generation for one B200.

Public face, in the manner of wlejon/brolm's C++ API
(include/brolm/gemma2.h:67-143, include/brolm/detail/generate.h:29-123):

    cfg    = brolm_b200.load_config(folder)            # Gemma2Config::from_safetensors_dir
    model  = brolm_b200.Model(cfg, dtype="bfloat16")   # Gemma2Model(cfg)
    model.load_weights(folder)                         # load_weights
    engine = brolm_b200.Engine(model, max_tokens=...)  # allocate_cache
    out    = brolm_b200.generate(engine, prompts, eos_id, GenerateOptions(...))
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, Gemma2Config, ModelConfig, load_config, register_architecture
from .engine import DecoderModel, Engine, StepError, generate, load_model, write_random_model
from .parts import register_part
from .sampling import GenerateOptions, SamplingParams, Sampler
from .tokenizer import GemmaTokenizer
from .weights import WeightsError

Model = DecoderModel

__all__ = ["ConfigError", "Gemma2Config", "ModelConfig", "load_config", "register_architecture", "DecoderModel",
           "Model", "Engine", "StepError", "load_model", "write_random_model", "register_part", "WeightsError", "generate", "GenerateOptions", "SamplingParams",
           "Sampler", "GemmaTokenizer"]
