"""hfee_b200: a single-GPU inference engine for the dense Llama decoder on NVIDIA
B200 (sm_100a), assembled from parts so that other architectures can be added.

    from hfee_b200 import Engine, SamplingOptions
    engine = Engine("path/to/model_dir", dtype="bfloat16")
    results = engine.generate([[1, 2, 3]], SamplingOptions.greedy(num_predict=16))
"""
from .config import (ConfigError, EngineConfig, LayerSpec, LlamaConfig, ModelSpec, PartSpec, RunSpec,
                     register_architecture)
from .cache import CacheManager, FixedState, OutOfPages, PagedKV
from .engine import Engine, GenerationResult, ModelRunner, Request, Scheduler, StepEntry
from .parts import Block, Mixer, Part, Runtime, register_part
from .sampling import SamplingOptions
from .weights import TensorNeed, WeightError, write_random_model

__version__ = "0.1.0"

__all__ = ["ConfigError", "EngineConfig", "LayerSpec", "LlamaConfig", "ModelSpec", "PartSpec", "RunSpec",
           "register_architecture", "CacheManager", "FixedState", "OutOfPages", "PagedKV", "Engine",
           "GenerationResult", "ModelRunner", "Request", "Scheduler", "StepEntry", "Block", "Mixer", "Part", "Runtime",
           "register_part", "SamplingOptions", "TensorNeed", "WeightError", "write_random_model", "__version__"]
