"""airun_b200: a small, whole inference engine for one NVIDIA B200 (sm_100a).

Python entry point::

    import airun_b200
    eng = airun_b200.Engine.from_folder("model_dir", dtype="bfloat16")
    out = eng.generate([1, 2, 3], airun_b200.SamplingParams.greedy(), max_new_tokens=16)
    print(out.token_ids)

The model class is chosen by ``architectures[0]`` of config.json through the
registry in :mod:`airun_b200.config`.
"""
from .config import (ConfigError, ModelConfig, Qwen3Config, load_config, register_architecture,
                     registered_architectures)
from .engine.engine import Engine, EngineOptions, GenerationResult, GenerationStats
from .engine.step import StepEntry, StepRunner
from .parts import register_part
from .sampling.sampler import SamplingParams
from .weights import WeightError, write_model_folder

__all__ = ["Engine", "EngineOptions", "GenerationResult", "GenerationStats", "SamplingParams", "StepEntry",
           "StepRunner", "ConfigError", "WeightError", "ModelConfig", "Qwen3Config", "load_config",
           "register_architecture", "registered_architectures", "register_part", "write_model_folder"]
