"""velomind_b200: a small generation library for one GPU (NVIDIA B200, sm_100a), built from parts.

The library is C++ and CUDA (`include/velomind_b200/velomind.h`); this package is its thin Python binding.

    import velomind_b200 as vm
    engine = vm.load("path/to/model_folder", dtype="bfloat16")
    results = engine.generate([[1, 2, 3], [4, 5]], temperature=0.0, max_tokens=16)
"""
from .binding import (CacheError, ConfigError, Engine, EngineConfig, Entry, GenerationLoop, KernelError, KernelLibraryError, Model, OpTimes,
                      Request, Result, SamplingParams, TextEngine, Timing, Tokenizer, WeightError, check_model_folder, check_safetensors_header, describe_config, load,
                      load_model, pretokenize, registered_architectures, safetensors_info, smollm2_135m_config, weight_table, write_random_model)

__all__ = ["CacheError", "ConfigError", "Engine", "EngineConfig", "Entry", "GenerationLoop", "KernelError", "KernelLibraryError", "Model",
           "OpTimes", "Request", "Result", "SamplingParams", "TextEngine", "Timing", "Tokenizer", "WeightError", "check_model_folder", "check_safetensors_header", "safetensors_info",
           "describe_config", "load", "load_model", "pretokenize", "registered_architectures", "smollm2_135m_config", "weight_table",
           "write_random_model", "SMOLLM2_135M"]


def __getattr__(name):
    if name == "SMOLLM2_135M":          # examples/smollm2/model.h:11-22: the sizes the reference's `--synthetic` switch uses
        return smollm2_135m_config()
    raise AttributeError(name)
