"""velomind_b200: a small generation library for one GPU (NVIDIA B200, sm_100a), built from parts.

    import velomind_b200 as vm
    engine = vm.load("path/to/model_folder", dtype="bfloat16")
    results = engine.generate([[1, 2, 3], [4, 5]], temperature=0.0, max_tokens=16)
"""
from . import models  # noqa: F401
from .api import SMOLLM2_135M, EngineConfig, TextEngine, TextStreamer, load
from .engine.generate import GenerationLoop, Request, Result
from .engine.model import DecoderModel, load_model
from .engine.step import Engine, Entry
from .sampling.sampler import DeviceSampler, SamplingParams
from .weights.synthetic import write_random_model

__all__ = ["SMOLLM2_135M", "EngineConfig", "TextEngine", "TextStreamer", "load", "GenerationLoop", "Request", "Result",
           "DecoderModel", "load_model", "Engine", "Entry", "DeviceSampler", "SamplingParams", "write_random_model"]
