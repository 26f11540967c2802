from .arena import ArenaPlan, Workspace, plan_arena
from .generate import GenerationLoop, Request, Result, Timing, plan_batches
from .model import DecoderModel, load_model, weight_table
from .step import Engine, Entry, StepContext

__all__ = ["ArenaPlan", "Workspace", "plan_arena", "GenerationLoop", "Request", "Result", "Timing", "plan_batches",
           "DecoderModel", "load_model", "weight_table", "Engine", "Entry", "StepContext"]
