"""Model, step function, generation loop and the Python entry point."""
from .batch import StepContext, build_context
from .engine import Engine, load_model, random_model
from .generate import BatchTracker, DecodeLoop, GpuBackend, plan_batches, run_batch
from .model import CausalLM
from .runner import Runner

__all__ = ["StepContext", "build_context", "Engine", "load_model", "random_model", "BatchTracker", "DecodeLoop", "GpuBackend",
           "plan_batches", "run_batch", "CausalLM", "Runner"]
