from .context import StepContext
from .engine import DecodeGraph, Engine, EngineError, bucket_for, resolve_dtype

__all__ = ["StepContext", "DecodeGraph", "Engine", "EngineError", "bucket_for", "resolve_dtype"]
