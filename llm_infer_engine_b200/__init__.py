"""A small generation library for one GPU (NVIDIA B200, sm_100a) and one architecture family.

    from llm_infer_engine_b200 import Engine, SamplingParams, generate, write_random_model
    engine = Engine("path/to/model_dir", dtype="bfloat16")
    new_tokens = generate(engine, [[1, 5, 9], [1, 7]], max_new_tokens=32)

Layout: `config/` typed configuration and the architecture registry; `weights/` safetensors
reading, the loader and the random-weights mode; `parts/` mixers, feed-forwards, norms,
position encodings and block arrangements with their registries; `models/` the generic decoder
and the architectures expressed as specs; `cache/` slots, pages and per-sequence state;
`engine/` the step function, captured decode steps and the generation loop; `sampling/`;
`kernels/` the build and the Python faces of the CUDA code in `csrc/`; `cli/` the command line.
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, known_architectures, load_config, register_architecture
from .engine.engine import Engine, EngineError
from .engine.generate import GenerationStats, generate
from .sampling import SamplingParams, uniform_for
from .weights import WeightsError, write_random_model

__all__ = ["ConfigError", "known_architectures", "load_config", "register_architecture", "Engine", "EngineError",
           "GenerationStats", "generate", "SamplingParams", "uniform_for", "WeightsError", "write_random_model"]
