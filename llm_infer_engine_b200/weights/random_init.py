"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed. The folder is then loaded like any checkpoint, so random models go
through the same loader, names and checks as real ones. (The reference's random mode builds
the torch module with default initialisers in memory, main.py:418-434.)

Matrices ~ N(0, std); norm weights are ones unless `norm_range=(lo, hi)` asks for U(lo, hi).
Each tensor has its own generator seeded from (seed, index in sorted-name order), so a tensor's
values do not depend on the others. Values are stored in bfloat16 unless `dtype` says float32.
"""
from __future__ import annotations

import json
import os
from typing import Optional, Tuple

import torch

from ..config.registry import load_config
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from .safetensors_io import save_file

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(config_json: dict, seed: int, std: float = 0.02,
                   norm_range: Optional[Tuple[float, float]] = None, dtype: str = "bfloat16"):
    if dtype not in _STORE:
        raise ValueError(f"dtype must be one of {sorted(_STORE)}, got {dtype!r}")
    arch, cfg = load_config(config_json)
    spec = arch.to_spec(cfg)
    # the parts are built on the CPU only to ask them for their tensor names and shapes
    runtime = Runtime(device=torch.device("cpu"), dtype=torch.float32, max_positions=1)
    model = DecoderModel(spec, runtime)
    out = {}
    for index, (name, ps) in enumerate(sorted(model.param_specs().items())):
        g = torch.Generator().manual_seed((int(seed) * 1000003 + index) & 0x7FFFFFFFFFFFFFFF)
        kind = ps.init[0]
        if ps.role == "vector" and norm_range is not None and kind == "ones":
            t = torch.empty(ps.shape).uniform_(float(norm_range[0]), float(norm_range[1]), generator=g)
        elif kind == "ones":
            t = torch.ones(ps.shape)
        elif kind == "zeros":
            t = torch.zeros(ps.shape)
        elif kind == "uniform":
            t = torch.empty(ps.shape).uniform_(float(ps.init[1]), float(ps.init[2]), generator=g)
        elif kind == "normal":
            t = torch.randn(ps.shape, generator=g) * std
        else:
            raise ValueError(f"tensor {name!r}: unknown init {ps.init!r}")
        out[name] = t.to(torch.int32) if ps.role == "table" else t.to(_STORE[dtype])
    return out, cfg


def write_random_model(config_json: dict, out_dir: str, seed: int, std: float = 0.02,
                       norm_range: Optional[Tuple[float, float]] = None, dtype: str = "bfloat16") -> str:
    tensors, _ = random_tensors(config_json, seed, std, norm_range, dtype)
    os.makedirs(out_dir, exist_ok=True)
    cfg_out = dict(config_json)
    cfg_out["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg_out, f, indent=2)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed), "std": str(std)})
    return out_dir


def scratch_folder(prefix: str) -> str:
    """A new temporary folder that is deleted when the process exits (model folders of random
    weights are gigabytes; nothing else removes them)."""
    import atexit
    import shutil
    import tempfile
    folder = tempfile.mkdtemp(prefix=prefix)
    atexit.register(shutil.rmtree, folder, True)
    return folder
