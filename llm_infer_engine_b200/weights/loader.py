"""Loads a model folder (config.json, model.safetensors) into a model, by tensor name.

The model says which tensors it reads (`param_specs()`); the file says which it holds. Any
disagreement is ONE error that lists the missing tensors, the unexpected ones and the wrong
shapes together. (The reference tolerates missing tensors silently and reports unexpected
ones in a returned dict, src/loader.py:110-151; a wrong shape raises, :73-76.)

Precision policy: a tensor stored in bfloat16 (or float16) is kept in bfloat16 by a bfloat16
engine and widened to float32 by a float32 engine (exact). A tensor stored in 32-bit stays
in 32-bit in either engine. Integer tensors become int32. The one narrowing there is: float16 becomes
bfloat16 in a bfloat16 engine (same width, fewer mantissa bits), since the kernels know one 16-bit format.

A checkpoint of a model with a tied head that also stores the head matrix (as some exporters do) is
accepted when that tensor has the embedding's shape: it is not read, and the report says so, as the
reference reports and goes on (src/loader.py:147-151).
"""
from __future__ import annotations

import re
import sys
from typing import Dict, List

import torch

from ..config.registry import load_config
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from .safetensors_io import open_model_files

_INT_TYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool)


class WeightsError(ValueError):
    """The checkpoint does not match the model; `.missing`, `.unexpected`, `.wrong_shape` hold the lists."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong_shape: List[tuple]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"{where}: the checkpoint does not match the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}):")
            lines += [f"    {n}" for n in missing]
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}):")
            lines += [f"    {n}" for n in unexpected]
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}):")
            lines += [f"    {n}: expected {tuple(e)}, file has {tuple(g)}" for n, e, g in wrong_shape]
        super().__init__("\n".join(lines))


def target_dtype(stored: torch.dtype, engine: torch.dtype) -> torch.dtype:
    if stored in _INT_TYPES:
        return torch.int32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16 if engine == torch.bfloat16 else torch.float32


def compare(expected: Dict[str, tuple], found: Dict[str, tuple], ignore: List[str], where: str) -> None:
    """Raises WeightsError unless `found` holds exactly the expected names with the expected shapes."""
    patterns = [re.compile(p) for p in ignore]
    missing = sorted(n for n in expected if n not in found)
    unexpected = sorted(n for n in found if n not in expected and not any(p.match(n) for p in patterns))
    wrong = sorted((n, expected[n], found[n]) for n in expected if n in found and tuple(found[n]) != tuple(expected[n]))
    if missing or unexpected or wrong:
        raise WeightsError(where, missing, unexpected, wrong)


def load_weights(model: DecoderModel, model_dir: str) -> Dict[str, int]:
    files = open_model_files(model_dir)
    specs = model.param_specs()
    expected = {n: ps.shape for n, ps in specs.items()}
    found = {n: f.entries[n][1] for n, f in files.items()}
    ignore = list(model.spec.ignore_unexpected)
    skipped = []
    head, emb = model.spec.head_name, model.spec.embedding_name
    if model.spec.tie_head and head in found and emb in expected and tuple(found[head]) == tuple(expected[emb]):
        ignore.append(re.escape(head) + "$")
        skipped.append(head)
        print(f"[llm_infer_engine_b200] {model_dir}: the head is tied to the embedding; the stored {head} is not read",
              file=sys.stderr)
    compare(expected, found, ignore, model_dir)
    rt = model.runtime
    tensors = {}
    n_bytes = 0
    for name in specs:
        host = files[name].tensor(name)
        dtype = target_dtype(host.dtype, rt.dtype)
        tensors[name] = host.to(device=rt.device, dtype=dtype)
        n_bytes += tensors[name].numel() * tensors[name].element_size()
    model.load_tensors(tensors)
    return {"tensors": len(tensors), "bytes": n_bytes, "skipped": skipped}


def build_model(model_dir: str, dtype: torch.dtype, device, max_positions: int | None = None):
    """config.json -> architecture -> typed config -> spec -> model with weights. Returns
    (model, typed config)."""
    arch, cfg = load_config(model_dir)
    spec = arch.to_spec(cfg)
    limit = spec.max_position if max_positions is None else min(max_positions, spec.max_position)
    runtime = Runtime(device=torch.device(device), dtype=dtype, max_positions=limit)
    model = DecoderModel(spec, runtime)
    model.load_report = load_weights(model, model_dir)
    return model, cfg
