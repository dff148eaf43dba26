"""Tracing of a step: NVTX ranges with the reference's stage names, and a per-kernel timer.

The reference marks every stage of its forward pass and of its loop with NVTX ranges
(src/model.py:22,53,61,66,78,82,86,112,126,156,165,180; main.py:235,256,258,278) so that a timeline
reads "Prefill / Decode / Step_i / ModelForward / Layers / Attn_i / QKV_proj / RoPE / KV_cache /
FlashAttn | FlashDecode / Output_proj / FFN_i / FFN / Output / Sample". The same names are used here.
Ranges cost a call each, so they are off unless asked for (`enable_ranges`, `Engine(nvtx=True)`,
`--nvtx` on the command line).

`KernelTimer` brackets every launch of this library (and the library matrix products of the parts)
with CUDA events while it is installed, and keeps the name, the stage it ran in, its time, and the
bytes and floating-point operations the caller said it has to move and do. Captured steps cannot be
timed this way: run the eager step. Launches are not overlapped meanwhile (no programmatic dependent
launch across an event), so the sum is an upper bound of the step's time in a graph.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Dict, List, Optional, Tuple

import torch

RANGES = False
_stack: List[str] = []
timer: Optional["KernelTimer"] = None


def enable_ranges(on: bool = True) -> None:
    global RANGES
    RANGES = bool(on)


def active() -> bool:
    return RANGES or timer is not None


def push(name: str) -> None:
    if RANGES or timer is not None:
        _stack.append(name)
        if RANGES:
            torch.cuda.nvtx.range_push(name)


def pop() -> None:
    if RANGES or timer is not None:
        if _stack:
            _stack.pop()
        if RANGES:
            torch.cuda.nvtx.range_pop()


@contextmanager
def stage(name: str):
    push(name)
    try:
        yield
    finally:
        pop()


def generic_stage() -> str:
    """The innermost stage with the layer number taken off (Attn_3 -> Attn), for tables over all layers."""
    for name in reversed(_stack):
        head, _, tail = name.rpartition("_")
        return head if head and tail.isdigit() else name
    return ""


class KernelTimer:
    def __init__(self):
        self.records: List[Tuple[str, str, torch.cuda.Event, torch.cuda.Event, float, float]] = []
        self._pending = (0.0, 0.0)

    def note(self, nbytes: float = 0.0, flops: float = 0.0) -> None:
        """What the next launch has to read and write (bytes) and compute (flops), as the caller counts it."""
        self._pending = (float(nbytes), float(flops))

    def run(self, name: str, fn, args):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nbytes, flops = self._pending
        self._pending = (0.0, 0.0)
        start.record()
        out = fn(*args)
        end.record()
        self.records.append((name, generic_stage(), start, end, nbytes, flops))
        return out

    def table(self) -> List[Dict]:
        """One row per (stage, kernel): launches, total microseconds, bytes, flops. Synchronises."""
        torch.cuda.synchronize()
        rows: Dict[Tuple[str, str], Dict] = {}
        for name, where, start, end, nbytes, flops in self.records:
            row = rows.setdefault((where, name), {"stage": where, "kernel": name, "launches": 0, "us": 0.0,
                                                  "bytes": 0.0, "flops": 0.0})
            row["launches"] += 1
            row["us"] += start.elapsed_time(end) * 1e3
            row["bytes"] += nbytes
            row["flops"] += flops
        return list(rows.values())


@contextmanager
def timing():
    """Installs a KernelTimer for the block; programmatic dependent launch is off meanwhile."""
    global timer
    from . import ops
    was = ops.PDL
    ops.set_pdl(False)
    timer = KernelTimer()
    try:
        yield timer
    finally:
        timer = None
        ops.set_pdl(was)
