"""Reader and writer for the safetensors container, by tensor name.

Layout: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}`, then the
data bytes that the offsets index. The reference reads one such file whole into host memory
with `safetensors.torch.load_file` (src/loader.py:99); this reader maps the file and hands out
one tensor at a time, and checks everything the header claims before any byte is used.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


def _no_duplicates(pairs):
    out = {}
    for k, v in pairs:
        if k in out:
            raise SafetensorsError(f"duplicate tensor name {k!r} in header")
        out[k] = v
    return out


class SafetensorsFile:
    """One mapped file. `entries[name] = (dtype, shape)`; `tensor(name)` returns a CPU tensor
    that views the mapping (copy-on-write, the file is never modified)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._file = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._file.read(8))
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        raw = self._file.read(hlen)
        try:
            header = json.loads(raw.decode("utf-8"), object_pairs_hook=_no_duplicates)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
        self._spans: Dict[str, Tuple[int, int]] = {}
        for name, info in header.items():
            try:
                dtype_name, shape, (begin, end) = info["dtype"], info["shape"], info["data_offsets"]
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{path}: entry {name!r} lacks dtype/shape/data_offsets") from e
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype_name!r}")
            dtype = _DTYPES[dtype_name]
            if not all(isinstance(s, int) and s >= 0 for s in shape):
                raise SafetensorsError(f"{path}: tensor {name!r} has a bad shape {shape!r}")
            numel = 1
            for s in shape:
                numel *= s
            nbytes = numel * torch.empty((), dtype=dtype).element_size()
            if not (isinstance(begin, int) and isinstance(end, int)) or not 0 <= begin <= end <= data_len:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} has data_offsets [{begin}, {end}] outside the data "
                    f"section of {data_len} bytes (file truncated?)")
            if end - begin != nbytes:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {shape} and dtype {dtype_name} needs {nbytes} bytes "
                    f"but its data_offsets span {end - begin}")
            self.entries[name] = (dtype, tuple(shape))
            self._spans[name] = (begin, end)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape = self.entries[name]
        begin, end = self._spans[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._data_start + begin:self._data_start + end]
        return torch.frombuffer(view, dtype=dtype).view(shape)

    def close(self) -> None:
        # tensors handed out may still view the mapping; it is released with the last of them
        self._map = None
        self._file.close()


def open_model_files(model_dir: str) -> Dict[str, SafetensorsFile]:
    """Tensor name -> the mapped file that holds it. Reads `model.safetensors`, or the shards
    listed by `model.safetensors.index.json`."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        return {name: f for name in f.names()}
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as fh:
            weight_map = json.load(fh).get("weight_map")
        if not isinstance(weight_map, dict):
            raise SafetensorsError(f"{index}: no weight_map")
        files: Dict[str, SafetensorsFile] = {}
        out: Dict[str, SafetensorsFile] = {}
        for name, shard in weight_map.items():
            if shard not in files:
                files[shard] = SafetensorsFile(os.path.join(model_dir, shard))
            if name not in files[shard].entries:
                raise SafetensorsError(f"{index}: {name!r} is not in shard {shard!r}")
            out[name] = files[shard]
        for shard, f in files.items():
            for name in f.names():
                out.setdefault(name, f)
        return out
    raise SafetensorsError(f"no model.safetensors (or model.safetensors.index.json) in {model_dir!r}")


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] | None = None) -> None:
    """Writes tensors (any device; made contiguous on the host) in name order."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().to("cpu").contiguous()
            if t.numel():
                f.write(_tensor_bytes(t))
    os.replace(tmp, path)


def _tensor_bytes(t: torch.Tensor) -> memoryview:
    flat = t.reshape(-1).view(torch.uint8) if t.dtype != torch.bool else t.reshape(-1).to(torch.uint8)
    return memoryview(flat.numpy())
