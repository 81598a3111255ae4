"""Reader and writer of the safetensors container.

Layout: 8 bytes little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header), then the raw little-endian tensor bytes. Files are memory-mapped; a tensor is a
view of the map until it is copied to the device. The reference maps every
``*.safetensors`` of a folder the same way (src/hub/loader.jl:20-29).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped file: ``entries`` maps a tensor name to (dtype, shape, begin, end)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a safetensors header")
        self._file = open(path, "rb")
        # Copy-on-write: tensors may view the map without ever changing the file.
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_COPY)
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size} (truncated file?)")
        try:
            header = json.loads(self._map[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self._base = 8 + n
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            dtype = _DTYPES[info["dtype"]]
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(o) for o in info["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * dtype.itemsize:
                raise SafetensorsError(f"{path}: tensor {name} of shape {shape} {info['dtype']} needs "
                                       f"{count * dtype.itemsize} bytes, header gives {end - begin}")
            if self._base + end > size:
                raise SafetensorsError(f"{path}: tensor {name} ends at byte {self._base + end}, "
                                       f"file has {size} (truncated file?)")
            self.entries[name] = (dtype, shape, begin, end)

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        count = (end - begin) // dtype.itemsize
        flat = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + begin)
        return flat.reshape(shape)


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] = None) -> None:
    """Write ``tensors`` (CPU or device; made contiguous) to ``path``."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name} of dtype {t.dtype}")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())


def open_folder(model_dir: str) -> Tuple[Dict[str, SafetensorsFile], Iterable[SafetensorsFile]]:
    """Map every ``*.safetensors`` of ``model_dir``; returns (name -> file, files)."""
    paths = sorted(os.path.join(model_dir, f) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if not paths:
        raise SafetensorsError(f"{model_dir} holds no .safetensors file")
    by_name: Dict[str, SafetensorsFile] = {}
    files = []
    for p in paths:
        f = SafetensorsFile(p)
        files.append(f)
        for name in f.entries:
            if name in by_name:
                raise SafetensorsError(f"tensor {name} is stored twice: in {by_name[name].path} and {p}")
            by_name[name] = f
    return by_name, files
