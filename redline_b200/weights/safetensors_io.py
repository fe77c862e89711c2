"""Reading and writing safetensors files without any library of that name.

Layout: 8 bytes little-endian header length N, N bytes of JSON (tensor name ->
dtype, shape, data_offsets relative to the end of the header; ``__metadata__``
holds strings), then the raw little-endian data.  The reader maps the file and
hands out zero-copy CPU tensors.  Error cases follow the reference's reader
(src/core/safetensors.cpp:68-108): cannot open, too small, header length beyond
the file, header not JSON, tensor outside the file, byte size that does not match
dtype and shape.
"""

from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import torch

ST_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
}
ST_NAMES = {v[0]: k for k, v in ST_DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e.strerror}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too small to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: corrupt header: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: corrupt header: not an object")
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self._info: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, ent in header.items():
            try:
                dt, shape, (b, e) = ent["dtype"], tuple(int(s) for s in ent["shape"]), ent["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: corrupt header entry for tensor {name}") from None
            if dt not in ST_DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {dt}")
            numel = 1
            for s in shape:
                numel *= s
            if b < 0 or e < b or e > data_size:
                raise SafetensorsError(f"{path}: tensor {name} lies outside the file")
            if e - b != numel * ST_DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor {name} has {e - b} bytes but {dt}{list(shape)} needs "
                    f"{numel * ST_DTYPES[dt][1]}")
            self._info[name] = (dt, shape, b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> List[str]:
        return list(self._info.keys())

    def has(self, name: str) -> bool:
        return name in self._info

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        if name not in self._info:
            raise SafetensorsError(f"{self.path}: tensor {name} not found")
        dt, shape, _, _ = self._info[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that shares the mapped file's memory (read-only: clone before writing)."""
        dt, shape = self.info(name)
        _, _, b, e = self._info[name]
        tdt = ST_DTYPES[dt][0]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        buf = memoryview(self._mm)[self._data_start + b:self._data_start + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # "buffer is not writable": it is only read
            return torch.frombuffer(buf, dtype=tdt).view(shape)

    def close(self) -> None:
        # tensors handed out keep the map alive through their memoryview
        self._f.close()


class CheckpointReader:
    """All tensors of a model folder: ``model.safetensors``, or the shards named by
    ``model.safetensors.index.json``, or every ``*.safetensors`` in the folder."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            with open(index) as f:
                paths = sorted({os.path.join(model_dir, p) for p in json.load(f)["weight_map"].values()})
        else:
            paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        if not paths:
            raise SafetensorsError(f"{model_dir}: no model.safetensors (or shards) found")
        self.files = [SafetensorsFile(p) for p in paths]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self._where[n] = f

    def names(self) -> List[str]:
        return list(self._where.keys())

    def has(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str) -> Tuple[str, Tuple[int, ...]]:
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)


class SafetensorsWriter:
    """Writes tensors one at a time: declare all (name, dtype, shape) first, then
    stream the data in the same order, so a large model never sits in memory twice."""

    def __init__(self, path: str, plan: Iterable[Tuple[str, torch.dtype, Tuple[int, ...]]],
                 metadata: Optional[Dict[str, str]] = None):
        header: Dict[str, object] = {}
        if metadata:
            header["__metadata__"] = dict(metadata)
        off = 0
        self._plan = []
        for name, dtype, shape in plan:
            numel = 1
            for s in shape:
                numel *= int(s)
            nbytes = numel * ST_DTYPES[ST_NAMES[dtype]][1]
            header[name] = {"dtype": ST_NAMES[dtype], "shape": [int(s) for s in shape],
                            "data_offsets": [off, off + nbytes]}
            self._plan.append((name, dtype, tuple(int(s) for s in shape), nbytes))
            off += nbytes
        hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
        hj += b" " * ((8 - len(hj) % 8) % 8)
        self._f = open(path, "wb")
        self._f.write(struct.pack("<Q", len(hj)))
        self._f.write(hj)
        self._next = 0

    def write(self, name: str, tensor: torch.Tensor) -> None:
        want_name, dtype, shape, nbytes = self._plan[self._next]
        if name != want_name or tensor.dtype != dtype or tuple(tensor.shape) != shape:
            raise SafetensorsError(f"writer expected {want_name} {dtype}{list(shape)}, got {name} "
                                   f"{tensor.dtype}{list(tensor.shape)}")
        t = tensor.detach().cpu().contiguous()
        if t.numel():
            self._f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())
        self._next += 1

    def close(self) -> None:
        if self._next != len(self._plan):
            raise SafetensorsError(f"writer closed after {self._next} of {len(self._plan)} tensors")
        self._f.close()


def save_file(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    w = SafetensorsWriter(path, [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()], metadata)
    for n, t in tensors.items():
        w.write(n, t)
    w.close()
