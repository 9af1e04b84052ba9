"""Reading and writing safetensors files: an 8-byte little-endian header
length, a JSON header (tensor name -> dtype, shape, byte range) and the raw
payload (MisterTK/gibbs ``src/model/mod.rs:398-410``; single file or an
``*.index.json`` of shards, ``src/model/weights.rs:341-386``).  The payload is
memory-mapped; a tensor is materialised only when it is asked for.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Iterable

import numpy as np
import torch

# safetensors dtype tag -> (torch dtype as stored, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F64": (torch.float64, 8),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_TAGS = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """Header of one file plus lazy access to its tensors."""

    def __init__(self, path):
        self.path = Path(path)
        with open(self.path, "rb") as fh:
            head = fh.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{self.path}: truncated before the header length")
            (hlen,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if 8 + hlen > size:
                raise SafetensorsError(f"{self.path}: header of {hlen} bytes does not fit a file of {size} bytes")
            try:
                header = json.loads(fh.read(hlen))
            except json.JSONDecodeError as e:
                raise SafetensorsError(f"{self.path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self.base = 8 + hlen
        self.entries: dict[str, dict] = header
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor '{name}' has unsupported dtype {info['dtype']}")
            lo, hi = info["data_offsets"]
            want = int(np.prod(info["shape"], dtype=np.int64)) * _DTYPES[info["dtype"]][1]
            if hi - lo != want or self.base + hi > size:
                raise SafetensorsError(
                    f"{self.path}: tensor '{name}' {info['dtype']}{info['shape']} needs {want} bytes, "
                    f"its range [{lo}, {hi}) holds {hi - lo} (file size {size})")
        self._mm = None

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name) -> torch.Tensor:
        """A CPU tensor that views the mapped file (copy before the file goes away)."""
        if self._mm is None:
            with open(self.path, "rb") as fh:
                self._mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        info = self.entries[name]
        tdtype, _ = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        if hi == lo:
            return torch.empty(info["shape"], dtype=tdtype)
        buf = memoryview(self._mm)[self.base + lo : self.base + hi]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # the mapping is read-only; the tensor is never written
            t = torch.frombuffer(buf, dtype=tdtype)
        return t.reshape(info["shape"])


class Checkpoint:
    """All tensors of a model folder: ``model.safetensors``, or the shards an
    ``model.safetensors.index.json`` lists."""

    def __init__(self, folder):
        self.folder = Path(folder)
        single = self.folder / "model.safetensors"
        index = self.folder / "model.safetensors.index.json"
        self.files: list[SafetensorsFile] = []
        self.where: dict[str, SafetensorsFile] = {}
        if single.exists():
            self._add(SafetensorsFile(single))
        elif index.exists():
            weight_map = json.loads(index.read_text())["weight_map"]
            opened: dict[str, SafetensorsFile] = {}
            for shard in sorted(set(weight_map.values())):
                if not (self.folder / shard).exists():
                    raise SafetensorsError(f"{index} lists shard '{shard}', which is absent")
                opened[shard] = SafetensorsFile(self.folder / shard)
                self._add(opened[shard])
            absent = sorted(n for n in weight_map if n not in self.where)
            if absent:
                raise SafetensorsError(f"{index} lists tensors that no shard holds: {absent}")
        else:
            raise FileNotFoundError(f"{self.folder} has neither model.safetensors nor model.safetensors.index.json")

    def _add(self, f: SafetensorsFile):
        self.files.append(f)
        for n in f.names():
            if n in self.where:
                raise SafetensorsError(f"tensor '{n}' appears in {self.where[n].path.name} and {f.path.name}")
            self.where[n] = f

    def names(self) -> list[str]:
        return list(self.where)

    def shape(self, name):
        return self.where[name].shape(name)

    def dtype(self, name):
        return self.where[name].dtype(name)

    def tensor(self, name):
        return self.where[name].tensor(name)


class TensorDict:
    """The same read interface over tensors already in memory."""

    def __init__(self, tensors: dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return list(self.tensors)

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def dtype(self, name):
        return self.tensors[name].dtype

    def tensor(self, name):
        return self.tensors[name]


def write_safetensors(path, tensors: Iterable[tuple[str, torch.Tensor]], metadata: dict | None = None) -> None:
    """Write tensors in the order given.  The JSON header is padded with spaces
    to a multiple of 8 bytes (as the reference's test writer does,
    ``src/arch/testing.rs:71-88``)."""
    items = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header, off = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in items:
        if t.dtype not in _TAGS:
            raise SafetensorsError(f"tensor '{name}' has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAGS[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(hj)))
        fh.write(hj)
        for _, t in items:
            if t.numel():
                fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
