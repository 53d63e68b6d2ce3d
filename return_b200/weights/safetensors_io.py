"""Reader and writer of the safetensors container, by tensor name.

The format: eight bytes (little-endian length N), N bytes of JSON mapping each name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header), then the raw little-endian data.  The reader maps the file into memory and makes
one tensor per name on request, so a large checkpoint is never held twice.  A model folder
holds either ``model.safetensors`` or ``model.safetensors.index.json`` with shards.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {path}: {e}") from e
        head = self._fh.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file")
        try:
            meta = json.loads(self._fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
        self.metadata = meta.pop("__metadata__", {})
        self.entries: Dict[str, dict] = meta
        self._base = 8 + n
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for name, e in self.entries.items():
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has dtype {e['dtype']}, which is not handled")
            b, end = e["data_offsets"]
            want = int(np.prod(e["shape"], dtype=np.int64)) * _DTYPES[e["dtype"]][1]
            if end - b != want or self._base + end > size:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that copies the named data out of the mapping."""
        e = self.entries[name]
        dt, _ = _DTYPES[e["dtype"]]
        b, end = e["data_offsets"]
        if end == b:
            return torch.empty(e["shape"], dtype=dt)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=end - b, offset=self._base + b)
        return torch.from_numpy(buf.copy()).view(dt).reshape(e["shape"])

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._fh.close()


class ModelFiles:
    """All tensors of a model folder, over one file or an index of shards."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(single):
            f = SafetensorsFile(single)
            self._files[single] = f
            self._where = {n: single for n in f.names()}
        elif os.path.isfile(index):
            with open(index) as fh:
                weight_map = json.load(fh)["weight_map"]
            for name, shard in weight_map.items():
                path = os.path.join(model_dir, shard)
                if path not in self._files:
                    if not os.path.isfile(path):
                        raise SafetensorsError(f"{index} names the shard {shard}, which is missing")
                    self._files[path] = SafetensorsFile(path)
                if name not in self._files[path].entries:
                    raise SafetensorsError(f"{index} places {name} in {shard}, which does not hold it")
                self._where[name] = path
        else:
            raise SafetensorsError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return self._files[self._where[name]].shape(name)

    def dtype(self, name: str) -> torch.dtype:
        return self._files[self._where[name]].dtype(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Writes named CPU tensors.  ``tensors`` may be a generator, but it is walked twice: once for
    the header and once for the data, so pass a callable-backed list for large models."""
    items = list(tensors)
    header, offset = {}, 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name} has dtype {t.dtype}, which safetensors does not hold")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            c = t.detach().contiguous().cpu()
            fh.write(c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b"")
    os.replace(tmp, path)
