"""Reading and writing safetensors files.

File layout: an unsigned 64-bit little-endian header length, a JSON header
mapping each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}``
(offsets relative to the end of the header), then the raw little-endian data.
The reference's reader checks the same things: a truncated header or payload,
an unknown dtype, offsets outside the file, and an element count that does not
match the byte span (crates/airun-gguf/src/safetensors.rs:104-155, :184-192,
:229-320).  A folder may hold one ``model.safetensors`` or shards listed in
``model.safetensors.index.json``.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Tuple

import torch


class SafetensorsError(ValueError):
    pass


_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsFile:
    """One file, memory-mapped; tensors are read on demand."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: file of {size} bytes is too short for a safetensors header")
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise SafetensorsError(
                f"{path}: header length {hlen} does not fit the file ({size} bytes): truncated or not safetensors")
        try:
            header = json.loads(self._mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._base = 8 + hlen
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        payload = size - self._base
        for name, e in header.items():
            try:
                dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise SafetensorsError(f"{path}: entry {name!r} is malformed: {ex}") from ex
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt}")
            tdt, esz = _DTYPES[dt]
            n = 1
            for s in shape:
                n *= s
            if not (0 <= b <= en <= payload):
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans bytes [{b}, {en}) but the payload has {payload}: truncated file")
            if en - b != n * esz:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} of shape {list(shape)} {dt} needs {n * esz} bytes, has {en - b}")
            self.entries[name] = (tdt, shape, b, en)

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self.entries[name]
        return e[0], e[1]

    def read(self, name: str) -> torch.Tensor:
        """A fresh CPU tensor holding ``name`` in its stored dtype."""
        tdt, shape, b, en = self.entries[name]
        if en == b:
            return torch.empty(shape, dtype=tdt)
        buf = bytearray(self._mm[self._base + b:self._base + en])
        return torch.frombuffer(buf, dtype=tdt).reshape(shape)

    def close(self) -> None:
        self._mm.close()
        self._f.close()


class SafetensorsFolder:
    """All tensors of a model folder, whichever file they live in."""

    def __init__(self, model_dir: str):
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.files: List[SafetensorsFile] = []
        self.where: Dict[str, SafetensorsFile] = {}
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as f:
                wm = json.load(f).get("weight_map", {})
            paths = sorted({os.path.join(model_dir, p) for p in wm.values()})
        else:
            raise SafetensorsError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
        for p in paths:
            if not os.path.isfile(p):
                raise SafetensorsError(f"{p}: shard named by the index is missing")
            sf = SafetensorsFile(p)
            self.files.append(sf)
            for n in sf.names():
                if n in self.where:
                    raise SafetensorsError(f"tensor {n!r} appears in both {self.where[n].path} and {p}")
                self.where[n] = sf

    def names(self) -> List[str]:
        return list(self.where)

    def info(self, name: str):
        return self.where[name].info(name)

    def read(self, name: str) -> torch.Tensor:
        return self.where[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes ``tensors`` (CPU or device) in name order, data 8-byte aligned."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for n in order:
        t = tensors[n]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {n!r} has dtype {t.dtype}, which safetensors cannot hold")
        nbytes = t.numel() * t.element_size()
        header[n] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                     "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    hb = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for n in order:
            t = tensors[n].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
