"""Weights by tensor name: what a model expects, checking, loading, random filling.

Every part of a model declares the tensors it needs as :class:`WeightSpec`
(name, shape, storage rule).  Loading compares the declared set with what the
source holds and raises ONE :class:`WeightError` that lists every missing
tensor, every unexpected tensor and every wrong shape, in the manner of the
reference's MissingTensor / ShapeMismatch errors
(crates/airun-core/src/error.rs:59-74, crates/airun-core/src/model.rs:1895-2018).

Storage rules:
  ``compute``   matrices used by matrix products: kept in bfloat16 when the engine
                serves in bfloat16, widened to float32 for the 32-bit path;
  ``float32``   always float32 (norm weights; the reference widens norms to f32,
                crates/airun-core/src/model.rs:1828-1840);
  ``as_stored`` kept in the stored type: a tensor stored in 32-bit stays 32-bit,
                integer tables become int32.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Protocol, Sequence, Tuple

import numpy as np
import torch

from .safetensors_io import SafetensorsFolder, write_safetensors


class WeightError(ValueError):
    """Raised once per load with every problem listed."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_type: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_type = list(wrong_type)
        lines = ["the weights do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(found)}, expected {list(exp)}" for n, found, exp in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  unusable types ({len(self.wrong_type)}): " + ", ".join(
                f"{n} is {t}" for n, t in self.wrong_type))
        lines.append("  check that config.json and model.safetensors belong to the same model")
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    storage: str = "compute"          # compute | float32 | as_stored
    init: str = "normal"              # normal: N(0, 0.02); norm: 1 + N(0, 0.1); zeros; int
    optional: bool = False


class TensorSource(Protocol):
    def names(self) -> List[str]: ...
    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]: ...
    def read(self, name: str) -> torch.Tensor: ...


class DictSource:
    """Tensors already in memory (any device)."""

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self) -> List[str]:
        return list(self.tensors)

    def info(self, name: str):
        t = self.tensors[name]
        return t.dtype, tuple(t.shape)

    def read(self, name: str) -> torch.Tensor:
        return self.tensors[name]


_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def check_source(specs: Sequence[WeightSpec], source: TensorSource,
                 ignorable: Iterable[str] = ()) -> None:
    """Raises WeightError unless ``source`` holds exactly what ``specs`` declare."""
    have = set(source.names())
    ignorable = set(ignorable)
    wanted = {s.name for s in specs}
    missing = [s.name for s in specs if s.name not in have and not s.optional]
    unexpected = sorted(n for n in have if n not in wanted and n not in ignorable)
    wrong_shape, wrong_type = [], []
    for s in specs:
        if s.name in have:
            dt, shape = source.info(s.name)
            if tuple(shape) != tuple(s.shape):
                wrong_shape.append((s.name, tuple(shape), tuple(s.shape)))
            if s.storage in ("compute", "float32") and dt not in _FLOATS:
                wrong_type.append((s.name, str(dt)))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(missing, unexpected, wrong_shape, wrong_type)


def stored_dtype(spec: WeightSpec, found: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device."""
    if spec.storage == "compute":
        return compute_dtype
    if spec.storage == "float32":
        return torch.float32
    if found in _INTS:
        return torch.int32
    if found in (torch.float32, torch.float64):
        return torch.float32
    return found if compute_dtype != torch.float32 else torch.float32


def load_tensors(specs: Sequence[WeightSpec], source: TensorSource,
                 compute_dtype: torch.dtype, device: torch.device | str,
                 ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Checks ``source`` against ``specs`` and returns the tensors on ``device``."""
    check_source(specs, source, ignorable)
    have = set(source.names())
    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in have:
            continue
        t = source.read(s.name)
        want = stored_dtype(s, t.dtype, compute_dtype)
        out[s.name] = t.to(device=device, dtype=want).contiguous()
    return out


_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


def _mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor: the seed mixed with the FNV-1a hash of its name."""
    h = 0xCBF29CE484222325
    for byte in name.encode("utf-8"):
        h = ((h ^ byte) * 0x100000001B3) & _M64
    return _mix64((h ^ ((int(seed) * _GOLDEN) & _M64)) & _M64)


def _np_mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def fill_random_host(n: int, key: int, kind: str, scale: float) -> np.ndarray:
    """Element i of the tensor with ``key`` as a function of (key, i) alone: the arithmetic of
    ``fill_random_kernel`` (csrc/elementwise.cu), integer up to one float32 product (and one sum
    for ``kind == "norm"``), so the device fills the same tensor bit for bit.  Returns float32
    (``normal``: z * scale, ``norm``: 1 + z * scale) or int32 (``int``)."""
    out = np.empty(n, dtype=np.int32 if kind == "int" else np.float32)
    step = 1 << 22
    gold, k = np.uint64(_GOLDEN), np.uint64(key)
    with np.errstate(over="ignore"):
        for s in range(0, n, step):
            e = min(n, s + step)
            c = np.arange(s, e, dtype=np.uint64) * np.uint64(3)
            h0 = _np_mix(k + c * gold)
            if kind == "int":
                out[s:e] = (h0 & np.uint64(0x7FFF)).astype(np.int32)
                continue
            h1 = _np_mix(k + (c + np.uint64(1)) * gold)
            h2 = _np_mix(k + (c + np.uint64(2)) * gold)
            total = np.zeros(e - s, dtype=np.int64)
            for h in (h0, h1, h2):
                for f in range(4):
                    total += ((h >> np.uint64(16 * f)) & np.uint64(0xFFFF)).astype(np.int64)
            z = (total - 393210).astype(np.float32) * np.float32(1.0 / 65536.0)
            w = z * np.float32(scale)
            if kind == "norm":
                w = np.float32(1.0) + w
            out[s:e] = w
    return out


def _fill_random_device(t: torch.Tensor, key: int, kind: str, scale: float) -> None:
    import ctypes
    from ..csrc import build
    lib = build.load("elementwise")
    f = lib.airun_fill_random
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_float,
                  ctypes.c_void_p]
    f.restype = ctypes.c_int
    dt = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}[t.dtype]
    with torch.cuda.device(t.device):
        rc = f(t.data_ptr(), dt, t.numel(), key, {"normal": 0, "norm": 1, "int": 2}[kind], float(scale),
               torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise RuntimeError(f"fill_random: status {rc}")


def random_tensors(specs: Sequence[WeightSpec], seed: int,
                   device: torch.device | str = "cpu",
                   matrix_dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_std: float = 0.1) -> Dict[str, torch.Tensor]:
    """Seeded random weights: matrices N(0, std) stored in ``matrix_dtype``, norm weights
    1 + N(0, norm_std) in float32.  Element i of tensor ``name`` depends on (seed, name, i) only (a
    counter-based generator, ``fill_random_host``), so the order of the specs does not matter and a
    tensor filled on the GPU by ``fill_random_kernel`` equals the one made here on the CPU bit for
    bit: a plain implementation can make the weights of a model again without a file."""
    out: Dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for s in specs:
        n = 1
        for d in s.shape:
            n *= int(d)
        kind = {"norm": "norm", "int": "int", "zeros": "zeros"}.get(s.init, "normal")
        dtype = torch.int32 if kind == "int" else (matrix_dtype if s.storage == "compute" else torch.float32)
        if kind == "zeros":
            out[s.name] = torch.zeros(s.shape, device=dev, dtype=dtype)
            continue
        key = tensor_key(seed, s.name)
        scale = norm_std if kind == "norm" else std
        if dev.type == "cuda":
            t = torch.empty(s.shape, device=dev, dtype=dtype)
            _fill_random_device(t, key, kind, scale)
        else:
            t = torch.from_numpy(fill_random_host(n, key, kind, scale)).view(s.shape).to(dtype)
        out[s.name] = t
    return out


def write_model_folder(model_dir: str, config, specs: Sequence[WeightSpec], seed: int,
                       matrix_dtype: torch.dtype = torch.bfloat16) -> None:
    """Random-weights mode: writes config.json and model.safetensors for ``config``."""
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=1)
    tensors = random_tensors(specs, seed, "cpu", matrix_dtype)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})


def open_model_folder(model_dir: str) -> SafetensorsFolder:
    return SafetensorsFolder(model_dir)
