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

import hashlib
import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Protocol, Sequence, Tuple

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


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(specs: Sequence[WeightSpec], seed: int,
                   device: torch.device | str = "cpu",
                   matrix_dtype: torch.dtype = torch.bfloat16,
                   std: float = 0.02, norm_std: float = 0.1) -> Dict[str, torch.Tensor]:
    """Seeded random weights, one generator per tensor name so the order of the
    specs does not matter: matrices N(0, std) stored in ``matrix_dtype``, norm
    weights 1 + N(0, norm_std) in float32."""
    out: Dict[str, torch.Tensor] = {}
    dev = torch.device(device)
    for s in specs:
        g = torch.Generator(device=dev)
        g.manual_seed(_seed_for(seed, s.name))
        if s.init == "norm":
            t = 1.0 + norm_std * torch.randn(s.shape, generator=g, device=dev, dtype=torch.float32)
        elif s.init == "zeros":
            t = torch.zeros(s.shape, device=dev, dtype=torch.float32)
        elif s.init == "int":
            t = torch.randint(0, 2 ** 15, s.shape, generator=g, device=dev, dtype=torch.int32)
        else:
            t = std * torch.randn(s.shape, generator=g, device=dev, dtype=torch.float32)
        if s.storage == "compute":
            t = t.to(matrix_dtype)
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
