"""Weights from safetensors, by tensor name.

Every tensor the model expects is looked up by its checkpoint name; shapes are
checked before anything is copied and *one* error lists all missing tensors, all
unexpected ones and all wrong shapes.  On the device a matrix is kept in the compute
dtype (bfloat16 in serving), a per-channel vector in float32 (lossless for bfloat16
storage; a tensor stored in 32-bit stays 32-bit), an integer table in int32.
Parity: qwen3_runtime/utils/loader.py:33-102 (names, index file or ``*.safetensors``,
conversion while moving), with the errors made explicit.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable, Protocol

import torch

from ..parts.base import ParamSpec


class WeightError(RuntimeError):
    """Checkpoint and model do not fit; the message lists every problem."""


class TensorSource(Protocol):
    def names(self) -> Iterable[str]: ...

    def shape(self, name: str) -> tuple[int, ...]: ...

    def get(self, name: str) -> torch.Tensor: ...


class SafetensorsDir:
    """The tensors of a model folder (``model.safetensors.index.json`` or ``*.safetensors``)."""

    def __init__(self, model_dir: str | Path):
        from safetensors import safe_open

        self.path = Path(model_dir)
        index = self.path / "model.safetensors.index.json"
        if index.exists():
            weight_map = json.loads(index.read_text()).get("weight_map") or {}
            files = sorted(set(weight_map.values()))
            if not files:
                raise FileNotFoundError(f"empty weight_map in {index}")
        else:
            files = sorted(p.name for p in self.path.glob("*.safetensors"))
            if not files:
                raise FileNotFoundError(f"no .safetensors files in {self.path}")
        self._handles = {}
        self._where: dict[str, str] = {}
        for name in files:
            handle = safe_open(str(self.path / name), framework="pt", device="cpu")
            self._handles[name] = handle
            for key in handle.keys():
                self._where[key] = name

    def names(self):
        return self._where.keys()

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self._handles[self._where[name]].get_slice(name).get_shape())

    def get(self, name: str) -> torch.Tensor:
        return self._handles[self._where[name]].get_tensor(name)


class DictSource:
    """Tensors already in memory (tests, weight generators)."""

    def __init__(self, tensors: dict[str, torch.Tensor]):
        self.tensors = tensors

    def names(self):
        return self.tensors.keys()

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def get(self, name):
        return self.tensors[name]


def check_tensors(expected: dict[str, ParamSpec], source: TensorSource, ignorable: set[str] = frozenset()) -> None:
    have = set(source.names())
    missing = [n for n in expected if n not in have]
    unexpected = sorted(have - set(expected) - set(ignorable))
    wrong = [
        f"{n}: checkpoint {list(source.shape(n))}, model {list(ps.shape)}"
        for n, ps in expected.items()
        if n in have and tuple(source.shape(n)) != tuple(ps.shape)
    ]
    if missing or unexpected or wrong:
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        raise WeightError("\n".join(lines))


def place(tensor: torch.Tensor, spec: ParamSpec, dtype: torch.dtype, device) -> torch.Tensor:
    """Move one stored tensor to the device in the dtype its kind calls for."""
    if spec.kind == "int":
        if tensor.is_floating_point():
            raise WeightError("an integer table is stored as floating point")
        return tensor.to(device=device, dtype=torch.int32)
    if not tensor.is_floating_point():
        raise WeightError("a floating-point tensor is stored as integers")
    if spec.kind == "vector":
        return tensor.to(device=device, dtype=torch.float32)
    return tensor.to(device=device, dtype=dtype)


def load_into(model, source: TensorSource) -> None:
    """Check ``source`` against ``model.expected_tensors()`` and load every tensor.  Each tensor
    is moved to the device when the part that owns it asks for it, so a part that fuses stored
    tensors (q/k/v, gate/up) holds the separate copies only while it fuses them."""
    expected = model.expected_tensors()
    check_tensors(expected, source, model.ignorable_tensors())
    ctx = model.ctx
    model.load_from(lambda name: place(source.get(name), expected[name], ctx.dtype, ctx.device))
