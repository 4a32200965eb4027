"""Random weights from a configuration and a seed.

Tensors are drawn in the model's fixed checkpoint-name order from one seeded CPU
generator, so a seed names a model regardless of how parts fuse their tensors:
matrices N(0, std), per-channel vectors (norm weights) 1 + N(0, vector_std).
:func:`write_random_model` writes a model folder (``config.json``,
``model.safetensors``) that the ordinary loader reads back.  The reference's only
random mode is ``LLM(model=None)`` with default initialisers and unit norm weights
(qwen3_runtime/llm.py:111-121).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config.registry import architecture_for_config
from ..parts.base import BuildContext, ParamSpec
from ..parts.model import DecoderModel

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def expected_tensors_for(config) -> dict[str, ParamSpec]:
    """Checkpoint names and shapes of the model a typed config describes (no device needed)."""
    arch = architecture_for_config(config)
    ctx = BuildContext(dtype=torch.float32, device=torch.device("cpu"), ops=None)
    return DecoderModel(arch.build_spec(config), ctx).expected_tensors()


def random_tensor(spec: ParamSpec, generator: torch.Generator, std: float, vector_std: float,
                  store_dtype: torch.dtype) -> torch.Tensor:
    if spec.kind == "int":
        raise ValueError("integer tables have no random initialiser")
    t = torch.randn(spec.shape, generator=generator, dtype=torch.float32)
    t = 1.0 + vector_std * t if spec.kind == "vector" else std * t
    return t.to(store_dtype)


def random_state(config, seed: int, *, std: float = 0.02, vector_std: float = 0.02,
                 store_dtype: str = "bfloat16") -> dict[str, torch.Tensor]:
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    return {
        name: random_tensor(ps, generator, std, vector_std, _STORE[store_dtype])
        for name, ps in expected_tensors_for(config).items()
    }


def write_random_model(config, folder: str | Path, seed: int, *, std: float = 0.02, vector_std: float = 0.02,
                       store_dtype: str = "bfloat16") -> Path:
    """Write ``config.json`` and ``model.safetensors`` for a random model; return the folder."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_hf_config()
    raw["torch_dtype"] = store_dtype
    (folder / "config.json").write_text(json.dumps(raw, indent=2) + "\n")
    state = random_state(config, seed, std=std, vector_std=vector_std, store_dtype=store_dtype)
    save_file({k: v.contiguous() for k, v in state.items()}, str(folder / "model.safetensors"))
    return folder


class RandomDeviceSource:
    """Random tensors generated on the device, one at a time (large benchmark models:
    no file, no host copy).  Same distributions as :func:`random_state`; the values
    differ from the CPU generator's."""

    def __init__(self, expected: dict[str, ParamSpec], seed: int, device, *, std: float = 0.02,
                 vector_std: float = 0.02, store_dtype: str = "bfloat16"):
        self.expected = expected
        self.device = device
        self.std, self.vector_std = std, vector_std
        self.store_dtype = _STORE[store_dtype]
        self.generator = torch.Generator(device=device)
        self.generator.manual_seed(int(seed))

    def names(self):
        return self.expected.keys()

    def shape(self, name):
        return tuple(self.expected[name].shape)

    def get(self, name):
        ps = self.expected[name]
        t = torch.empty(ps.shape, dtype=torch.float32, device=self.device)
        t.normal_(0.0, 1.0, generator=self.generator)
        t = 1.0 + self.vector_std * t if ps.kind == "vector" else self.std * t
        return t.to(self.store_dtype)
