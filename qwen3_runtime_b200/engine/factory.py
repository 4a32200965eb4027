"""Build a model, its cache and an engine from a model folder (or a config and a
tensor source).  Parity: qwen3_runtime/engine/factory.py:110-186 (``build_engine``
keyword names ``max_num_seqs``, ``max_num_batched_tokens``, ``block_size``,
``cuda_graph``, ``kv_budget``) and :75-107 (pages from free memory, at least 32)."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.engine_config import EngineConfig, canonical_dtype
from ..config.registry import architecture_for_config, load_config, read_config_json
from ..parts.base import BuildContext
from ..parts.model import DecoderModel
from ..sampling.sampler import Sampler
from ..weights.loader import SafetensorsDir, load_into
from .engine import Engine
from .runner import ModelRunner

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def default_ops(groups=None):
    from ..ops.cuda import CudaOps

    return CudaOps(groups)


def build_model(config, source, *, dtype: str = "bfloat16", device="cuda", ops=None) -> DecoderModel:
    """A loaded :class:`DecoderModel` for a typed config and a tensor source."""
    arch = architecture_for_config(config)
    ops = ops if ops is not None else default_ops()
    ctx = BuildContext(dtype=_TORCH_DTYPE[canonical_dtype(dtype)], device=torch.device(device), ops=ops)
    model = DecoderModel(arch.build_spec(config), ctx)
    if hasattr(ops, "prepare"):
        ops.prepare(model.kernel_groups())
    load_into(model, source)
    return model


def load_model(model_dir: str | Path, *, dtype: str = "bfloat16", device="cuda", ops=None,
               pin_path: str | Path | None = None):
    """``(model, typed config, raw config.json)`` from a folder with config.json and safetensors.
    ``pin_path``: a config.json that the folder's model has to match (checked before any weight
    is read)."""
    _arch, config = load_config(model_dir, pin_path)
    model = build_model(config, SafetensorsDir(model_dir), dtype=dtype, device=device, ops=ops)
    return model, config, read_config_json(model_dir)


@dataclass
class Runtime:
    """Model, cache and step function wired together (what the engine and trace replay share)."""

    model: DecoderModel
    cache: CacheManager
    storage: CacheStorage
    runner: ModelRunner
    max_positions: int


UNLIMITED_POSITIONS = 1 << 30  # a model none of whose parts limits the positions


def build_runtime(model: DecoderModel, *, max_positions: int | None = None, block_size: int,
                  num_kv_blocks: int | list[int] | None, max_num_seqs: int, cuda_graph: bool = False,
                  kv_budget: int | None = None, kv_memory_fraction: float = 0.85,
                  max_num_batched_tokens: int | None = None) -> Runtime:
    """Cache and step function for a loaded model.  ``max_positions`` defaults to what the
    model's own parts can serve (the shortest position table among them).  ``num_kv_blocks``:
    pages of every paged group, one count per paged group, or None to size the pools from
    ``kv_budget`` bytes (default: ``kv_memory_fraction`` of the free device memory)."""
    if max_positions is None:
        max_positions = model.position_limit() or UNLIMITED_POSITIONS
    layout = model.cache_layout()
    ctx = model.ctx
    dtype_bytes = torch.empty((), dtype=ctx.dtype).element_size()
    if num_kv_blocks is None:
        if kv_budget is None:
            if ctx.device.type != "cuda":
                kv_budget = 256 * 1024 * 1024
            else:
                free, _total = torch.cuda.mem_get_info(ctx.device)
                kv_budget = int(free * kv_memory_fraction)
        elif kv_budget <= 0:
            raise ValueError(f"kv_budget must be positive, got {kv_budget!r}")
        counts = layout.pages_for_budget(kv_budget, block_size, dtype_bytes, max_num_seqs=max_num_seqs,
                                         max_step_tokens=max_num_batched_tokens)
        num_kv_blocks = [max(32, n) for n in counts]
    cache = CacheManager(layout.group_specs, block_size, num_kv_blocks, max_num_seqs)
    storage = CacheStorage(layout, block_size, num_kv_blocks, max_num_seqs, ctx.dtype, ctx.device)
    runner = ModelRunner(model, cache, storage, max_positions=max_positions, cuda_graph=cuda_graph)
    return Runtime(model, cache, storage, runner, max_positions)


def eos_from_config(raw: dict) -> int | None:
    """First element when ``eos_token_id`` is a list (qwen3_runtime/engine/factory.py:64-72)."""
    eos = raw.get("eos_token_id")
    if isinstance(eos, list):
        eos = eos[0] if eos else None
    return int(eos) if eos is not None else None


def build_engine(model_dir: str | Path | None = None, *, max_num_seqs: int = 8, max_num_batched_tokens: int = 2048,
                 block_size: int = 16, dtype: str = "bfloat16", num_kv_blocks: int | None = None,
                 kv_budget: int | None = None, cuda_graph: bool | None = None, eos_token_id: int | None = None,
                 device="cuda", ops=None, model: DecoderModel | None = None, config=None,
                 max_positions: int | None = None, pin_path: str | Path | None = None,
                 run_ahead: bool = True, kv_memory_fraction: float = 0.85) -> Engine:
    """An :class:`Engine` for a model folder (or an already built ``model``; its ``config`` is
    kept on the engine for the caller's reference only)."""
    dtype = canonical_dtype(dtype)
    raw: dict = {}
    if model is None:
        if model_dir is None:
            raise ValueError("give a model folder or a built model")
        model, config, raw = load_model(model_dir, dtype=dtype, device=device, ops=ops, pin_path=pin_path)
    if cuda_graph is None:
        cuda_graph = model.ctx.device.type == "cuda"
    if eos_token_id is None:
        eos_token_id = eos_from_config(raw)
    rt = build_runtime(model, max_positions=max_positions, block_size=block_size, num_kv_blocks=num_kv_blocks,
                       max_num_seqs=max_num_seqs, cuda_graph=cuda_graph, kv_budget=kv_budget,
                       kv_memory_fraction=kv_memory_fraction, max_num_batched_tokens=max_num_batched_tokens)
    cfg = EngineConfig(block_size=block_size, num_kv_blocks=min(rt.cache.num_pages) if rt.cache.num_pages else None,
                       max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens,
                       eos_token_id=eos_token_id, cuda_graph=bool(cuda_graph), dtype=dtype, run_ahead=bool(run_ahead),
                       kv_memory_fraction=kv_memory_fraction)
    engine = Engine(cfg, rt.runner, rt.cache, Sampler(model.ops, model.ctx.device))
    engine.runtime = rt
    engine.model_config = config
    return engine
