"""Produce tests/golden/*.safetensors from the reference's own model code, on the CPU.

Run once, where yuzheng310/qwen3-runtime is checked out (its tree is only read):

    PYTHONPATH=<qwen3-runtime checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py

For the tiny configurations A and B it builds the seeded random model of
tests/helpers.py, loads those tensors into the reference's ``Qwen3ForCausalLM``
through its own ``load_hf_state_dict`` (qwen3_runtime/utils/loader.py:33-54), and
stores (a) float32 logits of whole prompts from one packed forward
(qwen3_runtime/models/qwen3.py:222-266), (b) greedy token ids from the reference's
paged engine with chunked prefill (qwen3_runtime/engine/engine.py:359-366) and (c) the
logits of the same forward with the model converted to bfloat16 (``model.to(bfloat16)``:
bfloat16 weights, activations and residual stream, layers/ops.py:17-49), as float32.
tests/test_plain_model.py compares the plain implementation with these files.
"""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import torch
from safetensors.torch import save_file

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from helpers import TINY, make_model_dir, random_ids  # noqa: E402
from plain_model import read_model_dir  # noqa: E402

from qwen3_runtime.config import Config  # noqa: E402  (the reference)
from qwen3_runtime.engine.engine import Engine  # noqa: E402
from qwen3_runtime.engine.model_runner import PagedRunner  # noqa: E402
from qwen3_runtime.models.qwen3 import Qwen3ForCausalLM, Qwen3ModelConfig  # noqa: E402
from qwen3_runtime.utils.loader import load_hf_state_dict  # noqa: E402

PROMPTS = {"A": [7, 19], "B": [5, 13, 30]}


def main() -> None:
    tmp = Path(tempfile.mkdtemp())
    for name, lens in PROMPTS.items():
        folder = make_model_dir(tmp, name)
        raw, tensors = read_model_dir(folder)
        cfg = Qwen3ModelConfig.from_hf_config(raw)
        model = Qwen3ForCausalLM(cfg).eval()
        load_hf_state_dict(model, {k: v.float() for k, v in tensors.items()})
        out = {}
        with torch.no_grad():
            for i, n in enumerate(lens):
                ids = random_ids(cfg.vocab_size, n, seed=100 + i)
                logits = model(torch.tensor(ids), torch.arange(n), cu_seqlens=[0, n])
                out[f"prompt{i}.ids"] = torch.tensor(ids, dtype=torch.int32)
                out[f"prompt{i}.logits"] = logits.float().contiguous()
                engine = Engine(Config(block_size=TINY[name]["page_size"], num_kv_blocks=64, max_num_seqs=4,
                                       max_num_batched_tokens=6), PagedRunner(model))
                out[f"prompt{i}.greedy"] = torch.tensor(engine.generate(ids, max_tokens=8), dtype=torch.int32)
            low = Qwen3ForCausalLM(cfg).eval()
            load_hf_state_dict(low, {k: v.float() for k, v in tensors.items()})
            low = low.to(torch.bfloat16)
            for i, n in enumerate(lens):
                ids = out[f"prompt{i}.ids"].tolist()
                logits = low(torch.tensor(ids), torch.arange(n), cu_seqlens=[0, n])
                out[f"prompt{i}.logits_bf16"] = logits.float().contiguous()
        save_file(out, str(HERE / f"tiny_{name}.safetensors"))
        print(name, {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
