"""Public facade: ``LLM(...).generate(prompts, sampling, max_tokens)``.

Parity: qwen3_runtime/llm.py:87-165 -- a model folder, or ``model=None`` for a tiny
random model that needs no files; prompts as token ids (one list, or a list of
lists), or text when a tokenizer is given.  Lists of prompts run together as one
continuous batch here (the reference runs them one after another, :156-157); each
request's result does not depend on that.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Sequence

from .config.model_config import Qwen3Config
from .engine.factory import build_engine, build_model
from .sampling.params import SamplingParams
from .weights.loader import DictSource
from .weights.random_init import random_state


def tiny_config() -> Qwen3Config:
    """The sizes of the reference's built-in tiny model (qwen3_runtime/llm.py:168-181), with a
    head size the attention kernels accept."""
    return Qwen3Config(vocab_size=32, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                       num_key_value_heads=1, head_dim=16, intermediate_size=64, rms_norm_eps=1e-6,
                       rope_theta=10000.0, max_position_embeddings=128, tie_word_embeddings=True)


class LLM:
    def __init__(self, model: str | Path | None = None, *, tokenizer: Any = None, config: Qwen3Config | None = None,
                 max_num_seqs: int = 4, max_num_batched_tokens: int = 256, seed: int = 0, dtype: str = "bfloat16",
                 **factory_kwargs):
        self.tokenizer = tokenizer
        if model is None:
            config = config or tiny_config()
            built = build_model(config, DictSource(random_state(config, seed, std=0.2)), dtype=dtype,
                                device=factory_kwargs.get("device", "cuda"), ops=factory_kwargs.get("ops"))
            factory_kwargs.setdefault("block_size", 4)
            factory_kwargs.setdefault("num_kv_blocks", 64)
            self.engine = build_engine(model=built, config=config, max_num_seqs=max_num_seqs,
                                       max_num_batched_tokens=max_num_batched_tokens, dtype=dtype, **factory_kwargs)
        else:
            self.engine = build_engine(model, max_num_seqs=max_num_seqs,
                                       max_num_batched_tokens=max_num_batched_tokens, dtype=dtype, **factory_kwargs)

    def encode(self, prompt) -> list[int]:
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return [int(x) for x in prompt]
        if self.tokenizer is None:
            raise TypeError("text prompts need a tokenizer; pass token ids or LLM(tokenizer=...)")
        if isinstance(prompt, str):
            ids = self.tokenizer.encode(prompt)
        else:
            ids = self.tokenizer.apply_chat_template(prompt, add_generation_prompt=True, tokenize=True)
        if hasattr(ids, "tolist"):
            ids = ids.tolist()
        return [int(x) for x in ids]

    def decode(self, tokens: Sequence[int]) -> str:
        if self.tokenizer is None:
            return " ".join(str(t) for t in tokens)
        return self.tokenizer.decode(list(tokens), skip_special_tokens=True)

    def generate(self, prompts, sampling: SamplingParams | None = None, max_tokens: int = 16):
        """Token ids in, token ids out; text in, text out.  A list of prompts gives a list."""
        sampling = sampling or SamplingParams()
        if isinstance(prompts, list) and prompts and isinstance(prompts[0], list):
            return self.engine.generate_batch([self.encode(p) for p in prompts], max_tokens=max_tokens,
                                              sampling=sampling)
        if isinstance(prompts, list) and prompts and isinstance(prompts[0], int):
            return self.engine.generate(prompts, max_tokens=max_tokens, sampling=sampling)
        ids = self.encode(prompts)
        return self.decode(self.engine.generate(ids, max_tokens=max_tokens, sampling=sampling))
