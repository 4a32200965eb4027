"""The Python entry point: ``LLM(...).generate(prompts, sampling, max_tokens)``.

The call and its meanings follow qwen3_runtime/llm.py:87-165: a model folder, or
``model=None`` for a small random model that needs no files; a prompt is a list of
token ids, a string or a chat (both need a tokenizer), or a list of those.  What
differs: a list of prompts is served as one continuous batch (the reference runs them
one after another, :156-157; a request's tokens do not depend on its neighbours), and
text without a tokenizer is refused instead of being mapped character by character.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Sequence

from .config.registry import default_architecture, resolve_architecture
from .engine.factory import build_engine, build_model
from .sampling.params import SamplingParams
from .weights.loader import DictSource
from .weights.random_init import random_state


def _is_token_list(x) -> bool:
    return isinstance(x, (list, tuple)) and len(x) > 0 and all(isinstance(t, int) for t in x)


class LLM:
    def __init__(self, model: str | Path | None = None, *, tokenizer: Any = None, config: Any = None,
                 architecture: str | None = None, max_num_seqs: int = 4, max_num_batched_tokens: int = 256,
                 seed: int = 0, dtype: str = "bfloat16", **factory_kwargs):
        """``model=None``: random weights (``seed``) for ``config``, or for the tiny configuration
        that the registered ``architecture`` (default: the first registered) offers."""
        self.tokenizer = tokenizer
        common = dict(max_num_seqs=max_num_seqs, max_num_batched_tokens=max_num_batched_tokens, dtype=dtype)
        if model is not None:
            self.engine = build_engine(model, **common, **factory_kwargs)
            return
        if config is None:
            arch = (resolve_architecture({"architectures": [architecture]}) if architecture
                    else default_architecture())
            if arch.tiny_config is None:
                raise ValueError(f"architecture {arch.name!r} offers no tiny configuration; pass config=")
            config = arch.tiny_config()
        weights = DictSource(random_state(config, seed, std=0.2))
        built = build_model(config, weights, dtype=dtype, device=factory_kwargs.get("device", "cuda"),
                            ops=factory_kwargs.get("ops"))
        factory_kwargs.setdefault("block_size", 4)
        factory_kwargs.setdefault("num_kv_blocks", 64)
        self.engine = build_engine(model=built, config=config, **common, **factory_kwargs)

    # ---- text <-> ids (only with a tokenizer) ---------------------------------------------
    def encode(self, prompt) -> list[int]:
        if _is_token_list(prompt):
            return list(prompt)
        if self.tokenizer is None:
            raise TypeError("text prompts need a tokenizer; pass token ids or LLM(tokenizer=...)")
        if isinstance(prompt, str):
            ids = self.tokenizer.encode(prompt)
        else:  # a chat: a list of {"role", "content"} messages
            ids = self.tokenizer.apply_chat_template(prompt, add_generation_prompt=True, tokenize=True)
        return [int(t) for t in (ids.tolist() if hasattr(ids, "tolist") else ids)]

    def decode(self, tokens: Sequence[int]) -> str:
        if self.tokenizer is None:
            return " ".join(map(str, tokens))
        return self.tokenizer.decode(list(tokens), skip_special_tokens=True)

    # ---- generation -----------------------------------------------------------------------------
    def generate(self, prompts, sampling: SamplingParams | None = None, max_tokens: int = 16):
        """One prompt gives one result, a list of prompts a list of results, in order.  Token ids
        in give token ids out; text (or a chat) in gives text out."""
        sampling = sampling if sampling is not None else SamplingParams()
        many = isinstance(prompts, (list, tuple)) and len(prompts) > 0 and not _is_token_list(prompts) \
            and not isinstance(prompts[0], dict)
        items = list(prompts) if many else [prompts]
        as_ids = [_is_token_list(p) for p in items]
        outputs = self.engine.generate_batch([self.encode(p) for p in items], max_tokens=max_tokens,
                                             sampling=sampling)
        results = [out if ids else self.decode(out) for out, ids in zip(outputs, as_ids)]
        return results if many else results[0]
