"""Command line in the manner of the reference's ``python -m qwen3_runtime.reference.cli``
(qwen3_runtime/reference/cli.py:17-76): token ids in, generated ids out, with the
engine's sizes printed.

  QWEN3_RUNTIME_MODEL=/path/to/model python -m qwen3_runtime_b200.cli --max-tokens 8

``--model``, ``--max-tokens``, ``--prompt-tokens`` and ``--cuda-graph/--no-cuda-graph``
keep the reference's names and meanings.  ``--backend`` and ``--enable-prefix-cache``
are not taken: this engine has one set of kernels and no prefix cache.  The
comparison with Hugging Face that the reference runs afterwards is not part of this
engine.  ``python -m qwen3_runtime_b200.cli random --config C.json --seed S --out DIR``
writes a random model folder.
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def _generate(argv: list[str]) -> int:
    parser = argparse.ArgumentParser(prog="qwen3_runtime_b200.cli")
    parser.add_argument("--model", default=os.environ.get("QWEN3_RUNTIME_MODEL"))
    parser.add_argument("--pin-path", default=None,
                        help="a config.json that the model folder has to match (refuse any other model)")
    parser.add_argument("--max-tokens", type=int, default=8)
    parser.add_argument("--prompt-tokens", type=int, nargs="+", default=[151643, 8948, 198, 2610])
    parser.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=None,
                        help="Decode-only CUDA Graph. Default: on.")
    parser.add_argument("--run-ahead", action=argparse.BooleanOptionalAction, default=True,
                        help="put the next decode step on the device before reading this one's tokens")
    parser.add_argument("--dtype", default="bfloat16", help="bfloat16 (serving) or float32 (true 32-bit path)")
    parser.add_argument("--temperature", type=float, default=0.0, help="<= 0: greedy")
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--min-p", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=None, help="sampling seed")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-kv-blocks", type=int, default=None)
    parser.add_argument("--max-num-seqs", type=int, default=1)
    parser.add_argument("--max-num-batched-tokens", type=int, default=2048)
    args = parser.parse_args(argv)
    if not args.model:
        raise SystemExit("set --model or QWEN3_RUNTIME_MODEL")
    from .engine.factory import build_engine
    from .sampling.params import SamplingParams

    engine = build_engine(args.model, max_num_seqs=args.max_num_seqs,
                          max_num_batched_tokens=args.max_num_batched_tokens, block_size=args.block_size,
                          dtype=args.dtype, num_kv_blocks=args.num_kv_blocks, cuda_graph=args.cuda_graph,
                          pin_path=args.pin_path, run_ahead=args.run_ahead)
    sampling = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                              seed=args.seed)
    out = engine.generate(args.prompt_tokens, max_tokens=args.max_tokens, sampling=sampling)
    rt = engine.runtime
    dtype_bytes = 4 if engine.config.dtype == "float32" else 2
    print("runtime", out)
    print("bytes_per_block", sum(rt.model.cache_layout().page_bytes(args.block_size, dtype_bytes)))
    print("device", rt.model.ctx.device)
    print("dtype", engine.config.dtype)
    print("num_kv_blocks", rt.cache.num_pages)
    print("cuda_graph", engine.config.cuda_graph)
    return 0


def _random(argv: list[str]) -> int:
    parser = argparse.ArgumentParser(prog="qwen3_runtime_b200.cli random")
    parser.add_argument("--config", required=True, help="a config.json (architecture keys)")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--out", required=True)
    parser.add_argument("--std", type=float, default=0.02)
    parser.add_argument("--vector-std", type=float, default=0.02)
    parser.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = parser.parse_args(argv)
    from .config.registry import resolve_architecture
    from .weights.random_init import write_random_model

    raw = json.loads(open(args.config).read())
    config = resolve_architecture(raw).config_class.from_hf_config(raw)
    path = write_random_model(config, args.out, args.seed, std=args.std, vector_std=args.vector_std,
                              store_dtype=args.store_dtype)
    print("wrote", path)
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "random":
        return _random(argv[1:])
    if argv and argv[0] == "generate":
        argv = argv[1:]
    return _generate(argv)


if __name__ == "__main__":
    raise SystemExit(main())
