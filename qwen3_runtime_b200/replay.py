"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
model, cache manager, step function and kernels that generation uses.

  bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line::

  {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch.  For a step in which something is wanted,
``<out>/<step>.f32`` holds the logits at the wanted places, in the order of the entries
and of ``want``, as little-endian float32 ``[wanted, vocab]``.  After every step a line
``done <step>`` is printed and flushed.  ``--max-tokens`` sizes the page pool: the most
tokens live requests hold at any time, each request's count rounded up to a multiple
of 64, so pages are handed out again as requests end.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run")
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, help="bfloat16 or float32")
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (must divide 64)")
    parser.add_argument("--max-live", type=int, default=8, help="state slots: most requests live at a time")
    parser.add_argument("--cuda-graph", action=argparse.BooleanOptionalAction, default=None,
                        help="replay captured graphs for decode-only steps (default: as serving does)")
    args = parser.parse_args(argv)
    if 64 % args.page_size:
        raise SystemExit("--page-size must divide 64")

    import numpy as np
    import torch

    from .config.engine_config import canonical_dtype
    from .engine.batch import StepEntry
    from .engine.factory import build_runtime, load_model

    dtype = canonical_dtype(args.dtype)
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    print(f"[trace_run] loading {args.model} ({dtype})", file=sys.stderr, flush=True)
    model, config, _raw = load_model(args.model, dtype=dtype)
    num_pages = max(1, -(-args.max_tokens // args.page_size))
    cuda_graph = (dtype == "bfloat16") if args.cuda_graph is None else args.cuda_graph
    rt = build_runtime(model, block_size=args.page_size,
                       num_kv_blocks=num_pages, max_num_seqs=args.max_live, cuda_graph=cuda_graph)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            rid = item["id"]
            rc = live.get(rid)
            if rc is None:
                rc = live[rid] = rt.cache.open(rid)
            tokens = [int(t) for t in item["tokens"]]
            rt.cache.reserve(rc, len(tokens))
            entries.append(StepEntry(rc, tokens, [int(w) for w in item.get("want", [])]))
        if entries:
            logits = rt.runner.run(entries)
            if logits is not None:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                if hasattr(model.ops, "raise_if_kernel_error"):
                    model.ops.raise_if_kernel_error()
                np.ascontiguousarray(arr).tofile(out_dir / f"{step}.f32")
        for rid in record.get("end", []):
            rc = live.pop(rid, None)
            if rc is not None:
                rt.cache.close(rc)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
