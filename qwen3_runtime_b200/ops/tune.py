"""Measurements behind the constants of the kernel table's cost models.

    python -m qwen3_runtime_b200.ops.tune decode_splits [--out FILE] [--quick]
    python -m qwen3_runtime_b200.ops.tune decode_mixed

``decode_splits`` times the split-KV decode attention kernel alone (finished queries, the merge
by the last block) for 1..128 sequences x 256..16384 keys x every slice count, each case replayed
from a CUDA graph over key/value pools that together exceed the L2, and prints for each (sequences,
keys) the time with the slice count that :meth:`CudaOps.decode_splits` picks, the best time and
the regret.  The last line is the mean and the worst regret over the table; the JSON lines
written with ``--out`` hold every measured time, for fitting the model's constants again on
another device.  ``decode_mixed`` does the same for a few batches of mixed lengths (the kernel cuts a
shorter sequence into fewer slices; :meth:`CudaOps.decode_slices_for` picks the count).
"""

from __future__ import annotations

import argparse
import json
import math
import sys


def _time_graph(torch, launch, sets: int) -> float:
    """Microseconds per launch: ``sets`` launches over different pools captured once, replayed three times."""
    for i in range(2):
        launch(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(sets):
            launch(i)
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(3):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / (3 * sets) * 1e3


def decode_splits(out_path: str | None, quick: bool, num_heads=32, num_kv_heads=8, head_dim=128, page_size=16) -> int:
    import torch

    from .cuda import CudaOps

    ops = CudaOps()
    batches = (1, 8, 32, 64) if quick else (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128)
    lengths = (512, 1024, 4096) if quick else (256, 512, 768, 1024, 1536, 2048, 3072, 4096, 8192, 16384)
    candidates = (1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16, 20, 24, 32, 48, 64)
    out = open(out_path, "w") if out_path else None
    regrets = []
    for B in batches:
        for L in lengths:
            pool_bytes = B * L * num_kv_heads * head_dim * 2 * 2
            if pool_bytes > 2.2e9:
                continue
            pages_per_seq = L // page_size + 1
            pages = B * pages_per_seq + 2
            sets = min(8, max(2, int(300e6 // pool_bytes) + 1))
            gen = torch.Generator().manual_seed(0)
            table = torch.randperm(pages - 1, generator=gen)[: B * pages_per_seq].int().view(B, pages_per_seq).cuda()
            pools = [(torch.randn(pages, num_kv_heads, page_size, head_dim, device="cuda").bfloat16(),
                      torch.randn(pages, num_kv_heads, page_size, head_dim, device="cuda").bfloat16())
                     for _ in range(sets)]
            q = torch.randn(B, (num_heads + 2 * num_kv_heads) * head_dim, device="cuda").bfloat16()
            kv_lens = torch.full((B,), L, dtype=torch.int32, device="cuda")
            cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
            result = torch.empty(B, num_heads * head_dim, dtype=torch.bfloat16, device="cuda")
            picked = ops.decode_splits(B, num_kv_heads, L, head_dim)
            times = {}
            for s in sorted(set(candidates) | {picked}):
                if (s > 1 and L // s < 64) or B * num_kv_heads * s > 20000:
                    continue

                def launch(i, s=s):
                    k, v = pools[i % sets]
                    ops.paged_attention_decode(q, q.stride(0), num_heads=num_heads, num_kv_heads=num_kv_heads,
                                               head_dim=head_dim, k_pages=k, v_pages=v, block_table=table,
                                               kv_lens=kv_lens, cu_seqlens=cu, out=result, page_size=page_size,
                                               scale=1 / math.sqrt(head_dim), window=None, num_seqs=B, max_kv_len=L,
                                               num_splits=s)

                times[s] = round(_time_graph(torch, launch, sets), 2)
            best = min(times, key=times.get)
            regret = times[picked] / times[best] - 1
            regrets.append(regret)
            tbs = pool_bytes / times[picked] / 1e6
            print(f"sequences {B:3d} keys {L:5d}: picked {picked:2d} slices {times[picked]:7.2f} us "
                  f"({tbs:4.2f} TB/s), best {best:2d} slices {times[best]:7.2f} us, regret {regret:+.1%}", flush=True)
            if out:
                out.write(json.dumps(dict(sequences=B, keys=L, kv_heads=num_kv_heads, head_dim=head_dim,
                                          picked=picked, best=best, us=times)) + "\n")
                out.flush()
            del pools
            torch.cuda.empty_cache()
    ops.raise_if_kernel_error()
    print(f"regret of the picked slice counts: mean {sum(regrets) / len(regrets):.2%}, worst {max(regrets):.1%} "
          f"over {len(regrets)} cases")
    return 0


def decode_mixed(num_heads=32, num_kv_heads=8, head_dim=128, page_size=16) -> int:
    import random

    import torch

    from .cuda import CudaOps

    ops = CudaOps()
    rnd = random.Random(1)
    batches = [
        ("48 sequences of 192..4224 keys", [rnd.randint(64, 4096) + 128 for _ in range(48)]),
        ("16 sequences of 192..4224 keys", [rnd.randint(64, 4096) + 128 for _ in range(16)]),
        ("8 sequences of 192..4224 keys", [rnd.randint(64, 4096) + 128 for _ in range(8)]),
        ("64 sequences of 64..2048 keys", [rnd.randint(64, 2048) for _ in range(64)]),
        ("one of 4096 keys among 47 of 200", [4096] + [200] * 47),
        ("8 sequences of 4100 keys", [4100] * 8),
        ("64 sequences of 800 keys", [800] * 64),
    ]
    for label, lens in batches:
        B, L = len(lens), max(lens)
        pages_per_seq = L // page_size + 1
        pages = B * pages_per_seq + 2
        nbytes = sum(lens) * num_kv_heads * head_dim * 2 * 2
        sets = min(8, max(3, int(400e6 // (pages * num_kv_heads * page_size * head_dim * 4)) + 1))
        gen = torch.Generator().manual_seed(0)
        table = torch.randperm(pages - 1, generator=gen)[: B * pages_per_seq].int().view(B, pages_per_seq).cuda()
        pools = [(torch.randn(pages, num_kv_heads, page_size, head_dim, device="cuda").bfloat16(),
                  torch.randn(pages, num_kv_heads, page_size, head_dim, device="cuda").bfloat16())
                 for _ in range(sets)]
        q = torch.randn(B, (num_heads + 2 * num_kv_heads) * head_dim, device="cuda").bfloat16()
        kv_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
        cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        result = torch.empty(B, num_heads * head_dim, dtype=torch.bfloat16, device="cuda")
        picked = ops.decode_slices_for(lens, num_kv_heads, head_dim, None)
        times = {}
        for s in sorted({1, 2, 3, 4, 5, 6, 8, 12, 16, picked}):
            if s > 1 and L // s < 64:
                continue

            def launch(i, s=s):
                k, v = pools[i % sets]
                ops.paged_attention_decode(q, q.stride(0), num_heads=num_heads, num_kv_heads=num_kv_heads,
                                           head_dim=head_dim, k_pages=k, v_pages=v, block_table=table,
                                           kv_lens=kv_lens, cu_seqlens=cu, out=result, page_size=page_size,
                                           scale=1 / math.sqrt(head_dim), window=None, num_seqs=B, max_kv_len=L,
                                           num_splits=s)

            times[s] = round(_time_graph(torch, launch, sets), 1)
        best = min(times, key=times.get)
        print(f"{label}: picked {picked} slices {times[picked]} us ({nbytes / times[picked] / 1e6:.2f} TB/s), "
              f"best {best} slices {times[best]} us; all: {times}", flush=True)
        del pools
        torch.cuda.empty_cache()
    ops.raise_if_kernel_error()
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("what", choices=["decode_splits", "decode_mixed"])
    parser.add_argument("--out", default=None, help="write every measured time as JSON lines")
    parser.add_argument("--quick", action="store_true", help="a few sizes only")
    args = parser.parse_args(argv)
    if args.what == "decode_mixed":
        return decode_mixed()
    return decode_splits(args.out, args.quick)


if __name__ == "__main__":
    sys.exit(main())
