"""The decode-attention entry point for callers that may not allocate device memory
(csrc/no_alloc.h): called through its exported C symbol, compared with the ordinary entry
point, twice in a row (the fixed scratch array keeps the first call's contents when the second
one starts).  This file sorts last so that a run that stops at the first failure has already
run every other test; it also passes alone in a fresh process."""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 2 * 1024 * 1024
ERR_SCRATCH_TOO_SMALL = 4


@pytest.fixture(scope="module")
def lib():
    from qwen3_runtime_b200.ops import build

    handle = build.load_group("attention_decode")
    fn = handle.q3_paged_attention_decode_no_alloc
    fn.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    fn.restype = c_int
    handle.q3_no_alloc_last_error.restype = ctypes.c_char_p
    return handle


def problem(nq, nkv, D, ps, lens, seed):
    """A paged cache with random keys and values, one query token per sequence."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    maxp = max(-(-n // ps) for n in lens) + 1
    pages = B * maxp + 2
    bt = torch.randperm(pages, generator=g)[: B * maxp].int().view(B, maxp).contiguous().cuda()
    k = torch.randn((pages, nkv, ps, D), generator=g).bfloat16().cuda()
    v = torch.randn((pages, nkv, ps, D), generator=g).bfloat16().cuda()
    q = torch.randn((B, (nq + 2 * nkv) * D), generator=g).bfloat16().cuda()
    kv_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    cu = torch.arange(B + 1, dtype=torch.int32).cuda()
    return q, k, v, bt, kv_lens, cu


def call_no_alloc(lib, q, k, v, bt, kv_lens, cu, nq, nkv, D, ps, splits, window=0, seq_list=None):
    out = torch.zeros((q.shape[0], nq * D), dtype=torch.bfloat16, device="cuda")
    n = q.shape[0] if seq_list is None else seq_list.numel()
    code = lib.q3_paged_attention_decode_no_alloc(
        q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), bt.data_ptr(), bt.shape[1], kv_lens.data_ptr(),
        cu.data_ptr(), None if seq_list is None else seq_list.data_ptr(), out.data_ptr(), n, nq, nkv, D, ps,
        1 / math.sqrt(D), window, splits, torch.cuda.current_stream().cuda_stream)
    return code, out


def call_ordinary(q, k, v, bt, kv_lens, cu, nq, nkv, D, ps, splits, window=0, seq_list=None):
    from qwen3_runtime_b200.ops.cuda import CudaOps

    out = torch.zeros((q.shape[0], nq * D), dtype=torch.bfloat16, device="cuda")
    n = q.shape[0] if seq_list is None else seq_list.numel()
    CudaOps().paged_attention_decode(q, q.stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=k, v_pages=v,
                                     block_table=bt, kv_lens=kv_lens, cu_seqlens=cu, out=out, page_size=ps,
                                     scale=1 / math.sqrt(D), window=window or None, num_seqs=n,
                                     max_kv_len=int(kv_lens.max()), num_splits=splits, seq_list=seq_list)
    return out


def plain_statement(q, k, v, bt, kv_lens, nq, nkv, D, ps, window=0):
    """The same attention stated in plain torch (tests/emulated_ops.py): an oracle that shares no
    code with either entry point."""
    from emulated_ops import TorchOps

    B = q.shape[0]
    out = torch.zeros((B, nq * D), dtype=torch.bfloat16, device="cuda")
    TorchOps().paged_attention(q, q.stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=k, v_pages=v,
                               block_table=bt, token_seq=torch.arange(B, dtype=torch.int32, device="cuda"),
                               positions=(kv_lens - 1).int(), out=out, page_size=ps, scale=1 / math.sqrt(D),
                               window=window or None)
    return out


# sizes, lengths, slices, window, whether only a subset of the sequences is asked for
CASES = [
    (32, 8, 128, 16, [700, 64, 1000, 129, 333], 6, 0, False),
    (32, 8, 128, 16, [65, 300, 2], 3, 0, False),       # fewer, shorter: finds the first call's partials in the array
    (32, 8, 128, 16, [700, 64, 1000, 129, 333], 4, 100, False),   # a window
    (8, 8, 64, 8, [90, 17, 260, 5], 1, 0, False),      # head size 64, one slice: no scratch, nothing to merge
    (6, 2, 256, 16, [700, 64, 1000, 129, 333], 5, 0, True),       # a subset of the sequences (seq_list)
]


def test_no_alloc_entry_point_matches_the_ordinary_one_and_the_plain_statement(lib):
    # the calls follow one another on one stream: each finds the last one's partial results in
    # the shared scratch array
    for nq, nkv, D, ps, lens, splits, window, subset in CASES:
        args = problem(nq, nkv, D, ps, lens, len(lens) * splits)
        seq_list = torch.tensor([3, 0, 2], dtype=torch.int32).cuda() if subset else None
        for _ in range(2):  # twice in a row on the same problem, too
            code, got = call_no_alloc(lib, *args, nq, nkv, D, ps, splits, window, seq_list)
            assert code == 0, lib.q3_no_alloc_last_error().decode()
        want = call_ordinary(*args, nq, nkv, D, ps, splits, window, seq_list)
        plain = plain_statement(*args[:5], nq, nkv, D, ps, window)
        torch.cuda.synchronize()
        rows = seq_list.long() if subset else torch.arange(len(lens)).cuda()
        scale = max(1.0, float(plain.float().abs().max()))
        what = (nq, nkv, D, ps, splits, window, subset)
        assert float((got[rows].float() - plain[rows].float()).abs().max()) <= 1e-2 * scale, what
        assert torch.equal(got, want), f"{what}: same kernels, same slices: the two entry points agree bit for bit"
        if subset:
            assert float(got[1].float().abs().max()) == 0.0, "a sequence that was not asked for is not written"


def test_no_alloc_entry_point_refuses_what_does_not_fit(lib):
    nq, nkv, D, ps = 32, 8, 128, 16
    lens = [40] * 64
    args = problem(nq, nkv, D, ps, lens, 3)
    splits = SCRATCH_FLOATS // (64 * nq * (D + 1)) + 1
    code, out = call_no_alloc(lib, *args, nq, nkv, D, ps, splits)
    assert code == ERR_SCRATCH_TOO_SMALL
    msg = lib.q3_no_alloc_last_error().decode()
    assert "64 sequences x 32 heads" in msg and str(SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0, "nothing was launched"
    code, _ = call_no_alloc(lib, *args, nq, nkv, D, ps, splits - 1)
    assert code == 0 and lib.q3_no_alloc_last_error() == b""
    # sizes that make no sense are refused by this entry point itself, with a sentence
    for bad in (dict(nkv=0), dict(nkv=5), dict(ps=0), dict(window=-1)):
        kw = {"nkv": nkv, "ps": ps, "window": 0, **bad}
        code, out = call_no_alloc(lib, *args, nq, kw["nkv"], D, kw["ps"], 2, kw["window"])
        assert code != 0 and b"bad sizes" in lib.q3_no_alloc_last_error(), bad
