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


def call_no_alloc(lib, q, k, v, bt, kv_lens, cu, nq, nkv, D, ps, splits, window=0):
    out = torch.zeros((q.shape[0], nq * D), dtype=torch.bfloat16, device="cuda")
    code = lib.q3_paged_attention_decode_no_alloc(
        q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), bt.data_ptr(), bt.shape[1], kv_lens.data_ptr(),
        cu.data_ptr(), None, out.data_ptr(), q.shape[0], nq, nkv, D, ps, 1 / math.sqrt(D), window, splits,
        torch.cuda.current_stream().cuda_stream)
    return code, out


def call_ordinary(q, k, v, bt, kv_lens, cu, nq, nkv, D, ps, splits, window=0):
    from qwen3_runtime_b200.ops.cuda import CudaOps

    out = torch.zeros((q.shape[0], nq * D), dtype=torch.bfloat16, device="cuda")
    CudaOps().paged_attention_decode(q, q.stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=k, v_pages=v,
                                     block_table=bt, kv_lens=kv_lens, cu_seqlens=cu, out=out, page_size=ps,
                                     scale=1 / math.sqrt(D), window=window or None, num_seqs=q.shape[0],
                                     max_kv_len=int(kv_lens.max()), num_splits=splits)
    return out


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(lib):
    nq, nkv, D, ps = 32, 8, 128, 16
    # two different problems back to back: the second call finds the first one's partial results
    # in the shared scratch array (more slices, longer sequences first; then fewer and shorter)
    for lens, splits, seed in (([700, 64, 1000, 129, 333], 6, 1), ([65, 300, 2], 3, 2)):
        args = problem(nq, nkv, D, ps, lens, seed)
        code, got = call_no_alloc(lib, *args, nq, nkv, D, ps, splits)
        assert code == 0, lib.q3_no_alloc_last_error().decode()
        want = call_ordinary(*args, nq, nkv, D, ps, splits)
        torch.cuda.synchronize()
        scale = max(1.0, float(want.float().abs().max()))
        assert float((got.float() - want.float()).abs().max()) <= 1e-2 * scale
        assert torch.equal(got, want), "same kernels, same slices: the two entry points agree bit for bit"


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
