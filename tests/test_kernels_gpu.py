"""Each CUDA kernel alone against its plain torch statement (tests/emulated_ops.py), at sizes
other than the tiny models': real Qwen3 layer sizes and awkward ones (widths and vocabularies
that are no power of two, odd page sizes, head sizes in steps of 16, uneven head groups)."""

import math

import pytest
import torch

from emulated_ops import TorchOps

pytestmark = pytest.mark.gpu

REF = TorchOps()
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


def close(got, want, dtype, what, f32_tol=2e-5, bf16_tol=2e-2):
    tol = f32_tol if dtype == torch.float32 else bf16_tol
    scale = max(1.0, float(want.float().abs().max()))
    diff = float((got.float() - want.float()).abs().max())
    assert diff <= tol * scale, f"{what}: max |diff| {diff:.3g} > {tol * scale:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,T", [(2560, 33), (333, 7), (4096, 2), (80, 130), (12288, 3)])
def test_fused_norm_variants(ops, dtype, H, T):
    w = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(1))).cuda()
    eps = 1e-5
    # (a) residual add + norm, residual updated in place
    resid = rand((T, H), torch.float32, 2)
    pend = rand((T, H), dtype, 3)
    r1, r2 = resid.clone(), resid.clone()
    o1 = torch.empty((T, H), dtype=dtype, device="cuda")
    o2 = torch.empty_like(o1)
    ops.fused_norm(o1, w, eps, resid=r1, pending=pend)
    REF.fused_norm(o2, w, eps, resid=r2, pending=pend)
    close(o1, o2, dtype, "add+norm")
    assert torch.equal(r1, r2), "the residual sum is a float32 add of the same two numbers"
    # (b) embedding lookup + norm
    V = 1000
    table = rand((V, H), dtype, 4)
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(5)).int().cuda()
    r1 = torch.empty((T, H), dtype=torch.float32, device="cuda")
    r2 = torch.empty_like(r1)
    ops.fused_norm(o1, w, eps, resid=r1, ids=ids, table=table)
    REF.fused_norm(o2, w, eps, resid=r2, ids=ids, table=table)
    close(o1, o2, dtype, "embed+norm")
    assert torch.equal(r1, r2)
    # (c) gathered rows, residual untouched
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32).cuda()
    before = resid.clone()
    g1 = torch.empty((3, H), dtype=dtype, device="cuda")
    g2 = torch.empty_like(g1)
    ops.fused_norm(g1, w, eps, resid=resid, pending=pend, rows=rows, write_resid=False)
    REF.fused_norm(g2, w, eps, resid=resid.clone(), pending=pend, rows=rows, write_resid=False)
    close(g1, g2, dtype, "gather+add+norm")
    assert torch.equal(resid, before)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("I,T", [(9728, 5), (111, 64), (160, 1)])
def test_silu_mul(ops, dtype, I, T):
    gu = rand((T, 2 * I), dtype, 6, scale=3.0)
    a = torch.empty((T, I), dtype=dtype, device="cuda")
    b = torch.empty_like(a)
    ops.silu_mul(gu, a)
    REF.silu_mul(gu, b)
    close(a, b, dtype, "silu_mul", bf16_tol=1e-2)


def test_rope_table_matches_host_formula(ops):
    for D, theta, n in ((128, 1e6, 5000), (48, 1e4, 300)):
        inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float) / D))
        cos, sin = ops.rope_table(inv.cuda(), n)
        ang = torch.arange(n, dtype=torch.float)[:, None] * inv[None, :]
        assert float((cos.cpu() - ang.cos()).abs().max()) < 2e-6
        assert float((sin.cpu() - ang.sin()).abs().max()) < 2e-6


def make_cache(num_pages, nkv, ps, D, dtype, seed):
    k = rand((num_pages, nkv, ps, D), dtype, seed)
    v = rand((num_pages, nkv, ps, D), dtype, seed + 1)
    return k, v


@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,D,ps,rot,write", [(32, 8, 128, 16, 128, True), (6, 3, 48, 7, 48, True),
                                                    (5, 5, 80, 1, 32, True), (4, 1, 16, 32, 16, False),
                                                    (3, 1, 64, 8, 64, True), (2, 2, 256, 4, 256, True)])
def test_qk_norm_rope_store(ops, dtype, nq, nkv, D, ps, rot, write, pairing):
    T, B = 37, 3
    maxp = (21 + T) // ps + 1  # every position below has a page in the table
    g = torch.Generator().manual_seed(7)
    seq = torch.randint(0, B, (T,), generator=g).int()
    # distinct (seq, position) pairs so that no two tokens write the same slot
    pos = torch.zeros(T, dtype=torch.int32)
    used = {}
    for t in range(T):
        s = int(seq[t])
        used[s] = used.get(s, 20) + 1
        pos[t] = used[s]
    bt = torch.randperm(B * maxp, generator=g).int().view(B, maxp)
    width = (nq + 2 * nkv) * D if write else nq * D
    qkv = rand((T, width), dtype, 8)
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda()
    inv = 1.0 / (1e4 ** (torch.arange(0, rot, 2, dtype=torch.float) / rot))
    cos, sin = ops.rope_table(inv.cuda(), 256)
    outs = []
    for impl in (ops, REF):
        x = qkv.clone()
        k, v = make_cache(B * maxp, nkv, ps, D, dtype, 9)
        impl.qk_norm_rope_store(x, num_heads=nq, num_kv_heads=nkv, head_dim=D, q_weight=qw, k_weight=kw, eps=1e-6,
                                cos=cos, sin=sin, positions=pos.cuda(), token_seq=seq.cuda(), block_table=bt.cuda(),
                                k_pages=k, v_pages=v, page_size=ps, write_kv=write, pairing=pairing)
        outs.append((x, k, v))
    (x1, k1, v1), (x2, k2, v2) = outs
    close(x1[:, : nq * D], x2[:, : nq * D], dtype, "q")
    close(k1, k2, dtype, "k pages")
    assert torch.equal(v1, v2), "values are copied bit for bit"
    if write:  # slots that no token of the step owns are untouched
        k0, _ = make_cache(B * maxp, nkv, ps, D, dtype, 9)
        assert int((k1 != k0).any(dim=-1).any(dim=1).sum()) == T
    ops.raise_if_kernel_error()


def test_a_position_beyond_the_rotation_tables_is_reported_not_rotated(ops):
    """The store kernels never rotate a token with another position's angles: a position outside
    the tables leaves that token's q and k as they were and sets the error word, which the host
    turns into an exception.  A table of no rows at all is refused before any launch."""
    from qwen3_runtime_b200.ops.cuda import KernelError

    nq, nkv, ps = 2, 1, 4
    for D in (32, 48):  # the 16-byte kernel and the scalar one
        T = 3
        qkv = rand((T, (nq + 2 * nkv) * D), torch.bfloat16, 12)
        pos = torch.tensor([0, 1, 9], dtype=torch.int32).cuda()   # the table below has 8 rows
        seq = torch.zeros(T, dtype=torch.int32).cuda()
        bt = torch.tensor([[0, 1, 2]], dtype=torch.int32).cuda()
        k, v = make_cache(3, nkv, ps, D, torch.bfloat16, 13)
        inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float) / D))
        cos, sin = ops.rope_table(inv.cuda(), 8)
        x = qkv.clone()
        ops.qk_norm_rope_store(x, num_heads=nq, num_kv_heads=nkv, head_dim=D, q_weight=None, k_weight=None, eps=0.0,
                               cos=cos, sin=sin, positions=pos, token_seq=seq, block_table=bt, k_pages=k, v_pages=v,
                               page_size=ps, write_kv=True)
        with pytest.raises(KernelError, match="outside the rotation tables"):
            ops.raise_if_kernel_error()
        assert torch.equal(x[2, : nq * D], qkv[2, : nq * D]), "the out-of-range token's q is untouched"
        assert not torch.equal(x[1, : nq * D], qkv[1, : nq * D]), "the others were rotated"
        ops.raise_if_kernel_error()  # the word was cleared
        with pytest.raises(KernelError, match="bad argument"):
            ops.qk_norm_rope_store(x, num_heads=nq, num_kv_heads=nkv, head_dim=D, q_weight=None, k_weight=None,
                                   eps=0.0, cos=cos[:0], sin=sin[:0], positions=pos, token_seq=seq, block_table=bt,
                                   k_pages=k, v_pages=v, page_size=ps, write_kv=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_qk_norm_rope_store_without_norm_or_rotation(ops, dtype):
    T, nq, nkv, D, ps = 5, 2, 1, 32, 4
    qkv = rand((T, (nq + 2 * nkv) * D), dtype, 10)
    pos = torch.arange(T, dtype=torch.int32).cuda()
    seq = torch.zeros(T, dtype=torch.int32).cuda()
    bt = torch.tensor([[1, 0]], dtype=torch.int32).cuda()
    k, v = make_cache(2, nkv, ps, D, dtype, 11)
    x = qkv.clone()
    ops.qk_norm_rope_store(x, num_heads=nq, num_kv_heads=nkv, head_dim=D, q_weight=None, k_weight=None, eps=0.0,
                           cos=None, sin=None, positions=pos, token_seq=seq, block_table=bt, k_pages=k, v_pages=v,
                           page_size=ps, write_kv=True)
    assert torch.equal(x, qkv)
    assert torch.equal(k[1, 0, :4], qkv[:4, nq * D:(nq + 1) * D]) and torch.equal(k[0, 0, 0], qkv[4, nq * D:(nq + 1) * D])


def attention_problem(nq, nkv, D, ps, lens, qlens, dtype, seed, num_pages=None):
    """A ragged batch: sequence b has ``lens[b]`` keys in the cache and its last ``qlens[b]`` are queries."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    maxp = max(-(-n // ps) for n in lens) + 1
    num_pages = num_pages or B * maxp + 3
    perm = torch.randperm(num_pages, generator=g).int()
    bt = perm[: B * maxp].view(B, maxp).contiguous()
    k, v = make_cache(num_pages, nkv, ps, D, dtype, seed + 1)
    seq, pos = [], []
    for b, (n, ql) in enumerate(zip(lens, qlens)):
        seq += [b] * ql
        pos += list(range(n - ql, n))
    T = len(seq)
    q = rand((T, (nq + 2 * nkv) * D), dtype, seed + 2)
    return dict(q=q, k=k, v=v, bt=bt.cuda(), seq=torch.tensor(seq, dtype=torch.int32).cuda(),
                pos=torch.tensor(pos, dtype=torch.int32).cuda(), T=T)


def run_attention(impl, pr, nq, nkv, D, ps, dtype, window=None, scale=None):
    out = torch.zeros((pr["T"], nq * D), dtype=dtype, device="cuda")
    impl.paged_attention(pr["q"], pr["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=pr["k"],
                         v_pages=pr["v"], block_table=pr["bt"], token_seq=pr["seq"], positions=pr["pos"], out=out,
                         page_size=ps, scale=scale or 1 / math.sqrt(D), window=window)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,D,ps,window", [(32, 8, 128, 16, None), (6, 3, 48, 7, None), (8, 2, 64, 16, 33),
                                                 (4, 4, 16, 1, None), (5, 1, 80, 32, 100), (2, 1, 256, 8, None)])
def test_paged_attention_mixed_batch(ops, dtype, nq, nkv, D, ps, window):
    lens, qlens = [300, 1, 77, 129, 64], [1, 1, 77, 40, 2]  # decode, first token, whole prompt, portion, tiny portion
    pr = attention_problem(nq, nkv, D, ps, lens, qlens, dtype, 20)
    a = run_attention(ops, pr, nq, nkv, D, ps, dtype, window)
    b = run_attention(REF, pr, nq, nkv, D, ps, dtype, window)
    close(a, b, dtype, "attention", f32_tol=1e-5, bf16_tol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """Random keys give near-uniform weights that hide a wrong page or offset.  Here one key, far
    back, in the middle of a page, is made to carry all the weight; the output must be that
    key's value.  Then the key one position past the window's edge must be ignored."""
    nq, nkv, D, ps = 8, 2, 128, 16
    n = 700
    for far in (0, 5, 16 * 9 + 15, 16 * 10, n - 1):
        pr = attention_problem(nq, nkv, D, ps, [n], [1], dtype, 30 + far)
        q = pr["q"]
        q[:] = 0
        q[0, : nq * D] = 4.0  # every query head: a constant vector
        page, off = int(pr["bt"][0, far // ps]), far % ps
        pr["k"][:] = pr["k"] * 0.01
        pr["k"][page, :, off, :] = 4.0  # score 16 * 128 / sqrt(128) = 181 against ~0
        out = run_attention(ops, pr, nq, nkv, D, ps, dtype)
        want = pr["v"][page, :, off, :].float().repeat_interleave(nq // nkv, dim=0).reshape(-1)
        close(out[0], want, dtype, f"far key at {far}", f32_tol=1e-6, bf16_tol=1e-6)
        # a window that ends one key after `far` must not see it
        window = n - 1 - far
        if window >= 1:
            out_w = run_attention(ops, pr, nq, nkv, D, ps, dtype, window=window)
            ref_w = run_attention(REF, pr, nq, nkv, D, ps, dtype, window=window)
            close(out_w, ref_w, dtype, f"window edge excludes {far}", f32_tol=1e-5, bf16_tol=1e-2)
            assert float((out_w[0].float() - want).abs().max()) > 0.1
            out_in = run_attention(ops, pr, nq, nkv, D, ps, dtype, window=window + 1)
            close(out_in[0], want, dtype, f"window edge includes {far}", f32_tol=1e-6, bf16_tol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_ignores_what_lies_beyond_a_sequence(ops, dtype):
    """Slots after a sequence's last key (rest of its last page, pages of other requests) hold NaN."""
    nq, nkv, D, ps = 4, 2, 64, 16
    lens, qlens = [21, 40], [21, 1]
    pr = attention_problem(nq, nkv, D, ps, lens, qlens, dtype, 40)
    ref = run_attention(REF, pr, nq, nkv, D, ps, dtype)
    used = torch.zeros(pr["k"].shape[0], ps, dtype=torch.bool)
    for b, n in enumerate(lens):
        for j in range(n):
            used[int(pr["bt"][b, j // ps]), j % ps] = True
    mask = (~used).cuda()[:, None, :, None].expand_as(pr["k"])
    pr["k"][mask] = float("nan")
    pr["v"][mask] = float("nan")
    out = run_attention(ops, pr, nq, nkv, D, ps, dtype)
    assert torch.isfinite(out).all()
    close(out, ref, dtype, "attention with poisoned free slots", f32_tol=1e-5, bf16_tol=1e-2)


def step_for(lens, qlens):
    """The fields of a StepContext that the attention wrapper reads."""
    from types import SimpleNamespace

    cu = [0]
    for n in qlens:
        cu.append(cu[-1] + n)
    singles = [b for b, n in enumerate(qlens) if n == 1]
    return SimpleNamespace(
        decode_only=all(n == 1 for n in qlens), num_seqs=len(lens), host_cu_seqlens=cu, host_kv_lens=list(lens),
        kv_lens=torch.tensor(lens, dtype=torch.int32).cuda(), cu_seqlens=torch.tensor(cu, dtype=torch.int32).cuda(),
        single_seqs=torch.tensor(singles, dtype=torch.int32).cuda(), num_single=len(singles),
        max_kv_len=max(lens), extras={})


@pytest.mark.parametrize("nq,nkv,D,ps,window", [(32, 8, 128, 16, None), (8, 8, 64, 8, None), (6, 2, 128, 3, None),
                                                 (16, 1, 64, 32, 50), (14, 2, 128, 16, 129), (4, 4, 128, 64, 1)])
def test_prefill_attention_tensor_cores(ops, nq, nkv, D, ps, window):
    """Whole prompts, portions after cached tokens, tiny portions and single tokens in one batch."""
    lens = [300, 1, 77, 700, 64, 130, 2, 333]
    qlens = [1, 1, 77, 200, 2, 130, 2, 33]
    pr = attention_problem(nq, nkv, D, ps, lens, qlens, torch.bfloat16, 90)
    want = run_attention(REF, pr, nq, nkv, D, ps, torch.bfloat16, window)
    out = torch.full((pr["T"], nq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.paged_attention(pr["q"], pr["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=pr["k"],
                        v_pages=pr["v"], block_table=pr["bt"], token_seq=pr["seq"], positions=pr["pos"], out=out,
                        page_size=ps, scale=1 / math.sqrt(D), window=window, step=step_for(lens, qlens))
    assert torch.isfinite(out).all(), "every row is written"
    close(out, want, torch.bfloat16, "prefill attention", bf16_tol=1e-2)


@pytest.mark.parametrize("nq,nkv,ps", [(32, 8, 16), (8, 8, 8), (16, 1, 64), (8, 2, 32), (32, 8, 16)])
def test_prefill_attention_tcgen05_matches_mma_kernel(ops, nq, nkv, ps):
    """head_dim 128 without a window takes the tcgen05/TMEM kernel; the mma.sync kernel and the
    plain statement are the references."""
    D = 128
    lens = [300, 1, 77, 700, 64, 130, 2, 1333, 128]
    qlens = [1, 1, 77, 200, 2, 130, 2, 1333, 128]
    pr = attention_problem(nq, nkv, D, ps, lens, qlens, torch.bfloat16, 92)
    step = step_for(lens, qlens)

    def run(which):
        ops.prefill_attention = which
        out = torch.full((pr["T"], nq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.paged_attention(pr["q"], pr["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=pr["k"],
                            v_pages=pr["v"], block_table=pr["bt"], token_seq=pr["seq"], positions=pr["pos"], out=out,
                            page_size=ps, scale=1 / math.sqrt(D), window=None, step=step)
        ops.prefill_attention = "tcgen05"
        return out

    tc, mma = run("tcgen05"), run("mma")
    ops.raise_if_kernel_error()
    assert torch.isfinite(tc).all(), "every row is written"
    want = run_attention(REF, pr, nq, nkv, D, ps, torch.bfloat16)
    close(mma, want, torch.bfloat16, "mma.sync prefill", bf16_tol=1e-2)
    close(tc, want, torch.bfloat16, "tcgen05 prefill", bf16_tol=1e-2)


def test_attention_kernels_at_long_contexts(ops, decode_loader):
    """Tens of thousands of keys: many slices and pages for the split-KV kernel, many tiles and an
    odd number of row blocks for the tcgen05 kernel (checked against the mma.sync kernel, the
    plain statement being too slow here)."""
    nq, nkv, D, ps = 8, 2, 128, 16
    lens = [30000, 17, 4097]
    pr = decode_problem(nq, nkv, D, ps, lens, 95)
    want = run_attention(REF, pr, nq, nkv, D, ps, torch.bfloat16)
    for splits in (None, 7, 23):
        got = run_decode(ops, pr, nq, nkv, D, ps, lens, splits=splits)
        close(got, want, torch.bfloat16, f"decode attention at 30000 keys, splits={splits}", bf16_tol=1e-2)
    lens, qlens = [9000, 300], [4100, 300]   # a portion of a long prompt after 4900 cached tokens
    pr = attention_problem(nq, nkv, D, ps, lens, qlens, torch.bfloat16, 96)
    step = step_for(lens, qlens)
    outs = {}
    for which in ("tcgen05", "mma"):
        ops.prefill_attention = which
        outs[which] = torch.full((pr["T"], nq * D), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.paged_attention(pr["q"], pr["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=pr["k"],
                            v_pages=pr["v"], block_table=pr["bt"], token_seq=pr["seq"], positions=pr["pos"],
                            out=outs[which], page_size=ps, scale=1 / math.sqrt(D), window=None, step=step)
    ops.prefill_attention = "tcgen05"
    ops.raise_if_kernel_error()
    assert torch.isfinite(outs["tcgen05"]).all()
    close(outs["tcgen05"], outs["mma"].float(), torch.bfloat16, "tcgen05 prefill at 9000 keys", bf16_tol=1e-2)


def test_prefill_attention_far_key_diagonal_and_poison(ops):
    nq, nkv, D, ps = 8, 2, 128, 16
    lens, qlens = [900, 257], [300, 257]
    pr = attention_problem(nq, nkv, D, ps, lens, qlens, torch.bfloat16, 91)
    used = torch.zeros(pr["k"].shape[0], ps, dtype=torch.bool)
    for b, n in enumerate(lens):
        for j in range(n):
            used[int(pr["bt"][b, j // ps]), j % ps] = True
    mask = (~used).cuda()[:, None, :, None].expand_as(pr["k"])
    pr["k"][mask] = float("nan")
    pr["v"][mask] = float("nan")
    step = step_for(lens, qlens)

    def run(p):
        out = torch.zeros((p["T"], nq * D), dtype=torch.bfloat16, device="cuda")
        ops.paged_attention(p["q"], p["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D, k_pages=p["k"],
                            v_pages=p["v"], block_table=p["bt"], token_seq=p["seq"], positions=p["pos"], out=out,
                            page_size=ps, scale=1 / math.sqrt(D), window=None, step=step)
        return out

    assert torch.isfinite(run(pr)).all()
    # one key carries all the weight for every query that can see it, none for the others
    for far in (0, 599, 600, 777, 899):
        p2 = dict(pr, k=pr["k"] * 0.01, q=pr["q"].clone())
        p2["q"][:300, : nq * D] = 4.0
        page, off = int(pr["bt"][0, far // ps]), far % ps
        p2["k"][page, :, off, :] = 4.0
        out = run(p2)
        want = p2["v"][page, :, off, :].float().repeat_interleave(nq // nkv, dim=0).reshape(-1)
        sees = torch.arange(600, 900) >= far  # query i of the portion sits at position 600 + i
        got = out[:300].float().cpu()
        assert float((got[sees] - want.cpu()).abs().max()) <= 1e-6 * max(1.0, float(want.abs().max()))
        if (~sees).any():
            assert float((got[~sees] - want.cpu()).abs().max()) > 0.05


def decode_problem(nq, nkv, D, ps, lens, seed):
    pr = attention_problem(nq, nkv, D, ps, lens, [1] * len(lens), torch.bfloat16, seed)
    pr["kv_lens"] = torch.tensor(lens, dtype=torch.int32).cuda()
    pr["cu"] = torch.arange(len(lens) + 1, dtype=torch.int32).cuda()
    return pr


MERGE_KERNEL = False  # set by the decode_loader fixture: the slices are merged by a second kernel


def run_decode(ops, pr, nq, nkv, D, ps, lens, window=None, splits=None, seq_list=None, out=None, merge_kernel=None,
               longest=None):
    out = out if out is not None else torch.zeros((pr["T"], nq * D), dtype=torch.bfloat16, device="cuda")
    n = len(lens) if seq_list is None else seq_list.numel()
    ops.paged_attention_decode(pr["q"], pr["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D,
                               k_pages=pr["k"], v_pages=pr["v"], block_table=pr["bt"], kv_lens=pr["kv_lens"],
                               cu_seqlens=pr["cu"], out=out, page_size=ps, scale=1 / math.sqrt(D), window=window,
                               num_seqs=n, max_kv_len=max(lens), seq_list=seq_list, num_splits=splits,
                               merge_kernel=MERGE_KERNEL if merge_kernel is None else merge_kernel, longest=longest)
    return out


@pytest.fixture(params=["last block merges", "merge kernel"])
def decode_loader(ops, request):
    """The slices of a sequence and kv head are merged by the block that finishes last, or by a
    second kernel (what callers without ticket words get)."""
    global MERGE_KERNEL
    MERGE_KERNEL = request.param == "merge kernel"
    yield request.param
    MERGE_KERNEL = False
    ops.raise_if_kernel_error()
    assert ops._tickets is None or not bool(ops._tickets.any()), "every ticket word is zero again after a launch"


@pytest.mark.parametrize("nq,nkv,D,ps", [(32, 8, 128, 16), (8, 8, 64, 8), (16, 1, 128, 32), (6, 2, 256, 16),
                                          (14, 2, 64, 3), (40, 8, 128, 64), (4, 2, 128, 128), (16, 4, 256, 8)])
@pytest.mark.parametrize("splits", [None, 1, 3, 8, 11])
def test_decode_attention_split_kv(ops, decode_loader, nq, nkv, D, ps, splits):
    lens = [1, 63, 64, 65, 700, 129, 2, 1000]
    pr = decode_problem(nq, nkv, D, ps, lens, 80)
    want = run_attention(REF, pr, nq, nkv, D, ps, torch.bfloat16)
    got = run_decode(ops, pr, nq, nkv, D, ps, lens, splits=splits)
    close(got, want, torch.bfloat16, f"decode attention splits={splits}", bf16_tol=1e-2)
    for window in (1, 64, 100):
        want = run_attention(REF, pr, nq, nkv, D, ps, torch.bfloat16, window=window)
        got = run_decode(ops, pr, nq, nkv, D, ps, lens, window=window, splits=splits)
        close(got, want, torch.bfloat16, f"decode attention window={window} splits={splits}", bf16_tol=1e-2)


@pytest.mark.parametrize("nq,nkv,D,ps", [(32, 8, 128, 16), (14, 2, 64, 3), (6, 2, 256, 16)])
def test_decode_attention_merge_by_last_block_gives_the_bits_of_the_merge_kernel(ops, nq, nkv, D, ps):
    """Whichever block of a pair finishes last merges the slices; the result does not depend on
    which one it was, and equals the merge kernel's bit for bit.  Ticket words are zero afterwards,
    also with empty slices (windows, lengths far below the slice count)."""
    lens = [1, 63, 64, 65, 700, 129, 2, 1000, 4096, 333]
    pr = decode_problem(nq, nkv, D, ps, lens, 81)
    for splits in (2, 6, 13):
        for window in (None, 100):
            want = run_decode(ops, pr, nq, nkv, D, ps, lens, window=window, splits=splits, merge_kernel=True)
            for _ in range(3):
                got = run_decode(ops, pr, nq, nkv, D, ps, lens, window=window, splits=splits, merge_kernel=False)
                assert torch.equal(got, want), (splits, window)
            # the longest length handed in by the caller: the same slices as when the blocks find it
            # (with a window the blocks look for the longest visible span, which need not be the
            # longest sequence's: the cut may differ by a tile then, the result only by rounding)
            known = torch.tensor([max(lens)], dtype=torch.int32, device="cuda")
            for merge_kernel in (False, True):
                got = run_decode(ops, pr, nq, nkv, D, ps, lens, window=window, splits=splits,
                                 merge_kernel=merge_kernel, longest=known)
                if window is None:
                    assert torch.equal(got, want), (splits, window, "longest given")
                else:
                    close(got, want, torch.bfloat16, "longest given, window", bf16_tol=1e-2)
            assert not bool(ops._tickets.any())


@pytest.mark.parametrize("nq,nkv,D,ps", [(32, 8, 128, 64), (8, 8, 64, 8), (16, 1, 128, 32), (6, 2, 256, 16),
                                          (14, 2, 64, 3), (32, 8, 128, 16)])
@pytest.mark.parametrize("norm,rotate", [(True, True), (False, True), (True, False), (False, False),
                                         (True, "interleaved")])
def test_decode_attention_makes_the_newest_token_itself(ops, decode_loader, nq, nkv, D, ps, norm, rotate):
    """One kernel (per-head norm, rotation, cache write, attention) against the two kernels it
    replaces: the same bits in the output and in the pages, for every split count and window."""
    lens = [1, 63, 64, 65, 700, 129, 2, 1000]
    g = torch.Generator().manual_seed(5)
    qw = (1 + 0.1 * torch.randn(D, generator=g)).cuda() if norm else None
    kw = (1 + 0.1 * torch.randn(D, generator=g)).cuda() if norm else None
    cos = sin = None
    pairing = rotate if isinstance(rotate, str) else "half"
    if rotate:
        inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, dtype=torch.float) / D))
        cos, sin = ops.rope_table(inv.cuda(), 1024)
    assert ops.decode_new_token_ok(torch.empty((1, (nq + 2 * nkv) * D), dtype=torch.bfloat16, device="cuda"),
                                   num_heads=nq, num_kv_heads=nkv, head_dim=D, cos=cos, q_weight=qw, k_weight=kw)
    for splits, window in [(None, None), (1, None), (3, None), (8, 100), (2, 1), (5, 64)]:
        pr = decode_problem(nq, nkv, D, ps, lens, 90)
        two = dict(pr, q=pr["q"].clone(), k=pr["k"].clone(), v=pr["v"].clone())
        ops.qk_norm_rope_store(two["q"], num_heads=nq, num_kv_heads=nkv, head_dim=D, q_weight=qw, k_weight=kw,
                               eps=1e-6, cos=cos, sin=sin, positions=pr["pos"], token_seq=pr["seq"],
                               block_table=pr["bt"], k_pages=two["k"], v_pages=two["v"], page_size=ps, write_kv=True,
                               pairing=pairing)
        want = run_decode(ops, two, nq, nkv, D, ps, lens, window=window, splits=splits)
        one = dict(pr, q=pr["q"].clone(), k=pr["k"].clone(), v=pr["v"].clone())
        raw = one["q"].clone()
        got = torch.zeros_like(want)
        ops.paged_attention_decode(one["q"], one["q"].stride(0), num_heads=nq, num_kv_heads=nkv, head_dim=D,
                                   k_pages=one["k"], v_pages=one["v"], block_table=pr["bt"], kv_lens=pr["kv_lens"],
                                   cu_seqlens=pr["cu"], out=got, page_size=ps, scale=1 / math.sqrt(D), window=window,
                                   num_seqs=len(lens), max_kv_len=max(lens), num_splits=splits,
                                   new_token=dict(q_weight=qw, k_weight=kw, eps=1e-6, cos=cos, sin=sin,
                                                  pairing=pairing), merge_kernel=MERGE_KERNEL)
        what = f"splits={splits} window={window}"
        assert torch.equal(got, want), what
        assert torch.equal(one["k"], two["k"]) and torch.equal(one["v"], two["v"]), what
        assert torch.equal(one["q"], raw), "the projection's output is read only"
        assert not torch.equal(one["k"], pr["k"])


def test_decode_attention_far_key_poison_and_subset(ops, decode_loader):
    nq, nkv, D, ps = 32, 8, 128, 16
    lens = [900, 333, 64]
    pr = decode_problem(nq, nkv, D, ps, lens, 81)
    # everything that is not a live key is NaN
    used = torch.zeros(pr["k"].shape[0], ps, dtype=torch.bool)
    for b, n in enumerate(lens):
        for j in range(n):
            used[int(pr["bt"][b, j // ps]), j % ps] = True
    mask = (~used).cuda()[:, None, :, None].expand_as(pr["k"])
    clean_k, clean_v = pr["k"].clone(), pr["v"].clone()
    pr["k"][mask] = float("nan")
    pr["v"][mask] = float("nan")
    got = run_decode(ops, pr, nq, nkv, D, ps, lens, splits=5)
    assert torch.isfinite(got).all()
    pr2 = dict(pr, k=torch.where(mask, torch.zeros_like(clean_k), clean_k), v=torch.where(mask, torch.zeros_like(clean_v), clean_v))
    close(got, run_attention(REF, pr2, nq, nkv, D, ps, torch.bfloat16), torch.bfloat16, "poisoned pool", bf16_tol=1e-2)
    # one far key carries all the weight
    for far in (0, 77, 16 * 20 + 15, 899):
        pr3 = dict(pr2, k=pr2["k"] * 0.01, q=pr2["q"].clone())
        pr3["q"][0, : nq * D] = 4.0
        page, off = int(pr["bt"][0, far // ps]), far % ps
        pr3["k"][page, :, off, :] = 4.0
        got = run_decode(ops, pr3, nq, nkv, D, ps, lens, splits=4)
        want = pr3["v"][page, :, off, :].float().repeat_interleave(nq // nkv, dim=0).reshape(-1)
        close(got[0], want, torch.bfloat16, f"far key {far}", bf16_tol=1e-6)
    # a subset of the sequences (a mixed step hands the one-token sequences to this kernel)
    seqs = torch.tensor([2, 0], dtype=torch.int32).cuda()
    out = torch.full((3, nq * D), 7.0, dtype=torch.bfloat16, device="cuda")
    run_decode(ops, pr2, nq, nkv, D, ps, lens, splits=3, seq_list=seqs, out=out)
    full = run_attention(REF, pr2, nq, nkv, D, ps, torch.bfloat16)
    close(out[[0, 2]], full[[0, 2]], torch.bfloat16, "subset", bf16_tol=1e-2)
    assert bool((out[1] == 7.0).all())


@pytest.mark.parametrize("M,N,K", [(1, 2560, 2560), (7, 333, 130), (64, 96, 64), (65, 160, 96), (300, 301, 80),
                                   (2, 1000, 9)])
def test_gemm_f32_is_exact_fp32_and_row_invariant(ops, M, N, K):
    x = rand((M, K), torch.float32, 50)
    w = rand((N, K), torch.float32, 51)
    got = ops.linear(x, w)
    want = (x.double() @ w.double().t())
    assert float((got.double() - want).abs().max()) <= 2e-6 * math.sqrt(K) * float(want.abs().max() + 1)
    # TF32 would be off by ~1e-3 relative: make sure we are far below it
    assert float((got.double() - want).abs().max()) < 1e-4 * float(want.abs().max())
    # a row's result does not depend on how many rows are computed with it
    alone = ops.linear(x[M - 1:M].contiguous(), w)
    assert torch.equal(alone[0], got[M - 1])
    if M > 2:
        part = ops.linear(x[1:M].contiguous(), w)
        assert torch.equal(part, got[1:])


@pytest.mark.parametrize("M,N,K", [(1, 2560, 2560), (8, 19456, 2560), (300, 304, 96), (5, 151936, 64)])
def test_linear_bf16(ops, M, N, K):
    x = rand((M, K), torch.bfloat16, 52)
    w = rand((N, K), torch.bfloat16, 53, scale=0.05)
    want = x.float() @ w.float().t()
    close(ops.linear(x, w), want, torch.bfloat16, "linear bf16", bf16_tol=1e-2)
    f32 = ops.linear(x, w, out_dtype=torch.float32)
    assert f32.dtype == torch.float32
    close(f32, want, torch.float32, "linear bf16 -> f32", f32_tol=1e-4)


@pytest.fixture(params=["stream", "registers", "auto"])
def small_gemm(ops, request):
    """Both kernels for products of at most 16 tokens: the shared-memory stream and the older
    register stream (which also takes what the first refuses)."""
    before = ops.small_gemm
    ops.small_gemm = request.param
    yield request.param
    ops.small_gemm = before
    ops.raise_if_kernel_error()


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(2560, 2560), (6144, 2560), (2560, 9728), (2560, 4096), (301, 80), (160, 96),
                                 (151936, 64), (24, 8), (17, 4096), (40, 20480), (40, 20488), (1000, 5128), (64, 40960), (8, 40968)])
def test_gemm_small_m(ops, small_gemm, M, N, K):
    x = rand((M, K), torch.bfloat16, 54)
    w = rand((N, K), torch.bfloat16, 55, scale=0.05)
    assert ops._small_m_ok(x, w)
    want = x.float() @ w.float().t()
    close(ops.linear(x, w), want, torch.bfloat16, "small-M linear", bf16_tol=1e-2)
    close(ops.linear(x, w, out_dtype=torch.float32), want, torch.float32, "small-M linear fp32 out", f32_tol=2e-5)
    # a view with a row stride (the q rows of the fused qkv weight) and a strided input
    wide = rand((M, K + 8), torch.bfloat16, 56)
    close(ops.linear(wide[:, :K], w[: max(1, N // 2)]), wide[:, :K].float() @ w[: max(1, N // 2)].float().t(),
          torch.bfloat16, "strided", bf16_tol=1e-2)
    # the same bits every time
    first = ops.linear(x, w, out_dtype=torch.float32)
    for _ in range(3):
        assert torch.equal(ops.linear(x, w, out_dtype=torch.float32), first)


def test_gemm_stream_rows_do_not_depend_on_the_other_tokens(ops):
    """A token's result is the same bits alone, among 8 and among 16 tokens."""
    for N, K in [(2560, 2560), (2560, 9728), (304, 96)]:
        x = rand((16, K), torch.bfloat16, 66)
        w = rand((N, K), torch.bfloat16, 67, scale=0.05)
        ops.small_gemm = "stream"
        full = ops.linear(x, w, out_dtype=torch.float32)
        for m in (1, 5, 8, 9):
            assert torch.equal(ops.linear(x[:m], w, out_dtype=torch.float32), full[:m]), (N, K, m)
    ops.small_gemm = "auto"
    ops.raise_if_kernel_error()


@pytest.mark.parametrize("M", [1, 7, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(2560, 4096), (2560, 9728), (301, 80), (17, 4096), (40, 20488), (1000, 5128),
                                 (8, 40968), (2560, 2560), (48, 64)])
def test_gemm_stream_partial_sums(ops, M, N, K):
    """The planes are the products over consecutive ranges of K (multiples of 32 wide) and add
    up to the product; the norm kernel adds them in order, then the residual."""
    x = rand((M, K), torch.bfloat16, 68)
    w = rand((N, K), torch.bfloat16, 69, scale=0.05)
    planes = ops.linear(x, w, partial_sums=True)
    want = x.float() @ w.float().t()
    if planes.dim() == 2:  # the kernel keeps K whole for these sizes: a finished product
        assert ops._stream_parts(M, N, K) <= 1
        close(planes, want, torch.bfloat16, "finished product", bf16_tol=1e-2)
        return
    parts = planes.shape[0]
    assert planes.dtype == torch.float32 and planes.shape == (parts, M, N) and parts in (2, 4, 8)
    width = (-(-K // parts) + 31) // 32 * 32
    for p in range(parts):
        a, b = p * width, min(K, (p + 1) * width)
        close(planes[p], x[:, a:b].float() @ w[:, a:b].float().t(), torch.float32, f"plane {p}", f32_tol=2e-5)
    close(planes.sum(0), want, torch.float32, "sum of the planes", f32_tol=2e-5)
    assert torch.equal(ops.linear(x, w, partial_sums=True), planes), "the same bits every time"
    if M > 1:  # a token's planes do not depend on the other tokens
        assert torch.equal(ops.linear(x[:1], w, partial_sums=True), planes[:, :1])
    # consumed by the norm: bfloat16 and float32 outputs, whole and gathered rows
    for dtype in DTYPES:
        g = (1 + 0.1 * torch.randn(N, generator=torch.Generator().manual_seed(70))).cuda()
        resid = rand((M, N), torch.float32, 71)
        r1, r2 = resid.clone(), resid.clone()
        o1 = torch.empty((M, N), dtype=dtype, device="cuda")
        o2 = torch.empty_like(o1)
        ops.fused_norm(o1, g, 1e-6, resid=r1, pending=planes)
        REF.fused_norm(o2, g, 1e-6, resid=r2, pending=planes)
        close(o1, o2, dtype, "partial sums + add + norm")
        assert torch.equal(r1, r2), "planes are added in order, then to the residual, all in float32"
        rows = torch.tensor([M - 1, 0], dtype=torch.int32).cuda()
        g1 = torch.empty((2, N), dtype=dtype, device="cuda")
        g2 = torch.empty_like(g1)
        ops.fused_norm(g1, g, 1e-6, resid=resid, pending=planes, rows=rows, write_resid=False)
        REF.fused_norm(g2, g, 1e-6, resid=resid.clone(), pending=planes, rows=rows, write_resid=False)
        close(g1, g2, dtype, "partial sums + gather + norm")
    # without leave, or with the register kernel, the product comes finished
    assert ops.linear(x, w).dim() == 2
    ops.partial_sums = False
    try:
        assert ops.linear(x, w, partial_sums=True).dim() == 2
    finally:
        ops.partial_sums = True
    ops.raise_if_kernel_error()


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(9728, 2560), (112, 80), (160, 96), (24, 4096), (301, 2560), (6, 9728)])
def test_gated_linear_small_m(ops, small_gemm, M, I, K):
    x = rand((M, K), torch.bfloat16, 57)
    w = rand((2 * I, K), torch.bfloat16, 58, scale=0.05)
    out = torch.empty((M, I), dtype=torch.bfloat16, device="cuda")
    ops.gated_linear(x, w, out)
    g, u = x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t()
    close(out, torch.nn.functional.silu(g) * u, torch.bfloat16, "fused SwiGLU", bf16_tol=1e-2)
    # more tokens than the fused kernel takes: product, then the SwiGLU kernel
    xb = rand((40, K), torch.bfloat16, 59)
    outb = torch.empty((40, I), dtype=torch.bfloat16, device="cuda")
    ops.gated_linear(xb, w, outb)
    gb, ub = xb.float() @ w[:I].float().t(), xb.float() @ w[I:].float().t()
    close(outb, torch.nn.functional.silu(gb.bfloat16().float()) * ub.bfloat16().float(), torch.bfloat16,
          "unfused SwiGLU", bf16_tol=2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (2048, 6144, 2560),
                                   (300, 2560, 4096), (17, 304, 96), (64, 2560, 9728), (1000, 1000, 72),
                                   (129, 151936, 64), (2048, 2560, 4096), (2048, 2500, 96), (1900, 2564, 200)])
@pytest.mark.parametrize("pair", [False, True], ids=["one SM", "two SMs"])
def test_gemm_tcgen05(ops, M, N, K, pair):
    x = rand((M, K), torch.bfloat16, 62)
    w = rand((N, K), torch.bfloat16, 63, scale=0.05)
    want = x.float() @ w.float().t()
    got = ops.linear_tcgen05(x, w, pair=pair)
    ops.raise_if_kernel_error()
    close(got, want, torch.bfloat16, "tcgen05 linear", bf16_tol=1e-2)
    got32 = ops.linear_tcgen05(x, w, out_dtype=torch.float32, pair=pair)
    ops.raise_if_kernel_error()
    close(got32, want, torch.float32, "tcgen05 linear fp32 out", f32_tol=2e-5 * max(1.0, K / 256))


@pytest.mark.parametrize("M,I,K", [(128, 128, 64), (2048, 9728, 2560), (300, 112, 80), (77, 1000, 256)])
@pytest.mark.parametrize("pair", [False, True], ids=["one SM", "two SMs"])
def test_gemm_tcgen05_swiglu(ops, M, I, K, pair):
    x = rand((M, K), torch.bfloat16, 64)
    w = rand((2 * I, K), torch.bfloat16, 65, scale=0.05)
    out = torch.empty((M, I), dtype=torch.bfloat16, device="cuda")
    ops.linear_tcgen05(x, w, out=out, mode=2, pair=pair)
    ops.raise_if_kernel_error()
    g, u = x.float() @ w[:I].float().t(), x.float() @ w[I:].float().t()
    close(out, torch.nn.functional.silu(g) * u, torch.bfloat16, "tcgen05 fused SwiGLU", bf16_tol=1e-2)


@pytest.mark.parametrize("V,R", [(151936, 3), (301, 5), (32, 1), (4099, 64), (151936, 8), (151937, 1), (40000, 33),
                                 (151936, 200), (8192, 2)])
def test_argmax_lowest_index_on_ties(ops, V, R):
    """One block per row, or (few rows, long rows) a row cut into slices whose last block merges."""
    logits = rand((R, V), torch.float32, 60)
    logits[0, V // 3] = 50.0
    logits[0, V - 1] = 50.0  # tie, in different slices of a long row: the lower index wins
    if R > 1:
        logits[1, 5] = logits[1, 6] = 60.0  # tie of neighbours
    if R > 2:
        logits[2] = float("nan")  # nothing comparable: token 0, as the one-block kernel answers
    tok, lp = ops.argmax(logits, want_logprob=True)
    plain = [r for r in range(R) if r not in (0, 1, 2)]
    want = logits.argmax(-1)
    assert tok[0].item() == V // 3
    if R > 1:
        assert tok[1].item() == 5
    if R > 2:
        assert tok[2].item() == 0
    assert torch.equal(tok.long()[plain], want[plain])
    rows = [r for r in range(R) if r != 2]
    ref_lp = torch.log_softmax(logits, -1).gather(1, tok.long()[:, None])[:, 0]
    assert float((lp[rows] - ref_lp[rows]).abs().max()) < 1e-4
    only_tok, none = ops.argmax(logits)
    assert none is None and torch.equal(only_tok, tok)
    assert ops._argmax_tickets is None or not bool(ops._argmax_tickets.any())


@pytest.mark.parametrize("V,R", [(151936, 4), (301, 16), (4099, 3), (151936, 8), (151937, 1), (40000, 33), (8192, 70),
                                 (151936, 200)])
def test_sample_inverse_cdf(ops, V, R):
    """One block per row, or (few long rows) slices whose last block finds the slice to scan."""
    g = torch.Generator().manual_seed(61)
    logits = rand((R, V), torch.float32, 62, scale=3.0)
    lowest = torch.finfo(torch.float32).min
    logits[0, : V // 2] = lowest  # what the filters leave behind: whole slices without mass
    if R > 1:
        logits[1, V // 3:] = float("-inf")
    temp = (0.5 + torch.rand(R, generator=g)).cuda()
    for trial in range(5):
        u = torch.rand(R, generator=g).cuda()
        if trial == 4:
            u[0] = 0.0
            u[-1] = 0.99999994  # the largest float below one
        tok, lp = ops.sample(logits, temp, u, want_logprob=True)
        probs = torch.softmax(logits.double() / temp.double()[:, None], -1)
        cdf = probs.cumsum(-1)
        for r in range(R):
            t = int(tok[r])
            lo = float(cdf[r, t - 1]) if t > 0 else 0.0
            assert lo - 2e-6 <= float(u[r]) <= float(cdf[r, t]) + 2e-6, (r, t, float(u[r]), lo, float(cdf[r, t]))
            assert abs(float(lp[r]) - math.log(float(probs[r, t]))) < 1e-3
    # u = 0 picks the first token with any probability; u just below 1 the last one
    tok, _ = ops.sample(logits, temp, torch.zeros(R).cuda())
    assert tok.tolist() == [V // 2] + [0] * (R - 1)  # row 0 has no mass in its first half
    peaked = torch.full((1, V), -1e4).cuda()
    peaked[0, V - 2] = 0.0
    tok, _ = ops.sample(peaked, torch.ones(1).cuda(), torch.tensor([0.9999]).cuda())
    assert tok.item() == V - 2


def test_kernels_refuse_sizes_they_do_not_support(ops):
    from qwen3_runtime_b200.ops.cuda import KernelError

    pr = attention_problem(2, 1, 264, 16, [5], [1], torch.float32, 70)
    with pytest.raises(KernelError, match="head_dim=264"):
        run_attention(ops, pr, 2, 1, 264, 16, torch.float32)
    with pytest.raises(KernelError):
        ops.linear(torch.zeros(2, 8).cuda(), torch.zeros(4, 9).cuda())
    with pytest.raises(KernelError, match="float32 and bfloat16"):
        ops.silu_mul(torch.zeros(2, 8, dtype=torch.float16).cuda(), torch.zeros(2, 4, dtype=torch.float16).cuda())


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_stays_usable(ops):
    """The give-up path of a kernel that waits on mbarriers, run for real.  A second build of
    the tcgen05 product, under another name, leaves the weight boxes of every stage out, so a
    stage's barrier is a flag that nothing sets, and has short limits (about 1 ms for a wait,
    10 ms for the wait on what is still in flight).  The kernel must come back by itself with
    the error word set; the host must raise on it; and the next ordinary launch must be right."""
    from ctypes import c_int, c_void_p

    from qwen3_runtime_b200.ops import build
    from qwen3_runtime_b200.ops.cuda import _SIGNATURES, KernelError

    path = build.compile_group("gemm_tcgen05", variant="_withheld_box",
                               defines=("-DQ3_WAIT_LIMIT_CYCLES=2000000ll", "-DQ3_DRAIN_LIMIT_CYCLES=20000000ll",
                                        "-DQ3_TEST_WITHHOLD_A_BOX"))
    import ctypes

    fn = ctypes.CDLL(str(path)).q3_gemm_tcgen05
    fn.argtypes, fn.restype = _SIGNATURES["gemm_tcgen05"]["q3_gemm_tcgen05"], c_int
    x = rand((128, 64), torch.bfloat16, 301)
    w = rand((256, 64), torch.bfloat16, 302, scale=0.05)
    out = torch.zeros((128, 256), dtype=torch.bfloat16, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    code = fn(0, x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), 128, 256, 64,
              err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    stop.record()
    assert code == 0
    torch.cuda.synchronize()  # returns: every wait in the kernel is bounded
    assert int(err.item()) == 1, "the wait that ran out is reported"
    assert start.elapsed_time(stop) < 2000.0
    # the kernel table's own word in the same state: the host raises, once
    ops._error_word(x.device).copy_(err)
    with pytest.raises(KernelError, match="bounded wait"):
        ops.raise_if_kernel_error()
    ops.raise_if_kernel_error()
    # the context is intact: the ordinary build of the same kernel gives the right product
    got = ops.linear_tcgen05(x, w, pair=False)
    close(got, x.float() @ w.float().t(), torch.bfloat16, "product after the aborted one", bf16_tol=1e-2)
    ops.raise_if_kernel_error()


def test_the_sweep_behind_the_slice_count_model_runs():
    """`python -m qwen3_runtime_b200.ops.tune decode_splits --quick`: the measurement that the
    constants of CudaOps.decode_splits were fitted to, on a few sizes."""
    from qwen3_runtime_b200.ops import tune

    assert tune.main(["decode_splits", "--quick"]) == 0
