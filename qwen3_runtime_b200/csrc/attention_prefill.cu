// Causal attention of prompt portions over the paged cache, bfloat16, on the tensor cores.
//
// Work item: (sequence, kv head, block of 128 rows), where the rows of a (sequence, kv head)
// are its (query token, head of the group) pairs in token-major order -- so the group's
// heads share every key and value tile that is loaded (grouped-query attention as one
// tall matrix).  A block has 8 warps of 16 rows; keys and values arrive in tiles of 64
// through a 3-stage cp.async pipeline into XOR-swizzled shared memory; S = Q K^T and
// O += P V run as m16n8k16 MMAs with fp32 accumulators, the softmax is online in fp32
// (exp2 with the scale folded in), probabilities are rounded to bfloat16 for P V as in the
// reference (attention/pytorch.py:45).  The query at absolute position p sees keys
// max(0, p - window + 1) .. p; p = kv_len - q_len + its index in the portion
// (attention/pytorch.py:12-15).  Keys the block does not need are zero-filled, never read.
//
// The block finds its work item by walking cu_seqlens (sequences with one token can be left
// to the decode kernel: skip_single).
#include "common.cuh"
#include "mma_tiles.cuh"

namespace {

constexpr int BLOCK_M = 128;
constexpr int TILE = 64;
constexpr int WARPS = BLOCK_M / 16;
constexpr int THREADS = WARPS * 32;
constexpr int STAGES = 3;

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
prefill_attention_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kpages,
                         const bf16* __restrict__ vpages, const int* __restrict__ block_table, int max_pages,
                         const int* __restrict__ kv_lens, const int* __restrict__ cu_seqlens,
                         bf16* __restrict__ out, int num_seqs, int nq, int nkv, int ps, float scale_log2,
                         int window, int skip_single) {
  constexpr int CHUNKS = D / 8;
  constexpr int TILE_BYTES = TILE * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                       // [BLOCK_M][D]
  unsigned char* kv_s = smem + BLOCK_M * D * 2;    // STAGES x (K tile, V tile)
  __shared__ int s_item[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  const int G = nq / nkv;

  if (tid == 0) {
    int acc = 0, found = -1, rb = 0;
    const int w = blockIdx.x;
    for (int s = 0; s < num_seqs; ++s) {
      const int ql = cu_seqlens[s + 1] - cu_seqlens[s];
      if (ql <= 0 || (skip_single && ql == 1)) continue;
      const int nb = (ql * G + BLOCK_M - 1) / BLOCK_M;
      if (w < acc + nb) {
        found = s;
        rb = w - acc;
        break;
      }
      acc += nb;
    }
    s_item[0] = found;
    s_item[1] = rb;
  }
  __syncthreads();
  const int seq = s_item[0];
  if (seq < 0) return;
  const int row0 = s_item[1] * BLOCK_M;
  const int tok0 = cu_seqlens[seq];
  const int q_len = cu_seqlens[seq + 1] - tok0;
  const int kv_len = kv_lens[seq];
  const int rows = q_len * G;
  const int base_pos = kv_len - q_len;
  const int* bt = block_table + (long)seq * max_pages;

  // ---- queries of this block into shared memory (rows past the end are zero) ----------------
  for (int c = tid; c < BLOCK_M * CHUNKS; c += THREADS) {
    const int r = c / CHUNKS, chunk = c % CHUNKS;
    const int R = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < rows) {
      const int tk = R / G, hd = kvh * G + (R - tk * G);
      v = *reinterpret_cast<const uint4*>(q + (long)(tok0 + tk) * q_stride + (long)hd * D + chunk * 8);
    }
    *reinterpret_cast<uint4*>(q_s + swz<D>(r, chunk)) = v;
  }

  // ---- key range of the block -----------------------------------------------------------------
  const int last_row = min(rows, row0 + BLOCK_M) - 1;
  const int p_min = base_pos + row0 / G, p_max = base_pos + last_row / G;
  const int k_lo = window > 0 ? max(0, p_min - window + 1) : 0;
  const int t_begin = k_lo / TILE, t_end = p_max / TILE;  // inclusive
  const int num_tiles = t_end - t_begin + 1;

  constexpr int ROWS_PER_PASS = THREADS / CHUNKS * 8;
  const bool page_fast = (ps & 7) == 0;
  auto load_tile = [&](int tile, int stage) {
    unsigned char* k_dst = kv_s + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* v_dst = k_dst + TILE_BYTES;
    const int base = (t_begin + tile) * TILE;
    const int chunk = tid % CHUNKS;
    for (int r0 = (tid / CHUNKS) * 8; r0 < TILE; r0 += ROWS_PER_PASS) {
      const int j0 = base + r0;
      long src = 0;
      if (page_fast && j0 <= p_max && j0 + 8 > k_lo) {
        const int page = bt[j0 / ps];
        src = (((long)page * nkv + kvh) * ps + (j0 % ps)) * D + chunk * 8;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = j0 + i;
        const bool valid = j >= k_lo && j <= p_max;
        long s = src + (long)i * D;
        if (!page_fast && valid) {
          const int page = bt[j / ps];
          s = (((long)page * nkv + kvh) * ps + (j % ps)) * D + chunk * 8;
        }
        const int off = swz<D>(r0 + i, chunk);
        cp_async16(smem_u32(k_dst + off), kpages + (valid ? s : 0), valid ? 16 : 0);
        cp_async16(smem_u32(v_dst + off), vpages + (valid ? s : 0), valid ? 16 : 0);
      }
    }
  };

  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_tiles) load_tile(s, s);
    cp_async_commit();
  }
  __syncthreads();  // q_s complete

  uint32_t qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldmatrix_x4(qa[ks], smem_u32(q_s + swz<D>(warp * 16 + (lane & 15), 2 * ks + (lane >> 4))));

  // this thread's two rows and what they may see
  int pos[2], lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = row0 + warp * 16 + (lane >> 2) + r * 8;
    pos[r] = R < rows ? base_pos + R / G : -1;
    lo[r] = window > 0 ? max(0, pos[r] - window + 1) : 0;
  }
  // the warp's extremes (rows are in token order, so the first and last rows give them)
  const int Rw0 = row0 + warp * 16, Rw1 = min(rows, Rw0 + 16) - 1;
  const bool warp_live = Rw0 < rows;
  const int wp_min = base_pos + Rw0 / G, wp_max = warp_live ? base_pos + Rw1 / G : -1;
  const int wlo_min = window > 0 ? max(0, wp_min - window + 1) : 0;
  const int wlo_max = window > 0 ? max(0, wp_max - window + 1) : 0;

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};

  for (int tile = 0; tile < num_tiles; ++tile) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nxt = tile + STAGES - 1;
      if (nxt < num_tiles) load_tile(nxt, nxt % STAGES);
      cp_async_commit();
    }
    const int key0 = (t_begin + tile) * TILE;
    if (!warp_live || key0 > wp_max || key0 + TILE - 1 < wlo_min) continue;  // nothing for this warp
    const unsigned char* k_t = kv_s + (size_t)(tile % STAGES) * 2 * TILE_BYTES;
    const unsigned char* v_t = k_t + TILE_BYTES;

    float s[TILE / 8][4];
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int nn = 0; nn < TILE / 16; ++nn) {
        uint32_t kb[4];
        const int row = nn * 16 + (lane & 7) + ((lane >> 4) << 3);
        ldmatrix_x4(kb, smem_u32(k_t + swz<D>(row, 2 * ks + ((lane >> 3) & 1))));
        mma_bf16(s[2 * nn], qa[ks], kb[0], kb[1]);
        mma_bf16(s[2 * nn + 1], qa[ks], kb[2], kb[3]);
      }
    }
    // mask where the tile crosses the diagonal or the window's edge
    if (key0 + TILE - 1 > wp_min || key0 < wlo_max) {
#pragma unroll
      for (int n = 0; n < TILE / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + n * 8 + 2 * (lane & 3) + (e & 1);
          if (j > pos[e >> 1] || j < lo[e >> 1]) s[n][e] = -INFINITY;
        }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f((m_run[r] - m_use[r]) * scale_log2);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int n = 0; n < TILE / 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[n][e] = exp2f((s[n][e] - m_use[e >> 1]) * scale_log2);
        l_run[e >> 1] += s[n][e];
      }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
    }
#pragma unroll
    for (int kk = 0; kk < TILE / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        uint32_t vb[4];
        const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldmatrix_x4_trans(vb, smem_u32(v_t + swz<D>(row, 2 * i + (lane >> 4))));
        mma_bf16(o[2 * i], pa, vb[0], vb[1]);
        mma_bf16(o[2 * i + 1], pa, vb[2], vb[3]);
      }
    }
  }
  cp_async_wait<0>();

  // ---- normalise and store -----------------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    const int R = row0 + warp * 16 + (lane >> 2) + r * 8;
    if (R >= rows) continue;
    const int tk = R / G, hd = kvh * G + (R - tk * G);
    const float inv = 1.f / l_run[r];
    bf16* dst = out + ((long)(tok0 + tk) * nq + hd) * D + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
  }
}

template <int D>
int launch_prefill(const bf16* q, int q_stride, const bf16* kpages, const bf16* vpages, const int* block_table,
                   int max_pages, const int* kv_lens, const int* cu_seqlens, bf16* out, int num_seqs, int num_work,
                   int nq, int nkv, int ps, float scale, int window, int skip_single, cudaStream_t stream) {
  const size_t smem = (size_t)BLOCK_M * D * 2 + (size_t)STAGES * 2 * TILE * D * 2;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid(num_work, nkv);
  prefill_attention_kernel<D><<<grid, THREADS, smem, stream>>>(q, q_stride, kpages, vpages, block_table, max_pages,
                                                               kv_lens, cu_seqlens, out, num_seqs, nq, nkv, ps,
                                                               scale * 1.4426950408889634f, window, skip_single);
  return q3_launch_status();
}

}  // namespace

// num_work = sum over the sequences this launch serves of ceil(q_len * (nq / nkv) / 128).
// head_dim 64 or 128; bfloat16 only.  With skip_single, sequences of one token are left out
// (their rows of `out` are not written).
Q3_EXPORT int q3_paged_attention_prefill(const void* q, int q_stride, const void* kpages, const void* vpages,
                                         const int* block_table, int max_pages, const int* kv_lens,
                                         const int* cu_seqlens, void* out, int num_seqs, int num_work, int nq,
                                         int nkv, int D, int ps, float scale, int window, int skip_single,
                                         cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !kv_lens || !cu_seqlens || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1 || num_seqs < 0 || num_work < 0) return Q3_ERR_ARGUMENT;
  if (q_stride % 8 || nkv > 65535) return Q3_ERR_UNSUPPORTED;
  if (num_work == 0) return Q3_OK;
  if (D == 64)
    return launch_prefill<64>((const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages, block_table,
                              max_pages, kv_lens, cu_seqlens, (bf16*)out, num_seqs, num_work, nq, nkv, ps, scale,
                              window, skip_single, stream);
  if (D == 128)
    return launch_prefill<128>((const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages, block_table,
                               max_pages, kv_lens, cu_seqlens, (bf16*)out, num_seqs, num_work, nq, nkv, ps, scale,
                               window, skip_single, stream);
  return Q3_ERR_UNSUPPORTED;
}
