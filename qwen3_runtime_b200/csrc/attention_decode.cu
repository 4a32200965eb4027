// Split-KV decode attention over the paged cache, bfloat16, for sequences that bring
// exactly one query token.  Memory-bound: the job is to stream a sequence's keys and
// values once at full HBM bandwidth.
//
// Grid (split, kv head, sequence).  A block handles one slice of one sequence's keys for
// one kv head and all `group = nq / nkv` query heads that read it: the group's queries are
// the (zero-padded) 16 rows of an m16n8k16 tensor-core tile, so a key or value loaded once
// serves every head of the group (the reference's Triton kernel does the same with
// BLOCK_H = 16, kernels/triton_decode.py:280-444).  Keys and values arrive in tiles of 64
// through a 2-stage cp.async pipeline into XOR-swizzled shared memory; each of the 4 warps
// takes 16 keys of a tile, keeps its own online-softmax state (fp32, exp2 with the scale
// folded in) and the warps merge at the end.  Slots outside [lo, kv_len) are zero-filled,
// never read, so stale or poisoned pages cannot leak in.
//
// With more than one split a block writes a normalised partial result and its log-sum-exp
// to scratch (mid_o [seqs, nq, splits, D] fp32, mid_lse [seqs, nq, splits]) and the splits
// are merged (triton_decode.py:447-501): by a second kernel, or, when the caller gives a
// ticket word per (sequence, kv head), by whichever block of the pair finishes last -- it
// draws the last ticket, reads all partials back and writes the result, so no kernel has to
// start, wait for this one to drain and run just for the merge.  Slices are cut at multiples
// of 64 keys counted from the first visible key, so an empty slice writes lse = -inf.
#include "common.cuh"
#include "mma_tiles.cuh"
#include "rotary.cuh"

#define Q3_ERR_POSITION 16  // error word: a newest position outside the rotation tables

namespace {

// What the fused variant needs to make q, k and v of the newest token itself, from the raw
// output of the q/k/v projection (row layout: nq q heads, nkv k heads, nkv v heads of D):
// per-head RMSNorm weights (null: no norm), rotation tables [max_pos, D/2] (null: none) and which
// elements form a rotation pair (rotary.cuh).
struct NewToken {
  const float* q_w;
  const float* k_w;
  const float* cos_t;
  const float* sin_t;
  bf16* kpages;   // the same pages the kernel reads, writable
  bf16* vpages;
  float eps;
  int max_pos;
  int pairing;
};

constexpr int TILE = 64;     // keys per pipeline stage
constexpr int WARPS = 4;     // each takes 16 keys of a tile
constexpr int THREADS = WARPS * 32;

// ---- merge of the slices ------------------------------------------------------------------------------
// One output row: out[d] = sum_s w_s * mid_o[s][d] / sum_s w_s with w_s = 2^(lse_s - max lse), slices
// in order; a thread makes 4 consecutive values.  Shared by the merge kernel and the merge by the last
// block, so both give the same bits.  Loads go past L1 (the partials may have been written by other
// blocks of the same kernel), eight slices' loads in flight at a time; an empty slice (lse = -inf)
// never wrote its partial, which is loaded but not used.
template <int D>
__device__ __forceinline__ void merge_row(const float* __restrict__ mid_o, const float* __restrict__ lse,
                                          int num_splits, bf16* __restrict__ out_row, int first, int step) {
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, __ldcg(lse + s));
  for (int d = 4 * first; d < D; d += 4 * step) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    float wsum = 0.f;
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
      float4 v[8];
      float ls[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < num_splits) {
          ls[j] = __ldcg(lse + s0 + j);
          v[j] = __ldcg(reinterpret_cast<const float4*>(mid_o + (long)(s0 + j) * D + d));
        }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j < num_splits && ls[j] != -INFINITY) {
          const float w = exp2f(ls[j] - mx);
          wsum += w;
          acc[0] += w * v[j].x;
          acc[1] += w * v[j].y;
          acc[2] += w * v[j].z;
          acc[3] += w * v[j].w;
        }
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0] / wsum, acc[1] / wsum);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc[2] / wsum, acc[3] / wsum);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out_row + d) = packed;
  }
}

// Called by every thread of a block after its partials are written.  True in the block that
// drew the pair's last ticket: every other slice's partials are then visible to it.  That
// block puts the ticket word back to zero for the next launch.
__device__ __forceinline__ bool drew_last_ticket(int* ticket, int num_splits) {
  __shared__ int last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    last = atomicAdd(ticket, 1) == num_splits - 1;
    if (last) *ticket = 0;
  }
  __syncthreads();
  if (last) __threadfence();
  return last;
}

// The first `slices` of the `num_splits` places that each head's partial results have.
template <int D>
__device__ __forceinline__ void merge_pair(const float* __restrict__ mid_o, const float* __restrict__ mid_lse,
                                           long first_head, int G, int num_splits, int slices,
                                           bf16* __restrict__ out_rows) {
  constexpr int PER_ROW = D / 4 < 32 ? D / 4 : 32;  // threads on one row, 4 values each
  for (int g = threadIdx.x / PER_ROW; g < G; g += THREADS / PER_ROW)
    merge_row<D>(mid_o + (first_head + g) * num_splits * D, mid_lse + (first_head + g) * num_splits, slices,
                 out_rows + (long)g * D, threadIdx.x % PER_ROW, PER_ROW);
}

// The launch's slice count is made for its longest sequence.  A shorter sequence is cut into fewer
// slices of about that length (at least one), so that a batch of mixed lengths does not end up with
// many blocks of a few keys beside a few long ones.  Called by every thread of the block; `span` is
// this sequence's keys from the first visible tile on; `longest_len` (may be null) points at the
// length of the launch's longest sequence, which the blocks otherwise work out for themselves.
__device__ __forceinline__ int slices_of(const int* __restrict__ kv_lens, const int* __restrict__ seq_list,
                                         int num_seqs, int window, int num_splits, int span,
                                         const int* __restrict__ longest_len) {
  if (num_splits <= 1) return 1;
  int longest = 0;
  if (longest_len) {  // the caller knows the longest sequence of the launch: one load, nothing to agree on
    const int n = *longest_len;
    const int first = window > 0 ? max(0, n - window) : 0;
    longest = n - (first & ~(TILE - 1));
  } else {
    __shared__ int longest_of_warp[WARPS];
    for (int i = threadIdx.x; i < num_seqs; i += THREADS) {
      const int n = kv_lens[seq_list ? seq_list[i] : i];
      const int first = window > 0 ? max(0, n - window) : 0;
      longest = max(longest, n - (first & ~(TILE - 1)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
    if ((threadIdx.x & 31) == 0) longest_of_warp[threadIdx.x >> 5] = longest;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < WARPS; ++w) longest = max(longest, longest_of_warp[w]);
  }
  int slice = (longest + num_splits - 1) / num_splits;
  slice = max(TILE, (slice + TILE - 1) & ~(TILE - 1));
  return min(num_splits, max(1, (span + slice - 1) / slice));
}

// FUSED: `q` is the raw q/k/v projection; the block norms and rotates its own queries, and the
// block whose slice holds the newest position also makes that token's key and value, writes
// them to their page and patches them into its tile (q/k/v math as in rope_kv.cu, same order of
// operations, so both ways give the same bits).  Nothing the block reads before pdl_wait() is
// written by a kernel of the same step, so the first key tiles are in flight while the
// projection before this kernel is still finishing.
template <int D, bool FUSED>
__global__ void __launch_bounds__(THREADS)
decode_attention_kernel(const bf16* __restrict__ q, int q_stride, const bf16* kpages,
                        const bf16* vpages, const int* __restrict__ block_table, int max_pages,
                        const int* __restrict__ kv_lens, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ seq_list, bf16* __restrict__ out, float* __restrict__ mid_o,
                        float* __restrict__ mid_lse, int nq, int nkv, int ps, float scale_log2, int window,
                        int num_splits, int stages, NewToken nt, int* __restrict__ error_word,
                        int* __restrict__ tickets, const int* __restrict__ longest_len) {
  constexpr int CHUNKS = D / 8;
  constexpr int TILE_BYTES = TILE * D * 2;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_s = smem;                  // [16][D] bf16
  unsigned char* kv_s = smem + 16 * D * 2;    // stages x (K tile, V tile); 1024-byte aligned
  unsigned char* new_s = kv_s + (size_t)stages * 2 * TILE_BYTES;  // FUSED: the newest key, then value, [2][D]
  // after the last tile the ring is reused: the warps' results [WARPS][16][D + 8] + [WARPS][16][2]

  if (!FUSED) pdl_wait();  // keys and values of the newest token come from the kernel before this one
  const int split = blockIdx.x, kvh = blockIdx.y;
  const int slot = blockIdx.z;                // index into the partial buffers
  const int seq = seq_list ? seq_list[slot] : slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = nq / nkv;
  const int kv_len = kv_lens[seq];
  const int tok = cu_seqlens[seq];
  const int p = kv_len - 1;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int begin0 = lo & ~(TILE - 1);
  const int total = kv_len - begin0;
  const int slices = slices_of(kv_lens, seq_list, gridDim.z, window, num_splits, total, longest_len);
  if (split >= slices) return;  // a sequence shorter than the longest: fewer slices, this block has none
  int per = (total + slices - 1) / slices;
  per = (per + TILE - 1) & ~(TILE - 1);
  const int k_begin = begin0 + split * per;
  const int k_end = min(kv_len, k_begin + per);
  const int* bt = block_table + (long)seq * max_pages;

  int* ticket = tickets && slices > 1 ? tickets + (long)slot * nkv + kvh : nullptr;
  if (k_begin >= k_end) {  // nothing visible in this slice
    if (slices > 1 && tid < G)
      mid_lse[((long)slot * nq + kvh * G + tid) * num_splits + split] = -INFINITY;
    if (ticket) {
      if (FUSED) pdl_wait();  // the ticket words and `out` belong to the kernels before this one until then
      pdl_launch_dependents();
      if (drew_last_ticket(ticket, slices))
        merge_pair<D>(mid_o, mid_lse, (long)slot * nq + kvh * G, G, num_splits, slices,
                      out + ((long)tok * nq + kvh * G) * D);
    }
    return;
  }
  // FUSED: position p is not in the cache yet; its row is left out of the copies and patched in
  const bool owner = FUSED && p >= k_begin && p < k_end;
  const int skip = FUSED ? p : -1;

  // ---- the group's queries: rows 0..G-1 of a 16-row tile, the rest zero -----------------
  if (!FUSED) {
    for (int c = tid; c < 16 * CHUNKS; c += THREADS) {
      const int row = c / CHUNKS, chunk = c % CHUNKS;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < G) v = *reinterpret_cast<const uint4*>(q + (long)tok * q_stride + (long)(kvh * G + row) * D + chunk * 8);
      *reinterpret_cast<uint4*>(q_s + swz<D>(row, chunk)) = v;
    }
  } else {
    for (int c = tid; c < (16 - G) * CHUNKS; c += THREADS)
      *reinterpret_cast<uint4*>(q_s + swz<D>(G + c / CHUNKS, c % CHUNKS)) = make_uint4(0, 0, 0, 0);
  }

  const int num_tiles = (k_end - k_begin + TILE - 1) / TILE;
  // A thread copies one 16-byte chunk column of 8 consecutive keys.  When the page size is
  // a multiple of 8 those keys lie in one page: one block-table lookup per thread per tile.
  constexpr int ROWS_PER_PASS = THREADS / CHUNKS * 8;  // keys covered by one pass of the block
  const bool page_fast = (ps & 7) == 0;
  auto load_tile = [&](int tile, int stage) {
    unsigned char* k_dst = kv_s + (size_t)stage * 2 * TILE_BYTES;
    unsigned char* v_dst = k_dst + TILE_BYTES;
    const int base = k_begin + tile * TILE;
    const int chunk = tid % CHUNKS;
    for (int r0 = (tid / CHUNKS) * 8; r0 < TILE; r0 += ROWS_PER_PASS) {
      const int j0 = base + r0;
      if (page_fast) {
        long src = 0;
        if (j0 < k_end && j0 + 8 > lo) {
          const int page = bt[j0 / ps];
          src = (((long)page * nkv + kvh) * ps + (j0 % ps)) * D + chunk * 8;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = j0 + i;
          const bool valid = j >= lo && j < k_end && j != skip;
          const int off = swz<D>(r0 + i, chunk);
          cp_async16(smem_u32(k_dst + off), kpages + (valid ? src + (long)i * D : 0), valid ? 16 : 0);
          cp_async16(smem_u32(v_dst + off), vpages + (valid ? src + (long)i * D : 0), valid ? 16 : 0);
        }
      } else {
        for (int i = 0; i < 8; ++i) {
          const int j = j0 + i;
          const bool valid = j >= lo && j < k_end && j != skip;
          long src = 0;
          if (valid) {
            const int page = bt[j / ps];
            src = (((long)page * nkv + kvh) * ps + (j % ps)) * D + chunk * 8;
          }
          const int off = swz<D>(r0 + i, chunk);
          cp_async16(smem_u32(k_dst + off), kpages + src, valid ? 16 : 0);
          cp_async16(smem_u32(v_dst + off), vpages + src, valid ? 16 : 0);
        }
      }
    }
  };

  for (int s = 0; s < stages - 1; ++s) {
    if (s < num_tiles) load_tile(s, s);
    cp_async_commit();
  }
  if (FUSED) {
    pdl_wait();  // the q/k/v projection of this step
    // D/16 threads per head; a thread owns elements [8c, 8c+8) and their rotation partners
    // [8c + D/2, 8c + D/2 + 8).  Items: the group's q heads, then (owner only) the k and v head.
    constexpr int TPH = D / 16, HALF = D / 2, PER_PASS = THREADS / TPH;
    const int items = G + (owner ? 2 : 0);
    const bf16* row = q + (long)tok * q_stride;
    long cache_row = -1;
    if (owner && p / ps < max_pages) {
      const int page = bt[p / ps];
      if (page >= 0) cache_row = (((long)page * nkv + kvh) * ps + (p % ps)) * D;
    }
    // a position beyond the tables is reported, not rotated with another position's angles
    const bool rotate = nt.cos_t && p < nt.max_pos;
    if (nt.cos_t && !rotate && tid == 0 && error_word) atomicExch(error_word, Q3_ERR_POSITION);
    for (int base = 0; base < items; base += PER_PASS) {
      const int item = base + tid / TPH, c = tid % TPH;
      const bool live = item < items;
      const bool is_q = item < G, is_v = item == G + 1;
      const bf16* x = row + (is_q ? (long)(kvh * G + item) * D
                                  : (long)(nq + (is_v ? nkv : 0) + kvh) * D);
      float a[8], b[8];
      if (live) {
        load8(x + 8 * c, a);
        load8(x + HALF + 8 * c, b);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = b[e] = 0.f;
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
      for (int o = TPH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (!live) continue;
      if (!is_v) {
        const float* w = is_q ? nt.q_w : nt.k_w;
        if (w) {
          const float rstd = rsqrtf(ss / (float)D + nt.eps);
          float wa[8], wb[8];
          load8(w + 8 * c, wa);
          load8(w + HALF + 8 * c, wb);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            a[e] = (a[e] * rstd) * wa[e];
            b[e] = (b[e] * rstd) * wb[e];
          }
        }
        if (rotate)
          rotate_chunks(a, b, nt.cos_t + (long)p * HALF, nt.sin_t + (long)p * HALF, c, HALF, nt.pairing);
      }
      if (is_q) {
        store8(reinterpret_cast<bf16*>(q_s + swz<D>(item, c)), a);
        store8(reinterpret_cast<bf16*>(q_s + swz<D>(item, CHUNKS / 2 + c)), b);
      } else {
        bf16* side = reinterpret_cast<bf16*>(new_s) + (is_v ? D : 0);
        store8(side + 8 * c, a);
        store8(side + HALF + 8 * c, b);
        if (cache_row >= 0) {
          bf16* dst = (is_v ? nt.vpages : nt.kpages) + cache_row;
          store8(dst + 8 * c, a);
          store8(dst + HALF + 8 * c, b);
        }
      }
    }
  }
  __syncthreads();  // q_s (and the newest key and value) are complete

  uint32_t qa[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldmatrix_x4(qa[ks], smem_u32(q_s + swz<D>(lane & 15, 2 * ks + (lane >> 4))));

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};  // rows lane/4 and lane/4 + 8, in units of raw scores
  float l_run[2] = {0.f, 0.f};              // this thread's share of the row sums

  for (int tile = 0; tile < num_tiles; ++tile) {
    if (stages == 2) cp_async_wait<0>(); else cp_async_wait<1>();
    __syncthreads();
    {
      const int nxt = tile + stages - 1;
      if (nxt < num_tiles) load_tile(nxt, nxt % stages);
      cp_async_commit();
    }
    unsigned char* k_t = kv_s + (size_t)(tile % stages) * 2 * TILE_BYTES;
    unsigned char* v_t = k_t + TILE_BYTES;
    {
      const int base = k_begin + tile * TILE;
      if (FUSED && owner && tile == (p - k_begin) / TILE) {  // (uniform over the block)
        const int r = p - base;
        for (int c = tid; c < 2 * CHUNKS; c += THREADS) {
          const int chunk = c % CHUNKS;
          const uint4 v = *reinterpret_cast<const uint4*>(new_s + (c / CHUNKS) * D * 2 + chunk * 16);
          *reinterpret_cast<uint4*>((c < CHUNKS ? k_t : v_t) + swz<D>(r, chunk)) = v;
        }
        __syncthreads();
      }
    }
    const int key0 = k_begin + tile * TILE + warp * 16;  // this warp's 16 keys
    if (key0 >= k_end) continue;                          // (uniform per warp)

    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t kb[4];
      const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
      ldmatrix_x4(kb, smem_u32(k_t + swz<D>(row, 2 * ks + ((lane >> 3) & 1))));
      mma_bf16(s[0], qa[ks], kb[0], kb[1]);
      mma_bf16(s[1], qa[ks], kb[2], kb[3]);
    }
    // mask, running max
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = key0 + n * 8 + 2 * (lane & 3) + (e & 1);
        if (j < lo || j >= k_end) s[n][e] = -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[n][e]);
      }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;
      corr[r] = exp2f((m_run[r] - m_use[r]) * scale_log2);  // m_run = -inf -> 0
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
    uint32_t pa[4];
    {
      float pv[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          pv[n][e] = exp2f((s[n][e] - m_use[e >> 1]) * scale_log2);
          l_run[e >> 1] += pv[n][e];
        }
      pa[0] = pack_bf16(pv[0][0], pv[0][1]);
      pa[1] = pack_bf16(pv[0][2], pv[0][3]);
      pa[2] = pack_bf16(pv[1][0], pv[1][1]);
      pa[3] = pack_bf16(pv[1][2], pv[1][3]);
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {  // the running max moved
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0]; o[i][1] *= corr[0];
        o[i][2] *= corr[1]; o[i][3] *= corr[1];
      }
    }
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      uint32_t vb[4];
      const int row = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      ldmatrix_x4_trans(vb, smem_u32(v_t + swz<D>(row, 2 * i + (lane >> 4))));
      mma_bf16(o[2 * i], pa, vb[0], vb[1]);
      mma_bf16(o[2 * i + 1], pa, vb[2], vb[3]);
    }
  }

  // ---- merge the 4 warps ------------------------------------------------------------------
  pdl_launch_dependents();
  cp_async_wait<0>();
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  // rows of D + 8 floats: the 8 rows that a warp stores at once then fall into different banks
  constexpr int OS = D + 8;
  float* o_s = reinterpret_cast<float*>(kv_s);          // [WARPS][16][OS]
  float* ml_s = o_s + WARPS * 16 * OS;                  // [WARPS][16][2]
  {
    const int r0 = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      float* base = o_s + ((size_t)warp * 16) * OS + i * 8 + c0;
      *reinterpret_cast<float2*>(base + (size_t)r0 * OS) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(base + (size_t)(r0 + 8) * OS) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
      ml_s[(warp * 16 + r0) * 2] = m_run[0];
      ml_s[(warp * 16 + r0) * 2 + 1] = l_run[0];
      ml_s[(warp * 16 + r0 + 8) * 2] = m_run[1];
      ml_s[(warp * 16 + r0 + 8) * 2 + 1] = l_run[1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += THREADS) {
    const int g = idx / D, d = idx - g * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, ml_s[(w * 16 + g) * 2]);
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float mw = ml_s[(w * 16 + g) * 2];
      const float f = mw == -INFINITY ? 0.f : exp2f((mw - m) * scale_log2);
      l += ml_s[(w * 16 + g) * 2 + 1] * f;
      acc += o_s[((size_t)w * 16 + g) * OS + d] * f;
    }
    const int head = kvh * G + g;
    const float val = acc / l;
    if (slices == 1) {
      out[((long)tok * nq + head) * D + d] = __float2bfloat16_rn(val);
    } else {
      mid_o[(((long)slot * nq + head) * num_splits + split) * D + d] = val;
      if (d == 0) mid_lse[((long)slot * nq + head) * num_splits + split] = m * scale_log2 + log2f(l);
    }
  }
  if (ticket && drew_last_ticket(ticket, slices))
    merge_pair<D>(mid_o, mid_lse, (long)slot * nq + kvh * G, G, num_splits, slices,
                  out + ((long)tok * nq + kvh * G) * D);
}

// The merge as a kernel of its own: one block per (kv head, sequence).
template <int D>
__global__ void __launch_bounds__(THREADS)
decode_combine_kernel(const float* __restrict__ mid_o, const float* __restrict__ mid_lse,
                      const int* __restrict__ kv_lens, const int* __restrict__ cu_seqlens,
                      const int* __restrict__ seq_list, bf16* __restrict__ out, int nq, int nkv, int window,
                      int num_splits, const int* __restrict__ longest_len) {
  pdl_wait();
  pdl_launch_dependents();
  const int slot = blockIdx.y, kvh = blockIdx.x;
  const int seq = seq_list ? seq_list[slot] : slot;
  const int tok = cu_seqlens[seq];
  const int G = nq / nkv;
  const int kv_len = kv_lens[seq];
  const int lo = window > 0 ? max(0, kv_len - window) : 0;
  const int slices =
      slices_of(kv_lens, seq_list, gridDim.y, window, num_splits, kv_len - (lo & ~(TILE - 1)), longest_len);
  if (slices == 1) return;  // a sequence in one slice: its block wrote the result itself
  merge_pair<D>(mid_o, mid_lse, (long)slot * nq + kvh * G, G, num_splits, slices,
                out + ((long)tok * nq + kvh * G) * D);
}

template <int D, bool FUSED>
int launch_decode(const bf16* q, int q_stride, const bf16* kpages, const bf16* vpages, const int* block_table,
                  int max_pages, const int* kv_lens, const int* cu_seqlens, const int* seq_list, bf16* out,
                  float* mid_o, float* mid_lse, int num_seqs, int nq, int nkv, int ps, float scale, int window,
                  int num_splits, const NewToken& nt, int* error_word, int* tickets, const int* longest_len,
                  cudaStream_t stream) {
  const int stages = 2;  // more stages mean fewer blocks per SM; measured equal at best
  const size_t pipe = (size_t)stages * 2 * TILE * D * 2;
  const size_t merge = (size_t)WARPS * 16 * (D + 8) * 4 + WARPS * 16 * 2 * 4;
  const size_t smem = 16 * D * 2 + (FUSED ? 2 * D * 2 : 0) + (pipe > merge ? pipe : merge);
  if (smem > 227 * 1024) return Q3_ERR_UNSUPPORTED;
  if (num_splits > 1 && (!mid_o || !mid_lse)) return Q3_ERR_ARGUMENT;
  if (((uintptr_t)out & 7) || ((uintptr_t)mid_o & 15)) return Q3_ERR_UNSUPPORTED;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(decode_attention_kernel<D, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid(num_splits, nkv, num_seqs);
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int n = 0;
    if (q3_pdl_enabled()) {
      attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const float scale_log2 = scale * 1.4426950408889634f;
    if (cudaLaunchKernelEx(&cfg, decode_attention_kernel<D, FUSED>, q, q_stride, kpages, vpages, block_table,
                           max_pages, kv_lens, cu_seqlens, seq_list, out, mid_o, mid_lse, nq, nkv, ps, scale_log2,
                           window, num_splits, stages, nt, error_word, tickets, longest_len) != cudaSuccess)
      return Q3_ERR_LAUNCH;
  }
  if (num_splits > 1 && !tickets) {
    dim3 cgrid(nkv, num_seqs);
    if (launch_pdl(decode_combine_kernel<D>, cgrid, dim3(THREADS), 0, stream, (const float*)mid_o,
                   (const float*)mid_lse, kv_lens, cu_seqlens, seq_list, out, nq, nkv, window, num_splits,
                   longest_len) != cudaSuccess)
      return Q3_ERR_LAUNCH;
  }
  return Q3_OK;
}

template <bool FUSED>
int dispatch_decode(const void* q, int q_stride, const void* kpages, const void* vpages, const int* block_table,
                    int max_pages, const int* kv_lens, const int* cu_seqlens, const int* seq_list, void* out,
                    float* mid_o, float* mid_lse, int num_seqs, int nq, int nkv, int D, int ps, float scale,
                    int window, int num_splits, const NewToken& nt, int* error_word, int* tickets,
                    const int* longest_len, cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !kv_lens || !cu_seqlens || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1 || num_splits < 1) return Q3_ERR_ARGUMENT;
  if (nq / nkv > 16 || q_stride % 8) return Q3_ERR_UNSUPPORTED;
  if (num_seqs == 0) return Q3_OK;
  if (num_seqs > 65535 || nkv > 65535) return Q3_ERR_UNSUPPORTED;
#define Q3_DECODE_CASE(DIM)                                                                                       \
  case DIM:                                                                                                       \
    return launch_decode<DIM, FUSED>((const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages,          \
                                     block_table, max_pages, kv_lens, cu_seqlens, seq_list, (bf16*)out, mid_o,    \
                                     mid_lse, num_seqs, nq, nkv, ps, scale, window, num_splits, nt, error_word,   \
                                     tickets, longest_len, stream)
  switch (D) {
    Q3_DECODE_CASE(64);
    Q3_DECODE_CASE(128);
    Q3_DECODE_CASE(256);
    default:
      return Q3_ERR_UNSUPPORTED;
  }
#undef Q3_DECODE_CASE
}

}  // namespace

// Attention for `num_seqs` one-token sequences: those listed in seq_list (indices into
// kv_lens / cu_seqlens / block_table rows), or sequences 0..num_seqs-1 when it is null.
// Scratch: mid_o needs num_seqs*nq*num_splits*D floats and mid_lse num_seqs*nq*num_splits
// floats when num_splits > 1 (both may be null otherwise).  head_dim 64, 128 or 256;
// group size nq/nkv at most 16; bfloat16 only.
// tickets: null, or num_seqs * nkv ints that are zero before the call (and again after it): with
// them the slices of a sequence and kv head are merged by whichever of their blocks finishes
// last, without them by a second kernel; the bits are the same.  Calls that share ticket words
// must not overlap (one stream, or words of their own).
// num_splits is the slice count of the longest sequence; a shorter one is cut into fewer slices of
// about the same length.  longest_len: null, or a device pointer to the length of the longest of the
// `num_seqs` sequences (saves every block working it out from kv_lens).
Q3_EXPORT int q3_paged_attention_decode(const void* q, int q_stride, const void* kpages, const void* vpages,
                                        const int* block_table, int max_pages, const int* kv_lens,
                                        const int* cu_seqlens, const int* seq_list, void* out, float* mid_o,
                                        float* mid_lse, int num_seqs, int nq, int nkv, int D, int ps, float scale,
                                        int window, int num_splits, int* tickets, const int* longest_len,
                                        cudaStream_t stream) {
  return dispatch_decode<false>(q, q_stride, kpages, vpages, block_table, max_pages, kv_lens, cu_seqlens, seq_list,
                                out, mid_o, mid_lse, num_seqs, nq, nkv, D, ps, scale, window, num_splits, NewToken{},
                                nullptr, tickets, longest_len, stream);
}

// The same, with the work of q3_qk_norm_rope_store folded in: `qkv` is the raw output of the
// q/k/v projection (rows of nq + 2*nkv heads); each sequence's newest position is
// kv_lens[seq] - 1.  q_w / k_w (per-head RMSNorm weights, fp32 [D]) and cos_t / sin_t
// ([max_pos, D/2], rotation over the whole head; `pairing` as in q3_qk_norm_rope_store) may be
// null.  The key and value of the newest token are written to their pages; q is not written
// back.  `error_word` (may be null) is set to Q3_ERR_POSITION if a newest position lies beyond
// the tables; that token is then left unrotated and the result is invalid.
Q3_EXPORT int q3_paged_attention_decode_fused(const void* qkv, int q_stride, void* kpages, void* vpages,
                                              const int* block_table, int max_pages, const int* kv_lens,
                                              const int* cu_seqlens, const int* seq_list, void* out, float* mid_o,
                                              float* mid_lse, int num_seqs, int nq, int nkv, int D, int ps,
                                              float scale, int window, int num_splits, const float* q_w,
                                              const float* k_w, float eps, const float* cos_t, const float* sin_t,
                                              int max_pos, int pairing, int* error_word, int* tickets,
                                              const int* longest_len, cudaStream_t stream) {
  if ((cos_t && (!sin_t || max_pos < 1)) || (!q_w) != (!k_w) || pairing < 0 || pairing > 1) return Q3_ERR_ARGUMENT;
  const uintptr_t bits = (uintptr_t)qkv | (uintptr_t)kpages | (uintptr_t)vpages | (uintptr_t)q_w | (uintptr_t)k_w |
                         (uintptr_t)cos_t | (uintptr_t)sin_t;
  if (bits & 15) return Q3_ERR_UNSUPPORTED;
  NewToken nt{q_w, k_w, cos_t, sin_t, (bf16*)kpages, (bf16*)vpages, eps, max_pos, pairing};
  return dispatch_decode<true>(qkv, q_stride, kpages, vpages, block_table, max_pages, kv_lens, cu_seqlens, seq_list,
                               out, mid_o, mid_lse, num_seqs, nq, nkv, D, ps, scale, window, num_splits, nt,
                               error_word, tickets, longest_len, stream);
}

// ---------------------------------------------------------------------------------------------
// The same attention for callers that may not allocate: the slices' partial results live in
// a fixed array inside this library.  See no_alloc.h for who needs this and for the rules
// (shared array, first call outside stream capture, overlapping calls race).
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"
#include <mutex>
#include <stdio.h>

static __device__ __align__(256) float q3_no_alloc_scratch[Q3_NO_ALLOC_SCRATCH_FLOATS];

namespace {
constexpr int NO_ALLOC_MAX_DEVICES = 64;
float* g_no_alloc_ptr[NO_ALLOC_MAX_DEVICES];  // device address of the array, per device, once known
std::mutex g_no_alloc_mutex;
thread_local char g_no_alloc_error[256] = "";

// In host code `q3_no_alloc_scratch` is only a handle for the runtime, not an address a kernel
// can use; the address on the current device comes from cudaGetSymbolAddress.
int no_alloc_scratch(float** ptr) {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= NO_ALLOC_MAX_DEVICES) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "no current CUDA device (or device index above %d)",
             NO_ALLOC_MAX_DEVICES - 1);
    return Q3_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
  if (!g_no_alloc_ptr[device]) {
    void* address = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&address, q3_no_alloc_scratch);
    if (err != cudaSuccess || !address) {
      snprintf(g_no_alloc_error, sizeof g_no_alloc_error, "cudaGetSymbolAddress failed on device %d: %s", device,
               cudaGetErrorString(err));
      return Q3_ERR_LAUNCH;
    }
    g_no_alloc_ptr[device] = static_cast<float*>(address);
  }
  *ptr = g_no_alloc_ptr[device];
  return Q3_OK;
}
}  // namespace

Q3_EXPORT const char* q3_no_alloc_last_error(void) { return g_no_alloc_error; }

Q3_EXPORT int q3_paged_attention_decode_no_alloc(const void* q, int q_stride, const void* kpages, const void* vpages,
                                                 const int* block_table, int max_pages, const int* kv_lens,
                                                 const int* cu_seqlens, const int* seq_list, void* out, int num_seqs,
                                                 int nq, int nkv, int D, int ps, float scale, int window,
                                                 int num_splits, cudaStream_t stream) {
  g_no_alloc_error[0] = '\0';
  if (num_seqs < 0 || nq < 1 || nkv < 1 || nq % nkv || D < 1 || ps < 1 || window < 0 || num_splits < 1) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error,
             "decode attention without allocation: bad sizes (num_seqs=%d nq=%d nkv=%d D=%d page_size=%d window=%d "
             "num_splits=%d): counts must be positive, nq a multiple of nkv, the window zero (none) or positive",
             num_seqs, nq, nkv, D, ps, window, num_splits);
    return Q3_ERR_ARGUMENT;
  }
  const long long partials = (long long)num_seqs * nq * num_splits;
  const long long need = partials * ((long long)D + 1);
  if (need > Q3_NO_ALLOC_SCRATCH_FLOATS) {
    snprintf(g_no_alloc_error, sizeof g_no_alloc_error,
             "decode attention without allocation: %d sequences x %d heads x %d slices x (%d + 1) = %lld floats "
             "of scratch, but the fixed array holds %d; use fewer slices or the allocating entry point",
             num_seqs, nq, num_splits, D, need, Q3_NO_ALLOC_SCRATCH_FLOATS);
    return Q3_ERR_SCRATCH_TOO_SMALL;
  }
  float* scratch = nullptr;
  const int status = no_alloc_scratch(&scratch);
  if (status != Q3_OK) return status;
  float* mid_o = scratch;                  // [num_seqs, nq, num_splits, D]
  float* mid_lse = scratch + partials * D; // [num_seqs, nq, num_splits]
  return q3_paged_attention_decode(q, q_stride, kpages, vpages, block_table, max_pages, kv_lens, cu_seqlens,
                                   seq_list, out, mid_o, mid_lse, num_seqs, nq, nkv, D, ps, scale, window,
                                   num_splits, nullptr, nullptr, stream);
}
