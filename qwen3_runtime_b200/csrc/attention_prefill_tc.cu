// Causal attention of prompt portions over the paged cache on the 5th-generation tensor
// cores: S = Q K^T and O += P V are tcgen05.mma with accumulators in tensor memory, Q, K and V
// tiles arrive by TMA (128-byte swizzle) straight from the QKV buffer and the cache pages.
// bfloat16, head_dim 128, group size a divisor of 128, page size 8/16/32/64, no window; the
// mma.sync kernel of attention_prefill.cu serves everything else.
//
// Work item: (sequence, kv head, two consecutive blocks of 128 rows, A and B); rows are the
// (query token, head of the group) pairs in token-major order, so one 3-D TMA box
// [128/G tokens, G heads, 64] is half a Q tile and the group's heads share every K/V tile.  Keys
// come in tiles of 64 (64/page_size pages, one TMA box per page and half of D), and each tile
// is used by both row blocks.  Per 64-key tile a row block's chain is long (TMEM load, exp2
// on the special-function unit, shared-memory stores, fences, barrier round trips) and
// leaves the tensor core and the exp2 unit idle most of the time; two blocks in flight hide
// each other's chain.  Eleven warps:
//   warp 0           : TMA producer (Q of both blocks once, then K and V tiles through 3-stage
//                      rings; the lanes issue a tile's page boxes side by side);
//   warps 1 and 10,  : MMA issuers of block A and of block B.  Order per block: S_0, S_1, then
//   one lane each      per tile j: P_j ready -> PV_j, S_(j+2).  S has two TMEM buffers per block,
//                      so the tensor core works for one block while the other block's softmax
//                      runs;
//   warps 2..5, 6..9 : softmax of block A and of block B, one thread per row: reads S from
//                      TMEM, masks, online softmax in fp32 (exp2, scale folded in), writes P
//                      (bf16) to shared memory (two buffers per block) in the swizzled K-major
//                      layout that the PV MMA reads; O stays in TMEM (the MMAs accumulate into
//                      it) and is rescaled there only when a row's maximum has grown by more
//                      than 2^8; finally stores O / l.
// Tensor memory: all 512 columns, per block S0 [0,64), S1 [64,128), O [128,256).
// V is the B operand of PV in MN-major form (rows = keys): descriptor with the halves of D
// 8 KB apart (leading offset) and 8-key groups 1 KB apart (stride offset); 16 keys = 2 KB.
// Keys past a block's last position are zeroed in shared memory before PV (stale or poisoned
// page contents must not meet a zero probability).  Every mbarrier wait is bounded; on expiry
// the block raises its abort flag and the global error word, frees TMEM and returns.
#include "async_tiles.cuh"

namespace {

constexpr int D = 128;
constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 64;
constexpr int THREADS = 352;
constexpr int Q_BYTES = BLOCK_M * D * 2;        // 32 KB: two halves of [128 rows][128 B]
constexpr int KV_BYTES = BLOCK_N * D * 2;       // 16 KB: two halves of [64 rows][128 B]
constexpr int P_BYTES = BLOCK_M * BLOCK_N * 2;  // 16 KB: [128 rows][128 B]
constexpr int KV_STAGES = 3;                    // key tiles and value tiles in flight
constexpr int SMEM_BYTES = 2 * Q_BYTES + 2 * KV_STAGES * KV_BYTES + 4 * P_BYTES + 1024;
constexpr int TMEM_COLS = 512;                  // per row block: S0 [0,64), S1 [64,128), O [128,256)
constexpr int TMEM_BLOCK = 256;

// 2^x in one instruction (exp2f adds range fix-ups around the same instruction; results
// below 2^-126 become zero here, which is what a probability that small is worth)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

enum { BAR_Q = 0, BAR_K_FULL = 1, BAR_K_EMPTY = BAR_K_FULL + KV_STAGES, BAR_V_FULL = BAR_K_EMPTY + KV_STAGES,
       BAR_V_EMPTY = BAR_V_FULL + KV_STAGES, BAR_S_FULL = BAR_V_EMPTY + KV_STAGES,  // [block][buffer]
       BAR_P_FULL = BAR_S_FULL + 4, BAR_PV_FULL = BAR_P_FULL + 2, NUM_BARS = BAR_PV_FULL + 2 };

__global__ void __launch_bounds__(THREADS, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                            const __grid_constant__ CUtensorMap tmap_v, const int* __restrict__ block_table,
                            int max_pages, const int* __restrict__ kv_lens, const int* __restrict__ cu_seqlens,
                            bf16* __restrict__ out, int num_seqs, int num_work, int nq, int nkv, int ps,
                            float scale_log2, int skip_single, int* __restrict__ error_word) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;                         // 2 blocks x [2 halves][128 rows][128 B]
  unsigned char* k_s = q_s + 2 * Q_BYTES;            // KV_STAGES x [2 halves][64 rows][128 B]
  unsigned char* v_s = k_s + KV_STAGES * KV_BYTES;   // KV_STAGES x [2 halves][64 rows][128 B]
  unsigned char* p_s = v_s + KV_STAGES * KV_BYTES;   // 2 blocks x 2 buffers x [128 rows][128 B]
  __shared__ __align__(8) unsigned long long bars[NUM_BARS];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;
  __shared__ int s_item[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // heavy items first over the whole grid: all kv heads of the heaviest item, then the next ...
  const int kvh = blockIdx.x % nkv;
  const int G = nq / nkv;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

  if (tid == 0) {
    abort_flag = 0;
    // heavy work (late rows of long prompts) first: walk the work list from its end
    int acc = 0, found = -1, rb = 0;
    const int w = num_work - 1 - (int)(blockIdx.x / nkv);
    for (int s = 0; s < num_seqs; ++s) {
      const int ql = cu_seqlens[s + 1] - cu_seqlens[s];
      if (ql <= 0 || (skip_single && ql == 1)) continue;
      const int nb = ((ql * G + BLOCK_M - 1) / BLOCK_M + 1) / 2;  // pairs of row blocks
      if (w < acc + nb) {
        found = s;
        rb = w - acc;
        break;
      }
      acc += nb;
    }
    s_item[0] = found;
    s_item[1] = rb;
    mbar_init(bar(BAR_Q), 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(bar(BAR_K_FULL + i), 1);
      mbar_init(bar(BAR_K_EMPTY + i), 2);  // both issuers
      mbar_init(bar(BAR_V_FULL + i), 1);
      mbar_init(bar(BAR_V_EMPTY + i), 2);
    }
    for (int i = 0; i < 4; ++i) mbar_init(bar(BAR_S_FULL + i), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(BAR_P_FULL + i), 128);
      mbar_init(bar(BAR_PV_FULL + i), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  const int seq = s_item[0];

  if (seq >= 0) {
    const int tok0 = cu_seqlens[seq];
    const int q_len = cu_seqlens[seq + 1] - tok0;
    const int kv_len = kv_lens[seq];
    const int rows = q_len * G;
    const int base_pos = kv_len - q_len;
    // row blocks A and B of this item; B may not exist (odd number of blocks)
    int row0[2], p_max[2], tiles[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      row0[x] = (2 * s_item[1] + x) * BLOCK_M;
      const bool live = row0[x] < rows;
      const int last_row = min(rows, row0[x] + BLOCK_M) - 1;
      p_max[x] = live ? base_pos + last_row / G : -1;
      tiles[x] = live ? p_max[x] / BLOCK_N + 1 : 0;
    }
    const int num_tiles = max(tiles[0], tiles[1]);  // B lies after A, so this is B's count when B exists
    const int p_last = max(p_max[0], p_max[1]);
    const int* bt = block_table + (long)seq * max_pages;
    const int pages_per_tile = BLOCK_N / ps;

    if (warp == 0) {  // ---- TMA producer: lane 0 waits and arms the barriers, the lanes share the loads ----
      if (lane == 0) {
        mbar_expect_tx(bar(BAR_Q), tiles[1] ? 2 * Q_BYTES : Q_BYTES);
        for (int x = 0; x < 2; ++x) {
          if (!tiles[x]) continue;
          const uint32_t dst = smem_addr(q_s) + x * Q_BYTES;
          tma_load_3d(dst, &tmap_q, bar(BAR_Q), 0, kvh * G, tok0 + row0[x] / G);
          tma_load_3d(dst + Q_BYTES / 2, &tmap_q, bar(BAR_Q), 64, kvh * G, tok0 + row0[x] / G);
        }
      }
      // a tile is 64 / ps pages x 2 halves of D: one box per lane (small boxes are slow to issue
      // one after another from a single thread)
      const int my_page = lane >> 1, my_half = lane & 1;
      int ok = 1;
      for (int j = 0; j < num_tiles && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t phase = (j / KV_STAGES) & 1;
        // pages of this tile that exist in the block table (the rest of the tile is masked)
        int page = -1;
        if (my_page < pages_per_tile) {
          const int pi = j * pages_per_tile + my_page;
          if (pi < max_pages && pi * ps <= p_last) page = bt[pi];
        }
        const uint32_t boxes = __popc(__ballot_sync(0xffffffffu, page >= 0));
        const uint32_t bytes = boxes * (uint32_t)ps * 128u;
        const int y = (page * nkv + kvh) * ps;
        const uint32_t off = st * KV_BYTES + my_half * (KV_BYTES / 2) + my_page * ps * 128;
        // keys
        if (lane == 0) {
          ok = mbar_wait(bar(BAR_K_EMPTY + st), phase ^ 1, &abort_flag);
          if (ok) mbar_expect_tx(bar(BAR_K_FULL + st), bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (page >= 0) tma_load_2d(smem_addr(k_s) + off, &tmap_k, bar(BAR_K_FULL + st), my_half * 64, y);
        // values
        if (lane == 0) {
          ok = mbar_wait(bar(BAR_V_EMPTY + st), phase ^ 1, &abort_flag);
          if (ok) mbar_expect_tx(bar(BAR_V_FULL + st), bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (page >= 0) tma_load_2d(smem_addr(v_s) + off, &tmap_v, bar(BAR_V_FULL + st), my_half * 64, y);
      }
    } else if (warp == 1 || warp == 10) {
      if (lane == 0) {  // ---- MMA issuers: warp 1 for block A, warp 10 for block B ------------------
        // Issuing is work too (descriptors, a dozen instructions per tile and block, barrier round
        // trips), so each block has its own issuing thread.  Both use every K and V tile: its
        // "empty" barrier counts two arrivals, a commit from an issuer that multiplied with the
        // tile and a plain arrival (after the tile's "full") from one that had no use for it.
        const int x = warp == 1 ? 0 : 1;
        const int my_tiles = tiles[x];
        constexpr uint32_t idesc_s = umma_idesc(BLOCK_M, BLOCK_N, 0);   // S = Q K^T: N = 64 keys
        constexpr uint32_t idesc_pv = umma_idesc(BLOCK_M, D, 1);        // PV: N = 128, V MN-major
        const uint32_t p_addr = smem_addr(p_s) + 2 * x * P_BYTES;
        const uint32_t q_addr = smem_addr(q_s) + x * Q_BYTES;
        const uint32_t tmem_x = tmem + x * TMEM_BLOCK;
        // S_j into TMEM buffer j & 1, or just the hand-back of key tile j
        auto keys = [&](int j) -> bool {
          const int st = j % KV_STAGES, sbuf = j & 1;
          if (!mbar_wait(bar(BAR_K_FULL + st), (j / KV_STAGES) & 1, &abort_flag)) return false;
          if (j >= my_tiles) {
            mbar_arrive(bar(BAR_K_EMPTY + st));
            return true;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t k_addr = smem_addr(k_s) + st * KV_BYTES;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t half = (k >> 2), sub = (k & 3) * 2;  // 4 steps of 32 bytes per 64-wide half
            umma_bf16(tmem_x + sbuf * BLOCK_N, umma_desc(q_addr + half * (Q_BYTES / 2)) + sub,
                 umma_desc(k_addr + half * (KV_BYTES / 2)) + sub, idesc_s, k > 0 ? 1u : 0u);
          }
          umma_commit(bar(BAR_K_EMPTY + st));           // this block is done with the key tile
          umma_commit(bar(BAR_S_FULL + 2 * x + sbuf));  // S_j is in TMEM
          return true;
        };
        bool ok = my_tiles == 0 || mbar_wait(bar(BAR_Q), 0, &abort_flag);
        for (int j = 0; j < 2 && j < num_tiles && ok; ++j) ok = keys(j);
        for (int j = 0; j < num_tiles && ok; ++j) {
          const int st = j % KV_STAGES, pbuf = j & 1;
          if (j < my_tiles) {
            ok = mbar_wait(bar(BAR_P_FULL + x), j & 1, &abort_flag);  // P_j written, S_j and PV_{j-1} consumed
            if (!ok) break;
          }
          ok = mbar_wait(bar(BAR_V_FULL + st), (j / KV_STAGES) & 1, &abort_flag);
          if (!ok) break;
          if (j < my_tiles) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t v_addr = smem_addr(v_s) + st * KV_BYTES;
#pragma unroll
            for (int k = 0; k < BLOCK_N / 16; ++k)  // 16 keys: 32 bytes along P's rows, 2 KB down V's rows
              umma_bf16(tmem_x + 2 * BLOCK_N, umma_desc(p_addr + pbuf * P_BYTES) + 2 * k,
                   umma_desc_mn_major(v_addr + k * 2048, KV_BYTES / 2), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
            umma_commit(bar(BAR_V_EMPTY + st));
            umma_commit(bar(BAR_PV_FULL + x));
          } else {
            mbar_arrive(bar(BAR_V_EMPTY + st));
          }
          if (j + 2 < num_tiles) ok = keys(j + 2);  // its TMEM buffer (j & 1) was read before P_j was signalled
        }
      }
    } else {  // ---- softmax: one thread per row; warps 2..5 block A, warps 6..9 block B ---------------
      const int x = (warp - 2) >> 2;
      const int quarter = warp & 3;
      const int r = quarter * 32 + lane;  // row of the tile = TMEM lane
      const int R = row0[x] + r;
      const bool row_ok = R < rows;
      const int pos = row_ok ? base_pos + R / G : -1;
      const int my_tiles = tiles[x];
      const uint32_t lane_base = tmem + x * TMEM_BLOCK + ((uint32_t)(quarter * 32) << 16);
      const uint32_t o_addr = lane_base + 2 * BLOCK_N;
      // O stays in TMEM and the MMAs accumulate into it.  The reference point of the exponentials
      // (m_ref) is only moved when a row's maximum exceeds it by more than 2^8 after scaling; then
      // O and l are rescaled.  Probabilities may therefore reach 2^8, which bf16 and fp32 hold easily,
      // and the final O / l is unchanged.
      const float slack = 8.f / scale_log2;
      float m_ref = -INFINITY, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const int st = j & 1;             // S buffer and P buffer of this tile
        const int vst = j % KV_STAGES;    // its value tile
        ok = mbar_wait(bar(BAR_S_FULL + 2 * x + st), (j >> 1) & 1, &abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t sa[32], sb[32];
        tmem_load32(lane_base + st * BLOCK_N, sa);
        tmem_load32(lane_base + st * BLOCK_N + 32, sb);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int key0 = j * BLOCK_N;
        float mx = -INFINITY;
        if (key0 + BLOCK_N - 1 > pos) {  // the tile crosses this row's diagonal
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            if (key0 + c > pos) sa[c] = 0xff800000u;       // -inf
            if (key0 + 32 + c > pos) sb[c] = 0xff800000u;
          }
        }
        {  // eight independent running maxima: a single chain of 64 would expose its latency
          float part[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) part[c] = fmaxf(__uint_as_float(sa[c]), __uint_as_float(sb[c]));
#pragma unroll
          for (int c = 8; c < 32; ++c)
            part[c & 7] = fmaxf(part[c & 7], fmaxf(__uint_as_float(sa[c]), __uint_as_float(sb[c])));
          mx = fmaxf(fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])),
                     fmaxf(fmaxf(part[4], part[5]), fmaxf(part[6], part[7])));
        }
        float corr = 1.f;
        if (mx > m_ref + slack || (m_ref == -INFINITY && mx > -INFINITY)) {
          corr = m_ref == -INFINITY ? 0.f : exp2f((m_ref - mx) * scale_log2);
          m_ref = mx;
        }
        const bool rescale = __any_sync(0xffffffffu, corr != 1.f) && j > 0;
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        // probabilities, rounded to bf16 as the MMA will see them, into the swizzled P tile; the
        // scaling and the row sum run on pairs of elements (packed fp32 instructions)
        float2 sums[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        unsigned char* p_row = p_s + (2 * x + st) * P_BYTES + r * 128;  // buffer j & 1: PV_{j-1} may still read the other
        const float2 scale2 = make_float2(scale_log2, scale_log2);
        const float2 neg2 = make_float2(-m_use * scale_log2, -m_use * scale_log2);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = ch * 8 + 2 * e;
            const float2 s2 = make_float2(__uint_as_float(c < 32 ? sa[c] : sb[c - 32]),
                                          __uint_as_float(c + 1 < 32 ? sa[c + 1] : sb[c + 1 - 32]));
            const float2 t2 = __ffma2_rn(s2, scale2, neg2);
            const float2 x2 = make_float2(ex2(t2.x), ex2(t2.y));
            sums[e] = __fadd2_rn(sums[e], x2);
            w[e] = pack2(x2.x, x2.y);
          }
          *reinterpret_cast<uint4*>(p_row + ((ch ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        {
          const float2 a = __fadd2_rn(sums[0], sums[1]), b = __fadd2_rn(sums[2], sums[3]);
          const float2 c = __fadd2_rn(a, b);
          l_run = l_run * corr + (c.x + c.y);
        }
        // PV_{j-1} must be finished before P_j is signalled: it keeps this barrier from running a
        // phase ahead of the waiters, and O must be at rest if it has to be rescaled
        if (j > 0) {
          ok = mbar_wait(bar(BAR_PV_FULL + x), (j - 1) & 1, &abort_flag);
          if (!ok) break;
          if (rescale) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t ov[32];
              tmem_load32(o_addr + c0, ov);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * corr);
              asm volatile(
                  "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                  "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                  "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                  ::"r"(o_addr + c0), "r"(ov[0]), "r"(ov[1]), "r"(ov[2]), "r"(ov[3]), "r"(ov[4]), "r"(ov[5]),
                  "r"(ov[6]), "r"(ov[7]), "r"(ov[8]), "r"(ov[9]), "r"(ov[10]), "r"(ov[11]), "r"(ov[12]), "r"(ov[13]),
                  "r"(ov[14]), "r"(ov[15]), "r"(ov[16]), "r"(ov[17]), "r"(ov[18]), "r"(ov[19]), "r"(ov[20]),
                  "r"(ov[21]), "r"(ov[22]), "r"(ov[23]), "r"(ov[24]), "r"(ov[25]), "r"(ov[26]), "r"(ov[27]),
                  "r"(ov[28]), "r"(ov[29]), "r"(ov[30]), "r"(ov[31])
                  : "memory");
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          }
        }
        // keys of this tile past the item's last position hold whatever the page held: zero their
        // value rows before PV reads them (both blocks do, each before its own PV; keys between the
        // blocks' last positions are real and only masked)
        if (key0 + BLOCK_N - 1 > p_last) {
          ok = mbar_wait(bar(BAR_V_FULL + vst), (j / KV_STAGES) & 1, &abort_flag);
          if (!ok) break;
          const int vrow = r & 63, half = r >> 6;
          if (key0 + vrow > p_last) {
            uint4* dst = reinterpret_cast<uint4*>(v_s + vst * KV_BYTES + half * (KV_BYTES / 2) + vrow * 128);
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) dst[ch] = make_uint4(0, 0, 0, 0);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P (and zeroed V) visible to the MMA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(bar(BAR_P_FULL + x));
      }
      if (ok && my_tiles) ok = mbar_wait(bar(BAR_PV_FULL + x), (my_tiles - 1) & 1, &abort_flag);
      if (ok && my_tiles) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = 1.f / l_run;
        bf16* dst = row_ok ? out + ((long)(tok0 + R / G) * nq + kvh * G + R % G) * D : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t ov[32];
          tmem_load32(o_addr + c0, ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (row_ok) {
#pragma unroll
            for (int c = 0; c < 32; c += 8) {
              float v8[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v8[e] = __uint_as_float(ov[c + e]) * inv;
              store8(dst + c0 + c, v8);
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
  if (tid == 0 && abort_flag && error_word) atomicExch(error_word, 2);
}

}  // namespace

// q: the QKV buffer, [num_tokens, *] bf16 with row stride q_stride (elements), head h at column
// h * 128.  kpages / vpages: [num_rows_kv / (nkv * ps), nkv, ps, 128] bf16 of one layer, num_rows_kv
// rows of 128 in all.  num_work = sum over served sequences of ceil(ceil(q_len * (nq / nkv) / 128) / 2).
// Returns Q3_ERR_UNSUPPORTED for shapes this kernel does not take (the caller then uses the
// mma.sync kernel).  error_word: device int set to 2 if a wait inside the kernel expired.
Q3_EXPORT int q3_paged_attention_prefill_tc(const void* q, int q_stride, int num_tokens, const void* kpages,
                                            const void* vpages, long num_rows_kv, const int* block_table,
                                            int max_pages, const int* kv_lens, const int* cu_seqlens, void* out,
                                            int num_seqs, int num_work, int nq, int nkv, int head_dim, int ps,
                                            float scale, int skip_single, int* error_word, cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !kv_lens || !cu_seqlens || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv) return Q3_ERR_ARGUMENT;
  const int G = nq / nkv;
  if (head_dim != D || BLOCK_M % G || (ps != 8 && ps != 16 && ps != 32 && ps != 64) || q_stride % 8 ||
      nkv > 65535 || (((uintptr_t)q | (uintptr_t)kpages | (uintptr_t)vpages) & 15))
    return Q3_ERR_UNSUPPORTED;
  if (num_work == 0) return Q3_OK;
  Q3EncodeTiledFn fn = q3_encode_tiled();
  if (!fn) return Q3_ERR_LAUNCH;
  CUtensorMap tq, tk, tv;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)nq, (cuuint64_t)num_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(BLOCK_M / G)};
    const cuuint32_t es[3] = {1, 1, 1};
    if (fn(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return Q3_ERR_LAUNCH;
  }
  // pages as a matrix [rows of all pages and kv heads][D], read in boxes of one page x 64 dims
  if (!q3_bf16_map(&tk, kpages, num_rows_kv, D, D, ps, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) ||
      !q3_bf16_map(&tv, vpages, num_rows_kv, D, D, ps, CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
    return Q3_ERR_LAUNCH;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid((unsigned)num_work * nkv);
  prefill_attention_tc_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, block_table, max_pages, kv_lens,
                                                                    cu_seqlens, (bf16*)out, num_seqs, num_work, nq,
                                                                    nkv, ps, scale * 1.4426950408889634f,
                                                                    skip_single, error_word);
  return q3_launch_status();
}
