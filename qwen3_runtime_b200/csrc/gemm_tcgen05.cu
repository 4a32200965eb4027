// out[M, N] = x[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory (TMEM), operands staged in shared
// memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), completion tracked by mbarriers.
// This is the matrix product of prompt portions (more tokens than the weight-streaming
// kernel of gemm_small_m.cu takes); the reference uses the library's product here
// (qwen3_runtime/models/qwen3.py:76-77, 134-135).
//
// A block computes 128 x 256 output tiles (128 tokens x 256 features), K in slices of 64,
// through a 4-stage ring of shared-memory tiles; it is persistent (one block per SM walks the
// tiles) and keeps two accumulators in TMEM so that the epilogue of a tile overlaps the MMAs
// of the next.  Six warps, three roles:
//   warp 0, one lane : TMA producer   - waits for a free stage, arms its "full" barrier with
//                                       the byte count, issues the loads of the A and B tiles;
//   warp 1, one lane : MMA issuer     - waits for "full", issues 4 tcgen05.mma (K = 16 each)
//                                       per stage, tcgen05.commit frees the stage; a final
//                                       commit signals the epilogue;  warp 1 also owns TMEM;
//   warps 2..5       : epilogue       - each reads its 32-lane quarter of TMEM with
//                                       tcgen05.ld, converts and stores.
// Epilogues: bf16 out; fp32 out; SwiGLU -- the block loads the gate rows and the up rows of
// the same 128 features as two B tiles, accumulates them in two TMEM column ranges and writes
// silu(gate) * up (models/qwen3.py:137-138), so the [M, 2I] intermediate never exists.
//
// Every wait on an mbarrier is bounded (about a second of SM clock): on expiry the waiter
// raises the block's abort flag and a global error word, every role leaves its loop, TMEM is
// freed and the block returns; the host reports the error.  Before it frees anything the
// one-CTA kernel waits (bounded again, with a limit of its own) for what it still has in
// flight: the producer for the boxes it issued into shared memory, the MMA thread for the MMAs
// it issued into tensor memory.  No load uses cluster multicast.
#include "async_tiles.cuh"

namespace {

enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_SWIGLU = 2 };
constexpr int BM = 128;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int THREADS = 192;

// NV values of one output row, columns [col, col + NV) as far as they exist: fp32 or bf16, with
// 16-byte stores where the row's alignment allows.
template <int MODE, int NV>
__device__ __forceinline__ void store_row(void* __restrict__ out, int ldo, int row, int col, int N,
                                          const float (&v)[NV]) {
  if (MODE == OUT_F32) {
    float* dst = reinterpret_cast<float*>(out) + (long)row * ldo + col;
    if (col + NV <= N && (ldo & 3) == 0) {
#pragma unroll
      for (int e = 0; e < NV; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
    } else {
      for (int e = 0; e < NV && col + e < N; ++e) dst[e] = v[e];
    }
  } else {
    bf16* dst = reinterpret_cast<bf16*>(out) + (long)row * ldo + col;
    if (col + NV <= N && (ldo & 7) == 0) {
#pragma unroll
      for (int e = 0; e < NV; e += 8) {
        float chunk[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) chunk[x] = v[e + x];
        store8(dst + e, chunk);
      }
    } else {
      for (int e = 0; e < NV && col + e < N; ++e) dst[e] = __float2bfloat16_rn(v[e]);
    }
  }
}

// BN: features per MMA (N of the instruction).  NB: B tiles per stage (2 for SwiGLU: gate, up).
// Persistent: block b computes tiles b, b + gridDim.x, ...; the accumulator is double-buffered
// in TMEM (2 x 256 columns) so that the epilogue of one tile overlaps the MMAs of the next.
template <int BN, int NB, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                    void* __restrict__ out, int ldo, int M, int N, int K, int up_row_offset,
                    int* __restrict__ error_word) {
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + NB * B_BYTES;
  constexpr int ACC_COLS = 256;          // columns per accumulator buffer (BN * NB of them are used)
  constexpr int TMEM_COLS = 2 * ACC_COLS;  // 512: the whole tensor memory of the SM
  static_assert(BN * NB <= ACC_COLS && BN % 32 == 0 && (BN * NB) % 16 == 0, "tile width");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * STAGES + 5];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;
  int issued = 0;  // producer thread: k-slices whose boxes it has issued

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[STAGES]);
  const uint32_t acc_full0 = smem_addr(&bars[2 * STAGES]), acc_empty0 = smem_addr(&bars[2 * STAGES + 2]);
  const uint32_t drained = smem_addr(&bars[2 * STAGES + 4]);  // give-up path: the issued MMAs have finished

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
    }
    mbar_init(drained, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // TMEM allocation is a warp-wide instruction; the same warp frees it at the end
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer -------------------------------------------------------
      int g = 0;  // k-slices issued so far, over all tiles of this block
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;  // token tiles fastest: a weight tile stays in L2
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int s = g % STAGES;
          const uint32_t phase = (g / STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, phase ^ 1, &abort_flag);
          if (!ok) break;
          const uint32_t a_dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, full0 + 8 * s, kb * BK, m0);
#ifndef Q3_TEST_WITHHOLD_A_BOX  // (a test build leaves the weight boxes out: the stage never fills, a wait runs out)
          tma_load_2d(a_dst + A_BYTES, &tmap_w, full0 + 8 * s, kb * BK, n0);
          if (NB == 2) tma_load_2d(a_dst + A_BYTES + B_BYTES, &tmap_w, full0 + 8 * s, kb * BK, up_row_offset + n0);
#endif
          issued = g + 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ---------------------------------------------------------
      // the B tiles of a stage lie one after the other, which is the layout of one tile of
      // NB * BN rows: one MMA over all of them reads the A tile once instead of NB times
      constexpr uint32_t idesc = umma_idesc(BM, NB * BN);
      int g = 0, i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++i) {
        const int buf = i & 1;
        ok = mbar_wait(acc_empty0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_flag);  // epilogue has drained it
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int s = g % STAGES;
          const uint32_t phase = (g / STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, phase, &abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr);
          const uint64_t b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 bytes = 2 descriptor units along K
            umma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);  // arrives when these MMAs have read the stage
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);  // arrives when the tile's MMAs have written TMEM
      }
    }
  } else {  // ---- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 31 ---------------------------
    const int quarter = warp & 3;
    int i = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++i) {
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;  // token tiles fastest: a weight tile stays in L2
      const int buf = i & 1;
      const int row = m0 + quarter * 32 + lane;
      ok = mbar_wait(acc_full0 + 8 * buf, (i >> 1) & 1, &abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const bool last = c0 + 32 >= BN || n0 + c0 + 32 >= N;
        if (n0 + c0 < N) {  // (uniform)
          uint32_t acc[32];
          tmem_load32(lane_addr + c0, acc);
          float v[32];
          if (MODE == OUT_SWIGLU) {
            uint32_t up[32];
            tmem_load32(lane_addr + BN + c0, up);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float gate = __uint_as_float(acc[e]);
              v[e] = (gate / (1.f + expf(-gate))) * __uint_as_float(up[e]);
            }
          } else {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(acc[e]);
          }
          if (last) {  // everything of this buffer is in registers: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
          }
          if (row < M) store_row<MODE, 32>(out, ldo, row, n0 + c0, N, v);
        }
        if (last) break;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (abort_flag) {
    // The block has given up.  Nothing of its own may still be under way when it frees its tensor
    // memory and leaves its shared memory to the next block: the boxes of the last STAGES
    // k-slices that were issued land on their stages' barriers (an earlier slice of a stage had
    // landed before the stage was issued again), and a last commit arrives when every MMA issued
    // so far has finished.
    if (warp == 0 && lane == 0)
      for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; ++j)
        mbar_wait_drain(full0 + 8 * (j % STAGES), (j / STAGES) & 1);
    if (warp == 1 && lane == 0) {
      umma_commit(drained);
      mbar_wait_drain(drained, 0);
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_word) atomicExch(error_word, 1);
}

// ---- the same product on pairs of SMs (cta_group::2) -------------------------------------------------
// One MMA of 256 x 256 over two CTAs of a cluster: each CTA holds 128 token rows of A and 128
// of the 256 feature rows of B (for SwiGLU: the leader the gate rows, its peer the up rows of
// the same 128 features) and gets the accumulator rows of its own tokens in its own tensor
// memory.  Per 16 k-values a CTA's shared memory is read for 4 KB of A and 4 KB of B instead
// of 4 KB + 8 KB, which is what keeps the one-CTA kernel below 70 % of the tensor pipe.
//   warp 0, one lane : TMA producer of this CTA's A and B boxes (6-stage ring).  Both CTAs'
//                      loads complete their bytes on the leader's "full" barrier of the stage
//                      (cp.async.bulk.tensor with .cta_group::2), which the leader arms for
//                      both; a relay through the peer's own barrier cost several hundred
//                      cycles per stage;
//   warp 1, one lane : leader only: MMA issuer; it releases a stage, and hands over a finished
//                      accumulator, in both CTAs at once with multicast commits;
//   warps 2..5       : epilogue of this CTA's 128 rows; "accumulator drained" goes to the
//                      leader (8 arrivals: 4 warps of each CTA).
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_BN = 256;

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                         void* __restrict__ out, int ldo, int M, int N, int K, int up_row_offset,
                         int* __restrict__ error_word) {
  constexpr int A_BYTES = BM * BK * 2;       // this CTA's 128 token rows
  constexpr int B_BYTES = 128 * BK * 2;      // this CTA's 128 feature rows
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int ACC_COLS = 256;
  constexpr int TMEM_COLS = 2 * ACC_COLS;
  constexpr int TILE_N = MODE == OUT_SWIGLU ? 128 : PAIR_BN;  // output columns per tile
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * PAIR_STAGES + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_n = (N + TILE_N - 1) / TILE_N, tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[PAIR_STAGES]);
  const uint32_t acc_full0 = smem_addr(&bars[2 * PAIR_STAGES]), acc_empty0 = smem_addr(&bars[2 * PAIR_STAGES + 2]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 8);  // one arrival per epilogue warp of both CTAs (used in the leader)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // both CTAs of the pair execute the pair-wide allocation, and later the release
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer -------------------------------------------------------
      const uint32_t leader_full0 = map_to_cta(full0, 0);
      int g = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % tiles_m) * (2 * BM) + rank * BM;  // token tiles fastest: a weight tile stays in L2
        const int n0 = (tile / tiles_m) * TILE_N;
        const int w_row = MODE == OUT_SWIGLU ? (rank ? up_row_offset + n0 : n0) : n0 + rank * 128;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int s = g % PAIR_STAGES;
          const uint32_t phase = (g / PAIR_STAGES) & 1;
          ok = mbar_wait(empty0 + 8 * s, phase ^ 1, &abort_flag);
          if (!ok) break;
          const uint32_t a_dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);  // this CTA's boxes and the peer's
          tma_load_2d_pair(a_dst, &tmap_a, leader_full0 + 8 * s, kb * BK, m0);
          tma_load_2d_pair(a_dst + A_BYTES, &tmap_w, leader_full0 + 8 * s, kb * BK, w_row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---- MMA issuer of the pair ------------------------------------
      constexpr uint32_t idesc = umma_idesc(2 * BM, PAIR_BN);
      int g = 0, i = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++i) {
        const int buf = i & 1;
        ok = mbar_wait(acc_empty0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_flag);  // both epilogues have drained it
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int s = g % PAIR_STAGES;
          const uint32_t phase = (g / PAIR_STAGES) & 1;
          ok = mbar_wait(full0 + 8 * s, phase, &abort_flag);  // both CTAs' boxes of the stage have landed
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_pair(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty0 + 8 * s);  // both CTAs may refill the stage once these MMAs have read it
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * buf);  // both epilogues: the tile is in tensor memory
      }
    }
  } else {  // ---- epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 31 of this CTA ------------------
    const int quarter = warp & 3;
    const uint32_t leader_acc_empty0 = map_to_cta(acc_empty0, 0);
    int i = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++i) {
      const int m0 = (tile % tiles_m) * (2 * BM) + rank * BM, n0 = (tile / tiles_m) * TILE_N;
      const int buf = i & 1;
      const int row = m0 + quarter * 32 + lane;
      ok = mbar_wait(acc_full0 + 8 * buf, (i >> 1) & 1, &abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < TILE_N; c0 += 32) {
        const bool last = c0 + 32 >= TILE_N || n0 + c0 + 32 >= N;
        if (n0 + c0 < N) {  // (uniform)
          uint32_t acc[32];
          tmem_load32(lane_addr + c0, acc);
          float v[32];
          if (MODE == OUT_SWIGLU) {
            uint32_t up[32];
            tmem_load32(lane_addr + 128 + c0, up);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float gate = __uint_as_float(acc[e]);
              v[e] = (gate / (1.f + expf(-gate))) * __uint_as_float(up[e]);
            }
          } else {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(acc[e]);
          }
          if (last) {  // everything of this buffer is in registers: hand it back to the MMA issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            if (lane == 0) remote_arrive(leader_acc_empty0 + 8 * buf);
          }
          if (row < M) store_row<MODE, 32>(out, ldo, row, n0 + c0, N, v);
        }
        if (last) break;
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();  // nobody leaves while the other still reads its shared memory or signals its barriers
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_word) atomicExch(error_word, 1);
}

// ---- pairs of SMs, tiles of 256 tokens x 320 features --------------------------------------------
// For outputs whose width leaves the 256-wide tiles one round short of filling the machine
// (2560 features x 2048 tokens: 80 tiles for 74 pairs, two rounds) a wider tile can do it in
// one: 64 tiles of 320.  An MMA takes at most 256 features, so a stage is multiplied by two MMAs
// of 160 (80 feature rows from each CTA); the accumulator has 320 columns and a single buffer
// (tensor memory has 512), so a pair's next tile waits for its epilogue.  Plain products only.
// Accumulator column c belongs to MMA c / 160; inside it columns [0,80) are the leader's rows and
// [80,160) the peer's: feature = n0 + 160 * (c % 160 / 80) + 80 * (c / 160) + c % 80.
constexpr int WIDE = 320;
constexpr int WIDE_STAGES = 5;

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_pair_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                              void* __restrict__ out, int ldo, int M, int N, int K, int* __restrict__ error_word) {
  static_assert(MODE != OUT_SWIGLU, "plain products only");
  constexpr int HALF = WIDE / 2;             // feature rows of this CTA: 160
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = HALF * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 512;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * WIDE_STAGES + 2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_n = (N + WIDE - 1) / WIDE, tiles_m = (M + 2 * BM - 1) / (2 * BM);
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[WIDE_STAGES]);
  const uint32_t acc_full = smem_addr(&bars[2 * WIDE_STAGES]), acc_empty = smem_addr(&bars[2 * WIDE_STAGES + 1]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < WIDE_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer -------------------------------------------------------
      const uint32_t leader_full0 = map_to_cta(full0, 0);
      int g = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % tiles_m) * (2 * BM) + rank * BM;
        const int w_row = (tile / tiles_m) * WIDE + rank * HALF;
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int s = g % WIDE_STAGES;
          ok = mbar_wait(empty0 + 8 * s, ((g / WIDE_STAGES) & 1) ^ 1, &abort_flag);
          if (!ok) break;
          const uint32_t a_dst = smem_addr(tiles + (size_t)s * STAGE_BYTES);
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
          tma_load_2d_pair(a_dst, &tmap_a, leader_full0 + 8 * s, kb * BK, m0);
          tma_load_2d_pair(a_dst + A_BYTES, &tmap_w, leader_full0 + 8 * s, kb * BK, w_row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ---- MMA issuer of the pair ------------------------------------
      constexpr uint32_t idesc = umma_idesc(2 * BM, HALF);  // N = 160: 80 feature rows of each CTA
      int g = 0, i = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++i) {
        ok = mbar_wait(acc_empty, (i & 1) ^ 1, &abort_flag);  // both epilogues have drained the accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < num_kb; ++kb, ++g) {
          const int s = g % WIDE_STAGES;
          ok = mbar_wait(full0 + 8 * s, (g / WIDE_STAGES) & 1, &abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_addr(tiles + (size_t)s * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint64_t b_desc = umma_desc(a_addr + A_BYTES + j * (HALF / 2) * 128);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_pair(tmem_base + j * HALF, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty0 + 8 * s);
        }
        if (ok) umma_commit_pair(acc_full);
      }
    }
  } else {  // ---- epilogue ------------------------------------------------------------------------------
    const int quarter = warp & 3;
    const uint32_t leader_acc_empty = map_to_cta(acc_empty, 0);
    int i = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++i) {
      const int m0 = (tile % tiles_m) * (2 * BM) + rank * BM, n0 = (tile / tiles_m) * WIDE;
      const int row = m0 + quarter * 32 + lane;
      ok = mbar_wait(acc_full, i & 1, &abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < WIDE; c0 += 16) {
        const int within = c0 % HALF;
        const int col = n0 + HALF * (within / (HALF / 2)) + (HALF / 2) * (c0 / HALF) + within % (HALF / 2);
        uint32_t acc[16];
        tmem_load16(lane_addr + c0, acc);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 16 >= WIDE) {  // the accumulator is in registers: hand it back to the MMA issuer
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          if (lane == 0) remote_arrive(leader_acc_empty);
        }
        if (row < M && col < N) {
          float v[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(acc[e]);
          store_row<MODE, 16>(out, ldo, row, col, N, v);
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_word) atomicExch(error_word, 1);
}

// ---- host side ------------------------------------------------------------------------------------

int sm_count() {
  static int count_on[Q3_MAX_DEVICES];
  int& count = count_on[q3_current_device()];
  if (!count) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count < 2) count = 148;
  }
  return count;
}

template <int BN, int NB, int MODE>
int launch(const CUtensorMap& ta, const CUtensorMap& tw, void* out, int ldo, int M, int N, int K, int up_offset,
           int* error_word, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + NB * BN * BK * 2) + 1024;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, NB, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  const int num_sms = sm_count();
  const int tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  const int grid = tiles < num_sms ? tiles : num_sms;  // one persistent block per SM
  gemm_tcgen05_kernel<BN, NB, MODE><<<grid, THREADS, smem, stream>>>(ta, tw, out, ldo, M, N, K, up_offset, error_word);
  return q3_launch_status();
}

template <int MODE>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tw, void* out, int ldo, int M, int N, int K, int up_offset,
                int* error_word, cudaStream_t stream) {
  constexpr size_t smem = (size_t)PAIR_STAGES * (BM * BK * 2 + 128 * BK * 2) + 1024;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  static int pairs_on[Q3_MAX_DEVICES];  // pairs of SMs the device runs at once with this kernel
  int& pairs = pairs_on[q3_current_device()];
  if (!pairs) {
    const int sms = sm_count();
    cfg.gridDim = dim3(sms / 2 * 2);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_pair_kernel<MODE>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      return Q3_ERR_UNSUPPORTED;
    }
    pairs = n < sms / 2 ? n : sms / 2;
  }
  constexpr int TILE_N = MODE == OUT_SWIGLU ? 128 : PAIR_BN;
  const int tiles = ((N + TILE_N - 1) / TILE_N) * ((M + 2 * BM - 1) / (2 * BM));
  cfg.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs));
  const cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel<MODE>, ta, tw, out, ldo, M, N, K,
                                             up_offset, error_word);
  return err == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

// pairs of SMs that run at once (clusters of two blocks that each take a whole SM)
int resident_pairs(const void* kernel, size_t smem) {
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms / 2 * 2);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    return 0;
  }
  return n < sms / 2 ? n : sms / 2;
}

template <int MODE>
int launch_pair_wide(const CUtensorMap& ta, const CUtensorMap& tw, void* out, int ldo, int M, int N, int K,
                     int* error_word, cudaStream_t stream) {
  constexpr size_t smem = (size_t)WIDE_STAGES * (BM * BK * 2 + (WIDE / 2) * BK * 2) + 1024;
  static int pairs_on[Q3_MAX_DEVICES];  // 0: not asked yet, -1: none
  int& pairs = pairs_on[q3_current_device()];
  if (pairs == 0) {
    if (cudaFuncSetAttribute(gemm_tcgen05_pair_wide_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    pairs = resident_pairs((const void*)gemm_tcgen05_pair_wide_kernel<MODE>, smem);
    if (pairs < 1) pairs = -1;
  }
  if (pairs < 1) return Q3_ERR_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int tiles = ((N + WIDE - 1) / WIDE) * ((M + 2 * BM - 1) / (2 * BM));
  cfg.gridDim = dim3(2 * (tiles < pairs ? tiles : pairs));
  const cudaError_t err =
      cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_wide_kernel<MODE>, ta, tw, out, ldo, M, N, K, error_word);
  return err == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

}  // namespace

// The same product on pairs of SMs (tcgen05 cta_group::2, tiles of 256 tokens x 256 features, for
// SwiGLU 256 tokens x 128 gate + 128 up; 256 x 320 where that saves a round of tiles): same
// arguments and modes as q3_gemm_tcgen05.
Q3_EXPORT int q3_gemm_tcgen05_pair(int mode, const void* x, int ldx, const void* W, int ldw, void* out, int ldo,
                                   int M, int N, int K, int* error_word, cudaStream_t stream) {
  if (!x || !W || !out || N < 1 || K < 1 || M < 0 || mode < 0 || mode > 2) return Q3_ERR_ARGUMENT;
  if (ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  CUtensorMap ta, tw;
  const long w_rows = mode == OUT_SWIGLU ? 2L * N : N;
  if (mode != OUT_SWIGLU) {
    // tile width: rounds of one tile per pair x columns per tile (+24 when the wide tile's
    // epilogue cannot overlap the next tile's MMAs)
    const long tiles_m = (M + 2 * BM - 1) / (2 * BM);
    const long pairs = sm_count() / 2;
    const long cost_256 = ((tiles_m * ((N + PAIR_BN - 1) / PAIR_BN) + pairs - 1) / pairs) * PAIR_BN;
    const long cost_wide = ((tiles_m * ((N + WIDE - 1) / WIDE) + pairs - 1) / pairs) * (WIDE + 24);
    if (cost_wide < cost_256) {
      if (!q3_bf16_map(&ta, x, M, K, ldx, BM) || !q3_bf16_map(&tw, W, w_rows, K, ldw, WIDE / 2)) return Q3_ERR_LAUNCH;
      return mode == OUT_F32 ? launch_pair_wide<OUT_F32>(ta, tw, out, ldo, M, N, K, error_word, stream)
                             : launch_pair_wide<OUT_BF16>(ta, tw, out, ldo, M, N, K, error_word, stream);
    }
  }
  if (!q3_bf16_map(&ta, x, M, K, ldx, BM) || !q3_bf16_map(&tw, W, w_rows, K, ldw, 128)) return Q3_ERR_LAUNCH;
  if (mode == OUT_SWIGLU) return launch_pair<OUT_SWIGLU>(ta, tw, out, ldo, M, N, K, N, error_word, stream);
  if (mode == OUT_F32) return launch_pair<OUT_F32>(ta, tw, out, ldo, M, N, K, 0, error_word, stream);
  return launch_pair<OUT_BF16>(ta, tw, out, ldo, M, N, K, 0, error_word, stream);
}

// mode 0: out bf16 [M, N]; 1: out fp32 [M, N]; 2: W is [2 * N, K] (gate rows, then up rows from
// row N), out bf16 [M, N] = silu(x W_gate^T) * (x W_up^T).  x, W bf16 with 16-byte aligned bases
// and row strides (elements) that are multiples of 8.  error_word: device int, set to 1 if a
// wait inside the kernel expired (may be null).
Q3_EXPORT int q3_gemm_tcgen05(int mode, const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M,
                              int N, int K, int* error_word, cudaStream_t stream) {
  if (!x || !W || !out || N < 1 || K < 1 || M < 0) return Q3_ERR_ARGUMENT;
  if (ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  CUtensorMap ta, tw;
  int bn = 128;
  if (mode != OUT_SWIGLU) {
    // tile width: the one that needs the fewest rounds of one-tile-per-SM, counted in columns
    // (+24 for what a tile costs beyond its MMAs); narrow outputs get narrower tiles
    const int tiles_m = (M + BM - 1) / BM;
    long best = -1;
    for (int cand : {256, 192, 160, 128}) {
      const long tiles = (long)tiles_m * ((N + cand - 1) / cand);
      const long cost = ((tiles + sm_count() - 1) / sm_count()) * (cand + 24);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand;
      }
    }
  }
  const long w_rows = mode == OUT_SWIGLU ? 2L * N : N;
  if (!q3_bf16_map(&ta, x, M, K, ldx, BM) || !q3_bf16_map(&tw, W, w_rows, K, ldw, bn)) return Q3_ERR_LAUNCH;
  if (mode == OUT_SWIGLU) return launch<128, 2, OUT_SWIGLU>(ta, tw, out, ldo, M, N, K, N, error_word, stream);
#define Q3_TC_CASE(BN_)                                                                                   \
  if (bn == BN_)                                                                                          \
    return mode == OUT_F32 ? launch<BN_, 1, OUT_F32>(ta, tw, out, ldo, M, N, K, 0, error_word, stream)    \
                           : launch<BN_, 1, OUT_BF16>(ta, tw, out, ldo, M, N, K, 0, error_word, stream)
  if (mode == OUT_BF16 || mode == OUT_F32) {
    Q3_TC_CASE(256);
    Q3_TC_CASE(192);
    Q3_TC_CASE(160);
    Q3_TC_CASE(128);
  }
#undef Q3_TC_CASE
  return Q3_ERR_ARGUMENT;
}
