// out[M, N] = x[M, K] * W[N, K]^T for 17..64 tokens, bfloat16, on tcgen05 with the roles of the
// operands swapped: a decode step of a few dozen sequences.
//
// With so few tokens the product is still a stream over the weights, but the tokens no longer
// fit a warp's registers (gemm_stream.cu) and a tile of 128 tokens x 256 features
// (gemm_tcgen05.cu) gives too few tiles to keep every SM reading.  So the weights are the
// 128-row operand of the MMA and the tokens its 64 columns: D[128 features, 64 tokens] in tensor
// memory, A = a [128 features x 64 k] box of W, B = the [64 tokens x 64 k] box of x (rows past M
// read as zero), both by TMA with the 128-byte swizzle.  A work item is one tile of 128 features
// x one range of K; K is cut into as many ranges as it takes to give every SM an item, and an
// item with a range of its own writes an fp32 plane out[range][token][feature] -- the sum over
// the ranges is the product, added up by the norm kernel (csrc/norm.cu) or by
// q3_sum_planes below.  One block per SM, persistent over its items.  A stage of the ring holds
// three k-blocks (three weight boxes of 16 KB and three token boxes of 8 KB) behind one barrier,
// three stages: a round trip over a stage's barriers costs about 0.7 us here whatever the stage
// holds, so with one k-block per stage the kernel ran at 3.3 TB/s, with three at 5.0.
// Roles as in gemm_tcgen05.cu: warp 0 lane 0 issues the TMA loads, warp 1 lane 0 the
// MMAs (and owns the tensor memory), warps 2..5 read the accumulator (each its 32 lanes =
// 32 features) and store, one token at a time, 32 consecutive features per warp.
//
// Every wait on an mbarrier is bounded: on expiry the waiter raises the block's abort flag and
// the error word, every role leaves its loop, the tensor memory is freed and the block returns.
#include "async_tiles.cuh"

namespace {

enum { SK_BF16 = 0, SK_F32 = 1, SK_PLANES = 2 };
constexpr int SK_BM = 128;     // features per tile
constexpr int SK_NT = 64;      // token columns of the MMA
constexpr int SK_BK = 64;
constexpr int SK_KSUB = 3;      // k-blocks per stage (per barrier round trip)
constexpr int SK_STAGES = 3;
constexpr int SK_THREADS = 192;
constexpr int SK_A_BYTES = SK_BM * SK_BK * 2;
constexpr int SK_B_BYTES = SK_NT * SK_BK * 2;
constexpr int SK_SUB_BYTES = SK_A_BYTES + SK_B_BYTES;
constexpr int SK_STAGE_BYTES = SK_KSUB * SK_SUB_BYTES;

template <int MODE>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   void* __restrict__ out, int ldo, int M, int N, int K, int kb_per_range, int ranges,
                   int* __restrict__ error_word) {
  // An MMA of 128 x 64 x 16 is short, and MMAs that add to the same accumulator run one after the
  // other: a single chain of them is bound by their latency, not by memory.  So the four k-steps of
  // a 64-wide k-block go to four accumulators of their own (four independent chains), which the
  // epilogue adds up.  Two such sets, so that the epilogue of an item overlaps the next: all 512
  // columns of the tensor memory.
  constexpr int CHAINS = SK_BK / 16;
  constexpr int ACC_COLS = CHAINS * SK_NT;
  constexpr int TMEM_COLS = 2 * ACC_COLS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long bars[2 * SK_STAGES + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_f = (N + SK_BM - 1) / SK_BM;
  const int num_items = tiles_f * ranges;  // item = range * tiles_f + tile: neighbours share a range of x
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[SK_STAGES]);
  const uint32_t acc_full0 = smem_addr(&bars[2 * SK_STAGES]), acc_empty0 = smem_addr(&bars[2 * SK_STAGES + 2]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < SK_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
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
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {  // ---- TMA producer -------------------------------------------------------
      // the g-th stage of this block's items: which features, which k-blocks (SK_KSUB of them, fewer
      // at the end of a range)
      auto locate = [&](int g, int& f0, int& kb, int& cnt) -> bool {
        int base = 0;
        for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
          const int lo = (item / tiles_f) * kb_per_range, n = min(num_kb, lo + kb_per_range) - lo;
          const int stages_n = (n + SK_KSUB - 1) / SK_KSUB;
          if (g < base + stages_n) {
            f0 = (item % tiles_f) * SK_BM;
            kb = lo + (g - base) * SK_KSUB;
            cnt = min(SK_KSUB, lo + n - kb);
            return true;
          }
          base += stages_n;
        }
        return false;
      };
      // The weights do not depend on the kernel before this one: the ring is filled with weight
      // boxes before the wait for it, the token boxes of those stages follow.
      int f0 = 0, kb = 0, cnt = 0, early = 0;
      for (; early < SK_STAGES && locate(early, f0, kb, cnt); ++early) {
        mbar_expect_tx(full0 + 8 * early, cnt * SK_SUB_BYTES);
        for (int j = 0; j < cnt; ++j)
          tma_load_2d(smem_addr(tiles + (size_t)early * SK_STAGE_BYTES + j * SK_SUB_BYTES), &tmap_w, full0 + 8 * early,
                      (kb + j) * SK_BK, f0);
      }
      pdl_wait();
      for (int g = 0; g < early; ++g) {
        locate(g, f0, kb, cnt);
        for (int j = 0; j < cnt; ++j)
          tma_load_2d(smem_addr(tiles + (size_t)g * SK_STAGE_BYTES + j * SK_SUB_BYTES) + SK_A_BYTES, &tmap_x,
                      full0 + 8 * g, (kb + j) * SK_BK, 0);
      }
      for (int g = early; locate(g, f0, kb, cnt); ++g) {
        const int s = g % SK_STAGES;
        if (!mbar_wait(empty0 + 8 * s, ((g / SK_STAGES) & 1) ^ 1, &abort_flag)) break;
        mbar_expect_tx(full0 + 8 * s, cnt * SK_SUB_BYTES);
        for (int j = 0; j < cnt; ++j) {
          const uint32_t a_dst = smem_addr(tiles + (size_t)s * SK_STAGE_BYTES + j * SK_SUB_BYTES);
          tma_load_2d(a_dst, &tmap_w, full0 + 8 * s, (kb + j) * SK_BK, f0);
          tma_load_2d(a_dst + SK_A_BYTES, &tmap_x, full0 + 8 * s, (kb + j) * SK_BK, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- MMA issuer ---------------------------------------------------------
      constexpr uint32_t idesc = umma_idesc(SK_BM, SK_NT);
      int g = 0, i = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++i) {
        const int range = item / tiles_f;
        const int kb_lo = range * kb_per_range, kb_hi = min(num_kb, kb_lo + kb_per_range);
        const int buf = i & 1;
        ok = mbar_wait(acc_empty0 + 8 * buf, ((i >> 1) & 1) ^ 1, &abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem_base + buf * ACC_COLS;
        for (int kb = kb_lo; kb < kb_hi; kb += SK_KSUB, ++g) {
          const int s = g % SK_STAGES;
          ok = mbar_wait(full0 + 8 * s, (g / SK_STAGES) & 1, &abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const int cnt = min(SK_KSUB, kb_hi - kb);
          for (int j = 0; j < cnt; ++j) {
            const uint32_t a_addr = smem_addr(tiles + (size_t)s * SK_STAGE_BYTES + j * SK_SUB_BYTES);
            const uint64_t a_desc = umma_desc(a_addr);
            const uint64_t b_desc = umma_desc(a_addr + SK_A_BYTES);
#pragma unroll
            for (int k = 0; k < SK_BK / 16; ++k)
              umma_bf16(acc + k * SK_NT, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb_lo || j > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);
      }
    }
  } else {  // ---- epilogue: warp w has TMEM lanes 32 * (w % 4) .. + 31 = 32 features of the tile --------
    const int quarter = warp & 3;
    int i = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++i) {
      const int f = (item % tiles_f) * SK_BM + quarter * 32 + lane, range = item / tiles_f;
      const int buf = i & 1;
      ok = mbar_wait(acc_full0 + 8 * buf, (i >> 1) & 1, &abort_flag);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + buf * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {  // tokens 0..31, then 32..63
        float v[32];
#pragma unroll
        for (int chain = 0; chain < CHAINS; ++chain) {
          uint32_t raw[32];
          tmem_load32(lane_addr + chain * SK_NT + 32 * half, raw);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = chain == 0 ? __uint_as_float(raw[e]) : v[e] + __uint_as_float(raw[e]);
        }
        if (half == 1) {  // everything of this set is in registers: hand it back to the MMA warp
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
        }
        if (f < N) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int c = 32 * half + e;
            if (c < M) {  // (uniform) token c: 32 consecutive features per warp
              if (MODE == SK_PLANES)
                reinterpret_cast<float*>(out)[((long)range * M + c) * ldo + f] = v[e];
              else if (MODE == SK_F32)
                reinterpret_cast<float*>(out)[(long)c * ldo + f] = v[e];
              else
                reinterpret_cast<bf16*>(out)[(long)c * ldo + f] = __float2bfloat16_rn(v[e]);
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0 && abort_flag && error_word) atomicExch(error_word, 1);
}

// out[i] = sum over the planes, in order, rounded once (bf16) or kept (fp32): finishes a product
// that was cut over ranges of K where nobody else adds the planes up.
template <typename T>
__global__ void sum_planes_kernel(const float* __restrict__ planes, int parts, long plane_stride,
                                  T* __restrict__ out, long n4) {
  pdl_wait();
  pdl_launch_dependents();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 acc = *reinterpret_cast<const float4*>(planes + 4 * i);
  for (int p = 1; p < parts; ++p) {
    const float4 v = *reinterpret_cast<const float4*>(planes + (long)p * plane_stride + 4 * i);
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
  }
  if (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + 4 * i) = acc;
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + 4 * i) = packed;
  }
}

int skinny_sm_count() {
  static int count_on[Q3_MAX_DEVICES];
  int& count = count_on[q3_current_device()];
  if (!count) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || count < 2) count = 148;
  }
  return count;
}

// Ranges of K: as many as give every SM an item, each a whole number of 64-wide k-blocks.
void skinny_plan(int N, int K, int max_ranges, int* kb_per_range, int* ranges) {
  const int tiles_f = (N + SK_BM - 1) / SK_BM;
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  int want = skinny_sm_count() / tiles_f;
  want = want < 1 ? 1 : (want > max_ranges ? max_ranges : want);
  if (want > num_kb) want = num_kb;
  *kb_per_range = (num_kb + want - 1) / want;
  *ranges = (num_kb + *kb_per_range - 1) / *kb_per_range;
}

template <int MODE>
int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, void* out, int ldo, int M, int N, int K,
                  int kb_per_range, int ranges, int* error_word, cudaStream_t stream) {
  constexpr size_t smem = (size_t)SK_STAGES * SK_STAGE_BYTES + 1024;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  const int items = ((N + SK_BM - 1) / SK_BM) * ranges;
  const int sms = skinny_sm_count();
  const int grid = items < sms ? items : sms;
  return launch_pdl(gemm_skinny_kernel<MODE>, dim3(grid), dim3(SK_THREADS), smem, stream, tw, tx, out, ldo, M, N, K,
                    kb_per_range, ranges, error_word) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

}  // namespace

// How many planes q3_gemm_skinny writes for these sizes when it may cut K (max_ranges >= 1).
Q3_EXPORT int q3_gemm_skinny_ranges(int N, int K, int max_ranges) {
  if (N < 1 || K < 1 || max_ranges < 1) return 0;
  int per = 0, ranges = 0;
  skinny_plan(N, K, max_ranges, &per, &ranges);
  return ranges;
}

// x bf16 [M, K] (1 <= M <= 64), W bf16 [N, K]; leading dimensions in elements, multiples of 8;
// bases 16-byte aligned.  ranges = 1: out is bf16 (mode 0) or fp32 (mode 1) [M, N] with row
// stride ldo.  ranges > 1 (what q3_gemm_skinny_ranges answered for the same max_ranges): out is
// fp32 [ranges, M, N] (ldo = N) whose planes add up to the product; mode must be 2.
// error_word: device int, set non-zero if a bounded wait expired.
Q3_EXPORT int q3_gemm_skinny(int mode, const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M,
                             int N, int K, int ranges, int* error_word, cudaStream_t stream) {
  if (!x || !W || !out || N < 1 || K < 1 || M < 0 || ranges < 1 || mode < 0 || mode > 2) return Q3_ERR_ARGUMENT;
  if (M > SK_NT || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return Q3_ERR_UNSUPPORTED;
  if ((mode == SK_PLANES) != (ranges > 1) && !(mode == SK_PLANES && ranges == 1)) return Q3_ERR_ARGUMENT;
  if (M == 0) return Q3_OK;
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  if (ranges > num_kb) return Q3_ERR_ARGUMENT;
  const int per = (num_kb + ranges - 1) / ranges;
  if ((num_kb + per - 1) / per != ranges) return Q3_ERR_ARGUMENT;
  CUtensorMap tw, tx;
  if (!q3_bf16_map(&tw, W, N, K, ldw, SK_BM) || !q3_bf16_map(&tx, x, M, K, ldx, SK_NT)) return Q3_ERR_LAUNCH;
  if (mode == SK_PLANES) return launch_skinny<SK_PLANES>(tw, tx, out, ldo, M, N, K, per, ranges, error_word, stream);
  if (mode == SK_F32) return launch_skinny<SK_F32>(tw, tx, out, ldo, M, N, K, per, ranges, error_word, stream);
  return launch_skinny<SK_BF16>(tw, tx, out, ldo, M, N, K, per, ranges, error_word, stream);
}

// out (bf16 for dtype 1, fp32 for dtype 0) [n] = planes[0] + planes[1] + ... ; n a multiple of 4,
// planes `plane_stride` floats apart, everything 16-byte aligned (out 8-byte for bf16).
Q3_EXPORT int q3_sum_planes(int dtype, const float* planes, int parts, long plane_stride, void* out, long n,
                            cudaStream_t stream) {
  if (!planes || !out || parts < 1 || n < 0) return Q3_ERR_ARGUMENT;
  if (n % 4 || plane_stride % 4 || ((uintptr_t)planes & 15) || ((uintptr_t)out & 7)) return Q3_ERR_UNSUPPORTED;
  if (n == 0) return Q3_OK;
  const long n4 = n / 4;
  const unsigned blocks = (unsigned)((n4 + 255) / 256);
  cudaError_t err;
  if (dtype == Q3_DTYPE_F32)
    err = launch_pdl(sum_planes_kernel<float>, dim3(blocks), dim3(256), 0, stream, planes, parts, plane_stride,
                     (float*)out, n4);
  else if (dtype == Q3_DTYPE_BF16)
    err = launch_pdl(sum_planes_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, planes, parts, plane_stride,
                     (bf16*)out, n4);
  else
    return Q3_ERR_ARGUMENT;
  return err == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
