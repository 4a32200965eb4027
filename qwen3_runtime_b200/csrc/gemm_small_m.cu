// out[M, N] = x[M, K] * W[N, K]^T for a handful of tokens (M <= 16), bfloat16 in, fp32
// accumulate: the decode-step matrix products.  With so few tokens the product is a pure
// stream over the weights, so the kernel is built around reading W once at full HBM
// bandwidth: weights are the 16-row side of m16n8k16 tensor-core tiles ("swap-AB": output
// features on M, tokens on N = 8 or 16), and both operands go from global memory straight
// into fragment registers with 16-byte loads -- no shared-memory staging.  That works
// because the contraction index may be permuted freely as long as both operands use the
// same permutation: a thread's 8 consecutive k-values of a weight row (one 16-byte load)
// are paired with the same 8 k-values of its token row and spread over two MMAs.
//
// A block has 8 or 16 warps = (warps / KS) output tiles of 16 features x KS slices of K; the slices
// of a tile are summed through shared memory.  KS is chosen by the launcher so that
// narrow products (N = hidden) still give every SM several warps.
// Epilogues: bf16 out; fp32 out (logits); SwiGLU (the block computes gate and up rows of the
// same features and writes silu(gate) * up, models/qwen3.py:137-138, layers/ops.py:23-25).
#include "common.cuh"

namespace {

enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_SWIGLU = 2 };
constexpr int MAX_WARPS = 16;

__device__ __forceinline__ uint4 ldg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg16_cached(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: token tiles of 8 (1 or 2).  MODE: epilogue.  SETS: 2 for SwiGLU (gate and up), else 1.
// WARPS_ x MINB_ is chosen so that the register cap is 64: two 16-warp blocks or four 8-warp
// blocks per SM, which lets every shape of the model run as a single wave of blocks.
template <int NT, int MODE, int WARPS_, int MINB_>
__global__ void __launch_bounds__(WARPS_ * 32, MINB_)
gemm_small_m_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw,
                    void* __restrict__ out, int ldo, int M, int N, int K, int KS, int kper, int up_offset,
                    int prefetch_l2) {
  constexpr int SETS = MODE == OUT_SWIGLU ? 2 : 1;
  constexpr int U = 2;  // k-blocks of 32 in flight per thread (64 registers: many warps instead)
  __shared__ float red[MAX_WARPS][SETS * NT * 4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int MT = (blockDim.x >> 5) / KS;
  const int tile = blockIdx.x * MT + warp / KS;
  const int ks = warp % KS;
  const int row0 = tile * 16;
  const int k_lo = ks * kper, k_hi = min(K, k_lo + kper);

  float acc[SETS][NT][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[s][n][0] = acc[s][n][1] = acc[s][n][2] = acc[s][n][3] = 0.f;

  if (row0 < N) {
    // weight rows of this thread: row0 + g and row0 + g + 8 (clamped; rows >= N are never stored)
    const bf16* w_lo[SETS];
    const bf16* w_hi[SETS];
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
      const int base = row0 + s * up_offset;
      w_lo[s] = W + (long)min(base + g, N + s * up_offset - 1) * ldw;
      w_hi[s] = W + (long)min(base + g + 8, N + s * up_offset - 1) * ldw;
    }
    const bf16* x_row[NT];
    bool x_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      x_ok[n] = n * 8 + g < M;
      x_row[n] = x + (long)(x_ok[n] ? n * 8 + g : 0) * ldx;
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // The first weights are fetched before waiting for the kernel that produces x: weights do
    // not depend on it, so this overlaps the predecessor's tail (programmatic dependent launch).
    uint4 wl[SETS][U], wh[SETS][U], xv[NT][U];
    auto load_w = [&](int k0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + 32 * u + 8 * t;
        const bool ok = k < k_hi;  // K and kper are multiples of 8, so a chunk is all in or all out
#pragma unroll
        for (int s = 0; s < SETS; ++s) {
          wl[s][u] = ok ? ldg16(w_lo[s] + k) : zero;
          wh[s][u] = ok ? ldg16(w_hi[s] + k) : zero;
        }
      }
    };
    load_w(k_lo);
    // ... and the rest of this warp's weight slice is requested into L2, one 128-byte line per
    // request, so that HBM keeps streaming while the predecessor finishes (only for weights
    // that fit in L2 with room to spare: requested too far ahead, lines are evicted again)
    for (int s = 0; s < SETS && prefetch_l2; ++s) {
      const bf16* row = W + (long)min(row0 + s * up_offset + (lane & 15), N + s * up_offset - 1) * ldw;
      for (int k = k_lo + 32 * U + 64 * (lane >> 4); k < k_hi; k += 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(row + k));
    }
    pdl_wait();
    for (int k0 = k_lo; k0 < k_hi; k0 += 32 * U) {
      if (k0 != k_lo) load_w(k0);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + 32 * u + 8 * t;
        const bool ok = k < k_hi;
#pragma unroll
        for (int n = 0; n < NT; ++n) xv[n][u] = (ok && x_ok[n]) ? ldg16_cached(x_row[n] + k) : zero;
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int s = 0; s < SETS; ++s)
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            mma_bf16(acc[s][n], wl[s][u].x, wh[s][u].x, wl[s][u].y, wh[s][u].y, xv[n][u].x, xv[n][u].y);
            mma_bf16(acc[s][n], wl[s][u].z, wh[s][u].z, wl[s][u].w, wh[s][u].w, xv[n][u].z, xv[n][u].w);
          }
    }
  } else {
    pdl_wait();
  }
  pdl_launch_dependents();

  // ---- sum the K slices of each tile, then the epilogue ---------------------------------------
  if (KS > 1) {
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[warp][(s * NT + n) * 4 + e][lane] = acc[s][n][e];
    __syncthreads();
    if (ks != 0) return;
    for (int o = 1; o < KS; ++o)
#pragma unroll
      for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[s][n][e] += red[warp + o][(s * NT + n) * 4 + e][lane];
  }
  if (row0 >= N) return;
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int feature = row0 + g + (e >> 1) * 8;
      const int token = n * 8 + 2 * t + (e & 1);
      if (feature >= N || token >= M) continue;
      float v = acc[0][n][e];
      if (MODE == OUT_SWIGLU) v = (v / (1.f + expf(-v))) * acc[SETS - 1][n][e];
      if (MODE == OUT_F32)
        reinterpret_cast<float*>(out)[(long)token * ldo + feature] = v;
      else
        reinterpret_cast<bf16*>(out)[(long)token * ldo + feature] = __float2bfloat16_rn(v);
    }
}

template <int NT, int MODE>
int launch(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int M, int N, int K, int up_offset,
           cudaStream_t stream) {
  const int tiles = (N + 15) / 16;
  // split K until there are about 16 warps per SM, but keep slices of at least 256
  int KS = 1;
  while (KS < MAX_WARPS && tiles * KS < 16 * 148 && K / (KS * 2) >= 256) KS *= 2;
  int kper = (K + KS - 1) / KS;
  kper = (kper + 31) & ~31;
  const int warps = KS > 8 ? 16 : 8;  // blocks of 8 warps balance better; 16 only to split K further
  const int MT = warps / KS;
  const int blocks = (tiles + MT - 1) / MT;
  cudaError_t err;
  const int prefetch_l2 = (long)N * K * 2 * (MODE == OUT_SWIGLU ? 2 : 1) <= (64L << 20);
  if (warps == 16)
    err = launch_pdl(gemm_small_m_kernel<NT, MODE, 16, 2>, dim3(blocks), dim3(512), 0, stream, x, ldx, W, ldw, out,
                     ldo, M, N, K, KS, kper, up_offset, prefetch_l2);
  else
    err = launch_pdl(gemm_small_m_kernel<NT, MODE, 8, 4>, dim3(blocks), dim3(256), 0, stream, x, ldx, W, ldw, out,
                     ldo, M, N, K, KS, kper, up_offset, prefetch_l2);
  return err == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}

}  // namespace

// mode 0: out bf16 [M, N]; 1: out fp32 [M, N]; 2: W is [2 * N, K] with gate rows first and up
// rows from row `N`, out bf16 [M, N] = silu(x W_gate^T) * (x W_up^T).
// M <= 16; K a multiple of 8; leading dimensions in elements (ldx, ldw multiples of 8).
Q3_EXPORT int q3_gemm_small_m(int mode, const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M,
                              int N, int K, cudaStream_t stream) {
  if (!x || !W || !out || N < 1 || K < 1 || M < 0) return Q3_ERR_ARGUMENT;
  if (M > 16 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
#define Q3_GEMM_CASE(NT, MODE) return launch<NT, MODE>(xp, ldx, wp, ldw, out, ldo, M, N, K, mode == 2 ? N : 0, stream)
  if (M <= 8) {
    if (mode == OUT_BF16) Q3_GEMM_CASE(1, OUT_BF16);
    if (mode == OUT_F32) Q3_GEMM_CASE(1, OUT_F32);
    if (mode == OUT_SWIGLU) Q3_GEMM_CASE(1, OUT_SWIGLU);
  } else {
    if (mode == OUT_BF16) Q3_GEMM_CASE(2, OUT_BF16);
    if (mode == OUT_F32) Q3_GEMM_CASE(2, OUT_F32);
    if (mode == OUT_SWIGLU) Q3_GEMM_CASE(2, OUT_SWIGLU);
  }
#undef Q3_GEMM_CASE
  return Q3_ERR_ARGUMENT;
}
