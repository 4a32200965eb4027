// out[M, N] = x[M, K] * W[N, K]^T for at most 16 tokens, bfloat16 in, fp32 accumulate: the
// matrix products of a decode step, built as a stream over the weights.
//
// With so few tokens the product is memory bound, and what decides its speed is how many
// bytes of W each SM keeps in flight.  Registers cannot hold enough, so the weights go
// through shared memory: one producer lane per row issues bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier) of whole row segments into a ring of
// stages that fills most of the SM's shared memory (about 160-190 KB in flight per SM), and
// 16 consumer warps feed them to mma.sync.  One block per SM, persistent over its units.
//
// Work: W is cut into panels of 8 rows (4 gate rows and the 4 up rows of the same features
// for the SwiGLU product) and K into `parts` (1, 2, 4 or 8) equal ranges; a unit is one panel x one range and fills one
// stage.  Block b always has range b % parts, so the tokens' values for that range live in
// registers for the whole kernel: consumer warp w owns the 32-wide k-blocks w, w+16, ... of
// the range.  The MMA is m16n8k16 with the tokens as its 16 rows and the panel's 8 weight
// rows as its 8 columns; a thread pairs 8 consecutive k-values of its weight row (one
// 16-byte shared-memory read, conflict free because the row pitch is 64 mod 128 bytes) with
// the same 8 k-values of its token rows, which is a valid contraction because both operands
// use the same permutation of k.  After a stage the 16 warps' partial tiles are summed
// through shared memory in warp order.
//
// A finished product (modes 0..2) is made with one range of K (parts = 1): a block owns whole
// rows of the result and nobody waits for anybody.  K is cut into ranges only for partial sums
// (mode 3): the block of range p writes its fp32 partial of every unit to
// out[p][token][feature], and whoever reads the product adds the `parts` planes in order; in a
// decode step that is the norm kernel that folds the product into the residual sum, which
// reads a few fp32 rows more and saves the blocks any exchange among themselves.
//
// Every mbarrier wait is bounded; on expiry the waiter sets the error word and carries on
// (the result is then invalid, and the host raises), so no barrier is ever abandoned.
#define Q3_WAIT_LIMIT_CYCLES 400000000ll
#include "async_tiles.cuh"

namespace {

enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_SWIGLU = 2, OUT_PARTIAL = 3 };
constexpr int CONSUMER_WARPS = 16;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_LIMIT = 226 * 1024;     // dynamic; the barriers are static
constexpr int RED_BYTES = 2 * CONSUMER_WARPS * 4 * 32 * 4;  // two buffers of the warps' tiles

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Plan {
  int parts;       // ranges of K
  int range;       // k-values per range (multiple of 32; the last range may be shorter)
  int pitch;       // bytes between rows of a stage, 64 mod 128
  int stages;
  int blocks;      // multiple of parts
  int panels;
};

// k-blocks of 32 per consumer warp: what its registers hold of the tokens' values
template <bool HI> struct Blocks { static constexpr int value = 5; };

// MODE: epilogue.  HI: tokens 8..15 exist (M > 8).
template <int MODE, bool HI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ W, int ldw, void* __restrict__ out,
                   int ldo, int M, int N, int K, int up_offset, Plan plan, int* __restrict__ error_word) {
  constexpr int ROWS = 8;
  constexpr int XB = Blocks<HI>::value;
  constexpr int FPP = MODE == OUT_SWIGLU ? 4 : 8;  // output features per panel
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES];
  const int stage_bytes = ROWS * plan.pitch;
  float* red = reinterpret_cast<float*>(smem + (size_t)plan.stages * stage_bytes);  // [2][warps][4][32]
  const uint32_t full0 = smem_addr(bars), empty0 = smem_addr(bars + MAX_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = blockIdx.x % plan.parts;
  const int k_lo = part * plan.range, k_hi = min(K, k_lo + plan.range);
  const int klen = k_hi - k_lo;                        // > 0 by construction
  const int first_panel = blockIdx.x / plan.parts, panel_step = plan.blocks / plan.parts;
  const int my_units = first_panel < plan.panels ? (plan.panels - 1 - first_panel) / panel_step + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < plan.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, CONSUMER_WARPS);
    }
    mbar_init_fence();
  }
  if (K & 31) {  // the tail of the last k-block is read but never copied: keep it finite
    for (int i = threadIdx.x * 16; i < plan.stages * stage_bytes; i += THREADS * 16)
      *reinterpret_cast<uint4*>(smem + i) = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp == CONSUMER_WARPS) {
    // ---- producer: weights do not depend on the kernel before this one, so it starts at once ----
    const uint32_t bytes_row = (uint32_t)klen * 2;
    for (int u = 0; u < my_units; ++u) {
      const int s = u % plan.stages;
      if (u >= plan.stages) mbar_wait_report(empty0 + 8 * s, ((u / plan.stages) & 1) ^ 1, error_word, 1);
      const int row0 = (first_panel + u * panel_step) * FPP;
      const int rows_live = min(FPP, N - row0);  // per half for SwiGLU: gate rows, then up rows
      if (lane == 0) mbar_expect_tx(full0 + 8 * s, bytes_row * rows_live * (ROWS / FPP));
      __syncwarp();
      if (lane < ROWS && (lane % FPP) < rows_live) {
        const long row = row0 + (lane % FPP) + (lane / FPP) * up_offset;
        bulk_copy(smem_addr(smem + (size_t)s * stage_bytes + lane * plan.pitch), W + row * ldw + k_lo, bytes_row,
                  full0 + 8 * s);
      }
    }
    return;
  }

  // ---- consumers ----------------------------------------------------------------------------------
  const int g = lane >> 2, t = lane & 3;
  pdl_wait();  // x comes from the kernel before this one
  uint4 xg[XB], xh[XB];
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int i = 0; i < XB; ++i) {
    const int k = 32 * (warp + CONSUMER_WARPS * i) + 8 * t;
    const bool ok = k < klen;
    xg[i] = (ok && g < M) ? __ldg(reinterpret_cast<const uint4*>(x + (long)g * ldx + k_lo + k)) : zero;
    xh[i] = (HI && ok && g + 8 < M) ? __ldg(reinterpret_cast<const uint4*>(x + (long)(g + 8) * ldx + k_lo + k)) : zero;
  }
  const int my_blocks = (klen + 31) / 32;  // k-blocks of this range; this warp has w, w+16, ...

  for (int u = 0; u < my_units; ++u) {
    const int s = u % plan.stages;
    const int panel = first_panel + u * panel_step;
    mbar_wait_report(full0 + 8 * s, (u / plan.stages) & 1, error_word, 2);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const unsigned char* base = smem + (size_t)s * stage_bytes + g * plan.pitch + 16 * t;
#pragma unroll
    for (int i = 0; i < XB; ++i) {
      const int b = warp + CONSUMER_WARPS * i;
      if (b < my_blocks) {
        const uint4 w = *reinterpret_cast<const uint4*>(base + 64 * b);
        mma_bf16(acc, xg[i].x, xh[i].x, xg[i].y, xh[i].y, w.x, w.y);
        mma_bf16(acc, xg[i].z, xh[i].z, xg[i].w, xh[i].w, w.z, w.w);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * s);  // the stage may be refilled

    // sum the warps' tiles (warp order), two buffers so that one barrier per unit is enough
    float* rbuf = red + (size_t)(u & 1) * CONSUMER_WARPS * 4 * 32;
#pragma unroll
    for (int e = 0; e < 4; ++e) rbuf[(warp * 4 + e) * 32 + lane] = acc[e];
    consumer_sync();
    if (threadIdx.x < 128) {  // thread = (e, lane) of the tile: token g + 8 * (e >> 1), row 2t + (e & 1)
      const int e = threadIdx.x >> 5;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < CONSUMER_WARPS; ++w) v += rbuf[(w * 4 + e) * 32 + lane];
      // SwiGLU: rows 0..3 of the panel are gate rows, rows 4..7 the up rows of the same features,
      // held two lanes further on
      const float up = MODE == OUT_SWIGLU ? __shfl_down_sync(0xffffffffu, v, 2) : 0.f;
      const int token = g + 8 * (e >> 1);
      const int feature = panel * FPP + 2 * t + (e & 1);
      if (token < M && feature < N && (MODE != OUT_SWIGLU || t < 2)) {
        float r = v;
        if (MODE == OUT_SWIGLU) r = (r / (1.f + expf(-r))) * up;
        if (MODE == OUT_PARTIAL)
          reinterpret_cast<float*>(out)[((long)part * M + token) * ldo + feature] = r;
        else if (MODE == OUT_F32)
          reinterpret_cast<float*>(out)[(long)token * ldo + feature] = r;
        else
          reinterpret_cast<bf16*>(out)[(long)token * ldo + feature] = __float2bfloat16_rn(r);
      }
    }
  }
  // only now: a successor that starts earlier requests its own weights into L2 while this
  // kernel is still streaming through it, and loses them again before it can use them
  pdl_launch_dependents();
}

cudaError_t launch_stream(const void* kernel, int blocks, size_t smem, cudaStream_t stream, void** args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
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
  return cudaLaunchKernelExC(&cfg, kernel, args);
}

// Ranges of K: as few as keep a range within what a warp's registers hold and the ring at two
// stages or more; more only while that shortens the longest block's work (units x (range +
// a fixed part worth 256 k-values)).
// finished: the product is wanted whole, so K is not cut at all.
bool make_plan(bool finished, int N, int K, int features_per_panel, int max_range, int sm_count, Plan* plan) {
  const int panels = (N + features_per_panel - 1) / features_per_panel;
  long best_cost = 0;
  plan->parts = 0;
  for (int parts = 1; parts <= (finished ? 1 : 8); parts *= 2) {
    int range = (K + parts - 1) / parts;
    range = (range + 31) & ~31;
    if (range > max_range) continue;
    if ((long)(parts - 1) * range >= K) continue;  // an empty range
    const int sets = sm_count / parts;                   // sets of `parts` blocks that share panels
    if (sets < 1) continue;
    const int groups = sets < panels ? sets : panels;  // sets launched
    const int units = (panels + groups - 1) / groups;
    const int pitch = ((range * 2 + 127) & ~127) + 64;
    int stages = (SMEM_LIMIT - RED_BYTES) / (8 * pitch);
    if (stages < 2) continue;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    const long cost = (long)units * (range + 256);
    if (!plan->parts || cost < best_cost) {
      best_cost = cost;
      plan->parts = parts;
      plan->range = range;
      plan->pitch = pitch;
      plan->stages = stages;
      plan->blocks = groups * parts;
      plan->panels = panels;
    }
  }
  return plan->parts != 0;
}

template <int MODE, bool HI>
int launch(const bf16* x, int ldx, const bf16* W, int ldw, void* out, int ldo, int M, int N, int K, int up_offset,
           int sm_count, int only_large, int planes, int* error_word, cudaStream_t stream) {
  const void* kernel = (const void*)gemm_stream_kernel<MODE, HI>;
  static bool configured_on[Q3_MAX_DEVICES];
  bool& configured = configured_on[q3_current_device()];
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    configured = true;
  }
  Plan plan;
  if (!make_plan(MODE != OUT_PARTIAL, N, K, MODE == OUT_SWIGLU ? 4 : 8,
                 CONSUMER_WARPS * 32 * Blocks<HI>::value, sm_count, &plan))
    return Q3_ERR_UNSUPPORTED;
  if (MODE == OUT_PARTIAL && plan.parts != planes) return Q3_ERR_ARGUMENT;
  // A block owns its SM, so kernels do not overlap at their ends: short products (few units
  // per block) are faster on the kernel that streams through registers.
  if (MODE != OUT_PARTIAL && only_large && plan.panels < 8 * plan.blocks) return Q3_ERR_UNSUPPORTED;
  const size_t smem = (size_t)plan.stages * 8 * plan.pitch + RED_BYTES;
  void* args[] = {&x, &ldx, &W, &ldw, &out, &ldo, &M, &N, &K, &up_offset, &plan, &error_word};
  return launch_stream(kernel, plan.blocks, smem, stream, args) == cudaSuccess
             ? Q3_OK
             : Q3_ERR_LAUNCH;
}

int sm_count_of_current_device() {
  static int count_on[Q3_MAX_DEVICES];
  int& count = count_on[q3_current_device()];
  if (!count) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 8)
      count = 0;
  }
  return count;
}

}  // namespace

// mode 0: out bf16 [M, N]; 1: out fp32 [M, N]; 2: W is [2 * N, K] with gate rows first and up
// rows from row `N`, out bf16 [M, N] = silu(x W_gate^T) * (x W_up^T).
// M <= 16; K a multiple of 8 and at most 40960 (20480 when M > 8); leading dimensions in
// elements (ldx, ldw multiples of 8); x and W 16-byte aligned; anything else is refused as
// unsupported.  only_large != 0: also refuse the products for which q3_gemm_small_m is the
// faster kernel on a B200.  `error_word` is set non-zero if a bounded wait expired.
Q3_EXPORT int q3_gemm_stream(int mode, const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M,
                             int N, int K, int only_large, int* error_word, cudaStream_t stream) {
  if (!x || !W || !out || !error_word || N < 1 || K < 1 || M < 0 || mode < 0 || mode > 2) return Q3_ERR_ARGUMENT;
  if (M > 16 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldo < N) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  const int sms = sm_count_of_current_device();
  if (!sms) return Q3_ERR_LAUNCH;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  const int up = mode == OUT_SWIGLU ? N : 0;
#define Q3_STREAM_CASE(MODE)                                                                                  \
  return M > 8 ? launch<MODE, true>(xp, ldx, wp, ldw, out, ldo, M, N, K, up, sms, only_large, 0, error_word, stream)          \
               : launch<MODE, false>(xp, ldx, wp, ldw, out, ldo, M, N, K, up, sms, only_large, 0, error_word, stream)
  if (mode == OUT_BF16) Q3_STREAM_CASE(OUT_BF16);
  if (mode == OUT_F32) Q3_STREAM_CASE(OUT_F32);
  Q3_STREAM_CASE(OUT_SWIGLU);
#undef Q3_STREAM_CASE
}

// The number of K ranges that q3_gemm_stream_partial cuts this product into (its output has
// that many planes); 0 if the product is not supported.
Q3_EXPORT int q3_gemm_stream_parts(int M, int N, int K) {
  if (N < 1 || K < 1 || M < 1 || M > 16 || K % 8) return 0;
  const int sms = sm_count_of_current_device();
  Plan plan;
  if (!sms || !make_plan(false, N, K, 8, CONSUMER_WARPS * 32 * Blocks<true>::value, sms, &plan)) return 0;
  return plan.parts;
}

// out fp32 [parts, M, N] with out[p] = x[:, range p] * W[:, range p]^T, so that the product is
// the sum of the planes; `parts` must be what q3_gemm_stream_parts returns for these sizes.
// Otherwise as q3_gemm_stream.
Q3_EXPORT int q3_gemm_stream_partial(const void* x, int ldx, const void* W, int ldw, float* out, int parts, int M,
                                     int N, int K, int* error_word, cudaStream_t stream) {
  if (!x || !W || !out || !error_word || N < 1 || K < 1 || M < 0 || parts < 1) return Q3_ERR_ARGUMENT;
  if (M > 16 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K) return Q3_ERR_UNSUPPORTED;
  if (((uintptr_t)x | (uintptr_t)W) & 15) return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  const int sms = sm_count_of_current_device();
  if (!sms) return Q3_ERR_LAUNCH;
  const bf16* xp = (const bf16*)x;
  const bf16* wp = (const bf16*)W;
  return M > 8 ? launch<OUT_PARTIAL, true>(xp, ldx, wp, ldw, out, N, M, N, K, 0, sms, 0, parts, error_word, stream)
               : launch<OUT_PARTIAL, false>(xp, ldx, wp, ldw, out, N, M, N, K, 0, sms, 0, parts, error_word, stream);
}
