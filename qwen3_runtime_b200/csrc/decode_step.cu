// All layers of a decode step (every sequence brings one token; at most 16 sequences) as ONE
// persistent kernel, bfloat16, for blocks of the shape  x += attention(norm(x)); x += mlp(norm(x))
// with RMSNorm, grouped-query attention over the paged cache (optional per-head q/k norm, rotary
// position encoding) and a SwiGLU feed-forward, no biases, no window.
//
// Why one kernel.  A decode step is bound by memory: every weight and every cached key and value
// is read once.  As separate kernels (norm, q/k/v product, attention, o product, norm, gate/up
// product, down product: seven launches a layer) each one starts with an empty memory pipe and
// ends by draining it, and memory idles a quarter of the time.  Here one block per SM lives for
// the whole step.  A producer warp streams everything the block will need -- the rows of the
// four weight matrices it owns and the key/value tiles of its share of the attention, layer
// after layer -- through one ring of shared-memory stages with bulk asynchronous copies
// (cp.async.bulk, completion counted on mbarriers).  None of that data depends on what the step
// computes, so the producer never waits for anything but a free stage: while the consumer warps
// sit at a barrier over the grid or fetch their activations, the ring keeps filling, and memory
// stays busy across what used to be kernel boundaries.
//
// Work of a layer, in five phases separated by barriers over the grid (consumers only):
//   QKV   qkv = norm1(x) Wqkv^T                      panels of 8 weight rows x ranges of K
//   ATT   ctx = attention(q, cache + newest k, v)    tiles of 64 keys of one (sequence, kv head)
//   O     x  += ctx Wo^T                             panels x ranges; finished rows add into x
//   GU    mid = silu(norm2(x) Wg^T) * (norm2(x) Wu^T) panels of 4 gate + 4 up rows
//   DOWN  x  += mid Wd^T                             panels x ranges
// A product: block b owns the panels b, b + grid, ... whole, so nobody ever exchanges partial
// sums with anybody.  The tokens' values live in registers (16 consumer warps, mma.sync
// m16n8k16 with the tokens as the 16 rows, the warps' tiles summed through shared memory in
// warp order, as gemm_stream.cu), which holds 2560 k-values; a longer inner dimension is cut
// into chunks and the block goes through its panels once per chunk, adding up the panels' fp32
// tiles in shared memory in chunk order.  The epilogue of O and DOWN adds the finished values
// into the fp32 residual sum and leaves the panel's sum of squares per token; the next norm is
// then a scale by rsqrt(mean) applied while the tokens' values are loaded into registers (fp32
// arithmetic, one rounding, as norm.cu).
// Attention: the 64-key tiles of all (sequence, kv head) pairs are dealt out in equal runs to the
// blocks; keys and values arrive as TMA boxes of one page's rows x 64 dims with the 128-byte
// swizzle (free of bank conflicts for ldmatrix; one tensor map per layer for keys and one for
// values, kept in device memory); a team of 4 warps takes a tile (16 keys per warp, online softmax
// in fp32 as attention_decode.cu); a run that ends inside a pair leaves a partial result and the
// pair's last block merges them.  The block whose run holds a sequence's newest position makes
// that token's k and v (per-head norm, rotation: rotary.cuh), writes them to their page and
// patches them into its tile.
//
// Every wait is bounded (mbarriers and the barrier over the grid); on expiry the waiter sets the
// error word and carries on, later waits return at once, and the host raises.
#define Q3_WAIT_LIMIT_CYCLES 600000000ll
#include "async_tiles.cuh"
#include "mma_tiles.cuh"
#include "rotary.cuh"

namespace {

constexpr int CW = 16;                   // consumer warps
constexpr int CONSUMERS = CW * 32;
constexpr int THREADS = CONSUMERS + 32;  // + the producer warp
constexpr int XB = 5;                    // 32-wide k-blocks of a range per consumer warp
constexpr int MAX_RANGE = CW * 32 * XB;  // 2560 k-values of a range
constexpr int MAX_STAGES = 8;
constexpr int TILE = 64;                 // keys per attention tile
constexpr int D = 128;                   // head size this kernel is built for
constexpr int HALF_TILE = TILE * 128;    // bytes of 64 keys x 64 dims; a K (V) tile is D / 64 of them
constexpr int KV_TILE = (D / 64) * HALF_TILE;
constexpr int TILE_BYTES = 2 * KV_TILE;
constexpr int ACC_MAX_PANELS = 24;       // panels of a chunked product one block may own
constexpr int MAX_TOKENS = 16;
constexpr int ERR_WAIT = 7;              // error word: a bounded wait of this kernel expired
constexpr int ERR_POSITION = 16;         // a newest position outside the rotation tables

enum { PH_QKV = 0, PH_ATT = 1, PH_O = 2, PH_GU = 3, PH_DOWN = 4 };

struct LayerPtrs {
  const bf16* wqkv;   // [(nq + 2 nkv) D, H]
  const bf16* wo;     // [H, nq D]
  const bf16* wgu;    // [2 I, H]: gate rows, then up rows
  const bf16* wdown;  // [H, I]
  const float* norm1; // [H]
  const float* norm2; // [H]
  const float* qnorm; // [D] or null
  const float* knorm; // [D] or null
  bf16* kpages;       // [pages, nkv, ps, D]
  bf16* vpages;
};

struct Product {  // how one product is cut (host side: make_product)
  int N, K;       // output features (SwiGLU: per half), inner dimension
  int chunks;     // pieces of K a block goes through one after the other
  int range;      // k-values per chunk, a multiple of 32
  int pitch;      // bytes between rows of a stage, 64 mod 128
  int panels;
  int fpp;        // output features per panel: 8, or 4 for SwiGLU
};

struct StepArgs {
  const LayerPtrs* layers;
  int L, M, H, I, nq, nkv, ps, vocab;
  const int* token_ids;
  const bf16* embed;
  const int* kv_lens;
  const int* block_table;
  int max_pages;
  const float* cos_t;
  const float* sin_t;
  int max_pos, pairing;
  float eps, qk_eps, scale_log2;
  Product prod[5];    // indexed by phase (PH_ATT unused)
  int stages, stage_bytes, red_bytes;
  const CUtensorMap* maps;  // [L][2]: key pages, value pages as [rows of all pages and heads][D]
  // scratch, all written and read inside the kernel (activations go past L1)
  float* resid;       // [16, H]: the residual sum; the step's result
  float* sumsq;       // [2][H / 8][16]: per panel of 8 features, each token's sum of squares
  bf16* qkv;          // [16, (nq + 2 nkv) D]
  bf16* ctx;          // [16, nq D]
  bf16* mid;          // [16, I]
  float* att_o;       // [pairs + grid][G][D]
  float* att_lse;     // [pairs + grid][G]
  int* att_tickets;   // [pairs], zero between uses
  unsigned* barrier;  // zero at launch
  int* error_word;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }
__device__ __forceinline__ void quad_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }  // warps 0..3
__device__ __forceinline__ void team_sync(int team) {
  asm volatile("bar.sync %0, 128;" ::"r"(3 + team) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_volatile(const int* p) {
  int v;
  asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait on a stage barrier that gives up at once when the step has already failed.
__device__ __forceinline__ void stage_wait(uint32_t bar, uint32_t parity, int* error_word) {
  if (mbar_try_wait(bar, parity)) return;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    const long long waited = clock64() - start;
    if (waited > Q3_WAIT_LIMIT_CYCLES || ((waited & 0xffff) < 64 && ld_volatile(error_word) != 0)) {
      atomicCAS(error_word, 0, ERR_WAIT);
      return;
    }
  }
}

// Barrier over the grid for the consumer threads.  `epoch` counts arrivals expected so far.
__device__ __forceinline__ void grid_sync(const StepArgs& a, unsigned& epoch) {
  consumer_sync();
  if (threadIdx.x == 0) {
    epoch += gridDim.x;
    __threadfence();
    atomicAdd(a.barrier, 1u);
    if (ld_acquire(a.barrier) < epoch) {
      const long long start = clock64();
      while (ld_acquire(a.barrier) < epoch) {
        const long long waited = clock64() - start;
        if (waited > Q3_WAIT_LIMIT_CYCLES || ((waited & 0xfff) < 64 && ld_volatile(a.error_word) != 0)) {
          atomicCAS(a.error_word, 0, ERR_WAIT);
          break;
        }
      }
    }
    __threadfence();
  }
  consumer_sync();
}

// byte offset of 16-byte chunk `chunk` of key row `row` in a K (V) tile as the boxes land
__device__ __forceinline__ int kv_off(int row, int chunk) {
  return (chunk >> 3) * HALF_TILE + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

// ---- how the attention tiles are dealt out -------------------------------------------------------
struct AttPlan {
  int tiles_of[MAX_TOKENS];  // 64-key tiles of each sequence (per kv head)
  int total;                 // all tiles: nkv * sum(tiles_of)
};
__device__ __forceinline__ long tile_begin(const AttPlan& p, int cta) { return (long)cta * p.total / gridDim.x; }
__device__ __forceinline__ int cta_of_tile(const AttPlan& p, long t) {
  return (int)(((t + 1) * gridDim.x - 1) / p.total);
}
// with fewer tiles than blocks some blocks have none
__device__ __forceinline__ bool cta_has_tiles(const AttPlan& p, int cta) { return tile_begin(p, cta) < tile_begin(p, cta + 1); }

struct Ring {
  uint32_t full0, empty0;
  unsigned char* base;
  int stages, stage_bytes;
};

// ---- producer ------------------------------------------------------------------------------------
__device__ void produce(const StepArgs& a, const Ring& ring, const AttPlan& att, int lane) {
  unsigned u = 0;  // units issued so far (a unit fills one stage)
  auto acquire = [&](uint32_t bytes) -> unsigned char* {
    const int s = u % ring.stages;
    if (u >= (unsigned)ring.stages) stage_wait(ring.empty0 + 8 * s, ((u / ring.stages) & 1) ^ 1, a.error_word);
    if (lane == 0) mbar_expect_tx(ring.full0 + 8 * s, bytes);
    __syncwarp();
    return ring.base + (size_t)s * ring.stage_bytes;
  };
  for (int layer = 0; layer < a.L; ++layer) {
    const LayerPtrs lp = a.layers[layer];
    for (int phase = 0; phase < 5; ++phase) {
      if (phase == PH_ATT) {
        const CUtensorMap* maps = a.maps + 2 * layer;
        const long t0 = tile_begin(att, blockIdx.x), t1 = tile_begin(att, blockIdx.x + 1);
        // walk to the pair that holds tile t0
        int seq = 0, kvh = 0;
        long first = 0;  // first tile of the current pair
        while (seq < a.M && first + att.tiles_of[seq] <= t0) {
          first += att.tiles_of[seq];
          if (++kvh == a.nkv) kvh = 0, ++seq;
        }
        for (long t = t0; t < t1; ++t, ++u) {
          while (t >= first + att.tiles_of[seq]) {
            first += att.tiles_of[seq];
            if (++kvh == a.nkv) kvh = 0, ++seq;
          }
          const int key0 = (int)(t - first) * TILE;
          const int kv_len = a.kv_lens[seq];
          // boxes: (page part j, half h of the head, K or V); a box holds `box_rows` keys of one page
          const int box_rows = a.ps < TILE ? a.ps : TILE;
          const int live_parts = (min(TILE, kv_len - key0) + box_rows - 1) / box_rows;
          unsigned char* dst = acquire((uint32_t)live_parts * box_rows * 128 * (D / 64) * 2);
          const uint32_t bar = ring.full0 + 8 * (u % ring.stages);
          const int* bt = a.block_table + (long)seq * a.max_pages;
          const int boxes = live_parts * (D / 64) * 2;
          for (int b = lane; b < boxes; b += 32) {
            const int which = b & 1, h = (b >> 1) % (D / 64), jpart = b / (2 * (D / 64));
            const int key = key0 + jpart * box_rows;
            const int page = bt[key / a.ps];
            const int y = (page * a.nkv + kvh) * a.ps + key % a.ps;
            tma_load_2d(smem_addr(dst + which * KV_TILE + h * HALF_TILE + jpart * box_rows * 128), maps + which, bar,
                        h * 64, y);
          }
        }
        continue;
      }
      const Product& pr = a.prod[phase];
      const bf16* W = phase == PH_QKV ? lp.wqkv : phase == PH_O ? lp.wo : phase == PH_GU ? lp.wgu : lp.wdown;
      for (int chunk = 0; chunk < pr.chunks; ++chunk) {
        const int k_lo = chunk * pr.range, klen = min(pr.K, k_lo + pr.range) - k_lo;
        const uint32_t bytes_row = (uint32_t)klen * 2;
        for (int panel = blockIdx.x; panel < pr.panels; panel += gridDim.x, ++u) {
          const int row0 = panel * pr.fpp;
          const int live = min(pr.fpp, pr.N - row0);  // per half for SwiGLU
          unsigned char* dst = acquire(bytes_row * live * (8 / pr.fpp));
          const uint32_t bar = ring.full0 + 8 * (u % ring.stages);
          if (lane < 8 && (lane % pr.fpp) < live) {
            const long row = row0 + (lane % pr.fpp) + (long)(lane / pr.fpp) * pr.N;  // up rows start at row N
            bulk_copy(smem_addr(dst + lane * pr.pitch), W + row * pr.K + k_lo, bytes_row, bar);
          }
        }
      }
    }
  }
}

// ---- consumers: the tokens' values of a range, in registers ------------------------------------
struct XRegs {
  uint4 g[XB], h[XB];  // rows lane/4 and lane/4 + 8; 8 consecutive k-values each
};

// from a bfloat16 activation [16, ld] that another phase of this kernel wrote
template <bool HI>
__device__ __forceinline__ void load_x_bf16(XRegs& x, const bf16* src, int ld, int M, int k_lo, int klen, int warp, int g,
                                            int t) {
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int i = 0; i < XB; ++i) {
    const int k = 32 * (warp + CW * i) + 8 * t;
    const bool ok = k < klen;
    x.g[i] = (ok && g < M) ? __ldcg(reinterpret_cast<const uint4*>(src + (long)g * ld + k_lo + k)) : zero;
    x.h[i] = (HI && ok && g + 8 < M) ? __ldcg(reinterpret_cast<const uint4*>(src + (long)(g + 8) * ld + k_lo + k)) : zero;
  }
}

// from the fp32 residual sum, normalised: (v * rstd[token]) * w, one rounding (norm.cu)
template <bool HI>
__device__ __forceinline__ void load_x_norm(XRegs& x, const float* resid, int H, const float* w, const float* rstd_s, int M,
                                            int k_lo, int klen, int warp, int g, int t) {
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int i = 0; i < XB; ++i) {
    const int k = 32 * (warp + CW * i) + 8 * t;
    x.g[i] = x.h[i] = zero;
    if (k >= klen) continue;
    const float4 w0 = *reinterpret_cast<const float4*>(w + k_lo + k), w1 = *reinterpret_cast<const float4*>(w + k_lo + k + 4);
#pragma unroll
    for (int half = 0; half < (HI ? 2 : 1); ++half) {
      const int row = g + 8 * half;
      if (row >= M) continue;
      const float4 v0 = __ldcg(reinterpret_cast<const float4*>(resid + (long)row * H + k_lo + k));
      const float4 v1 = __ldcg(reinterpret_cast<const float4*>(resid + (long)row * H + k_lo + k + 4));
      const float rs = rstd_s[row];
      uint4 packed;
      packed.x = pack_bf16((v0.x * rs) * w0.x, (v0.y * rs) * w0.y);
      packed.y = pack_bf16((v0.z * rs) * w0.z, (v0.w * rs) * w0.w);
      packed.z = pack_bf16((v1.x * rs) * w1.x, (v1.y * rs) * w1.y);
      packed.w = pack_bf16((v1.z * rs) * w1.z, (v1.w * rs) * w1.w);
      if (half == 0) x.g[i] = packed; else x.h[i] = packed;
    }
  }
}

// rstd of every token from the panels' sums of squares (fixed order: lane-strided, then a tree)
__device__ __forceinline__ void make_rstd(const float* sumsq_site, int panels, int H, float eps, float* rstd_s, int warp,
                                          int lane) {
  if (warp < MAX_TOKENS) {
    float s = 0.f;
    for (int p = lane; p < panels; p += 32) s += __ldcg(sumsq_site + (long)p * MAX_TOKENS + warp);
    s = warp_sum(s);
    if (lane == 0) rstd_s[warp] = rsqrtf(s / (float)H + eps);
  }
  consumer_sync();
}

// ---- consumers: one product ---------------------------------------------------------------------
// SRC: where the tokens' values come from: 0 the residual sum through a norm, 1 a bfloat16 activation.
// EPI: 0 bf16 store into `out_bf16` [16, N]; 1 SwiGLU into `out_bf16` [16, N]; 2 add into the residual
// sum and leave the panel's sums of squares at `sumsq_site`.
template <int EPI, int SRC, bool HI>
__device__ __forceinline__ void consume_product(const StepArgs& a, const Ring& ring, unsigned& u, const Product& pr,
                                                const bf16* src, int src_ld, const float* norm_w, const float* rstd_s,
                                                bf16* out_bf16, float* sumsq_site, float* red, float* acc_s,
                                                float* misc_s) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  int local = 0;
  for (int chunk = 0; chunk < pr.chunks; ++chunk) {
    const int k_lo = chunk * pr.range, klen = min(pr.K, k_lo + pr.range) - k_lo;
    const int my_blocks = (klen + 31) / 32;
    XRegs x;
    if (SRC == 0) load_x_norm<HI>(x, a.resid, a.H, norm_w, rstd_s, a.M, k_lo, klen, warp, g, t);
    else load_x_bf16<HI>(x, src, src_ld, a.M, k_lo, klen, warp, g, t);
    int mine = 0;
    for (int panel = blockIdx.x; panel < pr.panels; panel += gridDim.x, ++u, ++local, ++mine) {
      const int s = u % ring.stages;
      stage_wait(ring.full0 + 8 * s, (u / ring.stages) & 1, a.error_word);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      const unsigned char* base = ring.base + (size_t)s * ring.stage_bytes + g * pr.pitch + 16 * t;
#pragma unroll
      for (int i = 0; i < XB; ++i) {
        const int b = warp + CW * i;
        if (b < my_blocks) {
          const uint4 w = *reinterpret_cast<const uint4*>(base + 64 * b);
          mma16816(acc, x.g[i].x, x.h[i].x, x.g[i].y, x.h[i].y, w.x, w.y);
          mma16816(acc, x.g[i].z, x.h[i].z, x.g[i].w, x.h[i].w, w.z, w.w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty0 + 8 * s);
      float* rbuf = red + (size_t)(local & 1) * CW * 4 * 32;
#pragma unroll
      for (int e = 0; e < 4; ++e) rbuf[(warp * 4 + e) * 32 + lane] = acc[e];
      consumer_sync();
      if (threadIdx.x < 128) {  // thread = (e, lane): token g + 8 (e >> 1), row 2t + (e & 1) of the panel
        const int e = threadIdx.x >> 5;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < CW; ++w) v += rbuf[(w * 4 + e) * 32 + lane];
        if (pr.chunks > 1) {  // the panel's tile so far, chunk by chunk
          float* slot = acc_s + mine * 128 + threadIdx.x;
          if (chunk > 0) v += *slot;
          if (chunk + 1 < pr.chunks) *slot = v;
        }
        if (chunk + 1 == pr.chunks) {
          const int token = g + 8 * (e >> 1);
          if (EPI == 1) {
            const float up = __shfl_down_sync(0xffffffffu, v, 2);
            const int feature = panel * 4 + 2 * t + (e & 1);
            if (token < a.M && feature < pr.N && t < 2)
              out_bf16[(long)token * pr.N + feature] = __float2bfloat16_rn((v / (1.f + expf(-v))) * up);
          } else {
            const int feature = panel * 8 + 2 * t + (e & 1);
            const bool live = token < a.M && feature < pr.N;
            if (EPI == 0) {
              if (live) out_bf16[(long)token * pr.N + feature] = __float2bfloat16_rn(v);
            } else {
              float sq = 0.f;
              if (live) {
                float* r = a.resid + (long)token * a.H + feature;
                v += __ldcg(r);
                __stcg(r, v);
                sq = v * v;
              }
              // the panel's sum of squares per token: the four lanes of a token, then the two warps
              sq += __shfl_xor_sync(0xffffffffu, sq, 1);
              sq += __shfl_xor_sync(0xffffffffu, sq, 2);
              if (t == 0) misc_s[e * 8 + g] = sq;
              quad_sync();
              if (t == 0 && (e & 1) == 0)
                __stcg(sumsq_site + (long)panel * MAX_TOKENS + token, misc_s[e * 8 + g] + misc_s[(e + 1) * 8 + g]);
              quad_sync();
            }
          }
        }
      }
    }
  }
}

// ---- consumers: attention ------------------------------------------------------------------------
// One run of tiles of one (sequence, kv head) pair: every team takes the tiles t with
// (t - run begin) % 4 == team.  On return warp 0 holds the run's result for heads 0..G-1.
struct AttState {
  float o[D / 8][2];  // rows lane/4 (the group's heads are rows 0..G-1, G <= 8): columns 8i + 2(lane&3), +1
  float m, l;         // running maximum (raw scores) and this thread's share of the sum
};

__device__ __forceinline__ void att_tile(AttState& st, const unsigned char* k_t, const unsigned char* v_t,
                                         const unsigned char* q_s, int key0, int kv_len, int wt, int lane,
                                         float scale_log2) {
  const int kbase = key0 + wt * 16;  // this warp's 16 keys
  if (kbase >= kv_len) return;
  float s[2][4];
#pragma unroll
  for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t qa[4], kb[4];
    ldmatrix_x4(qa, smem_u32(q_s + swz<D>(lane & 15, 2 * ks + (lane >> 4))));
    const int row = wt * 16 + (lane & 7) + ((lane >> 4) << 3);
    ldmatrix_x4(kb, smem_u32(k_t + kv_off(row, 2 * ks + ((lane >> 3) & 1))));
    mma_bf16(s[0], qa, kb[0], kb[1]);
    mma_bf16(s[1], qa, kb[2], kb[3]);
  }
  // rows 8..15 of the tile are padding (G <= 8): only s[n][0], s[n][1] (row lane/4) matter
  float mx = -INFINITY;
#pragma unroll
  for (int n = 0; n < 2; ++n)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int j = kbase + n * 8 + 2 * (lane & 3) + e;
      if (j >= kv_len) s[n][e] = -INFINITY;
      mx = fmaxf(mx, s[n][e]);
    }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  const float m_new = fmaxf(st.m, mx);
  const float m_use = m_new == -INFINITY ? 0.f : m_new;
  const float corr = exp2f((st.m - m_use) * scale_log2);
  st.m = m_new;
  st.l *= corr;
  float p[2][2];
#pragma unroll
  for (int n = 0; n < 2; ++n)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      p[n][e] = exp2f((s[n][e] - m_use) * scale_log2);
      st.l += p[n][e];
    }
  uint32_t pa[4];
  pa[0] = pack_bf16(p[0][0], p[0][1]);
  pa[1] = 0u;  // rows 8..15
  pa[2] = pack_bf16(p[1][0], p[1][1]);
  pa[3] = 0u;
  if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) st.o[i][0] *= corr, st.o[i][1] *= corr;
  }
#pragma unroll
  for (int i = 0; i < D / 16; ++i) {
    uint32_t vb[4];
    const int row = wt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
    ldmatrix_x4_trans(vb, smem_u32(v_t + kv_off(row, 2 * i + (lane >> 4))));
    float c0[4] = {st.o[2 * i][0], st.o[2 * i][1], 0.f, 0.f};
    float c1[4] = {st.o[2 * i + 1][0], st.o[2 * i + 1][1], 0.f, 0.f};
    mma_bf16(c0, pa, vb[0], vb[1]);
    mma_bf16(c1, pa, vb[2], vb[3]);
    st.o[2 * i][0] = c0[0], st.o[2 * i][1] = c0[1];
    st.o[2 * i + 1][0] = c1[0], st.o[2 * i + 1][1] = c1[1];
  }
}

// state of warp `w` += state of warp `w + h`, through `buf` ([h][G rows][D + 2] floats)
__device__ __forceinline__ void att_fold(AttState& st, float* buf, int h, int G, int warp, int lane, float scale_log2) {
  const int r = lane >> 2, c = 2 * (lane & 3);
  if (warp >= h && warp < 2 * h && r < G) {
    float* dst = buf + ((size_t)(warp - h) * G + r) * (D + 2);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) dst[8 * i + c] = st.o[i][0], dst[8 * i + c + 1] = st.o[i][1];
    if ((lane & 3) == 0) dst[D] = st.m, dst[D + 1] = st.l;
  }
  consumer_sync();
  if (warp < h && r < G) {
    const float* src = buf + ((size_t)warp * G + r) * (D + 2);
    const float m2 = src[D], l2 = src[D + 1];
    const float m = fmaxf(st.m, m2);
    const float f1 = st.m == -INFINITY ? 0.f : exp2f((st.m - m) * scale_log2);
    const float f2 = m2 == -INFINITY ? 0.f : exp2f((m2 - m) * scale_log2);
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      st.o[i][0] = st.o[i][0] * f1 + src[8 * i + c] * f2;
      st.o[i][1] = st.o[i][1] * f1 + src[8 * i + c + 1] * f2;
    }
    st.l = st.l * f1 + l2 * f2;
    st.m = m;
  }
  consumer_sync();
}

__device__ void consume_attention(const StepArgs& a, const Ring& ring, unsigned& u, const AttPlan& att,
                                  const LayerPtrs& lp, unsigned char* q_s, unsigned char* new_s, float* fold_s,
                                  int* flag_s) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int team = warp >> 2, wt = warp & 3;
  const int G = a.nq / a.nkv;
  const int qkv_ld = (a.nq + 2 * a.nkv) * D;
  const long t0 = tile_begin(att, blockIdx.x), t1 = tile_begin(att, blockIdx.x + 1);
  int seq = 0, kvh = 0;
  long first = 0;
  while (seq < a.M && first + att.tiles_of[seq] <= t0) {
    first += att.tiles_of[seq];
    if (++kvh == a.nkv) kvh = 0, ++seq;
  }
  long t = t0;
  while (t < t1) {
    while (t >= first + att.tiles_of[seq]) {
      first += att.tiles_of[seq];
      if (++kvh == a.nkv) kvh = 0, ++seq;
    }
    // ---- a run: tiles [t, run_end) of pair (seq, kvh) ---------------------------------------
    const long pair_end = first + att.tiles_of[seq];
    const long run_end = pair_end < t1 ? pair_end : t1;
    const int kv_len = a.kv_lens[seq];
    const int p = kv_len - 1;  // the newest position
    const bool owner = run_end == pair_end;  // the pair's last tile holds position p
    const int* bt = a.block_table + (long)seq * a.max_pages;
    // q of the group (and, in the owner, k and v of the newest token): D/16 threads per head
    {
      constexpr int TPH = D / 16, HALF = D / 2, CHUNKS = D / 8;
      for (int c = tid; c < (16 - G) * CHUNKS; c += CONSUMERS)
        *reinterpret_cast<uint4*>(q_s + swz<D>(G + c / CHUNKS, c % CHUNKS)) = make_uint4(0, 0, 0, 0);
      const int items = G + (owner ? 2 : 0);
      const bf16* row = a.qkv + (long)seq * qkv_ld;
      long cache_row = -1;
      if (owner && p / a.ps < a.max_pages) {
        const int page = bt[p / a.ps];
        if (page >= 0) cache_row = (((long)page * a.nkv + kvh) * a.ps + (p % a.ps)) * D;
      }
      const bool rotate = a.cos_t && p < a.max_pos;
      if (a.cos_t && !rotate && tid == 0) atomicCAS(a.error_word, 0, ERR_POSITION);
      const int item = tid / TPH, c = tid % TPH;
      const bool live = item < items;
      const bool is_q = item < G, is_v = item == G + 1;
      const bf16* xp = row + (is_q ? (long)(kvh * G + item) * D : (long)(a.nq + (is_v ? a.nkv : 0) + kvh) * D);
      float va[8], vb[8];
      if (live) {
        const uint4 ra = __ldcg(reinterpret_cast<const uint4*>(xp + 8 * c));
        const uint4 rb = __ldcg(reinterpret_cast<const uint4*>(xp + HALF + 8 * c));
        const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ra);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 fa = __bfloat1622float2(ha[e]), fb = __bfloat1622float2(hb[e]);
          va[2 * e] = fa.x, va[2 * e + 1] = fa.y, vb[2 * e] = fb.x, vb[2 * e + 1] = fb.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) va[e] = vb[e] = 0.f;
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += va[e] * va[e] + vb[e] * vb[e];
#pragma unroll
      for (int o = TPH >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (live) {
        if (!is_v) {
          const float* w = is_q ? lp.qnorm : lp.knorm;
          if (w) {
            const float rstd = rsqrtf(ss / (float)D + a.qk_eps);
            float wa[8], wb[8];
            load8(w + 8 * c, wa);
            load8(w + HALF + 8 * c, wb);
#pragma unroll
            for (int e = 0; e < 8; ++e) va[e] = (va[e] * rstd) * wa[e], vb[e] = (vb[e] * rstd) * wb[e];
          }
          if (rotate) rotate_chunks(va, vb, a.cos_t + (long)p * HALF, a.sin_t + (long)p * HALF, c, HALF, a.pairing);
        }
        if (is_q) {
          store8(reinterpret_cast<bf16*>(q_s + swz<D>(item, c)), va);
          store8(reinterpret_cast<bf16*>(q_s + swz<D>(item, CHUNKS / 2 + c)), vb);
        } else {
          bf16* side = reinterpret_cast<bf16*>(new_s) + (is_v ? D : 0);
          store8(side + 8 * c, va);
          store8(side + HALF + 8 * c, vb);
          if (cache_row >= 0) {
            bf16* dst = (is_v ? lp.vpages : lp.kpages) + cache_row;
            store8(dst + 8 * c, va);
            store8(dst + HALF + 8 * c, vb);
          }
        }
      }
    }
    consumer_sync();
    AttState st;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) st.o[i][0] = st.o[i][1] = 0.f;
    st.m = -INFINITY;
    st.l = 0.f;
    for (long tt = t; tt < run_end; ++tt, ++u) {
      const int s = u % ring.stages;
      stage_wait(ring.full0 + 8 * s, (u / ring.stages) & 1, a.error_word);
      if ((int)((tt - t) & 3) == team) {
        unsigned char* k_t = ring.base + (size_t)s * ring.stage_bytes;
        unsigned char* v_t = k_t + KV_TILE;
        const int key0 = (int)(tt - first) * TILE;
        if (tt == pair_end - 1) {  // the pair's last tile (uniform per team)
          // whole pages were fetched: rows past the sequence's end hold whatever the pages held
          // before; a probability of zero does not silence a NaN, so they are cleared
          const int tl = tid & 127;
          const int live = kv_len - key0, box_rows = a.ps < TILE ? a.ps : TILE;
          const int fetched = min(TILE, (live + box_rows - 1) / box_rows * box_rows);
          for (int c = tl; c < (fetched - live) * 2 * (D / 8); c += 128) {
            const int row = live + c / (2 * (D / 8)), which = (c / (D / 8)) & 1, chunk = c % (D / 8);
            *reinterpret_cast<uint4*>((which ? v_t : k_t) + kv_off(row, chunk)) = make_uint4(0, 0, 0, 0);
          }
          if (owner && tl < 2 * (D / 8)) {  // the newest key and value go into their row
            const int r = p - key0;
            const int which = tl / (D / 8), chunk = tl % (D / 8);
            const uint4 v = *reinterpret_cast<const uint4*>(new_s + which * D * 2 + chunk * 16);
            *reinterpret_cast<uint4*>((which ? v_t : k_t) + kv_off(r, chunk)) = v;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before the stage is refilled
          team_sync(team);
        }
        att_tile(st, k_t, v_t, q_s, key0, kv_len, wt, lane, a.scale_log2);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(ring.empty0 + 8 * s);
    }
    // ---- fold the 16 warps into warp 0 -------------------------------------------------------------
    st.l += __shfl_xor_sync(0xffffffffu, st.l, 1);
    st.l += __shfl_xor_sync(0xffffffffu, st.l, 2);
    for (int h = CW / 2; h >= 1; h >>= 1) att_fold(st, fold_s, h, G, warp, lane, a.scale_log2);
    const int pair = seq * a.nkv + kvh;
    const int first_cta = cta_of_tile(att, first), last_cta = cta_of_tile(att, pair_end - 1);
    const int r = lane >> 2, c = 2 * (lane & 3);
    if (first_cta == last_cta) {  // the whole pair was this block's: finished rows
      if (warp == 0 && r < G) {
        bf16* dst = a.ctx + (long)seq * a.nq * D + (long)(kvh * G + r) * D;
        const float inv = 1.f / st.l;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<uint32_t*>(dst + 8 * i + c) = pack_bf16(st.o[i][0] * inv, st.o[i][1] * inv);
      }
    } else {
      const long slot = (long)pair + blockIdx.x;  // unique: both grow along the tiles
      if (warp == 0 && r < G) {
        float* dst = a.att_o + (slot * G + r) * D;
        const float inv = 1.f / st.l;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) __stcg(reinterpret_cast<float2*>(dst + 8 * i + c), make_float2(st.o[i][0] * inv, st.o[i][1] * inv));
        if ((lane & 3) == 0) __stcg(a.att_lse + slot * G + r, st.m * a.scale_log2 + log2f(st.l));
      }
      if (warp == 0) {
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          int want = 0;
          for (int cta = first_cta; cta <= last_cta; ++cta) want += cta_has_tiles(att, cta);
          const int drawn = atomicAdd(a.att_tickets + pair, 1);
          *flag_s = drawn == want - 1;
          if (drawn == want - 1) a.att_tickets[pair] = 0;
        }
      }
      consumer_sync();
      if (*flag_s) {  // the pair's last block merges its runs, in block order
        __threadfence();
        for (int idx = tid; idx < G * (D / 4); idx += CONSUMERS) {
          const int head = idx / (D / 4), d = 4 * (idx % (D / 4));
          float mx = -INFINITY;
          for (int cta = first_cta; cta <= last_cta; ++cta)
            if (cta_has_tiles(att, cta)) mx = fmaxf(mx, __ldcg(a.att_lse + ((long)pair + cta) * G + head));
          float acc[4] = {0.f, 0.f, 0.f, 0.f}, wsum = 0.f;
          for (int cta = first_cta; cta <= last_cta; ++cta) {
            if (!cta_has_tiles(att, cta)) continue;
            const long sl = (long)pair + cta;
            const float ls = __ldcg(a.att_lse + sl * G + head);
            const float4 v = __ldcg(reinterpret_cast<const float4*>(a.att_o + (sl * G + head) * D + d));
            const float w = exp2f(ls - mx);
            wsum += w;
            acc[0] += w * v.x, acc[1] += w * v.y, acc[2] += w * v.z, acc[3] += w * v.w;
          }
          bf16* dst = a.ctx + (long)seq * a.nq * D + (long)(kvh * G + head) * D + d;
          uint2 packed;
          packed.x = pack_bf16(acc[0] / wsum, acc[1] / wsum);
          packed.y = pack_bf16(acc[2] / wsum, acc[3] / wsum);
          *reinterpret_cast<uint2*>(dst) = packed;
        }
      }
      consumer_sync();
    }
    t = run_end;
  }
}

template <bool HI>
__global__ void __launch_bounds__(THREADS, 1) decode_step_kernel(const __grid_constant__ StepArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[2 * MAX_STAGES];
  __shared__ float rstd_s[MAX_TOKENS];
  __shared__ float misc_s[32];
  __shared__ int flag_s;
  __shared__ AttPlan att;
  unsigned char* aligned = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  Ring ring;
  ring.full0 = smem_addr(bars);
  ring.empty0 = smem_addr(bars + MAX_STAGES);
  ring.base = aligned;
  ring.stages = a.stages;
  ring.stage_bytes = a.stage_bytes;
  unsigned char* after = aligned + (size_t)a.stages * a.stage_bytes;
  float* red = reinterpret_cast<float*>(after);              // products: [2][CW][4][32], then the chunks' tiles; attention: the fold buffer
  float* acc_s = red + 2 * CW * 4 * 32;
  unsigned char* q_s = after + a.red_bytes;                  // [16][D] bf16, swizzled
  unsigned char* new_s = q_s + 16 * D * 2;                   // the newest key, then value
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(ring.full0 + 8 * s, 1);
      mbar_init(ring.empty0 + 8 * s, CW);
    }
    mbar_init_fence();
    int total = 0;
    for (int m = 0; m < MAX_TOKENS; ++m) {
      att.tiles_of[m] = m < a.M ? (a.kv_lens[m] + TILE - 1) / TILE : 0;
      total += att.tiles_of[m];
    }
    att.total = total * a.nkv;
  }
  // stale shared memory is multiplied by zeros (masked keys, k-values past a range's end): keep it finite
  for (int i = threadIdx.x * 16; i < a.stages * a.stage_bytes; i += THREADS * 16)
    *reinterpret_cast<uint4*>(aligned + i) = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  if (warp == CW) {
    produce(a, ring, att, lane);
    return;
  }

  // ---- consumers -------------------------------------------------------------------------------
  const int g = lane >> 2, t = lane & 3;
  unsigned epoch = 0, u = 0;
  const int panelsH = a.H / 8;
  float* sumsq_a = a.sumsq;                                  // feeds norm1
  float* sumsq_b = a.sumsq + (long)panelsH * MAX_TOKENS;     // feeds norm2
  // the embedding rows start the residual sum
  for (int panel = blockIdx.x; panel < panelsH; panel += gridDim.x) {
    if (threadIdx.x < 128) {
      const int token = threadIdx.x >> 3, j = threadIdx.x & 7;
      float v = 0.f;
      if (token < a.M) {
        int id = a.token_ids[token];
        id = id < 0 ? 0 : (id >= a.vocab ? a.vocab - 1 : id);
        v = __bfloat162float(a.embed[(long)id * a.H + panel * 8 + j]);
        __stcg(a.resid + (long)token * a.H + panel * 8 + j, v);
      }
      float sq = v * v;
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      if (j == 0) __stcg(sumsq_a + (long)panel * MAX_TOKENS + token, sq);
    }
  }
  grid_sync(a, epoch);

  for (int layer = 0; layer < a.L; ++layer) {
    const LayerPtrs lp = a.layers[layer];
    make_rstd(sumsq_a, panelsH, a.H, a.eps, rstd_s, warp, lane);
    consume_product<0, 0, HI>(a, ring, u, a.prod[PH_QKV], nullptr, 0, lp.norm1, rstd_s, a.qkv, nullptr, red, acc_s, misc_s);
    grid_sync(a, epoch);
    consume_attention(a, ring, u, att, lp, q_s, new_s, red, &flag_s);
    grid_sync(a, epoch);
    consume_product<2, 1, HI>(a, ring, u, a.prod[PH_O], a.ctx, a.nq * D, nullptr, nullptr, nullptr, sumsq_b, red, acc_s, misc_s);
    grid_sync(a, epoch);
    make_rstd(sumsq_b, panelsH, a.H, a.eps, rstd_s, warp, lane);
    consume_product<1, 0, HI>(a, ring, u, a.prod[PH_GU], nullptr, 0, lp.norm2, rstd_s, a.mid, nullptr, red, acc_s, misc_s);
    grid_sync(a, epoch);
    consume_product<2, 1, HI>(a, ring, u, a.prod[PH_DOWN], a.mid, a.I, nullptr, nullptr, nullptr, sumsq_a, red, acc_s, misc_s);
    grid_sync(a, epoch);
  }
}

bool make_product(Product* pr, int N, int K, int fpp, int grid) {
  pr->N = N;
  pr->K = K;
  pr->fpp = fpp;
  pr->panels = (N + fpp - 1) / fpp;
  for (int chunks = 1; chunks <= 16; ++chunks) {
    const int range = ((K + chunks - 1) / chunks + 31) & ~31;
    if (range > MAX_RANGE) continue;
    if ((long)(chunks - 1) * range >= K) continue;
    if (chunks > 1 && (pr->panels + grid - 1) / grid > ACC_MAX_PANELS) return false;
    pr->chunks = chunks;
    pr->range = range;
    pr->pitch = ((range * 2 + 127) & ~127) + 64;
    return true;
  }
  return false;
}

// shared memory beside the ring: the warps' tiles of a product (two buffers) and the chunked
// products' running tiles, or the buffer the attention's warps fold through; q; the newest k, v
int red_bytes_for(const Product* prod, int grid, int G) {
  int acc_panels = 0;
  for (int ph : {PH_QKV, PH_O, PH_GU, PH_DOWN})
    if (prod[ph].chunks > 1) {
      const int mine = (prod[ph].panels + grid - 1) / grid;
      acc_panels = acc_panels > mine ? acc_panels : mine;
    }
  const int products = 2 * CW * 4 * 32 * 4 + acc_panels * 128 * 4;
  const int fold = (CW / 2) * G * (D + 2) * 4;
  return ((products > fold ? products : fold) + 127) & ~127;
}

struct DeviceInfo {
  int sms = 0;
  bool cooperative = false;
  bool configured[2] = {false, false};
};
DeviceInfo& device_info() {
  static DeviceInfo info[Q3_MAX_DEVICES];
  DeviceInfo& d = info[q3_current_device()];
  if (!d.sms) {
    int device = 0, coop = 0;
    if (cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess &&
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device) == cudaSuccess)
      d.cooperative = coop != 0;
    else
      d.sms = 0;
  }
  return d;
}

constexpr int SMEM_LIMIT = 226 * 1024;

}  // namespace

// Sizes of the scratch buffers a caller has to provide, in bytes, for these model sizes:
// out[0] att_o, out[1] att_lse, out[2] att_tickets, out[3] sumsq, out[4] the tensor maps of
// one layer (keys and values).  Returns Q3_ERR_UNSUPPORTED when the kernel does not take the sizes.
Q3_EXPORT int q3_decode_step_scratch(int H, int I, int nq, int nkv, int head_dim, long* out) {
  const DeviceInfo& dev = device_info();
  if (!dev.sms || !dev.cooperative || !out) return Q3_ERR_UNSUPPORTED;
  const int grid = dev.sms;
  if (head_dim != D || nq % nkv || nq / nkv > 8 || H % 8 || I % 8) return Q3_ERR_UNSUPPORTED;
  Product pr[5];
  if (!make_product(&pr[PH_QKV], (nq + 2 * nkv) * D, H, 8, grid) || !make_product(&pr[PH_O], H, nq * D, 8, grid) ||
      !make_product(&pr[PH_GU], I, H, 4, grid) || !make_product(&pr[PH_DOWN], H, I, 8, grid))
    return Q3_ERR_UNSUPPORTED;
  const int G = nq / nkv;
  const long slots = (long)MAX_TOKENS * nkv + grid;
  out[0] = slots * G * D * 4;
  out[1] = slots * G * 4;
  out[2] = (long)MAX_TOKENS * nkv * 4;
  out[3] = 2L * (H / 8) * MAX_TOKENS * 4;
  out[4] = 2L * sizeof(CUtensorMap);
  return Q3_OK;
}

// The tensor maps the kernel fetches keys and values through: for each of the L layers one map
// of its key pages and one of its value pages, each seen as a matrix [pages * nkv * ps rows][D]
// read in boxes of [min(ps, 64) rows][64 dims] with the 128-byte swizzle.  `kpages`, `vpages`:
// host arrays of L device pointers.  The maps are written to `maps_device` (L * 2 maps, in
// device memory, 64-byte aligned) with a synchronous copy: call it once per cache, outside any
// stream capture.
Q3_EXPORT int q3_decode_step_maps(const void* const* kpages, const void* const* vpages, int L, long pages, int nkv,
                                  int ps, int head_dim, void* maps_device) {
  if (!kpages || !vpages || !maps_device || L < 1 || pages < 1 || nkv < 1 || ps < 1) return Q3_ERR_ARGUMENT;
  if (head_dim != D || ps % 8 || (TILE % ps && ps % TILE) || ((uintptr_t)maps_device & 63)) return Q3_ERR_UNSUPPORTED;
  const long rows = pages * nkv * ps;
  if (rows >= (1L << 31)) return Q3_ERR_UNSUPPORTED;
  const int box_rows = ps < TILE ? ps : TILE;
  CUtensorMap* host = static_cast<CUtensorMap*>(malloc(sizeof(CUtensorMap) * 2 * L));
  if (!host) return Q3_ERR_LAUNCH;
  bool ok = true;
  for (int l = 0; l < L && ok; ++l) {
    if (((uintptr_t)kpages[l] | (uintptr_t)vpages[l]) & 15) ok = false;
    ok = ok && q3_bf16_map(&host[2 * l], kpages[l], rows, D, D, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) &&
         q3_bf16_map(&host[2 * l + 1], vpages[l], rows, D, D, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
  }
  if (ok) ok = cudaMemcpy(maps_device, host, sizeof(CUtensorMap) * 2 * L, cudaMemcpyHostToDevice) == cudaSuccess;
  free(host);
  return ok ? Q3_OK : Q3_ERR_LAUNCH;
}

// All layers of a decode step.  `layers`: device array of L LayerPtrs (ten pointers each, in the
// order of the struct above); `maps`: what q3_decode_step_maps wrote for the same pages.
// Activation scratch: resid fp32 [16, H] (the result: the residual sum after the last layer),
// qkv [16, (nq + 2 nkv) D], ctx [16, nq D], mid [16, I] bfloat16; the rest as
// q3_decode_step_scratch says; att_tickets zero before the first call (the kernel leaves them
// zero); `barrier` one unsigned that this call sets to zero itself.
// Refuses (Q3_ERR_UNSUPPORTED) what it is not built for: more than 16 tokens, head sizes other
// than 128, groups of more than 8 query heads per kv head, page sizes that are neither a divisor
// nor a multiple of 64 (or not a multiple of 8), a device without cooperative launch.
Q3_EXPORT int q3_decode_step(const void* layers, const void* maps, int L, int M, int H, int I, int nq, int nkv,
                             int head_dim, int ps, int vocab, const int* token_ids, const void* embed,
                             const int* kv_lens, const int* block_table, int max_pages, const float* cos_t,
                             const float* sin_t, int max_pos, int pairing, float eps, float qk_eps, float scale,
                             float* resid, float* sumsq, void* qkv, void* ctx, void* mid, float* att_o, float* att_lse,
                             int* att_tickets, unsigned* barrier, int* error_word, cudaStream_t stream) {
  if (!layers || !maps || !token_ids || !embed || !kv_lens || !block_table || !resid || !sumsq || !qkv || !ctx ||
      !mid || !att_o || !att_lse || !att_tickets || !barrier || !error_word)
    return Q3_ERR_ARGUMENT;
  if (L < 1 || M < 0 || nq < 1 || nkv < 1 || ps < 1 || (cos_t && (!sin_t || max_pos < 1)) || pairing < 0 || pairing > 1)
    return Q3_ERR_ARGUMENT;
  if (M > MAX_TOKENS || head_dim != D || nq % nkv || nq / nkv > 8 || H % 8 || I % 8 || ps % 8 ||
      (TILE % ps && ps % TILE))
    return Q3_ERR_UNSUPPORTED;
  if (M == 0) return Q3_OK;
  DeviceInfo& dev = device_info();
  if (!dev.sms || !dev.cooperative) return Q3_ERR_UNSUPPORTED;
  const int grid = dev.sms;
  StepArgs a = {};
  if (!make_product(&a.prod[PH_QKV], (nq + 2 * nkv) * D, H, 8, grid) || !make_product(&a.prod[PH_O], H, nq * D, 8, grid) ||
      !make_product(&a.prod[PH_GU], I, H, 4, grid) || !make_product(&a.prod[PH_DOWN], H, I, 8, grid))
    return Q3_ERR_UNSUPPORTED;
  int stage_bytes = TILE_BYTES;
  for (int ph : {PH_QKV, PH_O, PH_GU, PH_DOWN}) stage_bytes = stage_bytes > 8 * a.prod[ph].pitch ? stage_bytes : 8 * a.prod[ph].pitch;
  stage_bytes = (stage_bytes + 1023) & ~1023;
  const int red_bytes = red_bytes_for(a.prod, grid, nq / nkv);
  const int fixed = 1024 + red_bytes + 16 * D * 2 + 2 * D * 2;  // 1024: the ring starts on a 1024-byte boundary
  int stages = (SMEM_LIMIT - fixed) / stage_bytes;
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) return Q3_ERR_UNSUPPORTED;
  const size_t smem = (size_t)stages * stage_bytes + fixed;
  a.layers = static_cast<const LayerPtrs*>(layers);
  a.maps = static_cast<const CUtensorMap*>(maps);
  a.L = L, a.M = M, a.H = H, a.I = I, a.nq = nq, a.nkv = nkv, a.ps = ps, a.vocab = vocab;
  a.token_ids = token_ids, a.embed = static_cast<const bf16*>(embed), a.kv_lens = kv_lens;
  a.block_table = block_table, a.max_pages = max_pages;
  a.cos_t = cos_t, a.sin_t = sin_t, a.max_pos = max_pos, a.pairing = pairing;
  a.eps = eps, a.qk_eps = qk_eps, a.scale_log2 = scale * 1.4426950408889634f;
  a.stages = stages, a.stage_bytes = stage_bytes, a.red_bytes = red_bytes;
  a.resid = resid, a.sumsq = sumsq, a.qkv = static_cast<bf16*>(qkv), a.ctx = static_cast<bf16*>(ctx);
  a.mid = static_cast<bf16*>(mid), a.att_o = att_o, a.att_lse = att_lse;
  a.att_tickets = att_tickets, a.barrier = barrier, a.error_word = error_word;
  const bool hi = M > 8;
  const void* kernel = hi ? (const void*)decode_step_kernel<true> : (const void*)decode_step_kernel<false>;
  if (!dev.configured[hi]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT) != cudaSuccess)
      return Q3_ERR_LAUNCH;
    dev.configured[hi] = true;
  }
  if (cudaMemsetAsync(barrier, 0, sizeof(unsigned), stream) != cudaSuccess) return Q3_ERR_LAUNCH;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  void* params[] = {&a};
  return cudaLaunchKernelExC(&cfg, kernel, params) == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
}
