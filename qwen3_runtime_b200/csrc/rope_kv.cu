// Per-head q/k RMSNorm, rotary position encoding and the write of keys and values
// into their cache pages, in one pass over the QKV projection's output.
//
// One warp handles one (token, head).  For a q or k head (models/qwen3.py:101-103):
//   y = (x * rsqrt(mean(x^2) + eps)) * w          over the head's D values, fp32
//   rotation of the first 2*rot_half dims by cos/sin[position][i]; which two elements form
//   pair i is the position part's choice: `pairing` 0 = halves, (i, i + rot_half)
//   (layers/rope.py:7-11, what Qwen3 uses); 1 = interleaved, (2i, 2i + 1)
// q is written back in place (the attention kernels read it from the QKV buffer);
// k goes to its slot of the key pages; v heads are copied to the value pages
// unchanged (kv/paged.py:74-84).  Slot of position p: page = block_table[seq][p / ps],
// row p % ps.  Page layout [pages, kv_heads, page_size, D].
//
// A position outside the rotation tables (p < 0 or p >= max_pos) is never rotated with another
// position's angles: the (token, head) is left untouched and `error_word` (if given) is set to
// Q3_ERR_POSITION, which the host reads with the step's other error reports.
#include "common.cuh"
#include "rotary.cuh"

#define Q3_ERR_POSITION 16

template <typename T, int WARPS>
__global__ void qk_norm_rope_store_kernel(T* __restrict__ qkv, int row_stride, int nq, int nkv, int D,
                                          const float* __restrict__ q_w, const float* __restrict__ k_w,
                                          float eps, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int rot_half, int max_pos,
                                          const int* __restrict__ positions, const int* __restrict__ token_seq,
                                          const int* __restrict__ block_table, int max_pages,
                                          T* __restrict__ kpages, T* __restrict__ vpages, int ps,
                                          int num_tokens, int write_kv, int pairing, int* __restrict__ error_word) {
  extern __shared__ float stage[];  // WARPS * D
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = write_kv ? nq + 2 * nkv : nq;
  const long item = (long)blockIdx.x * WARPS + warp;
  if (item >= (long)num_tokens * heads) return;
  const int t = (int)(item / heads);
  const int hi = (int)(item - (long)t * heads);
  T* x = qkv + (long)t * row_stride + (long)hi * D;
  const int p = positions[t];
  if (cos_t && hi < nq + nkv && (p < 0 || p >= max_pos)) {
    if (error_word && lane == 0) atomicExch(error_word, Q3_ERR_POSITION);
    return;
  }
  long cache_row = 0;
  if (hi >= nq) {
    const int kvh = hi < nq + nkv ? hi - nq : hi - nq - nkv;
    if (p < 0 || p / ps >= max_pages) return;  // no page in the table for this position: write nothing
    const int page = block_table[(long)token_seq[t] * max_pages + p / ps];
    if (page < 0) return;
    cache_row = (((long)page * nkv + kvh) * ps + (p % ps)) * D;
  }
  if (hi >= nq + nkv) {  // value head: plain copy
    T* dst = vpages + cache_row;
    for (int d = lane; d < D; d += 32) dst[d] = x[d];
    return;
  }
  float* xs = stage + warp * D;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float v = to_f32(x[d]);
    xs[d] = v;
    ss += v * v;
  }
  const float* w = hi < nq ? q_w : k_w;
  const float rstd = w ? rsqrtf(warp_sum(ss) / (float)D + eps) : 1.f;
  __syncwarp();
  const float* cs = cos_t ? cos_t + (long)p * rot_half : nullptr;
  const float* sn = cos_t ? sin_t + (long)p * rot_half : nullptr;
  T* dst = hi < nq ? x : kpages + cache_row;
  for (int d = lane; d < D; d += 32) {
    float y = w ? (xs[d] * rstd) * w[d] : xs[d];
    if (cs && d < 2 * rot_half) {
      const bool first = pairing ? (d & 1) == 0 : d < rot_half;  // the pair's first element
      const int i = pairing ? d >> 1 : (first ? d : d - rot_half);
      const int pd = pairing ? d ^ 1 : (first ? d + rot_half : d - rot_half);
      const float yp = w ? (xs[pd] * rstd) * w[pd] : xs[pd];
      y = first ? y * cs[i] - yp * sn[i] : y * cs[i] + yp * sn[i];
    }
    dst[d] = from_f32<T>(y);
  }
}

// The same with 16-byte accesses, for head sizes 16, 32, 64, 128, 256 with the rotation over
// the whole head (or none): D/16 threads per (token, head); a thread owns elements
// [8c, 8c+8) and [8c + D/2, 8c + D/2 + 8): with the halves pairing each element's partner is in
// the other chunk, with the interleaved pairing it is its neighbour in the same chunk.
template <typename T>
__global__ void qk_norm_rope_store_vec_kernel(T* __restrict__ qkv, int row_stride, int nq, int nkv, int D,
                                              const float* __restrict__ q_w, const float* __restrict__ k_w,
                                              float eps, const float* __restrict__ cos_t,
                                              const float* __restrict__ sin_t, int max_pos,
                                              const int* __restrict__ positions,
                                              const int* __restrict__ token_seq,
                                              const int* __restrict__ block_table, int max_pages,
                                              T* __restrict__ kpages, T* __restrict__ vpages, int ps,
                                              int tph_shift, int write_kv, int pairing,
                                              int* __restrict__ error_word) {
  // grid (tokens, blocks over one token's heads): no division finds a thread's token and head
  const int tph = D / 16;  // threads per head: a power of two, at most 16
  const int heads = write_kv ? nq + 2 * nkv : nq;
  pdl_wait();
  pdl_launch_dependents();
  const int u = blockIdx.y * blockDim.x + threadIdx.x;
  const int t = blockIdx.x;
  const int hi_raw = u >> tph_shift;
  const int c = u & (tph - 1);
  const bool live = hi_raw < heads;
  const int hi = live ? hi_raw : 0;
  const int half = D / 2;
  T* x = qkv + (long)t * row_stride + (long)hi * D;
  const int p = positions[t];
  long cache_row = -1;
  if (live && hi >= nq && p >= 0 && p / ps < max_pages) {
    const int kvh = hi < nq + nkv ? hi - nq : hi - nq - nkv;
    const int page = block_table[(long)token_seq[t] * max_pages + p / ps];
    if (page >= 0) cache_row = (((long)page * nkv + kvh) * ps + (p % ps)) * D;
  }
  float a[8], b[8];
  if (live) {
    load8(x + 8 * c, a);
    load8(x + half + 8 * c, b);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = b[e] = 0.f;
  }
  const bool is_v = hi >= nq + nkv;
  const float* w = hi < nq ? q_w : k_w;
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
  for (int o = tph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!live) return;
  if (is_v) {
    if (cache_row >= 0) {
      store8(vpages + cache_row + 8 * c, a);
      store8(vpages + cache_row + half + 8 * c, b);
    }
    return;
  }
  if (w) {
    const float rstd = rsqrtf(ss / (float)D + eps);
    float wa[8], wb[8];
    load8(w + 8 * c, wa);
    load8(w + half + 8 * c, wb);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      a[e] = (a[e] * rstd) * wa[e];
      b[e] = (b[e] * rstd) * wb[e];
    }
  }
  if (cos_t) {
    if (p < 0 || p >= max_pos) {
      if (error_word && c == 0) atomicExch(error_word, Q3_ERR_POSITION);
      return;
    }
    rotate_chunks(a, b, cos_t + (long)p * half, sin_t + (long)p * half, c, half, pairing);
  }
  if (hi < nq) {
    store8(x + 8 * c, a);
    store8(x + half + 8 * c, b);
  } else if (cache_row >= 0) {
    store8(kpages + cache_row + 8 * c, a);
    store8(kpages + cache_row + half + 8 * c, b);
  }
}

static inline bool rk_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

Q3_EXPORT int q3_qk_norm_rope_store(int dtype, void* qkv, int row_stride, int nq, int nkv, int D,
                                    const float* q_w, const float* k_w, float eps, const float* cos_t,
                                    const float* sin_t, int rot_half, int max_pos, const int* positions,
                                    const int* token_seq, const int* block_table, int max_pages, void* kpages,
                                    void* vpages, int ps, int num_tokens, int write_kv, int pairing,
                                    int* error_word, cudaStream_t stream) {
  if (!qkv || !positions || nq < 1 || nkv < 1 || D < 1 || pairing < 0 || pairing > 1) return Q3_ERR_ARGUMENT;
  if (cos_t && max_pos < 1) return Q3_ERR_ARGUMENT;
  if (write_kv && (!token_seq || !block_table || !kpages || !vpages || ps < 1)) return Q3_ERR_ARGUMENT;
  if (cos_t && (!sin_t || rot_half < 1 || 2 * rot_half > D)) return Q3_ERR_ARGUMENT;
  if (num_tokens == 0) return Q3_OK;
  const int tph = D / 16;
  const bool vec = D % 16 == 0 && tph >= 1 && tph <= 16 && (tph & (tph - 1)) == 0 && row_stride % 8 == 0 &&
                   (!cos_t || 2 * rot_half == D) && rk_aligned16(qkv) && rk_aligned16(kpages) &&
                   rk_aligned16(vpages) && rk_aligned16(q_w) && rk_aligned16(k_w) && rk_aligned16(cos_t) &&
                   rk_aligned16(sin_t);
  if (vec) {
    // a token's threads in blocks of 128 (Qwen3 sizes: 48 heads x 8 threads = 3 blocks, none idle)
    const int per_token = (write_kv ? nq + 2 * nkv : nq) * tph;
    int tph_shift = 0;
    while ((1 << tph_shift) < tph) ++tph_shift;
    const int vthreads = 128;
    const dim3 vgrid((unsigned)num_tokens, (unsigned)((per_token + vthreads - 1) / vthreads));
    if (vgrid.y > 65535) return Q3_ERR_UNSUPPORTED;
    cudaError_t err;
    if (dtype == Q3_DTYPE_F32)
      err = launch_pdl(qk_norm_rope_store_vec_kernel<float>, vgrid, dim3(vthreads), 0, stream, (float*)qkv,
                       row_stride, nq, nkv, D, q_w, k_w, eps, cos_t, sin_t, max_pos, positions, token_seq,
                       block_table, max_pages, (float*)kpages, (float*)vpages, ps, tph_shift, write_kv, pairing,
                       error_word);
    else if (dtype == Q3_DTYPE_BF16)
      err = launch_pdl(qk_norm_rope_store_vec_kernel<bf16>, vgrid, dim3(vthreads), 0, stream, (bf16*)qkv,
                       row_stride, nq, nkv, D, q_w, k_w, eps, cos_t, sin_t, max_pos, positions, token_seq,
                       block_table, max_pages, (bf16*)kpages, (bf16*)vpages, ps, tph_shift, write_kv, pairing,
                       error_word);
    else
      return Q3_ERR_ARGUMENT;
    return err == cudaSuccess ? Q3_OK : Q3_ERR_LAUNCH;
  }
  constexpr int WARPS = 4;
  const size_t smem = (size_t)WARPS * D * sizeof(float);
  if (smem > 48 * 1024) return Q3_ERR_UNSUPPORTED;
  const long items = (long)num_tokens * (write_kv ? nq + 2 * nkv : nq);
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == Q3_DTYPE_F32)
    qk_norm_rope_store_kernel<float, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (float*)qkv, row_stride, nq, nkv, D, q_w, k_w, eps, cos_t, sin_t, rot_half, max_pos, positions,
        token_seq, block_table, max_pages, (float*)kpages, (float*)vpages, ps, num_tokens, write_kv, pairing,
                       error_word);
  else if (dtype == Q3_DTYPE_BF16)
    qk_norm_rope_store_kernel<bf16, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (bf16*)qkv, row_stride, nq, nkv, D, q_w, k_w, eps, cos_t, sin_t, rot_half, max_pos, positions,
        token_seq, block_table, max_pages, (bf16*)kpages, (bf16*)vpages, ps, num_tokens, write_kv, pairing,
                       error_word);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// cos/sin tables [max_pos, half]: angle = float(p) * inv_freq[j], as an fp32 product
// (layers/rope.py:17-22); accurate cosf/sinf (this file is never built with fast math).
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, float* __restrict__ cos_t,
                                  float* __restrict__ sin_t, int max_pos, int half) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)max_pos * half) return;
  const int p = (int)(idx / half), j = (int)(idx % half);
  const float angle = (float)p * inv_freq[j];
  cos_t[idx] = cosf(angle);
  sin_t[idx] = sinf(angle);
}

Q3_EXPORT int q3_rope_table(const float* inv_freq, float* cos_t, float* sin_t, int max_pos, int half,
                            cudaStream_t stream) {
  if (!inv_freq || !cos_t || !sin_t || max_pos < 1 || half < 1) return Q3_ERR_ARGUMENT;
  const long total = (long)max_pos * half;
  rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(inv_freq, cos_t, sin_t, max_pos, half);
  return q3_launch_status();
}
