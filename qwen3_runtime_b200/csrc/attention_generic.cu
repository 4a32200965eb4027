// Causal attention over the paged cache for any mix of prompt portions and single
// decoded tokens: the general kernel (any head_dim that is a multiple of 8 up to
// 256, any head counts, any page size, optional window), used by the fp32 path and
// wherever a specialised kernel refuses a size.
//
// One warp per (token, query head).  The query at absolute position p attends to
// keys lo..p of its own sequence (lo = p - window + 1 with a window, else 0), which
// the cache holds already because keys are stored before attention runs
// (attention/pytorch.py:12-47).  Keys are visited in tiles of 32 aligned to
// absolute positions, each lane scoring one key, with an online softmax in fp32
// and exact expf.  The order of every reduction depends only on (p, window), so
// the result of a token does not depend on how the work was cut into steps or on
// what else is in the batch.
#include "common.cuh"

template <typename T, int WARPS>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, int q_stride,
                                               const T* __restrict__ kpages, const T* __restrict__ vpages,
                                               const int* __restrict__ block_table, int max_pages,
                                               const int* __restrict__ token_seq,
                                               const int* __restrict__ positions, T* __restrict__ out,
                                               int num_tokens, int nq, int nkv, int D, int ps, float scale,
                                               int window) {
  extern __shared__ float qs_all[];  // WARPS * D
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * WARPS + warp;
  if (item >= (long)num_tokens * nq) return;
  const int t = (int)(item / nq);
  const int h = (int)(item - (long)t * nq);
  const int kvh = h / (nq / nkv);
  const int p = positions[t];
  const int* bt = block_table + (long)token_seq[t] * max_pages;
  float* qs = qs_all + warp * D;
  const T* qrow = q + (long)t * q_stride + (long)h * D;
  for (int d = lane; d < D; d += 32) qs[d] = to_f32(qrow[d]);
  __syncwarp();
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  for (int j0 = lo & ~31; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j >= lo && j <= p;
    long row = 0;
    float s = -INFINITY;
    if (valid) {
      const int page = bt[j / ps];
      row = (((long)page * nkv + kvh) * ps + (j % ps)) * D;
      const T* kr = kpages + row;
      float dot = 0.f;
      for (int d = 0; d < D; d += 8) {
        float kv[8];
        load8(kr + d, kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(qs[d + e], kv[e], dot);
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pl = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(pl);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] *= corr;
    const int count = min(32, p - j0 + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, pl, jj);
      const long rj = __shfl_sync(0xffffffffu, row, jj);
      if (pj == 0.f) continue;  // keys before the window, or fully underflowed
      const T* vr = vpages + rj;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int d = lane + 32 * c;
        if (d < D) acc[c] = fmaf(pj, to_f32(vr[d]), acc[c]);
      }
    }
    m = m_new;
  }
  T* orow = out + ((long)t * nq + h) * D;
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int d = lane + 32 * c;
    if (d < D) orow[d] = from_f32<T>(acc[c] * inv);
  }
}

// q: [num_tokens, *] with row stride q_stride (elements), head h at column h*D.
// out: [num_tokens, nq*D].  window <= 0: none.
Q3_EXPORT int q3_paged_attention_generic(int dtype, const void* q, int q_stride, const void* kpages,
                                         const void* vpages, const int* block_table, int max_pages,
                                         const int* token_seq, const int* positions, void* out,
                                         int num_tokens, int nq, int nkv, int D, int ps, float scale,
                                         int window, cudaStream_t stream) {
  if (!q || !kpages || !vpages || !block_table || !token_seq || !positions || !out) return Q3_ERR_ARGUMENT;
  if (nq < 1 || nkv < 1 || nq % nkv || ps < 1) return Q3_ERR_ARGUMENT;
  if (D < 8 || D % 8 || D > 256) return Q3_ERR_UNSUPPORTED;
  if (num_tokens == 0) return Q3_OK;
  constexpr int WARPS = 4;
  const size_t smem = (size_t)WARPS * D * sizeof(float);
  const long items = (long)num_tokens * nq;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == Q3_DTYPE_F32)
    paged_attention_generic_kernel<float, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (const float*)q, q_stride, (const float*)kpages, (const float*)vpages, block_table, max_pages,
        token_seq, positions, (float*)out, num_tokens, nq, nkv, D, ps, scale, window);
  else if (dtype == Q3_DTYPE_BF16)
    paged_attention_generic_kernel<bf16, WARPS><<<blocks, WARPS * 32, smem, stream>>>(
        (const bf16*)q, q_stride, (const bf16*)kpages, (const bf16*)vpages, block_table, max_pages,
        token_seq, positions, (bf16*)out, num_tokens, nq, nkv, D, ps, scale, window);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}
