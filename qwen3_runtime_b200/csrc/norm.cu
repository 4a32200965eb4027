// RMSNorm fused with what feeds it: the residual add, the embedding lookup and a
// row gather.  All arithmetic is fp32; one rounding at the store.
//
//   v   = (ids ? table[ids[r]] : resid[r]) + (pending ? pending[r] : 0)      (fp32)
//         pending is either [rows, H] of the output's type or, with parts > 0, fp32
//         [parts, rows, H] (planes `part_stride` elements apart) whose planes are the
//         partial sums of a product over ranges of its inner dimension
//         (csrc/gemm_stream.cu); they are added in plane order, then to the residual
//   resid[r] = v                                  (when write_resid)
//   out[i]  = (v * rsqrt(mean(v^2) + eps)) * w    (qwen3_runtime/layers/ops.py:17-37)
//
// `rows` (optional) selects which source rows are processed; output row i then
// comes from source row rows[i] (used for the final norm, which only runs on the
// rows whose logits are wanted, qwen3_runtime/models/qwen3.py:263-264).
#include "common.cuh"

template <typename T>
__global__ void fused_norm_kernel(const void* __restrict__ pending, int parts, long part_stride,
                                  float* __restrict__ resid, const int* __restrict__ ids,
                                  const T* __restrict__ table, const int* __restrict__ rows,
                                  const float* __restrict__ w, T* __restrict__ out, int H, float eps,
                                  int write_resid, int vocab) {
  extern __shared__ float vals[];  // H floats, then 33 for the reduction
  float* red = vals + H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  const T* trow = nullptr;
  if (ids) {
    int id = ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    trow = table + (long)id * H;
  }
  const T* prow = pending && !parts ? static_cast<const T*>(pending) + src * H : nullptr;
  const float* frow = pending && parts ? static_cast<const float*>(pending) + src * H : nullptr;
  float* rrow = resid ? resid + src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = trow ? to_f32(trow[i]) : rrow[i];
    if (prow) v += to_f32(prow[i]);
    if (frow) {
      float sum = frow[i];
      for (int p = 1; p < parts; ++p) sum += frow[p * part_stride + i];
      v += sum;
    }
    if (write_resid) rrow[i] = v;
    vals[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)H + eps);
  T* orow = out + (long)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) orow[i] = from_f32<T>((vals[i] * rstd) * w[i]);
}

// The same with 16-byte accesses: H a multiple of 8 and every row 16-byte aligned.
// REGS: the block has a thread for every 8 elements of a row, so a thread's 8 values stay in
// registers between the two passes (no staging through shared memory).
// PLANES: what is pending may be partial-sum planes (a variant of its own, so that the common one
// keeps its registers).
template <typename T, bool REGS, bool PLANES>
__global__ void __launch_bounds__(512) fused_norm_vec_kernel(const void* __restrict__ pending, int parts, long part_stride,
                                      float* __restrict__ resid, const int* __restrict__ ids,
                                      const T* __restrict__ table, const int* __restrict__ rows,
                                      const float* __restrict__ w, T* __restrict__ out, int H, float eps,
                                      int write_resid, int vocab) {
  extern __shared__ float vals[];
  float* red = REGS ? vals : vals + H;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const long src = rows ? rows[r] : r;
  const T* trow = nullptr;
  if (ids) {
    int id = ids[src];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    trow = table + (long)id * H;
  }
  const T* prow = pending && !parts ? static_cast<const T*>(pending) + src * H : nullptr;
  const float* frow = PLANES && pending && parts ? static_cast<const float*>(pending) + src * H : nullptr;
  float* rrow = resid ? resid + src * H : nullptr;
  float ss = 0.f;
  float mine[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8];
    if (trow) load8(trow + i, v); else load8(rrow + i, v);
    if (prow) {
      float pv[8];
      load8(prow + i, pv);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += pv[e];
    }
    if (PLANES && frow) {  // four planes' loads in flight at a time; added in plane order
      float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p0 = 0; p0 < parts; p0 += 4) {
        float pv[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < parts) load8(frow + (p0 + j) * part_stride + i, pv[j]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < parts) {
#pragma unroll
            for (int e = 0; e < 8; ++e) sum[e] += pv[j][e];
          }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += sum[e];
    }
    if (write_resid) store8(rrow + i, v);
    if (REGS) {
#pragma unroll
      for (int e = 0; e < 8; ++e) mine[e] = v[e];
    } else {
      store8(vals + i, v);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)H + eps);
  T* orow = out + (long)r * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], wv[8];
    if (REGS) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = mine[e];
    } else {
      load8(vals + i, v);
    }
    load8(w + i, wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = (v[e] * rstd) * wv[e];
    store8(orow + i, v);
  }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int launch_fused_norm(const void* pending, int parts, long part_stride, float* resid, const int* ids,
                             const void* table, const int* rows, const float* w, void* out, int num_rows, int H,
                             float eps, int write_resid, int vocab, cudaStream_t stream) {
  if (num_rows == 0) return Q3_OK;
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  if (smem > 200 * 1024) return Q3_ERR_UNSUPPORTED;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(fused_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const bool vec = H % 8 == 0 && part_stride % 4 == 0 && aligned16(pending) && aligned16(resid) &&
                   aligned16(table) && aligned16(w) && aligned16(out);
  if (vec) {
    int threads = ((H / 8 + 31) / 32) * 32;
    threads = threads > 512 ? 512 : threads;
    const bool regs = threads * 8 >= H;  // one chunk per thread: the values stay in registers
    const size_t vec_smem = regs ? 33 * sizeof(float) : smem;
    void (*kernel)(const void*, int, long, float*, const int*, const T*, const int*, const float*, T*, int, float, int,
                   int);
    if (parts)
      kernel = regs ? fused_norm_vec_kernel<T, true, true> : fused_norm_vec_kernel<T, false, true>;
    else
      kernel = regs ? fused_norm_vec_kernel<T, true, false> : fused_norm_vec_kernel<T, false, false>;
    if (vec_smem > 48 * 1024)
      cudaFuncSetAttribute((const void*)kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)vec_smem);
    return launch_pdl(kernel, dim3(num_rows), dim3(threads), vec_smem, stream, pending, parts, part_stride, resid, ids,
                      (const T*)table, rows, w, (T*)out, H, eps, write_resid, vocab) == cudaSuccess
               ? Q3_OK
               : Q3_ERR_LAUNCH;
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  fused_norm_kernel<T><<<num_rows, threads, smem, stream>>>(
      pending, parts, part_stride, resid, ids, (const T*)table, rows, w, (T*)out, H, eps, write_resid, vocab);
  return q3_launch_status();
}

// out[num_rows, H]; resid fp32 [*, H] (may be null only when ids is given and
// write_resid is 0); table/out have `dtype`; w is fp32 [H].  pending has `dtype` when
// pending_parts is 0, else it is fp32 with pending_parts planes, part_stride elements apart.
Q3_EXPORT int q3_fused_norm(int dtype, const void* pending, int pending_parts, long part_stride, float* resid,
                            const int* ids, const void* table,
                            const int* rows, const float* w, void* out, int num_rows, int H, float eps,
                            int write_resid, int vocab, cudaStream_t stream) {
  if (!w || !out || H < 1) return Q3_ERR_ARGUMENT;
  if (!ids && !resid) return Q3_ERR_ARGUMENT;
  if (ids && !table) return Q3_ERR_ARGUMENT;
  if (write_resid && !resid) return Q3_ERR_ARGUMENT;
  if (pending_parts < 0 || (pending_parts && (!pending || part_stride < 0))) return Q3_ERR_ARGUMENT;
  if (dtype == Q3_DTYPE_F32)
    return launch_fused_norm<float>(pending, pending_parts, part_stride, resid, ids, table, rows, w, out, num_rows, H, eps, write_resid,
                                    vocab, stream);
  if (dtype == Q3_DTYPE_BF16)
    return launch_fused_norm<bf16>(pending, pending_parts, part_stride, resid, ids, table, rows, w, out, num_rows, H, eps, write_resid,
                                   vocab, stream);
  return Q3_ERR_ARGUMENT;
}

// ---- SwiGLU product: out[t, i] = silu(gu[t, i]) * gu[t, I + i]  (layers/ops.py:23-25) ----
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long total, int I) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long t = idx / I;
  const int i = (int)(idx - t * I);
  const float g = to_f32(gu[t * 2 * I + i]);
  const float u = to_f32(gu[t * 2 * I + I + i]);
  out[idx] = from_f32<T>((g / (1.f + expf(-g))) * u);
}

template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, long chunks, int I) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunks) return;
  const int per_row = I / 8;
  const long t = idx / per_row;
  const int i = (int)(idx - t * per_row) * 8;
  float g[8], u[8];
  load8(gu + t * 2 * I + i, g);
  load8(gu + t * 2 * I + I + i, u);
#pragma unroll
  for (int e = 0; e < 8; ++e) g[e] = (g[e] / (1.f + expf(-g[e]))) * u[e];
  store8(out + t * I + i, g);
}

Q3_EXPORT int q3_silu_mul(int dtype, const void* gu, void* out, int num_rows, int I, cudaStream_t stream) {
  if (!gu || !out || I < 1) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * I;
  if (total == 0) return Q3_OK;
  const int threads = 256;
  if (I % 8 == 0 && aligned16(gu) && aligned16(out)) {
    const long chunks = total / 8;
    const unsigned vblocks = (unsigned)((chunks + threads - 1) / threads);
    if (dtype == Q3_DTYPE_F32)
      silu_mul_vec_kernel<float><<<vblocks, threads, 0, stream>>>((const float*)gu, (float*)out, chunks, I);
    else if (dtype == Q3_DTYPE_BF16)
      silu_mul_vec_kernel<bf16><<<vblocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, chunks, I);
    else
      return Q3_ERR_ARGUMENT;
    return q3_launch_status();
  }
  const long blocks = (total + threads - 1) / threads;
  if (dtype == Q3_DTYPE_F32)
    silu_mul_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)gu, (float*)out, total, I);
  else if (dtype == Q3_DTYPE_BF16)
    silu_mul_kernel<bf16><<<(unsigned)blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, total, I);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// ---- small epilogues that an architecture may ask for (Qwen3 dense uses neither) ---------------------
// out[r][c] += bias[c]: the bias of a projection, added in fp32 to the product's rounded value.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, long ld, const float* __restrict__ bias, long total, int N) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long r = idx / N;
  const int c = (int)(idx - r * N);
  out[r * ld + c] = from_f32<T>(to_f32(out[r * ld + c]) + bias[c]);
}

Q3_EXPORT int q3_add_bias(int dtype, void* out, long ld, const float* bias, int num_rows, int N, cudaStream_t stream) {
  if (!out || !bias || N < 1 || ld < N) return Q3_ERR_ARGUMENT;
  const long total = (long)num_rows * N;
  if (total == 0) return Q3_OK;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == Q3_DTYPE_F32)
    add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)out, ld, bias, total, N);
  else if (dtype == Q3_DTYPE_BF16)
    add_bias_kernel<bf16><<<blocks, 256, 0, stream>>>((bf16*)out, ld, bias, total, N);
  else
    return Q3_ERR_ARGUMENT;
  return q3_launch_status();
}

// logits = logits * scale, then (cap > 0) cap * tanh(logits / cap), in place on fp32 logits.
__global__ void logit_scale_cap_kernel(float* __restrict__ logits, long total, float scale, float cap) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float v = logits[idx] * scale;
  if (cap > 0.f) v = cap * tanhf(v / cap);
  logits[idx] = v;
}

Q3_EXPORT int q3_logit_scale_cap(float* logits, long total, float scale, float cap, cudaStream_t stream) {
  if (!logits || total < 0 || cap < 0.f) return Q3_ERR_ARGUMENT;
  if (total == 0) return Q3_OK;
  logit_scale_cap_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(logits, total, scale, cap);
  return q3_launch_status();
}
