// Token choice from fp32 logit rows: greedy argmax and temperature sampling by
// inverse CDF with a uniform number drawn on the host.  One block per row.
// Parity: qwen3_runtime/sampling.py:28-32 (argmax, lowest id on ties), :260-270
// (softmax(logits / temperature)), :208-227 (first index whose cumulative
// probability exceeds u, clamped to the vocabulary).
#include "common.cuh"
#include <limits.h>

#define SAMPLE_THREADS 1024

// token[r] = argmax; logprob[r] = log_softmax(row)[token]   (logprob may be null)
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ token, float* __restrict__ logprob) {
  __shared__ float red[33];
  __shared__ int best_idx;
  const float* row = logits + (long)blockIdx.x * V;
  float best = -INFINITY;
  int idx = INT_MAX;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < idx)) {
      best = v;
      idx = i;
    }
  }
  const float top = block_max(best, red);
  if (threadIdx.x == 0) best_idx = INT_MAX;
  __syncthreads();
  if (best == top && idx != INT_MAX) atomicMin(&best_idx, idx);
  __syncthreads();
  int chosen = best_idx;
  if (chosen == INT_MAX) chosen = 0;  // a row without any comparable value (all NaN)
  if (threadIdx.x == 0) token[blockIdx.x] = chosen;
  if (logprob) {
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(row[i] - top);
    const float z = block_sum(s, red);
    if (threadIdx.x == 0) logprob[blockIdx.x] = row[chosen] - top - logf(z);
  }
}

// x = logits / temperature; p = softmax(x); token = first i with cumsum(p)[i] > u.
// The cumulative sum runs in index order: a chunk of blockDim * ITEMS consecutive
// elements at a time, each thread summing ITEMS consecutive ones, the block scanning
// the thread sums, a running prefix carried from chunk to chunk.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ token, float* __restrict__ logprob) {
  constexpr int ITEMS = 4;
  __shared__ float red[33];
  __shared__ float scan[SAMPLE_THREADS];
  __shared__ int found;
  const float* row = logits + (long)blockIdx.x * V;
  const float temp = temperature[blockIdx.x];
  const float u = uniform[blockIdx.x];
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] / temp);
  mx = block_max(mx, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(row[i] / temp - mx);
  const float z = block_sum(s, red);
  if (threadIdx.x == 0) found = INT_MAX;
  __syncthreads();
  float carried = 0.f;
  const int chunk = blockDim.x * ITEMS;
  for (int base = 0; base < V && found == INT_MAX; base += chunk) {
    const int first = base + threadIdx.x * ITEMS;
    float pr[ITEMS];
    float mine = 0.f;
#pragma unroll
    for (int e = 0; e < ITEMS; ++e) {
      pr[e] = first + e < V ? expf(row[first + e] / temp - mx) / z : 0.f;
      mine += pr[e];
    }
    scan[threadIdx.x] = mine;
    __syncthreads();
    for (int off = 1; off < blockDim.x; off <<= 1) {  // inclusive Hillis-Steele scan
      const float add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0.f;
      __syncthreads();
      scan[threadIdx.x] += add;
      __syncthreads();
    }
    float c = carried + scan[threadIdx.x] - mine;  // cumulative sum before my items
#pragma unroll
    for (int e = 0; e < ITEMS; ++e) {
      c += pr[e];
      if (first + e < V && c > u) {
        atomicMin(&found, first + e);
        break;
      }
    }
    carried += scan[blockDim.x - 1];
    __syncthreads();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int chosen = found == INT_MAX ? V - 1 : found;
    token[blockIdx.x] = chosen;
    if (logprob) logprob[blockIdx.x] = logf(fmaxf(expf(row[chosen] / temp - mx) / z, 1e-30f));
  }
}

Q3_EXPORT int q3_argmax(const float* logits, int num_rows, int V, int* token, float* logprob,
                        cudaStream_t stream) {
  if (!logits || !token || V < 1) return Q3_ERR_ARGUMENT;
  if (num_rows == 0) return Q3_OK;
  argmax_kernel<<<num_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, token, logprob);
  return q3_launch_status();
}

Q3_EXPORT int q3_sample(const float* logits, int num_rows, int V, const float* temperature,
                        const float* uniform, int* token, float* logprob, cudaStream_t stream) {
  if (!logits || !token || !temperature || !uniform || V < 1) return Q3_ERR_ARGUMENT;
  if (num_rows == 0) return Q3_OK;
  sample_kernel<<<num_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, uniform, token, logprob);
  return q3_launch_status();
}
