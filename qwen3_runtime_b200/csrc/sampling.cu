// Token choice from fp32 logit rows: greedy argmax and temperature sampling by
// inverse CDF with a uniform number drawn on the host.  One block per row.
// Parity: qwen3_runtime/sampling.py:28-32 (argmax, lowest id on ties), :260-270
// (softmax(logits / temperature)), :208-227 (first index whose cumulative
// probability exceeds u, clamped to the vocabulary).
#include "async_tiles.cuh"
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

// The same for few rows: with one block per row a batch of 8 keeps 8 SMs busy for tens of
// microseconds.  Here a row is cut into `slices` equal parts, one block each; a block leaves its
// best value, the lowest index that has it and (for the log-probability) sum exp(x - best) over
// its part, draws a ticket for its row, and the block that draws the last one merges the
// row's parts: greatest value, lowest index among equals; z = sum z_s * exp(best_s - top).
struct ArgmaxPart {
  float best;
  int idx;
  float z;
  int pad;
};

#define ARGMAX_SPLIT_THREADS 256

__global__ void __launch_bounds__(ARGMAX_SPLIT_THREADS)
argmax_split_kernel(const float* __restrict__ logits, int V, int slices, ArgmaxPart* __restrict__ parts,
                    int* __restrict__ tickets, int* __restrict__ token, float* __restrict__ logprob) {
  __shared__ float red[33];
  __shared__ int best_idx;
  __shared__ int last;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.y, s = blockIdx.x;
  const float* row = logits + (long)r * V;
  int per = (V + slices - 1) / slices;
  per = (per + 3) & ~3;
  const int lo = s * per, hi = min(V, lo + per);
  const bool vec = (V & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  float best = -INFINITY;
  int idx = INT_MAX;
  if (vec) {
    for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {  // hi - lo and lo are multiples of 4
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (e[k] > best) {  // ascending index: the first of equals stays
          best = e[k];
          idx = i + k;
        }
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const float v = row[i];
      if (v > best) {
        best = v;
        idx = i;
      }
    }
  }
  const float top = block_max(best, red);
  if (threadIdx.x == 0) best_idx = INT_MAX;
  __syncthreads();
  if (best == top && idx != INT_MAX) atomicMin(&best_idx, idx);
  __syncthreads();
  float z = 0.f;
  if (logprob && best_idx != INT_MAX) {
    float sum = 0.f;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) sum += expf(row[i] - top);
    z = block_sum(sum, red);
  }
  if (threadIdx.x == 0) {
    ArgmaxPart part;
    part.best = top;
    part.idx = best_idx;
    part.z = z;
    part.pad = 0;
    parts[(long)r * slices + s] = part;
    __threadfence();
    last = atomicAdd(tickets + r, 1) == slices - 1;
    if (last) tickets[r] = 0;  // for the next launch
  }
  __syncthreads();
  if (!last || threadIdx.x >= 32) return;
  __threadfence();
  // one warp merges the row's parts
  const float4* in = reinterpret_cast<const float4*>(parts + (long)r * slices);
  float mbest = -INFINITY;
  int midx = INT_MAX;
  for (int k = threadIdx.x; k < slices; k += 32) {
    const float4 raw = __ldcg(in + k);
    const float b = raw.x;
    const int i = __float_as_int(raw.y);
    if (i != INT_MAX && (b > mbest || (b == mbest && i < midx))) {
      mbest = b;
      midx = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, mbest, o);
    const int oi = __shfl_xor_sync(0xffffffffu, midx, o);
    if (oi != INT_MAX && (ob > mbest || (ob == mbest && oi < midx))) {
      mbest = ob;
      midx = oi;
    }
  }
  if (midx == INT_MAX) midx = 0;  // a row without any comparable value (all NaN)
  if (threadIdx.x == 0) token[r] = midx;
  if (logprob) {
    float zsum = 0.f;
    for (int k = threadIdx.x; k < slices; k += 32) {
      const float4 raw = __ldcg(in + k);
      if (__float_as_int(raw.y) != INT_MAX) zsum += raw.z * expf(raw.x - mbest);
    }
    zsum = warp_sum(zsum);
    if (threadIdx.x == 0) logprob[r] = row[midx] - mbest - logf(zsum);
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

// The same draw for few long rows: a row is cut into `slices` parts, one block each, which leave
// their maximum and sum exp(x - maximum); the block that draws the row's last ticket merges them
// to the row's maximum and normaliser, adds the parts' masses up in order to find the part in
// which the cumulative sum passes u, and scans only from there (carrying the mass before it).
__global__ void __launch_bounds__(ARGMAX_SPLIT_THREADS)
sample_split_kernel(const float* __restrict__ logits, int V, int slices, float2* __restrict__ parts,
                    int* __restrict__ tickets, const float* __restrict__ temperature,
                    const float* __restrict__ uniform, int* __restrict__ token, float* __restrict__ logprob) {
  constexpr int ITEMS = 4;
  constexpr int T = ARGMAX_SPLIT_THREADS;
  __shared__ float red[33];
  __shared__ float scan[T];
  __shared__ int found;
  __shared__ int last;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.y, s = blockIdx.x;
  const float* row = logits + (long)r * V;
  const float temp = temperature[r];
  const float u = uniform[r];
  int per = (V + slices - 1) / slices;
  per = (per + 3) & ~3;
  const int lo = s * per, hi = min(V, lo + per);
  float mx = -INFINITY;
  for (int i = lo + threadIdx.x; i < hi; i += T) mx = fmaxf(mx, row[i] / temp);
  mx = block_max(mx, red);
  float sum = 0.f;
  if (mx != -INFINITY)  // a part that the filters emptied weighs nothing (and -inf - -inf is no number)
    for (int i = lo + threadIdx.x; i < hi; i += T) sum += expf(row[i] / temp - mx);
  sum = block_sum(sum, red);
  if (threadIdx.x == 0) {
    parts[(long)r * slices + s] = make_float2(mx, lo < hi ? sum : 0.f);
    __threadfence();
    last = atomicAdd(tickets + r, 1) == slices - 1;
    if (last) tickets[r] = 0;  // for the next launch
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  // ---- the row's maximum and normaliser from the parts (fixed order: the same bits every time)
  const float2* in = parts + (long)r * slices;
  float top = -INFINITY;
  for (int k = threadIdx.x; k < slices; k += T) {
    const float2 p = __ldcg(in + k);
    if (p.y > 0.f) top = fmaxf(top, p.x);
  }
  top = block_max(top, red);
  float zpart = 0.f;
  for (int k = threadIdx.x; k < slices; k += T) {
    const float2 p = __ldcg(in + k);
    if (p.y > 0.f) zpart += p.y * expf(p.x - top);
  }
  const float z = block_sum(zpart, red);
  // ---- the part in which the cumulative mass passes u: thread t adds up parts [t*each, (t+1)*each)
  const int each = (slices + T - 1) / T;
  float mass[4];  // slices <= 1024 = 4 * T
  float mine = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int k = threadIdx.x * each + e;
    mass[e] = 0.f;
    if (e < each && k < slices) {
      const float2 p = __ldcg(in + k);
      if (p.y > 0.f) mass[e] = p.y * expf(p.x - top) / z;
    }
    mine += mass[e];
  }
  scan[threadIdx.x] = mine;
  if (threadIdx.x == 0) found = INT_MAX;
  __syncthreads();
  for (int off = 1; off < T; off <<= 1) {  // inclusive Hillis-Steele scan
    const float add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0.f;
    __syncthreads();
    scan[threadIdx.x] += add;
    __syncthreads();
  }
  {
    float c = scan[threadIdx.x] - mine;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = threadIdx.x * each + e;
      if (e < each && k < slices) {
        c += mass[e];
        if (c > u) {
          atomicMin(&found, k);
          break;
        }
      }
    }
  }
  __syncthreads();
  const int start_slice = found == INT_MAX ? slices - 1 : found;
  __syncthreads();
  // mass before that part, added up the same way
  float before = 0.f;
  {
    const int owner = start_slice / each;
    if ((int)threadIdx.x == owner) {
      float c = scan[threadIdx.x] - mine;
      for (int e = 0; e < start_slice - owner * each; ++e) c += mass[e];
      scan[0] = c;  // every thread has read its scan value
    }
    __syncthreads();
    before = scan[0];
    __syncthreads();
  }
  // ---- scan the elements from that part on (as sample_kernel does from the start of the row)
  if (threadIdx.x == 0) found = INT_MAX;
  __syncthreads();
  float carried = before;
  const int chunk = T * ITEMS;
  for (int base = start_slice * per; base < V && found == INT_MAX; base += chunk) {
    const int first = base + threadIdx.x * ITEMS;
    float pr[ITEMS];
    float my = 0.f;
#pragma unroll
    for (int e = 0; e < ITEMS; ++e) {
      pr[e] = first + e < V ? expf(row[first + e] / temp - top) / z : 0.f;
      my += pr[e];
    }
    scan[threadIdx.x] = my;
    __syncthreads();
    for (int off = 1; off < T; off <<= 1) {
      const float add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0.f;
      __syncthreads();
      scan[threadIdx.x] += add;
      __syncthreads();
    }
    float c = carried + scan[threadIdx.x] - my;
#pragma unroll
    for (int e = 0; e < ITEMS; ++e) {
      c += pr[e];
      if (first + e < V && c > u) {
        atomicMin(&found, first + e);
        break;
      }
    }
    carried += scan[T - 1];
    __syncthreads();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int chosen = found == INT_MAX ? V - 1 : found;
    token[r] = chosen;
    if (logprob) logprob[r] = logf(fmaxf(expf(row[chosen] / temp - top) / z, 1e-30f));
  }
}

// scratch / tickets (both may be null: one block per row): `slices` x 16 bytes per row, 16-byte
// aligned, and an int per row that is zero before the call and again after it.  slices <= 1024.
Q3_EXPORT int q3_argmax(const float* logits, int num_rows, int V, int* token, float* logprob, void* scratch,
                        int* tickets, int slices, cudaStream_t stream) {
  if (!logits || !token || V < 1 || slices < 0 || slices > 1024) return Q3_ERR_ARGUMENT;
  if (num_rows == 0) return Q3_OK;
  if (slices > 1 && scratch && tickets && num_rows <= 65535) {
    if (reinterpret_cast<uintptr_t>(scratch) & 15) return Q3_ERR_ARGUMENT;
    return launch_pdl(argmax_split_kernel, dim3(slices, num_rows), dim3(ARGMAX_SPLIT_THREADS), 0, stream, logits, V,
                      slices, static_cast<ArgmaxPart*>(scratch), tickets, token, logprob) == cudaSuccess
               ? Q3_OK
               : Q3_ERR_LAUNCH;
  }
  argmax_kernel<<<num_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, token, logprob);
  return q3_launch_status();
}

// scratch / tickets / slices as for q3_argmax (8 bytes of scratch per slice and row are used).
Q3_EXPORT int q3_sample(const float* logits, int num_rows, int V, const float* temperature,
                        const float* uniform, int* token, float* logprob, void* scratch, int* tickets, int slices,
                        cudaStream_t stream) {
  if (!logits || !token || !temperature || !uniform || V < 1 || slices < 0 || slices > 1024) return Q3_ERR_ARGUMENT;
  if (num_rows == 0) return Q3_OK;
  if (slices > 1 && scratch && tickets && num_rows <= 65535) {
    if (reinterpret_cast<uintptr_t>(scratch) & 7) return Q3_ERR_ARGUMENT;
    return launch_pdl(sample_split_kernel, dim3(slices, num_rows), dim3(ARGMAX_SPLIT_THREADS), 0, stream, logits, V,
                      slices, static_cast<float2*>(scratch), tickets, temperature, uniform, token, logprob) ==
                   cudaSuccess
               ? Q3_OK
               : Q3_ERR_LAUNCH;
  }
  sample_kernel<<<num_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, uniform, token, logprob);
  return q3_launch_status();
}

// ---------------------------------------------------------------------------------------------
// Logit processors, in place on one fp32 row per block, in the reference's order
// (qwen3_runtime/sampling.py:120-135): logit bias -> repetition / presence / frequency
// penalties -> (greedy stops) -> divide by temperature -> min_p -> top_k -> top_p.
// ---------------------------------------------------------------------------------------------

// Order-preserving map from float to unsigned: a > b  <=>  key(a) > key(b).
__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Bias and penalties (sampling.py:36-72).  counts: scratch of V ints for this row.
__global__ void __launch_bounds__(SAMPLE_THREADS)
bias_penalty_kernel(float* __restrict__ row, int V, const int* __restrict__ bias_ids,
                    const float* __restrict__ bias_vals, int n_bias, const int* __restrict__ seen_ids, int n_seen,
                    int* __restrict__ counts, float repetition, float presence, float frequency) {
  for (int i = threadIdx.x; i < n_bias; i += blockDim.x) {
    const int id = bias_ids[i];
    if (id >= 0 && id < V) atomicAdd(&row[id], bias_vals[i]);
  }
  if (n_seen == 0 || (repetition == 1.f && presence == 0.f && frequency == 0.f)) return;
  for (int i = threadIdx.x; i < V; i += blockDim.x) counts[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_seen; i += blockDim.x) {
    const int id = seen_ids[i];
    if (id >= 0 && id < V) atomicAdd(&counts[id], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const int c = counts[i];
    if (c == 0) continue;
    float v = row[i];
    if (repetition != 1.f) v = v > 0.f ? v / repetition : v * repetition;
    v -= presence;
    v -= frequency * (float)c;
    row[i] = v;
  }
}

// The same for several rows in one launch: block b works on row `row_index[b]` of `logits` with
// its own slice of the packed bias entries and seen ids (offsets[b] .. offsets[b + 1]), its own
// counts scratch and its own three penalties (params[3b .. 3b+2]).
__global__ void __launch_bounds__(SAMPLE_THREADS)
bias_penalty_rows_kernel(float* __restrict__ logits, int V, const int* __restrict__ row_index,
                         const int* __restrict__ bias_off, const int* __restrict__ bias_ids,
                         const float* __restrict__ bias_vals, const int* __restrict__ seen_off,
                         const int* __restrict__ seen_ids, int* __restrict__ counts, const float* __restrict__ params) {
  const int b = blockIdx.x;
  float* row = logits + (long)row_index[b] * V;
  for (int i = bias_off[b] + threadIdx.x; i < bias_off[b + 1]; i += blockDim.x) {
    const int id = bias_ids[i];
    if (id >= 0 && id < V) atomicAdd(&row[id], bias_vals[i]);
  }
  const float repetition = params[3 * b], presence = params[3 * b + 1], frequency = params[3 * b + 2];
  const int s0 = seen_off[b], s1 = seen_off[b + 1];
  if (s1 == s0 || (repetition == 1.f && presence == 0.f && frequency == 0.f)) return;
  int* cnt = counts + (long)b * V;
  for (int i = threadIdx.x; i < V; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  for (int i = s0 + threadIdx.x; i < s1; i += blockDim.x) {
    const int id = seen_ids[i];
    if (id >= 0 && id < V) atomicAdd(&cnt[id], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const int c = cnt[i];
    if (c == 0) continue;
    float v = row[i];
    if (repetition != 1.f) v = v > 0.f ? v / repetition : v * repetition;
    v -= presence;
    v -= frequency * (float)c;
    row[i] = v;
  }
}

// Smallest key k such that measure({i : key(x_i) > k}) <= limit, by bisection on the 32-bit key.
// count_mode: measure = number of elements; else measure = sum of exp(x_i - mx) / z.
__device__ unsigned cutoff_key(const float* row, int V, bool count_mode, float limit, float mx, float z, float* red) {
  unsigned lo = 0u, hi = 0xffffffffu;
  while (lo < hi) {
    const unsigned mid = lo + ((hi - lo) >> 1);
    float part = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (ordered_key(v) > mid) part += count_mode ? 1.f : expf(v - mx) / z;
    }
    const float total = block_sum(part, red);
    if (total <= limit) hi = mid; else lo = mid + 1;
  }
  return lo;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
filter_kernel(float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const float* __restrict__ min_p, const int* __restrict__ top_k, const float* __restrict__ top_p) {
  __shared__ float red[33];
  float* row = logits + (long)blockIdx.x * V;
  const float temp = temperature[blockIdx.x];
  const float mp = min_p[blockIdx.x], tp = top_p[blockIdx.x];
  const int tk = top_k[blockIdx.x];
  const float lowest = -3.4028234663852886e38f;  // finfo(float32).min, the reference's mask value
  if (temp != 1.f)
    for (int i = threadIdx.x; i < V; i += blockDim.x) row[i] = row[i] / temp;
  __syncthreads();
  if (mp > 0.f) {  // drop tokens whose probability is below min_p times the largest (sampling.py:75-81)
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (expf(row[i] - mx) < mp) row[i] = -INFINITY;
    __syncthreads();
  }
  if (tk > 0 && tk < V) {  // keep the k largest, ties with the k-th included (sampling.py:96-99)
    const unsigned cut = cutoff_key(row, V, true, (float)(tk - 1), 0.f, 1.f, red);
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (ordered_key(row[i]) < cut) row[i] = lowest;
    __syncthreads();
  }
  if (tp > 0.f && tp < 1.f) {  // nucleus: keep a token iff the mass ranked before it is <= top_p (:100-108)
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float s = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(row[i] - mx);
    const float z = block_sum(s, red);
    const unsigned cut = cutoff_key(row, V, false, tp, mx, z, red);
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (ordered_key(row[i]) < cut) row[i] = lowest;
  }
}

// The same filters with the row in registers: a cluster of 8 blocks holds one row (thread t of
// block b has elements b*512 + t + 4096*k), so a bisection step is arithmetic on registers and
// one sum over the cluster instead of a pass over memory by a single block (1.8 ms for a
// vocabulary of 152 K became tens of microseconds).  Sums over the cluster: every block
// reduces its own part, leaves it in its shared memory, and after a cluster barrier every block
// adds the 8 parts in rank order, so all blocks see the same bits and take the same branch.
// Two slots used in turn make one barrier per sum enough.
constexpr int FILTER_CLUSTER = 8;
constexpr int FILTER_THREADS = 512;  // 128 registers a thread: room for 40 elements of the row

struct ClusterReducer {
  float* red;        // [33] block scratch
  float* slots;      // [2] this block's part, by turn
  unsigned turn;
  __device__ __forceinline__ float finish(float mine, bool is_max) {
    float* slot = slots + (turn & 1);
    if (threadIdx.x == 0) *slot = mine;
    cluster_sync_all();
    float total = is_max ? -INFINITY : 0.f;
    for (int r = 0; r < FILTER_CLUSTER; ++r) {
      float v;
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(map_to_cta(smem_addr(slot), r)) : "memory");
      total = is_max ? fmaxf(total, v) : total + v;
    }
    ++turn;
    return total;
  }
  __device__ __forceinline__ float sum(float part) { return finish(block_sum(part, red), false); }
  __device__ __forceinline__ float max(float part) { return finish(block_max(part, red), true); }
};

// Sums of WAYS - 1 values at once over the cluster: warps by shuffles, the block's warps in warp
// order, the cluster's blocks in rank order; every thread of every block gets the same bits.
constexpr int FILTER_WAYS = 16;

struct ClusterVectorSum {
  float (*warp_part)[FILTER_WAYS];   // [warps][ways] block scratch
  float (*slots)[FILTER_WAYS];       // [2][ways] this block's sums, by turn
  float* total;                      // [ways]
  unsigned turn;
  __device__ __forceinline__ void run(float (&part)[FILTER_WAYS - 1]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < FILTER_WAYS - 1; ++j) {
      float v = warp_sum(part[j]);
      if (lane == 0) warp_part[warp][j] = v;
    }
    __syncthreads();
    float* slot = slots[turn & 1];
    if (threadIdx.x < FILTER_WAYS - 1) {
      float v = 0.f;
      for (int w = 0; w < FILTER_THREADS / 32; ++w) v += warp_part[w][threadIdx.x];
      slot[threadIdx.x] = v;
    }
    cluster_sync_all();
    if (threadIdx.x < FILTER_WAYS - 1) {
      float v = 0.f;
      for (int r = 0; r < FILTER_CLUSTER; ++r) {
        float got;
        asm volatile("ld.shared::cluster.f32 %0, [%1];"
                     : "=f"(got)
                     : "r"(map_to_cta(smem_addr(slot + threadIdx.x), r))
                     : "memory");
        v += got;
      }
      total[threadIdx.x] = v;
    }
    __syncthreads();
    ++turn;
  }
};

// smallest key k with measure({element : key(x) > k}) <= limit; the measure is the number of
// elements (count_mode) or the sum of exp(x - mx) / z.  Elements past the end of the row count
// for nothing.  A search that cuts the interval of keys into 16 at every step (15 thresholds,
// 15 sums at once), so 8 steps and 8 sums over the cluster instead of 32.
template <int ITEMS>
__device__ unsigned cutoff_key_regs(const float (&x)[ITEMS], int first, int V, bool count_mode, float limit, float mx,
                                    float z, ClusterVectorSum& cs) {
  constexpr int STEP = FILTER_CLUSTER * FILTER_THREADS;
  constexpr int T = FILTER_WAYS - 1;
  unsigned lo = 0u, hi = 0xffffffffu;
  float above = 0.f;  // the measure of {key > hi}: known from the step that set hi
  while (lo < hi) {
    const unsigned long long span = (unsigned long long)hi - lo;
    unsigned cut[T];  // non-decreasing, in [lo, hi)
#pragma unroll
    for (int j = 0; j < T; ++j) cut[j] = lo + (unsigned)((span * (j + 1)) / FILTER_WAYS);
    float part[T];
#pragma unroll
    for (int j = 0; j < T; ++j) part[j] = 0.f;
    // only keys in (lo, hi] can tell two thresholds apart; after the first steps that is almost
    // none of the row, and a warp skips an element that none of its lanes has in that interval
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const unsigned key = ordered_key(x[k]);
      if (first + k * STEP < V && key > lo && key <= hi) {
        const float wgt = count_mode ? 1.f : expf(x[k] - mx) / z;
#pragma unroll
        for (int j = 0; j < T; ++j)
          if (key > cut[j]) part[j] += wgt;
      }
    }
    cs.run(part);
    // the first threshold whose measure is within the limit bounds the answer from above, the
    // one before it from below
    int j = 0;
    while (j < T && !(above + cs.total[j] <= limit)) ++j;
    const unsigned new_hi = j < T ? cut[j] : hi;
    const unsigned new_lo = j > 0 ? cut[j - 1] + 1 : lo;
    if (j < T) above += cs.total[j];
    hi = new_hi;
    lo = new_lo;
    __syncthreads();  // everybody has read the sums before the next step overwrites them
  }
  return lo;
}

template <int ITEMS>
__global__ void __cluster_dims__(FILTER_CLUSTER, 1, 1) __launch_bounds__(FILTER_THREADS)
filter_cluster_kernel(float* __restrict__ logits, int V, const float* __restrict__ temperature,
                      const float* __restrict__ min_p, const int* __restrict__ top_k,
                      const float* __restrict__ top_p) {
  __shared__ float red[33];
  __shared__ float slots[2];
  __shared__ float warp_part[FILTER_THREADS / 32][FILTER_WAYS];
  __shared__ float vector_slots[2][FILTER_WAYS];
  __shared__ float vector_total[FILTER_WAYS];
  ClusterReducer cr{red, slots, 0u};
  ClusterVectorSum cs{warp_part, vector_slots, vector_total, 0u};
  const int r = blockIdx.y;
  float* row = logits + (long)r * V;
  const float temp = temperature[r];
  const float mp = min_p[r], tp = top_p[r];
  const int tk = top_k[r];
  const float lowest = -3.4028234663852886e38f;  // finfo(float32).min, the reference's mask value
  const int first = blockIdx.x * FILTER_THREADS + threadIdx.x;
  constexpr int STEP = FILTER_CLUSTER * FILTER_THREADS;
  // elements past the end are -inf, and left out of every count and sum
  float x[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = first + k * STEP;
    x[k] = i < V ? row[i] : -INFINITY;
    if (temp != 1.f && i < V) x[k] = x[k] / temp;
  }
  if (mp > 0.f) {  // drop tokens whose probability is below min_p times the largest (sampling.py:75-81)
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) mx = fmaxf(mx, x[k]);
    mx = cr.max(mx);
#pragma unroll
    for (int k = 0; k < ITEMS; ++k)
      if (expf(x[k] - mx) < mp) x[k] = -INFINITY;
  }
  if (tk > 0 && tk < V) {  // keep the k largest, ties with the k-th included (sampling.py:96-99)
    const unsigned cut = cutoff_key_regs<ITEMS>(x, first, V, true, (float)(tk - 1), 0.f, 1.f, cs);
#pragma unroll
    for (int k = 0; k < ITEMS; ++k)
      if (ordered_key(x[k]) < cut) x[k] = lowest;
  }
  if (tp > 0.f && tp < 1.f) {  // nucleus: keep a token iff the mass ranked before it is <= top_p (:100-108)
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) mx = fmaxf(mx, first + k * STEP < V ? x[k] : -INFINITY);
    mx = cr.max(mx);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < ITEMS; ++k)
      if (first + k * STEP < V) s += expf(x[k] - mx);
    const float z = cr.sum(s);
    const unsigned cut = cutoff_key_regs<ITEMS>(x, first, V, false, tp, mx, z, cs);
#pragma unroll
    for (int k = 0; k < ITEMS; ++k)
      if (ordered_key(x[k]) < cut) x[k] = lowest;
  }
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = first + k * STEP;
    if (i < V) row[i] = x[k];
  }
  cluster_sync_all();  // nobody leaves while a neighbour may still read its slot
}

template <int ITEMS>
static int launch_filter_cluster(float* logits, int num_rows, int V, const float* temperature, const float* min_p,
                                 const int* top_k, const float* top_p, cudaStream_t stream) {
  filter_cluster_kernel<ITEMS><<<dim3(FILTER_CLUSTER, num_rows), FILTER_THREADS, 0, stream>>>(
      logits, V, temperature, min_p, top_k, top_p);
  return q3_launch_status();
}

Q3_EXPORT int q3_bias_penalty(float* row, int V, const int* bias_ids, const float* bias_vals, int n_bias,
                              const int* seen_ids, int n_seen, int* counts, float repetition, float presence,
                              float frequency, cudaStream_t stream) {
  if (!row || V < 1 || (n_bias > 0 && (!bias_ids || !bias_vals)) || (n_seen > 0 && (!seen_ids || !counts)))
    return Q3_ERR_ARGUMENT;
  bias_penalty_kernel<<<1, SAMPLE_THREADS, 0, stream>>>(row, V, bias_ids, bias_vals, n_bias, seen_ids, n_seen, counts,
                                                       repetition, presence, frequency);
  return q3_launch_status();
}

// Bias and penalties for `n` rows of `logits` ([*, V] fp32) in one launch.  ints: row_index [n],
// bias_off [n + 1], seen_off [n + 1], bias_ids, seen_ids packed one after the other as the offsets
// say; floats: params [3 n] (repetition, presence, frequency), then bias_vals; counts: n * V ints.
Q3_EXPORT int q3_bias_penalty_rows(float* logits, int V, int n, const int* row_index, const int* bias_off,
                                   const int* bias_ids, const float* bias_vals, const int* seen_off,
                                   const int* seen_ids, int* counts, const float* params, cudaStream_t stream) {
  if (!logits || V < 1 || n < 0 || !row_index || !bias_off || !seen_off || !params || !counts) return Q3_ERR_ARGUMENT;
  if (n == 0) return Q3_OK;
  bias_penalty_rows_kernel<<<n, SAMPLE_THREADS, 0, stream>>>(logits, V, row_index, bias_off, bias_ids, bias_vals,
                                                            seen_off, seen_ids, counts, params);
  return q3_launch_status();
}

Q3_EXPORT int q3_filter(float* logits, int num_rows, int V, const float* temperature, const float* min_p,
                        const int* top_k, const float* top_p, cudaStream_t stream) {
  if (!logits || !temperature || !min_p || !top_k || !top_p || V < 1) return Q3_ERR_ARGUMENT;
  if (num_rows == 0) return Q3_OK;
  // rows that fit the registers of a cluster of 8 blocks (up to 163,840 elements) and are long
  // enough to be worth it; the others take one block per row and passes over memory
  constexpr int PER_ITEM = FILTER_CLUSTER * FILTER_THREADS;
  if (V > 4096 && num_rows <= 65535 && V <= 40 * PER_ITEM) {
    int status;
    if (V <= 8 * PER_ITEM)
      status = launch_filter_cluster<8>(logits, num_rows, V, temperature, min_p, top_k, top_p, stream);
    else if (V <= 20 * PER_ITEM)
      status = launch_filter_cluster<20>(logits, num_rows, V, temperature, min_p, top_k, top_p, stream);
    else
      status = launch_filter_cluster<40>(logits, num_rows, V, temperature, min_p, top_k, top_p, stream);
    if (status == Q3_OK) return Q3_OK;
    // a device that cannot place such a cluster refuses the launch (nothing ran): one block per row
  }
  filter_kernel<<<num_rows, SAMPLE_THREADS, 0, stream>>>(logits, V, temperature, min_p, top_k, top_p);
  return q3_launch_status();
}
