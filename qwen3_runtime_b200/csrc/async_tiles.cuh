// Helpers for the kernels that move tiles asynchronously on sm_100a: mbarriers with bounded
// waits, TMA (tiled tensor copies and plain bulk copies), tcgen05 MMAs with accumulators in
// tensor memory, and the pieces a thread-block cluster needs (remote barrier arrival, address
// of the same variable in another block, cluster-wide barrier).
//
// Every wait on an mbarrier is bounded.  Two conventions, one per kernel family:
//   mbar_wait(bar, parity, &abort_flag)            the block has a shared abort flag: on expiry the
//                                                  waiter raises it and returns false; every role
//                                                  that sees it leaves its loop, the block frees
//                                                  what it holds and reports through an error word;
//   mbar_wait_report(bar, parity, error_word, c)   no flag: on expiry the waiter writes code c to
//                                                  the error word and carries on, so that barriers
//                                                  which other threads still count on are not
//                                                  abandoned; the result is invalid and the host raises.
// The limit (SM clock cycles) is Q3_WAIT_LIMIT_CYCLES; define it before including to change it.
#pragma once
#include <cuda.h>

#include "common.cuh"

#ifndef Q3_WAIT_LIMIT_CYCLES
#define Q3_WAIT_LIMIT_CYCLES 2000000000ll
#endif

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarriers ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// the same, ordering what other blocks of the cluster wrote before their arrival
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  False: gave up (this or another role raised the abort flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - start > Q3_WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}
// After a block has given up: wait for something of its own that is still in flight (copies
// into its shared memory, MMAs into its tensor memory) before it frees and leaves.  The limit is
// a long one of its own, so that shortening Q3_WAIT_LIMIT_CYCLES does not cut this wait short.
#ifndef Q3_DRAIN_LIMIT_CYCLES
#define Q3_DRAIN_LIMIT_CYCLES 2000000000ll
#endif
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity))
    if (clock64() - start > Q3_DRAIN_LIMIT_CYCLES) return false;
  return true;
}
// Bounded wait; on expiry records `code` in the error word and returns (the caller carries on).
__device__ __forceinline__ void mbar_wait_report(uint32_t bar, uint32_t parity, int* error_word, int code) {
  if (mbar_try_wait(bar, parity)) return;
  const long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - start > Q3_WAIT_LIMIT_CYCLES) {
      if (error_word) atomicExch(error_word, code);
      return;
    }
  }
}

// ---- clusters ------------------------------------------------------------------------------------
// the address, in the cluster's shared-memory window, of this block's `addr` in block `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// the box lands in this CTA's shared memory, its bytes count on the pair leader's barrier
// (`leader_bar`: a cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
// untiled: `bytes` (a multiple of 16) from a 16-byte aligned global address
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// ---- tcgen05 ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major tile [rows][64] bf16 written by TMA with the
// 128-byte swizzle: rows are 128 bytes, groups of 8 rows are 1024 bytes apart.  16 more k-values
// are 32 bytes = 2 descriptor units further.
__device__ __forceinline__ uint64_t umma_desc(uint32_t tile_addr) {
  uint64_t d = (uint64_t)((tile_addr & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                                // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset: next group of 8 rows
  d |= (uint64_t)1 << 46;                                // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
  return d;
}
// MN-major operand (rows = K index, 64 contiguous N per 128-byte row), 128-byte swizzle:
// leading offset = distance between 64-wide blocks of N, stride offset = 8 rows of K.
__device__ __forceinline__ uint64_t umma_desc_mn_major(uint32_t addr, uint32_t n_block_bytes) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(n_block_bytes >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: D fp32, A and B bf16, A K-major, B K-major or MN-major, M x N
// (M is the pair's 256 for cta_group::2).
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, int b_mn_major = 0) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// one MMA over the two CTAs of a pair, issued by the leader
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on `bar` when the MMAs this thread has issued so far have completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// the same for a pair: arrives on the barrier at this shared-memory offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both)
               : "memory");
}
// 32 (16) consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// ---- host: tensor maps ---------------------------------------------------------------------------
typedef CUresult (*Q3EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
static inline Q3EncodeTiledFn q3_encode_tiled() {
  static Q3EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<Q3EncodeTiledFn>(ptr);
  }
  return fn;
}
// A row-major [rows, cols] bf16 matrix with row stride `ld` elements, read in boxes of
// [box_rows, 64] with the 128-byte swizzle; out-of-range elements read as zero.
static inline bool q3_bf16_map(CUtensorMap* map, const void* base, long rows, long cols, long ld, int box_rows,
                               CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_256B) {
  Q3EncodeTiledFn fn = q3_encode_tiled();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promotion,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
