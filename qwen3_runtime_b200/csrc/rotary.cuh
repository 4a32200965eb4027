// Rotation of one thread's share of a head by the angles of one position, shared by the kernel
// that rotates every token of a step (rope_kv.cu) and by the decode-attention kernel that makes
// the newest token's q and k itself (attention_decode.cu), so that both give the same bits.
//
// A head of D elements (D a multiple of 16, rotation over the whole head) is handled by D/16
// threads; thread c holds a[] = elements [8c, 8c+8) and b[] = elements [D/2 + 8c, D/2 + 8c + 8).
// `cos_row` / `sin_row` point at the D/2 angles of the token's position.
//   pairing 0 ("half"):        pair i = (i, i + D/2)  -- a[e] rotates with b[e], angle 8c + e
//   pairing 1 ("interleaved"): pair i = (2i, 2i + 1)  -- neighbours inside a[] (angles 4c ..)
//                                                        and inside b[] (angles D/4 + 4c ..)
#pragma once
#include "common.cuh"

__device__ __forceinline__ void rotate_chunks(float (&a)[8], float (&b)[8], const float* __restrict__ cos_row,
                                              const float* __restrict__ sin_row, int c, int half, int pairing) {
  float cs[8], sn[8];
  if (!pairing) {
    load8(cos_row + 8 * c, cs);
    load8(sin_row + 8 * c, sn);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ya = a[e], yb = b[e];
      a[e] = ya * cs[e] - yb * sn[e];
      b[e] = yb * cs[e] + ya * sn[e];
    }
    return;
  }
  const float4 ca = *reinterpret_cast<const float4*>(cos_row + 4 * c);
  const float4 sa = *reinterpret_cast<const float4*>(sin_row + 4 * c);
  const float4 cb = *reinterpret_cast<const float4*>(cos_row + half / 2 + 4 * c);
  const float4 sb = *reinterpret_cast<const float4*>(sin_row + half / 2 + 4 * c);
  cs[0] = ca.x, cs[1] = ca.y, cs[2] = ca.z, cs[3] = ca.w, cs[4] = cb.x, cs[5] = cb.y, cs[6] = cb.z, cs[7] = cb.w;
  sn[0] = sa.x, sn[1] = sa.y, sn[2] = sa.z, sn[3] = sa.w, sn[4] = sb.x, sn[5] = sb.y, sn[6] = sb.z, sn[7] = sb.w;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float a0 = a[2 * j], a1 = a[2 * j + 1], b0 = b[2 * j], b1 = b[2 * j + 1];
    a[2 * j] = a0 * cs[j] - a1 * sn[j];
    a[2 * j + 1] = a1 * cs[j] + a0 * sn[j];
    b[2 * j] = b0 * cs[4 + j] - b1 * sn[4 + j];
    b[2 * j + 1] = b1 * cs[4 + j] + b0 * sn[4 + j];
  }
}
