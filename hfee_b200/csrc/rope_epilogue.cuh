// The epilogue that the q/k/v product of prompt portions runs instead of a store, shared by the
// single-CTA and the paired tcgen05 GEMM kernels.
#pragma once

#include "tcgen05.cuh"

namespace tc {

// The product is the fused q/k/v projection of a prompt portion, columns [q heads | k heads |
// v heads] of head_dim each.  Instead of storing it, the epilogue rotates the query and key heads by
// the token's position (hostfog/hfee internal/llm/forward.go:181-196, pairs (i, i + head_dim/2), or
// (2i, 2i + 1) when `interleaved`) in float32, straight from the accumulator, writes the queries to
// q_out and keys and values to the cache pages of (slot, position): the rotary kernel's pass over
// the projection and the bfloat16 rounding between product and rotation fall away.
struct RopeEpi {
  const float2* cs;              // [token][head_dim/2] (cos, sin); null: no rotation
  const int* positions;          // [token]
  const int* slot_of_token;      // [token]
  __nv_bfloat16* q_out; long long ld_q;
  __nv_bfloat16* k_pool; __nv_bfloat16* v_pool;      // null: every head is a query head
  PagedCache cache;
  int heads, kv_heads, head_dim, interleaved;
};

// One epilogue warp's share of a tile of BN columns that starts at column n0: `tmem_rows` is the
// tensor-memory address of the warp's 32 accumulator rows (lane = row) at the tile's first column,
// `row` the thread's token, `half` which of the two warps of the lane quadrant this is.
template <int BN>
__device__ __forceinline__ void rope_epilogue(const RopeEpi& rope, uint32_t tmem_rows, int half, int row, int M, int N, int n0) {
  // A unit is 64 columns of a head: the chunk of 32 dims d0 .. d0 + 31 and the chunk that holds
  // their rotation partners (d + head_dim/2; with interleaved pairs simply the next chunk).  The two
  // warps of a lane quadrant take every other unit.  BN is a multiple of head_dim: whole heads.
  const int cph = rope.head_dim / 32;                    // chunks per head: 2 or 4
  const bool row_ok = row < M;
  int pos = 0, slot = 0;
  if (row_ok) { pos = rope.positions[row]; slot = rope.slot_of_token[row]; }
#pragma unroll 1
  for (int u = half; u < BN / 64; u += 2) {
    const int hh = (2 * u) / cph, pr = u % (cph / 2);
    const int step_b = rope.interleaved ? 1 : cph / 2;
    const int ch_a = rope.interleaved ? 2 * u : hh * cph + pr, ch_b = ch_a + step_b;
    const int h = n0 / rope.head_dim + hh;               // the head's number among q, k and v heads
    if (n0 + hh * rope.head_dim >= N) break;             // the same for the whole warp
    uint32_t va[32], vb[32];
    tc_ld32(tmem_rows + (uint32_t)(ch_a * 32), va);
    tc_ld32(tmem_rows + (uint32_t)(ch_b * 32), vb);
    tc_wait_ld();
    if (!row_ok) continue;
    __nv_bfloat16* dst;
    bool rotate = rope.cs != nullptr;
    if (h < rope.heads || rope.k_pool == nullptr) {
      dst = rope.q_out + (long long)row * rope.ld_q + (long long)h * rope.head_dim;
    } else if (h < rope.heads + rope.kv_heads) {
      dst = rope.k_pool + paged_offset(rope.cache, slot, pos, h - rope.heads);
    } else {
      dst = rope.v_pool + paged_offset(rope.cache, slot, pos, h - rope.heads - rope.kv_heads);
      rotate = false;
    }
    const int da = (ch_a - hh * cph) * 32, db = (ch_b - hh * cph) * 32;      // first dims of the two chunks
    if (rotate) {
      const float2* t = rope.cs + (long long)row * (rope.head_dim / 2);
      if (!rope.interleaved) {
        // va holds dims da + j, vb their partners da + j + head_dim/2; table entry da + j
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float4 c = __ldg(reinterpret_cast<const float4*>(t + da + j));
          const float x0 = __uint_as_float(va[j]), y0 = __uint_as_float(vb[j]);
          const float x1 = __uint_as_float(va[j + 1]), y1 = __uint_as_float(vb[j + 1]);
          va[j] = __float_as_uint(x0 * c.x - y0 * c.y);     vb[j] = __float_as_uint(x0 * c.y + y0 * c.x);
          va[j + 1] = __float_as_uint(x1 * c.z - y1 * c.w); vb[j + 1] = __float_as_uint(x1 * c.w + y1 * c.z);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 ca = __ldg(reinterpret_cast<const float4*>(t + (da + j) / 2));
          const float4 cb = __ldg(reinterpret_cast<const float4*>(t + (db + j) / 2));
          float x0 = __uint_as_float(va[j]), x1 = __uint_as_float(va[j + 1]);
          va[j] = __float_as_uint(x0 * ca.x - x1 * ca.y); va[j + 1] = __float_as_uint(x0 * ca.y + x1 * ca.x);
          x0 = __uint_as_float(va[j + 2]); x1 = __uint_as_float(va[j + 3]);
          va[j + 2] = __float_as_uint(x0 * ca.z - x1 * ca.w); va[j + 3] = __float_as_uint(x0 * ca.w + x1 * ca.z);
          x0 = __uint_as_float(vb[j]); x1 = __uint_as_float(vb[j + 1]);
          vb[j] = __float_as_uint(x0 * cb.x - x1 * cb.y); vb[j + 1] = __float_as_uint(x0 * cb.y + x1 * cb.x);
          x0 = __uint_as_float(vb[j + 2]); x1 = __uint_as_float(vb[j + 3]);
          vb[j + 2] = __float_as_uint(x0 * cb.z - x1 * cb.w); vb[j + 3] = __float_as_uint(x0 * cb.w + x1 * cb.z);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      uint4 oa, ob;
      __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(va[j]), __uint_as_float(va[j + 1]));
      __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(va[j + 2]), __uint_as_float(va[j + 3]));
      __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(va[j + 4]), __uint_as_float(va[j + 5]));
      __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(va[j + 6]), __uint_as_float(va[j + 7]));
      oa.x = *reinterpret_cast<uint32_t*>(&p0); oa.y = *reinterpret_cast<uint32_t*>(&p1);
      oa.z = *reinterpret_cast<uint32_t*>(&p2); oa.w = *reinterpret_cast<uint32_t*>(&p3);
      p0 = __floats2bfloat162_rn(__uint_as_float(vb[j]), __uint_as_float(vb[j + 1]));
      p1 = __floats2bfloat162_rn(__uint_as_float(vb[j + 2]), __uint_as_float(vb[j + 3]));
      p2 = __floats2bfloat162_rn(__uint_as_float(vb[j + 4]), __uint_as_float(vb[j + 5]));
      p3 = __floats2bfloat162_rn(__uint_as_float(vb[j + 6]), __uint_as_float(vb[j + 7]));
      ob.x = *reinterpret_cast<uint32_t*>(&p0); ob.y = *reinterpret_cast<uint32_t*>(&p1);
      ob.z = *reinterpret_cast<uint32_t*>(&p2); ob.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(dst + da + j) = oa;
      *reinterpret_cast<uint4*>(dst + db + j) = ob;
    }
  }
}

}  // namespace tc
