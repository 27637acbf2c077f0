// Causal grouped-query flash attention over the paged cache with bfloat16 tensor-core
// MMAs (mma.sync.m16n8k16) and a float32 online softmax, for prefill portions,
// single decoded tokens and mixtures of both in one launch.
//
// A CTA serves one (request, kv head, tile of query rows[, split of the keys]).  The
// rows of a tile are (token, query head of the kv head's group) pairs, so the group
// shares every key/value load.  Keys are visited in blocks of 64 positions aligned
// to absolute multiples of 64; a block's rows are fetched page by page with
// cp.async (double buffered), rows outside the tile's key range are zero-filled so
// that stale page content never reaches an MMA.  With num_splits > 1 the key blocks
// of a tile are divided among CTAs which write unnormalised partial results; the
// combine kernel merges them in split order.
// Reference: hostfog/hfee internal/llm/forward.go:146-178, internal/ggml/ops.go:136-150.
#include "common.cuh"

#ifndef HFEE_ATTN_EXPORT
#define HFEE_ATTN_EXPORT 1
#endif

namespace {

constexpr int BLOCK_N = 64;

struct AttnParams {
  const __nv_bfloat16* q; int ld_q;
  __nv_bfloat16* out; int ld_o;
  const __nv_bfloat16* k_pool; const __nv_bfloat16* v_pool;
  PagedCache cache;
  const int* cu_tokens;        // [R+1]
  const int* slots;            // [R]
  const int* context_before;   // [R]
  int heads, group;            // group = heads / kv_heads
  float scale_log2;            // scale * log2(e)
  int window;                  // 0: all keys
  int tokens_per_tile;         // query tokens per tile = rows / group
  int num_splits;
  float* part_o;               // [(token*heads + head)*num_splits + split][HD]
  float* part_ml;              // [...][2] = (max in log2 units, sum)
  // Fused rotary + cache write (decode steps with one new token per request): q is unused;
  // queries, the new key and the new value are taken from the projection rows
  // [q heads | k heads | v heads], rotated here, and the new key/value are also written to the cache.
  const __nv_bfloat16* rope_qkv; int ld_qkv;
  const float2* rope_cs;       // [token][rope_dim/2] (cos, sin); null: no rotation
  int rope_dim, rope_interleaved;
  __nv_bfloat16* k_write; __nv_bfloat16* v_write;      // the pools, writable; null: this run only reads the cache
};

// Rotates the 16-byte piece of a head that starts at dim `a` (a multiple of 8): pairs (i, i + half)
// when `interleaved` is 0, (2i, 2i + 1) otherwise; dims at or above rope_dim pass through.  With
// half-split pairing the piece at `a` < half is rotated together with its partner at a + half
// (returns 2: y0 belongs at a, y1 at a + half); the partner piece itself returns 0 (nothing to
// store); every other piece returns 1 (y0 at a).  Same arithmetic as the rotary kernel:
// internal/llm/forward.go:181-196.
__device__ __forceinline__ int rope_piece(const __nv_bfloat16* head, const float2* t, int a, int rope_dim,
                                          int interleaved, uint4& y0, uint4& y1) {
  const int half = rope_dim / 2;
  if (t == nullptr || a >= rope_dim) {
    y0 = *reinterpret_cast<const uint4*>(head + a);
    return 1;
  }
  union Piece { uint4 u; __nv_bfloat16 v[8]; };
  if (interleaved) {
    Piece x, y;
    x.u = *reinterpret_cast<const uint4*>(head + a);
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const float2 c = t[(a + e) / 2];
      const float x0 = __bfloat162float(x.v[e]), x1 = __bfloat162float(x.v[e + 1]);
      y.v[e] = __float2bfloat16_rn(x0 * c.x - x1 * c.y);
      y.v[e + 1] = __float2bfloat16_rn(x0 * c.y + x1 * c.x);
    }
    y0 = y.u;
    return 1;
  }
  if (a >= half) return 0;
  Piece x0, x1, o0, o1;
  x0.u = *reinterpret_cast<const uint4*>(head + a);
  x1.u = *reinterpret_cast<const uint4*>(head + a + half);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float2 c = t[a + e];
    const float u = __bfloat162float(x0.v[e]), v = __bfloat162float(x1.v[e]);
    o0.v[e] = __float2bfloat16_rn(u * c.x - v * c.y);
    o1.v[e] = __float2bfloat16_rn(u * c.y + v * c.x);
  }
  y0 = o0.u;
  y1 = o1.u;
  return 2;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (2 ulp; 2^-inf = 0), as flash-attention kernels use it.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// KSPLIT = false: each warp owns 16 query rows and visits all 64 keys of a block (prefill).
// KSPLIT = true: the tile has 16 rows; each warp visits 16 of a block's 64 keys with a softmax
// state of its own, and the warps' results are merged at the end (decode: few rows, many keys).
// STAGES key/value blocks are in flight per CTA (cp.async groups): decode CTAs, which do little
// arithmetic per block, keep more of them in flight than prefill CTAs.
template <int HD, int NWARPS, bool KSPLIT, int STAGES>
__global__ void __launch_bounds__(NWARPS * 32)
attention_mma_kernel(AttnParams p) {
  static_assert(!KSPLIT || NWARPS * 16 == BLOCK_N, "key-split mode needs 16 keys per warp");
  static_assert(STAGES >= 2, "at least double buffering");
  constexpr int ROWS = KSPLIT ? 16 : 16 * NWARPS;
  constexpr int WKEYS = KSPLIT ? 16 : BLOCK_N;        // keys of a block one warp visits
  constexpr int PITCH = HD + 8;                 // elements; odd number of 16-byte units: conflict-free ldmatrix
  constexpr int CHUNKS = HD / 8;                // 16-byte chunks per row
  constexpr int THREADS = NWARPS * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [ROWS][PITCH]
  __nv_bfloat16* k_s = q_s + ROWS * PITCH;                                // [STAGES][BLOCK_N][PITCH]
  __nv_bfloat16* v_s = k_s + STAGES * BLOCK_N * PITCH;                    // [STAGES][BLOCK_N][PITCH]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int wrow = KSPLIT ? 0 : warp * 16;            // first tile row of this warp
  const int wkey = KSPLIT ? warp * 16 : 0;            // first key (within a block) of this warp
  // CTAs start in the order of blockIdx.x, then y: the tiles with the most keys (the latest
  // positions) of every kv head first, the light ones last to fill the gaps at the end
  const int tile = (int)(gridDim.y / p.num_splits) - 1 - (int)(blockIdx.y / p.num_splits);
  const int split = blockIdx.y % p.num_splits;
  const int kvh = blockIdx.x, r = blockIdx.z;

  const int tok0 = p.cu_tokens[r], n_new = p.cu_tokens[r + 1] - tok0;
  const int t_first = tile * p.tokens_per_tile;
  if (t_first >= n_new) return;
  const int t_count = min(p.tokens_per_tile, n_new - t_first);
  const int slot = p.slots[r], before = p.context_before[r];
  const int pos_first = before + t_first, pos_last = pos_first + t_count - 1;
  const int key_lo = (p.window > 0 && pos_first + 1 > p.window) ? pos_first + 1 - p.window : 0;
  const int rows_used = t_count * p.group;

  // key blocks of this CTA
  int b_lo = key_lo / BLOCK_N, b_hi = pos_last / BLOCK_N;
  if (p.num_splits > 1) {
    // The launch (and a captured graph) fixes the number of splits for the longest context the
    // engine allows; a shorter context uses only as many of them as leave each at least two key
    // blocks, the rest find an empty range and write an empty partial result.
    const int blocks = b_hi - b_lo + 1;
    const int used = max(1, min(p.num_splits, blocks / 2));
    const int per = (blocks + used - 1) / used;
    b_lo = b_lo + split * per;
    b_hi = min(b_hi, b_lo + per - 1);
  }

  // The batch layout and the block table come from the host, not from the previous kernel: they
  // were read (and the table rows of this CTA's blocks pulled into cache) while that kernel may
  // still be running.  Queries and this step's keys/values are its output: wait for it now.
  // lowest and highest position among this warp's valid rows (warp-uniform), to tell which
  // blocks need no mask at all; a warp without valid rows masks everything
  int row_pos_min = pos_first + wrow / p.group;
  int row_pos_max = pos_first + min(wrow + 15, rows_used - 1) / p.group;
  if (wrow >= rows_used) { row_pos_min = -1; row_pos_max = -1; }
  else if (wrow + 15 >= rows_used) row_pos_min = -1;          // padding rows in the tile: keep masking

  if (b_lo <= b_hi && tid <= b_hi - b_lo) {
    int warm = p.cache.block_table[(long long)slot * p.cache.max_pages + (b_lo + tid) * BLOCK_N / p.cache.page_size];
    asm volatile("" ::"r"(warm));
  }
  // A block's 64 rows x CHUNKS 16-byte pieces are spread over the threads.  Page ids are looked
  // up first for all of a thread's pieces (independent loads), then the copies are issued.
  constexpr int PIECES = (BLOCK_N * CHUNKS + THREADS - 1) / THREADS;
  auto load_kv = [&](int block, int stage) {
    __nv_bfloat16* kd = k_s + stage * BLOCK_N * PITCH;
    __nv_bfloat16* vd = v_s + stage * BLOCK_N * PITCH;
    long long off[PIECES];
    bool ok[PIECES];
    if (p.cache.page_size >= BLOCK_N) {
      // a block lies inside one page (both are powers of two, blocks start at multiples of 64): one lookup
      const int pos0 = block * BLOCK_N;
      const int page = p.cache.block_table[(long long)slot * p.cache.max_pages + (pos0 >> p.cache.page_shift)];
      const long long base = (long long)page * p.cache.page_stride +
                             ((long long)kvh * p.cache.page_size + (pos0 & (p.cache.page_size - 1))) * HD;
#pragma unroll
      for (int i = 0; i < PIECES; ++i) {
        const int idx = tid + i * THREADS;
        const int row = idx / CHUNKS, ch = idx % CHUNKS;
        const int pos = pos0 + row;
        ok[i] = idx < BLOCK_N * CHUNKS && pos >= key_lo && pos <= pos_last;
        off[i] = ok[i] ? base + (long long)row * HD + ch * 8 : 0;
      }
    } else {
#pragma unroll
      for (int i = 0; i < PIECES; ++i) {
        const int idx = tid + i * THREADS;
        const int row = idx / CHUNKS, ch = idx % CHUNKS;
        const int pos = block * BLOCK_N + row;
        ok[i] = idx < BLOCK_N * CHUNKS && pos >= key_lo && pos <= pos_last;
        off[i] = ok[i] ? paged_offset(p.cache, slot, pos, kvh) + ch * 8 : 0;
      }
    }
#pragma unroll
    for (int i = 0; i < PIECES; ++i) {
      const int idx = tid + i * THREADS;
      if (idx < BLOCK_N * CHUNKS) {
        const int row = idx / CHUNKS, ch = idx % CHUNKS;
        cp_async16(kd + row * PITCH + ch * 8, p.k_pool + off[i], ok[i]);
        cp_async16(vd + row * PITCH + ch * 8, p.v_pool + off[i], ok[i]);
      }
    }
  };

  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // positions of this thread's two rows (g and g+8 of the warp's 16)
  int row_pos[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    int row = wrow + g + 8 * h;
    row_pos[h] = row < rows_used ? pos_first + row / p.group : -1;      // -1: every key masked
  }

  // one cp.async group per block, committed even when empty, so that "all but the newest
  // STAGES-1 groups are complete" always means "this iteration's block has landed".
  // Keys below context_before were written by earlier steps, not by the previous kernel: blocks
  // that hold only such keys are requested before the wait on that kernel.
  int requested = 0;
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (requested == i && b_lo + i <= b_hi && (b_lo + i + 1) * BLOCK_N <= before) {
      load_kv(b_lo + i, i);
      cp_async_commit();
      ++requested;
    }
  }
  pdl_wait();
  pdl_launch_dependents();

  // ---- stage Q (rows beyond rows_used are zero) with plain loads: it becomes visible with the
  // first block's barrier and belongs to no cp.async group
  const bool fused_rope = KSPLIT && p.rope_qkv != nullptr;
  const int rope_half = p.rope_dim / 2;
  for (int idx = tid; idx < ROWS * CHUNKS; idx += THREADS) {
    int row = idx / CHUNKS, ch = idx % CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0), v2 = v;
    int pieces = 1;
    if (row < rows_used) {
      int t = t_first + row / p.group, hg = row % p.group;
      if (fused_rope) {
        const __nv_bfloat16* head = p.rope_qkv + (long long)(tok0 + t) * p.ld_qkv + (long long)(kvh * p.group + hg) * HD;
        const float2* tab = p.rope_cs ? p.rope_cs + (long long)(tok0 + t) * rope_half : nullptr;
        pieces = rope_piece(head, tab, ch * 8, p.rope_dim, p.rope_interleaved, v, v2);
      } else {
        v = *reinterpret_cast<const uint4*>(p.q + (long long)(tok0 + t) * p.ld_q + (long long)(kvh * p.group + hg) * HD + ch * 8);
      }
    }
    if (pieces >= 1) *reinterpret_cast<uint4*>(q_s + row * PITCH + ch * 8) = v;
    if (pieces == 2) *reinterpret_cast<uint4*>(q_s + row * PITCH + ch * 8 + rope_half) = v2;
  }
  // The new token's key (rotated) and value: held in registers by the first threads of the CTA whose
  // key range ends at the new position, written to the cache now and into the shared-memory tile
  // once that block's copy from the cache (which holds nothing valid for this row yet) has landed.
  const bool patch_cta = fused_rope && p.k_write != nullptr && b_lo <= b_hi && pos_last / BLOCK_N == b_hi;
  uint4 new_k0 = make_uint4(0, 0, 0, 0), new_k1 = new_k0, new_v = new_k0;
  int new_k_pieces = 0;
  if (patch_cta && tid < 2 * CHUNKS) {
    const __nv_bfloat16* row = p.rope_qkv + (long long)tok0 * p.ld_qkv;
    const long long at = paged_offset(p.cache, slot, pos_last, kvh);
    if (tid < CHUNKS) {
      const float2* tab = p.rope_cs ? p.rope_cs + (long long)tok0 * rope_half : nullptr;
      new_k_pieces = rope_piece(row + (long long)(p.heads + kvh) * HD, tab, tid * 8, p.rope_dim, p.rope_interleaved, new_k0, new_k1);
      if (new_k_pieces >= 1) *reinterpret_cast<uint4*>(p.k_write + at + tid * 8) = new_k0;
      if (new_k_pieces == 2) *reinterpret_cast<uint4*>(p.k_write + at + tid * 8 + rope_half) = new_k1;
    } else {
      const int ch = tid - CHUNKS;
      new_v = *reinterpret_cast<const uint4*>(row + (long long)(p.heads + p.heads / p.group + kvh) * HD + ch * 8);
      *reinterpret_cast<uint4*>(p.v_write + at + ch * 8) = new_v;
    }
  }
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i >= requested) {
      if (b_lo + i <= b_hi) load_kv(b_lo + i, i);
      cp_async_commit();
    }
  }

  for (int b = b_lo; b <= b_hi; ++b) {
    int stage = (b - b_lo) % STAGES;
    if (b + STAGES - 1 <= b_hi) load_kv(b + STAGES - 1, (b - b_lo + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    if (patch_cta && b == b_hi) {                       // CTA-uniform
      const int r_new = pos_last % BLOCK_N;
      if (tid < CHUNKS) {
        __nv_bfloat16* dst = k_s + (stage * BLOCK_N + r_new) * PITCH + tid * 8;
        if (new_k_pieces >= 1) *reinterpret_cast<uint4*>(dst) = new_k0;
        if (new_k_pieces == 2) *reinterpret_cast<uint4*>(dst + rope_half) = new_k1;
      } else if (tid < 2 * CHUNKS) {
        *reinterpret_cast<uint4*>(v_s + (stage * BLOCK_N + r_new) * PITCH + (tid - CHUNKS) * 8) = new_v;
      }
      __syncthreads();
    }

    const __nv_bfloat16* kt = k_s + stage * BLOCK_N * PITCH;
    const __nv_bfloat16* vt = v_s + stage * BLOCK_N * PITCH;

    // ---- S = Q K^T for this warp's 16 rows x 64 keys
    float s[WKEYS / 8][4];
#pragma unroll
    for (int i = 0; i < WKEYS / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, q_s + (wrow + (lane & 15)) * PITCH + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < WKEYS / 16; ++np) {
        uint32_t kb[4];
        ldmatrix_x4(kb, kt + (wkey + np * 16 + (lane & 7) + ((lane >> 4) << 3)) * PITCH + ks * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], a, kb[0], kb[1]);
        mma_bf16(s[2 * np + 1], a, kb[2], kb[3]);
      }
    }

    // ---- mask (only in blocks that reach past a row's position or below its window), online
    // softmax on the raw scores: p = 2^(s*c - m*c) with c = scale*log2(e) folded into one FMA
    const float c_log2 = p.scale_log2;
    const int key0 = b * BLOCK_N + wkey;                       // first key this warp visits in the block
    const int row_lo = min(row_pos_min, row_pos_max), row_hi = row_pos_max;
    const bool need_mask = key0 + WKEYS - 1 > row_lo || (p.window > 0 && key0 <= row_hi - p.window);
    float m_new[2] = {m_run[0], m_run[1]};
    if (need_mask) {
#pragma unroll
      for (int nt = 0; nt < WKEYS / 8; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          int h = j >> 1;
          int key = key0 + nt * 8 + 2 * c + (j & 1);
          bool ok = key <= row_pos[h] && (p.window <= 0 || key > row_pos[h] - p.window);
          if (!ok) s[nt][j] = -INFINITY;
        }
    }
#pragma unroll
    for (int nt = 0; nt < WKEYS / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) m_new[j >> 1] = fmaxf(m_new[j >> 1], s[nt][j]);
    float alpha[2], neg_mc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      float m_use = m_new[h] == -INFINITY ? 0.f : m_new[h];
      // 0 when the row sees its first key; 1 while it has seen none (nothing to rescale, and padding rows stay out of the test below)
      alpha[h] = m_new[h] == -INFINITY ? 1.f : fast_exp2((m_run[h] - m_use) * c_log2);
      neg_mc[h] = -m_use * c_log2;
      m_run[h] = m_new[h];
    }
    float l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < WKEYS / 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int h = j >> 1;
        float e = fast_exp2(fmaf(s[nt][j], c_log2, neg_mc[h]));
        s[nt][j] = e;
        l_add[h] += e;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + l_add[h];
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {       // most blocks leave every maximum where it was
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
        o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
      }
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < WKEYS / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vt + (wkey + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + dp * 16 + (lane >> 4) * 8);
        mma_bf16(o_acc[2 * dp], a, vb[0], vb[1]);
        mma_bf16(o_acc[2 * dp + 1], a, vb[2], vb[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- row sums across the quad
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  if constexpr (KSPLIT) {
    // merge the warps' (max, sum, O) per row in warp order; the K/V stages are free now
    float* mo = reinterpret_cast<float*>(k_s);                 // [NWARPS][16][HD]
    float* mm = mo + NWARPS * 16 * HD;                         // [NWARPS][16] max
    float* ml = mm + NWARPS * 16;                              // [NWARPS][16] sum
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int row = g + 8 * h;
      float* dst = mo + (warp * 16 + row) * HD;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * c) = make_float2(o_acc[i][2 * h], o_acc[i][2 * h + 1]);
      // running maxima are in raw score units; merges and partial results use log2 units
      if (c == 0) { mm[warp * 16 + row] = m_run[h] * p.scale_log2; ml[warp * 16 + row] = l_run[h]; }
    }
    __syncthreads();
    for (int idx = tid; idx < rows_used * (HD / 2); idx += THREADS) {
      int row = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) m = fmaxf(m, mm[w * 16 + row]);
      float l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        float mw = mm[w * 16 + row];
        float sc = mw == -INFINITY ? 0.f : exp2f(mw - m);
        l += sc * ml[w * 16 + row];
        o0 += sc * mo[(w * 16 + row) * HD + d];
        o1 += sc * mo[(w * 16 + row) * HD + d + 1];
      }
      int t = t_first + row / p.group, head = kvh * p.group + row % p.group;
      if (p.num_splits == 1) {
        float inv = l > 0.f ? 1.f / l : 0.f;
        __nv_bfloat16* dst = p.out + (long long)(tok0 + t) * p.ld_o + (long long)head * HD;
        *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(o0 * inv, o1 * inv);
      } else {
        long long pi = ((long long)(tok0 + t) * p.heads + head) * p.num_splits + split;
        *reinterpret_cast<float2*>(p.part_o + pi * HD + d) = make_float2(o0, o1);
        if (d == 0) { p.part_ml[pi * 2] = m; p.part_ml[pi * 2 + 1] = l; }
      }
    }
  } else {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    int row = wrow + g + 8 * h;
    if (row >= rows_used) continue;
    int t = t_first + row / p.group, head = kvh * p.group + row % p.group;
    if (p.num_splits == 1) {
      float inv = l_run[h] > 0.f ? 1.f / l_run[h] : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(tok0 + t) * p.ld_o + (long long)head * HD;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(o_acc[i][2 * h] * inv, o_acc[i][2 * h + 1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + 2 * c) = v;
      }
    } else {
      long long idx = ((long long)(tok0 + t) * p.heads + head) * p.num_splits + split;
      float* dst = p.part_o + idx * HD;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i)
        *reinterpret_cast<float2*>(dst + i * 8 + 2 * c) = make_float2(o_acc[i][2 * h], o_acc[i][2 * h + 1]);
      if (c == 0) {
        p.part_ml[idx * 2] = m_run[h] * p.scale_log2;
        p.part_ml[idx * 2 + 1] = l_run[h];
      }
    }
  }
  }
}

// out[token, head, :] = sum_s w_s O_s / sum_s w_s l_s, w_s = 2^(m_s - max m), splits in order.
// One warp per (token, head): lane s holds split s's (max, sum); every lane owns four output dims
// per trip.  The partial outputs of up to 8 splits are requested together with the (max, sum)
// pairs, before anything is computed: one memory round trip instead of one per split.
constexpr int COMBINE_WARPS = 4;
__global__ void __launch_bounds__(COMBINE_WARPS * 32)
attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                         __nv_bfloat16* __restrict__ out, int ld_o, int heads, int hd, int num_splits, int pairs) {
  pdl_wait();
  pdl_launch_dependents();
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int pair = blockIdx.x * COMBINE_WARPS + warp;
  if (pair >= pairs) return;
  int token = pair / heads, head = pair % heads;
  long long base = (long long)pair * num_splits;
  float2 ml = lane < num_splits ? *reinterpret_cast<const float2*>(part_ml + (base + lane) * 2) : make_float2(-INFINITY, 0.f);
  // splits that found no keys (a context shorter than the launch was planned for) hold (-inf, 0) and
  // no output; they come last, so only the leading ones are read
  const unsigned live = __ballot_sync(0xffffffffu, ml.x != -INFINITY);
  num_splits = live ? 32 - __clz(live) : 0;
  float w = 0.f, inv = 0.f;
  bool have_w = false;
  for (int d0 = 0; d0 < hd; d0 += 128) {         // every lane takes every trip: the shuffles need the whole warp
    const int d = d0 + lane * 4;                 // hd is a multiple of 16, so a lane's four dims are all in or all out
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < num_splits; s0 += 8) {
      float4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        v[i] = (s0 + i < num_splits && d < hd) ? *reinterpret_cast<const float4*>(part_o + (base + s0 + i) * hd + d)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
      if (!have_w) {
        float m = warp_max(ml.x);
        w = ml.x == -INFINITY ? 0.f : exp2f(ml.x - m);
        float l = 0.f;
        for (int s = 0; s < num_splits; ++s) l += __shfl_sync(0xffffffffu, w * ml.y, s);     // split order
        inv = l > 0.f ? 1.f / l : 0.f;
        have_w = true;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float ws = __shfl_sync(0xffffffffu, w, (s0 + i) & 31);
        if (s0 + i < num_splits) {
          acc.x += ws * v[i].x; acc.y += ws * v[i].y; acc.z += ws * v[i].z; acc.w += ws * v[i].w;
        }
      }
    }
    if (d < hd) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
      uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      *reinterpret_cast<uint2*>(out + (long long)token * ld_o + (long long)head * hd + d) = pk;
    }
  }
}

template <int HD, bool KSPLIT, int STAGES>
int launch(const AttnParams& p, int q_tiles, int kv_heads, int requests, cudaStream_t stream) {
  constexpr int NWARPS = 4;
  constexpr int PITCH = HD + 8;
  constexpr int ROWS = KSPLIT ? 16 : 64;
  size_t smem = (size_t)(ROWS + 2 * STAGES * BLOCK_N) * PITCH * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_mma_kernel<HD, NWARPS, KSPLIT, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "attention_mma: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((unsigned)kv_heads, (unsigned)(q_tiles * p.num_splits), (unsigned)requests);
  hfee_launch(attention_mma_kernel<HD, NWARPS, KSPLIT, STAGES>, dim3(grid), dim3(NWARPS * 32), smem, stream, p);
  return hfee_check_launch("attention_mma");
}

template <int HD>
int dispatch_mode(const AttnParams& p, bool ksplit, int q_tiles, int kv_heads, int requests, cudaStream_t stream) {
  if (!ksplit) return launch<HD, false, 2>(p, q_tiles, kv_heads, requests, stream);
  // decode: keep four key blocks in flight per CTA when the grid is small enough that the larger
  // shared-memory footprint (fewer CTAs per SM) does not add a wave; otherwise two
  constexpr int DEEP = HD <= 64 ? 4 : (HD <= 128 ? 3 : 2);
  long long ctas = (long long)p.num_splits * kv_heads * requests;
  if (DEEP > 2 && ctas <= 3 * hfee_sm_count()) return launch<HD, true, DEEP>(p, q_tiles, kv_heads, requests, stream);
  return launch<HD, true, 2>(p, q_tiles, kv_heads, requests, stream);
}

}  // namespace

// Scratch floats needed for `num_splits` > 1: n_tokens * heads * num_splits * (head_dim + 2).
HFEE_API long long hfee_attention_mma_scratch_floats(int n_tokens, int heads, int head_dim, int num_splits) {
  return num_splits > 1 ? (long long)n_tokens * heads * num_splits * (head_dim + 2) : 0;
}

// max_new: most new tokens of any request in the batch.  num_splits > 1 needs max_new * group <= rows
// of one tile and `scratch`.  Returns HFEE_ERR_ARG for head sizes or groups it does not take.
namespace {
struct RopeFusion {
  const void* qkv; int ld_qkv; const float* cs; int rope_dim; int interleaved; void* k_write; void* v_write;
};

int attention_mma_impl(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                       const int* block_table, int max_pages, int page_size, const int* cu_tokens,
                       const int* slots, const int* context_before, void* out, int ld_o, int n_tokens,
                       int requests, int max_new, int heads, int kv_heads, int head_dim, float scale,
                       int window, int num_splits, float* scratch, const RopeFusion* rope, cudaStream_t stream) {
  if (n_tokens == 0 || requests == 0) return HFEE_OK;
  HFEE_REQUIRE(head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 256,
               "attention_mma: head_dim %d must be a multiple of 16 in 16..256", head_dim);
  HFEE_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "attention_mma: heads %d / kv_heads %d", heads, kv_heads);
  int group = heads / kv_heads;
  HFEE_REQUIRE(group <= 64, "attention_mma: %d query heads per kv head exceed 64", group);
  HFEE_REQUIRE(ld_o % 2 == 0, "attention_mma: the output's leading dimension must be even");
  HFEE_REQUIRE(rope != nullptr || (ld_q % 8 == 0 && (uintptr_t)q % 16 == 0), "attention_mma: q must be 16-byte aligned with ld %% 8 == 0");
  HFEE_REQUIRE(requests <= 65535, "attention_mma: too many requests for one grid");
  HFEE_REQUIRE(max_new > 0 && num_splits >= 1 && num_splits <= 32, "attention_mma: num_splits must be in 1..32");
  // when 16 rows hold every request's new tokens (decode) the warps split the keys instead
  bool ksplit = max_new * group <= 16;
  int rows = ksplit ? 16 : 64;
  int tokens_per_tile = rows / group;
  int q_tiles = (max_new + tokens_per_tile - 1) / tokens_per_tile;
  HFEE_REQUIRE((long long)q_tiles * num_splits <= 65535, "attention_mma: %d new tokens of one request exceed one grid", max_new);
  HFEE_REQUIRE(num_splits == 1 || (ld_o % 4 == 0 && (uintptr_t)out % 8 == 0 && (uintptr_t)scratch % 16 == 0),
               "attention_mma: with split keys the output needs 8-byte alignment (ld %% 4 == 0) and the scratch 16-byte alignment");
  HFEE_REQUIRE(num_splits == 1 || (q_tiles == 1 && scratch != nullptr),
               "attention_mma: splitting the keys needs one query tile per request and scratch memory");
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.ld_q = ld_q;
  p.out = (__nv_bfloat16*)out; p.ld_o = ld_o;
  p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  HFEE_REQUIRE(make_paged_cache(&p.cache, block_table, max_pages, page_size, kv_heads, head_dim),
               "attention_mma: page_size %d must be a power of two", page_size);
  p.cu_tokens = cu_tokens; p.slots = slots; p.context_before = context_before;
  p.heads = heads; p.group = group;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.tokens_per_tile = tokens_per_tile; p.num_splits = num_splits;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (long long)n_tokens * heads * num_splits * head_dim : nullptr;
  p.rope_qkv = nullptr; p.ld_qkv = 0; p.rope_cs = nullptr; p.rope_dim = 0; p.rope_interleaved = 0;
  p.k_write = nullptr; p.v_write = nullptr;
  if (rope != nullptr) {
    HFEE_REQUIRE(ksplit && max_new == 1, "attention_mma: rotary fusion is for decode steps of one token per request");
    HFEE_REQUIRE(rope->qkv != nullptr && (uintptr_t)rope->qkv % 16 == 0 && rope->ld_qkv % 8 == 0 &&
                 rope->ld_qkv >= (heads + (rope->k_write ? 2 * kv_heads : 0)) * head_dim,
                 "attention_mma: the projection rows must be 16-byte aligned, ld %% 8 == 0, and hold q, k and v heads");
    HFEE_REQUIRE(rope->rope_dim >= 0 && rope->rope_dim <= head_dim && rope->rope_dim % 16 == 0,
                 "attention_mma: rotary fusion needs rope_dim %% 16 == 0 and at most head_dim, got %d", rope->rope_dim);
    HFEE_REQUIRE((rope->k_write == nullptr) == (rope->v_write == nullptr), "attention_mma: key and value pools go together");
    p.rope_qkv = (const __nv_bfloat16*)rope->qkv; p.ld_qkv = rope->ld_qkv;
    p.rope_cs = (const float2*)rope->cs; p.rope_dim = rope->rope_dim; p.rope_interleaved = rope->interleaved;
    p.k_write = (__nv_bfloat16*)rope->k_write; p.v_write = (__nv_bfloat16*)rope->v_write;
  }
  int rc;
  switch (head_dim) {
#define HFEE_CASE(D) case D: rc = dispatch_mode<D>(p, ksplit, q_tiles, kv_heads, requests, stream); break;
    HFEE_CASE(16) HFEE_CASE(32) HFEE_CASE(48) HFEE_CASE(64) HFEE_CASE(80) HFEE_CASE(96) HFEE_CASE(112) HFEE_CASE(128)
    HFEE_CASE(144) HFEE_CASE(160) HFEE_CASE(176) HFEE_CASE(192) HFEE_CASE(208) HFEE_CASE(224) HFEE_CASE(240) HFEE_CASE(256)
#undef HFEE_CASE
    default: return hfee_fail(HFEE_ERR_ARG, "attention_mma: head_dim %d", head_dim);
  }
  if (rc != HFEE_OK || num_splits == 1) return rc;
  int pairs = n_tokens * heads;
  hfee_launch(attention_combine_kernel, dim3((unsigned)((pairs + COMBINE_WARPS - 1) / COMBINE_WARPS)),
              dim3(COMBINE_WARPS * 32), 0, stream, p.part_o, p.part_ml, p.out, ld_o, heads, head_dim, num_splits, pairs);
  return hfee_check_launch("attention_combine");
}
}  // namespace

// q [n_tokens, ld_q], out [n_tokens, ld_o]: bfloat16; pools [num_pages, kv_heads, page_size, head_dim].
// num_splits > 1 (only when max_new * group <= 16) needs `scratch` of
// n_tokens * heads * num_splits * (head_dim + 2) floats and launches the combine kernel too.
HFEE_API int hfee_attention_mma(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                const int* block_table, int max_pages, int page_size, const int* cu_tokens,
                                const int* slots, const int* context_before, void* out, int ld_o, int n_tokens,
                                int requests, int max_new, int heads, int kv_heads, int head_dim, float scale,
                                int window, int num_splits, float* scratch, cudaStream_t stream) {
  return attention_mma_impl(q, ld_q, k_pool, v_pool, block_table, max_pages, page_size, cu_tokens, slots, context_before,
                            out, ld_o, n_tokens, requests, max_new, heads, kv_heads, head_dim, scale, window, num_splits,
                            scratch, nullptr, stream);
}

// A decode step (one new token per request) with the rotary kernel's work done inside: queries,
// the new key and the new value come from the projection rows `qkv` [n_tokens, ld_qkv] =
// [q heads | k heads | v heads]; `cs` [n_tokens, rope_dim/2] holds (cos, sin) pairs (null: no
// rotation); the rotated key and the value are written to the cache pages of (slot, position)
// unless `write_cache` is 0 (a run that reads another run's cache: then qkv holds q heads only).
HFEE_API int hfee_attention_mma_rope(const void* qkv, int ld_qkv, const float* cs, int rope_dim, int interleaved,
                                     int write_cache, void* k_pool, void* v_pool, const int* block_table, int max_pages,
                                     int page_size, const int* cu_tokens, const int* slots, const int* context_before,
                                     void* out, int ld_o, int n_tokens, int requests, int heads, int kv_heads,
                                     int head_dim, float scale, int window, int num_splits, float* scratch,
                                     cudaStream_t stream) {
  RopeFusion rope{qkv, ld_qkv, cs, rope_dim, interleaved, write_cache ? k_pool : nullptr, write_cache ? v_pool : nullptr};
  return attention_mma_impl(nullptr, 0, k_pool, v_pool, block_table, max_pages, page_size, cu_tokens, slots,
                            context_before, out, ld_o, n_tokens, requests, 1, heads, kv_heads, head_dim, scale, window,
                            num_splits, scratch, &rope, stream);
}

// ------------------------------------------------------------------------------------------
// The same split-key attention for callers that cannot allocate: its partial results go to a
// fixed array in this library instead of caller-provided scratch.  See no_alloc.h.
#include "no_alloc.h"

namespace {

// Partial (max, sum, output) cells of one call.  A host-side name only stands in for this array;
// the kernels get its device address, looked up once per device below.
static __device__ __align__(256) float g_noalloc_scratch[HFEE_NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};

// Device address of the array on the current device (set-up on the first call per device).
int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "attention_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES)
    return hfee_fail(HFEE_ERR_ARG, "attention_decode_noalloc: device ordinal %d is outside 0..%d", dev, NOALLOC_MAX_DEVICES - 1);
  if (g_noalloc_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return hfee_fail(HFEE_ERR_CUDA, "attention_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return HFEE_OK;
}

}  // namespace

HFEE_API int hfee_attention_decode_noalloc(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                           const int* block_table, int max_pages, int page_size,
                                           const int* cu_tokens, const int* slots, const int* context_before,
                                           void* out, int ld_o, int n_tokens, int requests, int max_new, int heads,
                                           int kv_heads, int head_dim, float scale, int window, int num_splits,
                                           cudaStream_t stream) {
  if (n_tokens == 0 || requests == 0) return HFEE_OK;
  HFEE_REQUIRE(num_splits >= 2, "attention_decode_noalloc: num_splits=%d; this entry point is the split-key variant (>= 2)", num_splits);
  HFEE_REQUIRE(n_tokens > 0 && heads > 0 && head_dim > 0, "attention_decode_noalloc: bad sizes");
  long long need = (long long)n_tokens * heads * num_splits * (head_dim + 2);
  HFEE_REQUIRE(need <= (long long)HFEE_NOALLOC_SCRATCH_FLOATS,
               "attention_decode_noalloc: %d tokens x %d heads x %d splits x (%d + 2) = %lld floats of partial "
               "results exceed the built-in scratch of %d floats; use fewer splits or hfee_attention_mma with "
               "scratch of your own", n_tokens, heads, num_splits, head_dim, need, (int)HFEE_NOALLOC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc != HFEE_OK) return rc;
  return hfee_attention_mma(q, ld_q, k_pool, v_pool, block_table, max_pages, page_size, cu_tokens, slots,
                            context_before, out, ld_o, n_tokens, requests, max_new, heads, kv_heads, head_dim, scale,
                            window, num_splits, scratch, stream);
}
