// Causal grouped-query flash attention for prompt portions on the 5th-generation tensor cores:
// S = Q K^T and O_block = P V are tcgen05 MMAs with their accumulators in tensor memory, Q/K/V
// tiles arrive by TMA (K and V page by page through the block table), and a warpgroup of four
// softmax warps owns one query row per thread (so row maxima and sums need no shuffles).
//
// A CTA serves one (request, kv head, tile of 128 query rows); the rows are (token, query head of
// the group) pairs, so the group shares every key/value tile.  Keys go in blocks of 128:
//   warp 0     TMA producer   Q once; per block K and V (two 64-key page pieces each) into a
//                             3-stage ring
//   warp 1     MMA issuer     S_j = Q K_j^T into S buffer j%2 (issued one block ahead), then
//                             O_j = P_j V_j into O buffer j%2 once the softmax warps wrote P_j
//   warps 2-5  softmax        read S_j from TMEM (twice: row max, then exponentials), write P_j as
//                             bf16 into 128B-swizzled shared memory, keep the running max/sum and
//                             the output row in registers: o = o * alpha_j + O_j, read from TMEM
// Masks: causal and window, applied only in blocks that need them.  Head size 64, pages of at least
// 64 tokens (a power of two); other shapes use the mma.sync kernel.  Every barrier wait is bounded.
// Reference: hostfog/hfee internal/llm/forward.go:146-178, internal/ggml/ops.go:136-150.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int QM = 128;            // query rows per CTA
constexpr int KB = 128;            // keys per block
constexpr int HD = 64;             // head size
constexpr int KV_STAGES = 2;
constexpr int NBUF = 1;            // S, P and O buffers per CTA; two CTAs share an SM and overlap each other
constexpr int AT_THREADS = 192;
constexpr int Q_BYTES = QM * HD * 2;            // 16 KB
constexpr int KT_BYTES = KB * HD * 2;           // 16 KB each for K and V
constexpr int P_BYTES = QM * KB * 2;            // 32 KB: two slabs of [128 rows][64 keys]
constexpr int TILE_BYTES = Q_BYTES + KV_STAGES * 2 * KT_BYTES + NBUF * P_BYTES;
constexpr int AT_SMEM = TILE_BYTES + 256;       // + barriers; the base must come 1024-aligned (checked)
constexpr uint32_t TMEM_COLS = NBUF == 1 ? 256 : 512;     // S: NBUF x 128 columns, O: NBUF x 64 columns
constexpr uint32_t S_COL = 0, O_COL = NBUF * KB;

struct TcAttnParams {
  __nv_bfloat16* out; int ld_o;
  const int* block_table; int max_pages; int page_shift; int page_size;
  const int* cu_tokens;
  const int* slots;
  const int* context_before;
  int heads, group;
  float scale_log2;
  int window;
  int tokens_per_tile, q_tiles;
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Descriptor of an MN-major operand tile in the 128-byte swizzle: rows (the K index) are 128 bytes
// of 64 contiguous MN elements, 8-row groups are `sbo` bytes apart; `lbo` is the distance between
// 64-element chunks along MN (unused when the tile is 64 wide).
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, TcAttnParams p, int* __restrict__ status) {
  // no static shared memory: tiles first (1024-byte aligned for the swizzle), barriers behind them,
  // so that two CTAs fit one SM
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* base = smem_dyn;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + TILE_BYTES);
  uint64_t& q_full = bars[0];
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + KV_STAGES;
  uint64_t* s_full = kv_empty + KV_STAGES;
  uint64_t* s_empty = s_full + NBUF;
  uint64_t* p_full = s_empty + NBUF;
  uint64_t* p_empty = p_full + NBUF;
  uint64_t* o_full = p_empty + NBUF;
  uint64_t* o_empty = o_full + NBUF;
  uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(o_empty + NBUF);
  int& abort_flag = *reinterpret_cast<int*>(reinterpret_cast<uint32_t*>(o_empty + NBUF) + 1);
  static_assert((1 + 2 * KV_STAGES + 6 * NBUF) * 8 + 8 <= 256, "barrier area");
  unsigned char* q_s = base;
  unsigned char* kv_s = base + Q_BYTES;                                 // [stage][K | V]
  unsigned char* p_s = kv_s + KV_STAGES * 2 * KT_BYTES;                 // [2][P]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // CTAs start in the order of blockIdx.x, then y: the heaviest tiles (latest positions) of every
  // kv head first, the light ones last, so that they fill the gaps at the end
  const int tile = p.q_tiles - 1 - (int)blockIdx.y, kvh = blockIdx.x, r = blockIdx.z;
  const int tok0 = p.cu_tokens[r], n_new = p.cu_tokens[r + 1] - tok0;
  const int t_first = tile * p.tokens_per_tile;
  if (t_first >= n_new) return;
  const int t_count = min(p.tokens_per_tile, n_new - t_first);
  const int slot = p.slots[r], before = p.context_before[r];
  const int pos_first = before + t_first, pos_last = pos_first + t_count - 1;
  const int key_lo = (p.window > 0 && pos_first + 1 > p.window) ? pos_first + 1 - p.window : 0;
  const int b_lo = key_lo / KB, nb = pos_last / KB - b_lo + 1;

  if (threadIdx.x == 0) {
    abort_flag = (smem_u32(base) & 1023u) != 0 ? 1 : 0;       // misaligned tiles would corrupt the swizzle
    mbar_init(&q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < NBUF; ++b) {
      mbar_init(&s_full[b], 1); mbar_init(&s_empty[b], 4);
      mbar_init(&p_full[b], 4); mbar_init(&p_empty[b], 1);
      mbar_init(&o_full[b], 1); mbar_init(&o_empty[b], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();                       // queries and this step's keys/values come from the previous kernels
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // the box is tokens_per_tile x group rows (fewer than 128 when the group does not divide 128;
      // the rows left over are never read back)
      mbar_expect_tx(&q_full, (uint32_t)(p.tokens_per_tile * p.group * HD * 2));
      tma_load_4d(q_s, &map_q, 0, 0, kvh, tok0 + t_first, &q_full);
      bool ok = true;
      for (int j = 0; j < nb && ok; ++j) {
        const int s = j % KV_STAGES;
        ok = mbar_wait(&kv_empty[s], ((j / KV_STAGES) & 1u) ^ 1u, &abort_flag);
        if (!ok) break;
        unsigned char* k_dst = kv_s + s * 2 * KT_BYTES;
        mbar_expect_tx(&kv_full[s], 2 * KT_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c) {                       // two pieces of 64 keys
          const int key0 = (b_lo + j) * KB + c * 64;
          // a piece beyond the pages the request holds reads page -1: out of range, zero-filled
          const int page = (key0 >> p.page_shift) < p.max_pages
                               ? p.block_table[(long long)slot * p.max_pages + (key0 >> p.page_shift)] : -1;
          const int in_page = key0 & (p.page_size - 1);
          tma_load_4d(k_dst + c * (KT_BYTES / 2), &map_k, 0, in_page, kvh, page, &kv_full[s]);
          tma_load_4d(k_dst + KT_BYTES + c * (KT_BYTES / 2), &map_v, 0, in_page, kvh, page, &kv_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(QM, KB);                       // A, B K-major
      constexpr uint32_t idesc_o = make_idesc(QM, HD) | (1u << 16);          // B (V) MN-major
      const uint32_t q_addr = smem_u32(q_s);
      bool ok = mbar_wait(&q_full, 0, &abort_flag);
      auto issue_s = [&](int j) {
        const int s = j % KV_STAGES, sb = j % NBUF;
        ok = ok && mbar_wait(&kv_full[s], (j / KV_STAGES) & 1u, &abort_flag);
        ok = ok && mbar_wait(&s_empty[sb], ((j / NBUF) & 1u) ^ 1u, &abort_flag);
        if (!ok) return;
        tc_fence_after();
        const uint64_t dq = make_desc(q_addr), dk = make_desc(smem_u32(kv_s + s * 2 * KT_BYTES));
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          tc_mma(tmem_base + S_COL + sb * KB, dq + 2 * k, dk + 2 * k, idesc_s, k != 0);
        tc_commit(&s_full[sb]);
      };
      auto issue_pv = [&](int j) {
        const int s = j % KV_STAGES, sb = j % NBUF;
        ok = ok && mbar_wait(&p_full[sb], (j / NBUF) & 1u, &abort_flag);
        ok = ok && mbar_wait(&o_empty[sb], ((j / NBUF) & 1u) ^ 1u, &abort_flag);
        if (!ok) return;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(p_s + sb * P_BYTES);
        const uint32_t v_addr = smem_u32(kv_s + s * 2 * KT_BYTES + KT_BYTES);
#pragma unroll
        for (int kk = 0; kk < KB / 16; ++kk) {
          // P: slab kk/4 of [128 rows][64 keys], 16 keys = 32 bytes further along K
          const uint64_t dp = make_desc(p_addr + (kk / 4) * (P_BYTES / 2)) + 2 * (kk % 4);
          // V: 16 keys = two 8-row groups of 1024 bytes further
          const uint64_t dv = make_desc_mn(v_addr + kk * 2048, 16, 1024);
          tc_mma(tmem_base + O_COL + sb * HD, dp, dv, idesc_o, kk != 0);
        }
        tc_commit(&o_full[sb]);
        tc_commit(&kv_empty[s]);
        tc_commit(&p_empty[sb]);
      };
      if (ok) issue_s(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) issue_s(j + 1);
        issue_pv(j);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                       // tile row = TMEM lane
    const int rows_used = t_count * p.group;
    const bool valid = row < rows_used;
    const int pos = valid ? pos_first + row / p.group : -1;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float c_log2 = p.scale_log2;
    float o_reg[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) o_reg[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
    bool ok = true;

    // every lane of a warp must take the same path around the warp-wide TMEM loads, also when a
    // wait gives up
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {       // one lane waits, the warp follows
      int done = lane == 0 ? (int)mbar_wait(bar, parity, &abort_flag) : 0;
      return __shfl_sync(0xffffffffu, done, 0) != 0;
    };
    auto accumulate = [&](int j, float alpha) {            // o = o * alpha + O_j
      const int sb = j % NBUF;
      ok = ok && wait_all(&o_full[sb], (j / NBUF) & 1u);
      tc_fence_after();
      if (!ok) return;
#pragma unroll
      for (int ch = 0; ch < HD / 32; ++ch) {
        uint32_t v[32];
        tc_ld32(lane_addr + O_COL + sb * HD + ch * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_reg[ch * 32 + i] = fmaf(o_reg[ch * 32 + i], alpha, __uint_as_float(v[i]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty[sb]);
    };

    for (int j = 0; j < nb && ok; ++j) {
      const int sb = j % NBUF;
      const int key0 = (b_lo + j) * KB;
      ok = wait_all(&s_full[sb], (j / NBUF) & 1u);
      tc_fence_after();
      if (!ok) break;
      // keys this row may see: [key_min, pos]; blocks wholly inside need no per-element test
      const int key_min = p.window > 0 ? pos - p.window + 1 : -(1 << 30);
      const bool need_mask = key0 + KB - 1 > pos || key0 < key_min;
      // pass 1: row maximum (four independent chains)
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int ch = 0; ch < KB / 32; ++ch) {
        uint32_t v[32];
        tc_ld32(lane_addr + S_COL + sb * KB + ch * 32, v);
        tc_wait_ld();
        if (need_mask) {
          const int kb = key0 + ch * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool seen = kb + i <= pos && kb + i >= key_min;
            mx[i & 3] = fmaxf(mx[i & 3], seen ? __uint_as_float(v[i]) : -INFINITY);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[i]));
        }
      }
      const float m_new = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), m_run);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2((m_run - m_use) * c_log2);
      const float neg_mc = -m_use * c_log2;
      m_run = m_new;
      // the P buffer is free once the MMA that read it has completed
      ok = wait_all(&p_empty[sb], ((j / NBUF) & 1u) ^ 1u);
      if (!ok) break;
      // pass 2: exponentials -> bf16 P row in the 128-byte swizzle: 16-byte chunk c of row r sits
      // at chunk position c ^ (r % 8) of its 128-byte line
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned char* p_row = p_s + sb * P_BYTES + row * 128;
#pragma unroll 1
      for (int ch = 0; ch < KB / 32; ++ch) {
        uint32_t v[32];
        tc_ld32(lane_addr + S_COL + sb * KB + ch * 32, v);
        tc_wait_ld();
        float e[32];
        if (need_mask) {
          const int kb = key0 + ch * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool seen = kb + i <= pos && kb + i >= key_min;
            e[i] = seen ? fast_exp2(fmaf(__uint_as_float(v[i]), c_log2, neg_mc)) : 0.f;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) e[i] = fast_exp2(fmaf(__uint_as_float(v[i]), c_log2, neg_mc));
        }
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          ls[(i >> 1) & 3] += e[i] + e[i + 1];
          __nv_bfloat162 b = __floats2bfloat162_rn(e[i], e[i + 1]);
          packed[i / 2] = *reinterpret_cast<uint32_t*>(&b);
        }
        unsigned char* slab = p_row + (ch / 2) * (P_BYTES / 2);           // keys 0-63 | 64-127
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {                                   // four 16-byte chunks = 32 keys
          const int chunk = (ch % 2) * 4 + q4;
          *reinterpret_cast<uint4*>(slab + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      }
      const float l_add = (ls[0] + ls[1]) + (ls[2] + ls[3]);
      l_run = l_run * alpha + l_add;
      // S buffer read completely; P written: make it visible to the tensor core's (async) reads
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[sb]); mbar_arrive(&p_full[sb]); }
      // fold in the previous block's output while the tensor core works on this one
      if (j > 0) accumulate(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    if (ok && nb > 0) accumulate(nb - 1, alpha_prev);

    if (ok && valid) {
      const int t = t_first + row / p.group, head = kvh * p.group + row % p.group;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(tok0 + t) * p.ld_o + (long long)head * HD;
#pragma unroll
      for (int d = 0; d < HD; d += 8) {
        uint4 o;
        __nv_bfloat162 b0 = __floats2bfloat162_rn(o_reg[d] * inv, o_reg[d + 1] * inv);
        __nv_bfloat162 b1 = __floats2bfloat162_rn(o_reg[d + 2] * inv, o_reg[d + 3] * inv);
        __nv_bfloat162 b2 = __floats2bfloat162_rn(o_reg[d + 4] * inv, o_reg[d + 5] * inv);
        __nv_bfloat162 b3 = __floats2bfloat162_rn(o_reg[d + 6] * inv, o_reg[d + 7] * inv);
        o.x = *reinterpret_cast<uint32_t*>(&b0); o.y = *reinterpret_cast<uint32_t*>(&b1);
        o.z = *reinterpret_cast<uint32_t*>(&b2); o.w = *reinterpret_cast<uint32_t*>(&b3);
        *reinterpret_cast<uint4*>(dst + d) = o;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    for (int i = 0; i < 400; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 2);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Rank-4 bf16 tensor map with the 128-byte swizzle.  dims/box innermost first; strides (bytes) for dims 1..3.
int make_map_4d(CUtensorMap* map, const void* base, const cuuint64_t (&dims)[4], const cuuint64_t (&strides)[3],
                const cuuint32_t (&box)[4]) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return hfee_fail(HFEE_ERR_CUDA, "attention_tc: the driver has no cuTensorMapEncodeTiled");
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return hfee_fail(HFEE_ERR_CUDA, "attention_tc: cuTensorMapEncodeTiled failed with %d", (int)rc);
  return HFEE_OK;
}

}  // namespace

// 1 if hfee_attention_tc takes this shape (bfloat16 is implied).
HFEE_API int hfee_attention_tc_supports(int heads, int kv_heads, int head_dim, int page_size) {
  if (head_dim != HD || kv_heads <= 0 || heads % kv_heads != 0) return 0;
  int group = heads / kv_heads;
  if (group > QM) return 0;
  if (page_size < 64 || (page_size & (page_size - 1)) != 0) return 0;
  return 1;
}

// q [n_tokens, ld_q], out [n_tokens, ld_o]: bfloat16; pools [num_pages, kv_heads, page_size, head_dim].
HFEE_API int hfee_attention_tc(const void* q, int ld_q, const void* k_pool, const void* v_pool, int num_pages,
                               const int* block_table, int max_pages, int page_size, const int* cu_tokens,
                               const int* slots, const int* context_before, void* out, int ld_o, int n_tokens,
                               int requests, int max_new, int heads, int kv_heads, int head_dim, float scale,
                               int window, int* status, cudaStream_t stream) {
  if (n_tokens == 0 || requests == 0) return HFEE_OK;
  HFEE_REQUIRE(hfee_attention_tc_supports(heads, kv_heads, head_dim, page_size),
               "attention_tc: needs head_dim 64, at most 128 query heads per kv head and power-of-two pages >= 64 "
               "(got head_dim %d, heads %d/%d, page_size %d)", head_dim, heads, kv_heads, page_size);
  HFEE_REQUIRE(ld_q % 8 == 0 && ld_o % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)out % 16 == 0,
               "attention_tc: q and out must be 16-byte aligned with leading dimensions %% 8 == 0");
  HFEE_REQUIRE(requests <= 65535 && max_new > 0 && max_new / (QM / (heads / kv_heads)) < 65535 && num_pages > 0,
               "attention_tc: bad sizes");
  const int group = heads / kv_heads;
  TcAttnParams p;
  p.out = (__nv_bfloat16*)out; p.ld_o = ld_o;
  p.block_table = block_table; p.max_pages = max_pages; p.page_size = page_size;
  p.page_shift = 0;
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  p.cu_tokens = cu_tokens; p.slots = slots; p.context_before = context_before;
  p.heads = heads; p.group = group;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.tokens_per_tile = QM / group;
  p.q_tiles = (max_new + p.tokens_per_tile - 1) / p.tokens_per_tile;

  CUtensorMap mq, mk, mv;
  {
    // q as [token][kv head][head of group][d]; a tile is (tokens_per_tile x group) rows of 64 d
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)group, (cuuint64_t)kv_heads, (cuuint64_t)n_tokens};
    const cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)group * HD * 2, (cuuint64_t)ld_q * 2};
    const cuuint32_t box[4] = {(cuuint32_t)HD, (cuuint32_t)group, 1, (cuuint32_t)p.tokens_per_tile};
    int rc = make_map_4d(&mq, q, dims, strides, box);
    if (rc != HFEE_OK) return rc;
  }
  {
    const cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)page_size * HD * 2,
                                   (cuuint64_t)kv_heads * page_size * HD * 2};
    const cuuint32_t box[4] = {(cuuint32_t)HD, 64, 1, 1};
    int rc = make_map_4d(&mk, k_pool, dims, strides, box);
    if (rc != HFEE_OK) return rc;
    rc = make_map_4d(&mv, v_pool, dims, strides, box);
    if (rc != HFEE_OK) return rc;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "attention_tc: cannot get %d bytes of shared memory: %s", AT_SMEM, cudaGetErrorString(e));
    configured = true;
  }
  dim3 grid((unsigned)kv_heads, (unsigned)p.q_tiles, (unsigned)requests);
  hfee_launch(attention_tc_kernel, grid, dim3(AT_THREADS), AT_SMEM, stream, mq, mk, mv, p, status);
  return hfee_check_launch("attention_tc");
}
