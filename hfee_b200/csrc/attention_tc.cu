// Causal grouped-query flash attention for prompt portions on the 5th-generation tensor cores,
// head sizes 64 and 128.
//
// A CTA serves one (request, kv head) and NT tiles of 128 query rows; the rows are (token, query
// head of the group) pairs, so the whole group shares every key/value tile, and the NT tiles
// (adjacent token ranges) share them too.  Keys go in blocks of 128:
//   warp 0        TMA producer   Q tiles once; per block K then V (64-key page pieces through the
//                                block table, 64 head dims per load) into a ring of stages
//   warp 1        MMA issuer     S_t = Q_t K^T into tile t's 128 S columns of tensor memory, then,
//                                once tile t's softmax warps have turned S_t into P_t,
//                                O_t += P_t V with P_t read from tensor memory (it overwrites the
//                                first 64 columns of S_t as packed bfloat16) and directly the next
//                                S_t: while one tile's rows are in the softmax the tensor core
//                                works for the other tile
//   warps 4..     softmax        a warpgroup per tile, one query row per thread: the row of S is read
//                                from tensor memory once, max / exp2 / sum in registers, P written
//                                back with tcgen05.st (warps 2 and 3 only give their registers to
//                                the softmax warpgroups)
// O_t stays in tensor memory for the whole key loop (the MMA accumulates into it).  The running row
// maximum is moved only when it grew by more than 2^8 in the exponent (then that warp rescales its
// O rows in tensor memory); otherwise the old maximum keeps being used for P and for the row sum,
// which cancels in O / sum.
// Masks: causal and window, applied only in blocks that need them; V rows of positions behind the
// last token of the CTA are cleared in shared memory, so that whatever an earlier owner of the page
// left there (also a NaN) meets no MMA.  Pages of at least 64 tokens (a power of two); other shapes
// use the mma.sync kernel.  Every barrier wait is bounded.
// Reference: hostfog/hfee internal/llm/forward.go:146-178, internal/ggml/ops.go:136-150.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int QM = 128;            // query rows per tile
constexpr int KB = 128;            // keys per block
constexpr int SLAB_BYTES = 128 * 128;   // 128 rows of 64 bf16: one 128-byte-swizzled slab of Q, K or V
constexpr float RESCALE_LOG2 = 8.f;     // the row maximum moves only when it grew by more than this

template <int HD, int NT>
struct TcCfg {
  static constexpr int SLABS = HD / 64;
  static constexpr int Q_BYTES = QM * HD * 2;              // one query tile
  static constexpr int KT_BYTES = KB * HD * 2;             // K or V of one key block
  static constexpr int STAGES = HD == 64 ? 3 : 2;
  static constexpr int TILE_BYTES = NT * Q_BYTES + STAGES * 2 * KT_BYTES;
  static constexpr int SMEM = TILE_BYTES + 256;            // + barriers; the base must come 1024-aligned (checked)
  static constexpr int THREADS = 128 + NT * 128;      // warpgroup 0: producer and MMA warps; one warpgroup per tile
  // Tensor memory: S_t at t*128.  When the 512 columns allow it (head size 64) P_t has 64 columns of
  // its own, so that S_t is free again as soon as the softmax threads hold it in registers and the
  // next S_t is computed while they work; else P_t overwrites the first half of S_t.  O_t behind them.
  static constexpr bool SEP_P = NT * (KB + KB / 2 + HD) <= 512;
  static constexpr uint32_t S_COL = 0, P_COL = SEP_P ? NT * KB : 0, P_STRIDE = SEP_P ? KB / 2 : KB;
  static constexpr uint32_t O_COL = SEP_P ? NT * (KB + KB / 2) : NT * KB;      // O_t at O_COL + t*HD
  static constexpr uint32_t TMEM_COLS = O_COL + NT * HD <= 256 ? 256 : 512;
  static_assert(O_COL + NT * HD <= 512, "tensor memory");
  static constexpr int N_BARS = NT + 3 * STAGES + 5 * NT + 1;
  static_assert(N_BARS * 8 + 8 <= 256, "barrier area");
  static_assert(SMEM <= 227 * 1024, "shared memory");
};

struct TcAttnParams {
  __nv_bfloat16* out; int ld_o;
  const int* block_table; int max_pages; int page_shift; int page_size;
  const int* cu_tokens;
  const int* slots;
  const int* context_before;
  int heads, group;
  float scale_log2;
  int window;
  int tokens_per_tile, q_tiles, q_groups;      // q_groups = CTAs along the tokens = ceil(q_tiles / NT)
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Descriptor of an MN-major operand tile, 64 MN elements wide, in the 128-byte swizzle: rows (the K
// index) are 128 bytes of 64 contiguous MN elements, 8-row groups are `sbo` bytes apart.
__device__ __forceinline__ uint64_t make_desc_mn(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 bf16, two to a 32-bit column) comes from
// tensor memory.
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two float32 operations in one instruction.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)), "l"(reinterpret_cast<uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

template <int HD, int NT>
__global__ void __launch_bounds__(TcCfg<HD, NT>::THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, TcAttnParams p, int* __restrict__ status) {
  using C = TcCfg<HD, NT>;
  constexpr int ST = C::STAGES;
  // no static shared memory: tiles first (1024-byte aligned for the swizzle), barriers behind them
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* base = smem_dyn;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + C::TILE_BYTES);
  uint64_t* q_full = bars;                 // [NT]
  uint64_t* k_full = q_full + NT;          // [ST]
  uint64_t* v_full = k_full + ST;          // [ST]
  uint64_t* kv_empty = v_full + ST;        // [ST]
  uint64_t* s_full = kv_empty + ST;        // [NT]  S_t of the current block is in tensor memory
  uint64_t* p_full = s_full + NT;          // [NT]  P_t is in tensor memory (and O_t rescaled if it had to be)
  uint64_t* o_done = p_full + NT;          // [NT]  the MMAs O_t += P_t V of the current block have completed
  uint64_t* s_free = o_done + NT;          // [NT]  the softmax threads hold S_t in registers (SEP_P only)
  uint64_t* turn = s_free + NT;            // [NT]  tile t's softmax threads may compute their exponentials (SEP_P only)
  uint64_t* v_clean = turn + NT;           //       the last block's V rows behind the last position are cleared
  uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(v_clean + 1);
  int& abort_flag = *reinterpret_cast<int*>(reinterpret_cast<uint32_t*>(v_clean + 1) + 1);
  unsigned char* q_s = base;                                  // [NT][slab][128 rows][64]
  unsigned char* kv_s = base + NT * C::Q_BYTES;               // [stage][K | V][slab][128 keys][64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // CTAs start in the order of blockIdx.x, then y: the heaviest tiles (latest positions) of every
  // kv head first, the light ones last, so that they fill the gaps at the end
  const int qg = p.q_groups - 1 - (int)blockIdx.y, kvh = blockIdx.x, r = blockIdx.z;
  const int tok0 = p.cu_tokens[r], n_new = p.cu_tokens[r + 1] - tok0;
  if (qg * NT * p.tokens_per_tile >= n_new) return;
  const int slot = p.slots[r], before = p.context_before[r];
  // per tile: first token, token count, key blocks; all tiles walk the blocks from the first one
  // that the earliest tile can see
  int t_first[NT], t_count[NT], nb_t[NT];
  int nb = 0, pos_last_all = 0;
  const int pos_first0 = before + qg * NT * p.tokens_per_tile;
  const int key_lo = (p.window > 0 && pos_first0 + 1 > p.window) ? pos_first0 + 1 - p.window : 0;
  const int b_lo = key_lo / KB;
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    t_first[t] = (qg * NT + t) * p.tokens_per_tile;
    t_count[t] = min(p.tokens_per_tile, n_new - t_first[t]);
    nb_t[t] = 0;
    if (t_count[t] > 0) {
      const int pos_last = before + t_first[t] + t_count[t] - 1;
      nb_t[t] = pos_last / KB - b_lo + 1;
      nb = nb_t[t];
      pos_last_all = pos_last;
    }
  }

  if (threadIdx.x == 0) {
    abort_flag = (smem_u32(base) & 1023u) != 0 ? 1 : 0;       // misaligned tiles would corrupt the swizzle
    for (int t = 0; t < NT; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&s_full[t], 1); mbar_init(&p_full[t], 4); mbar_init(&o_done[t], 1); mbar_init(&s_free[t], 4); mbar_init(&turn[t], 4);
    }
    for (int s = 0; s < ST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(v_clean, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();                       // queries and this step's keys/values come from the previous kernels
  pdl_launch_dependents();
  // The softmax threads hold a whole row of S: they take registers the first warpgroup does not need.
  // The kernel starts with 168 registers per thread (65,536 / 384 rounded down to a multiple of 8);
  // setmaxnreg.inc waits until the CTA's pool holds what it asks for, so what the first warpgroup
  // gives up (168 - 64 each) must cover what the others take (216 - 168 each) or the CTA hangs.
  static_assert(128 * (168 - 64) >= NT * 128 * (216 - 168), "register hand-over");

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 0) {
      if (lane == 0) {
        // a query box is tokens_per_tile x group rows (fewer than 128 when the group does not divide
        // 128; the rows left over are never read back), 64 head dims per load
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          if (nb_t[t] == 0) continue;
          mbar_expect_tx(&q_full[t], (uint32_t)(p.tokens_per_tile * p.group * HD * 2));
#pragma unroll
          for (int h = 0; h < C::SLABS; ++h)
            tma_load_4d(q_s + t * C::Q_BYTES + h * SLAB_BYTES, &map_q, h * 64, 0, kvh, tok0 + t_first[t], &q_full[t]);
        }
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < nb && ok; ++j) {
          const int s = j % ST;
          ok = mbar_wait(&kv_empty[s], ((j / ST) & 1u) ^ 1u, &abort_flag);
          if (!ok) break;
          int page[2], in_page[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) {                       // two pieces of 64 keys
            const int key0 = (b_lo + j) * KB + c * 64;
            // a piece beyond the pages the request holds reads page -1: out of range, zero-filled
            page[c] = (key0 >> p.page_shift) < p.max_pages
                          ? p.block_table[(long long)slot * p.max_pages + (key0 >> p.page_shift)] : -1;
            in_page[c] = key0 & (p.page_size - 1);
          }
          unsigned char* k_dst = kv_s + s * 2 * C::KT_BYTES;
          mbar_expect_tx(&k_full[s], C::KT_BYTES);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int h = 0; h < C::SLABS; ++h)
              tma_load_4d(k_dst + h * SLAB_BYTES + c * (SLAB_BYTES / 2), &map_k, h * 64, in_page[c], kvh, page[c], &k_full[s]);
          mbar_expect_tx(&v_full[s], C::KT_BYTES);
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int h = 0; h < C::SLABS; ++h)
              tma_load_4d(k_dst + C::KT_BYTES + h * SLAB_BYTES + c * (SLAB_BYTES / 2), &map_v, h * 64, in_page[c], kvh,
                          page[c], &v_full[s]);
        }
      }
      __syncwarp();
      // The last block's V rows of positions behind the CTA's last token: their P is zero, but a page
      // that another request used before may hold anything there, and 0 * NaN is NaN.  Clear them.
      if (nb > 0) {
        const int j = nb - 1, s = j % ST;
        int done = lane == 0 ? (int)mbar_wait(&v_full[s], (j / ST) & 1u, &abort_flag) : 0;
        done = __shfl_sync(0xffffffffu, done, 0);
        const int first_row = pos_last_all - (b_lo + j) * KB + 1;       // 1..128
        if (done && first_row < KB) {
          unsigned char* v_dst = kv_s + s * 2 * C::KT_BYTES + C::KT_BYTES;
          const int per_slab = (KB - first_row) * 8;                    // 16-byte pieces
          for (int i = lane; i < per_slab * C::SLABS; i += 32) {
            const int h = i / per_slab, o = i % per_slab;
            *reinterpret_cast<uint4*>(v_dst + h * SLAB_BYTES + first_row * 128 + o * 16) = make_uint4(0, 0, 0, 0);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        if (lane == 0 && done) mbar_arrive(v_clean);
      }
    } else if (warp == 1) {
      // The whole warp walks the loop (so that control flow stays warp-uniform and addresses and
      // descriptors can live in uniform registers); one elected lane issues the MMAs and commits.
      constexpr uint32_t idesc_s = make_idesc(QM, KB);                       // A, B K-major
      constexpr uint32_t idesc_o = make_idesc(QM, 64) | (1u << 16);          // B (V) MN-major, 64 head dims per MMA
      bool ok = true;
      auto wait = [&](uint64_t* bar, uint32_t parity) {
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, &abort_flag));
        return ok;
      };
      const uint64_t q_desc = make_desc(smem_u32(q_s)), kv_desc = make_desc(smem_u32(kv_s));
      const uint64_t v_desc = make_desc_mn(smem_u32(kv_s) + C::KT_BYTES, 16, 1024);
      auto issue_s = [&](int t, int j) {
        const int s = j % ST;
        if (!wait(&k_full[s], (j / ST) & 1u)) return;
        tc_fence_after();
        if (elect_one()) {
          // descriptor addresses count 16-byte units
          const uint64_t dq = q_desc + (uint64_t)(t * (C::Q_BYTES >> 4)), dk = kv_desc + (uint64_t)(s * (2 * C::KT_BYTES >> 4));
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            // 16 head dims = 32 bytes further along a slab's rows; the next slab after four of them
            const uint32_t off = (ks / 4) * (SLAB_BYTES >> 4) + 2 * (ks % 4);
            tc_mma(tmem_base + C::S_COL + t * KB, dq + off, dk + off, idesc_s, ks != 0);
          }
          tc_commit(&s_full[t]);
        }
        __syncwarp();
      };
      auto issue_pv = [&](int t, int j) {
        const int s = j % ST;
        if (!wait(&p_full[t], j & 1u)) return;
        if (!wait(&v_full[s], (j / ST) & 1u)) return;
        if (j == nb - 1 && !wait(v_clean, 0)) return;
        tc_fence_after();
        if (elect_one()) {
          const uint64_t dv = v_desc + (uint64_t)(s * (2 * C::KT_BYTES >> 4));
          const uint32_t acc = j > 0 ? 1u : 0u;
#pragma unroll
          for (int kk = 0; kk < KB / 16; ++kk) {
            // P: 16 keys = 8 columns of packed bf16 further; V: 16 keys = two 8-row groups of 1024 bytes
#pragma unroll
            for (int h = 0; h < C::SLABS; ++h)
              tc_mma_ts(tmem_base + C::O_COL + t * HD + h * 64, tmem_base + C::P_COL + t * C::P_STRIDE + kk * 8,
                        dv + (uint64_t)(h * (SLAB_BYTES >> 4) + kk * (2048 >> 4)), idesc_o, kk != 0 ? 1u : acc);
          }
          tc_commit(&o_done[t]);
        }
        __syncwarp();
      };
#pragma unroll
      for (int t = 0; t < NT; ++t)
        if (nb_t[t] > 0) wait(&q_full[t], 0);
#pragma unroll
      for (int t = 0; t < NT; ++t)
        if (nb_t[t] > 0 && ok) issue_s(t, 0);
#pragma unroll 1
      for (int j = 0; j < nb && ok; ++j) {
        if (C::SEP_P) {
          // the next S_t as soon as the softmax threads have taken this one out of tensor memory
#pragma unroll
          for (int t = 0; t < NT; ++t)
            if (j + 1 < nb_t[t] && wait(&s_free[t], j & 1u)) issue_s(t, j + 1);
#pragma unroll
          for (int t = 0; t < NT; ++t)
            if (j < nb_t[t] && ok) issue_pv(t, j);
        } else {
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            if (j < nb_t[t] && ok) issue_pv(t, j);
            if (j + 1 < nb_t[t] && ok) issue_s(t, j + 1);
          }
        }
        if (ok && elect_one()) tc_commit(&kv_empty[j % ST]);
        __syncwarp();
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int t = (warp - 4) >> 2;                          // the tile this warpgroup serves
    const int quad = warp & 3;                              // the 32 TMEM lanes this warp may touch
    const int row = quad * 32 + lane;                       // tile row = TMEM lane
    const int my_nb = nb_t[t];
    const int rows_used = max(t_count[t], 0) * p.group;
    const bool valid = row < rows_used;
    const int pos_first = before + t_first[t];
    // rows past the tile's tokens compute like its last row and are never stored
    const int pos = pos_first + (valid ? row / p.group : max(t_count[t] - 1, 0));
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + C::S_COL + t * KB, o_addr = lane_addr + C::O_COL + t * HD;
    const uint32_t p_addr = lane_addr + C::P_COL + t * C::P_STRIDE;
    const float c_log2 = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    // With S_t ready ahead of time the two tiles' softmax threads would run in step and meet in the
    // special-function unit while the other pipes idle, then leave it idle together.  Tile 1 starts
    // its first exponentials when tile 0 has finished its own, which puts the two half a block apart:
    // one tile's exponentials then run beside the other's loads, maxima and waits.
    const int nb_turns = (C::SEP_P && NT == 2) ? min(1, min(nb_t[0], nb_t[NT - 1])) : 0;
    if (t == 1 && nb_turns > 0) {
      __syncwarp();
      if (lane == 0) mbar_arrive(&turn[0]);                // tile 0 begins
    }

    // every lane of a warp must take the same path around the warp-wide TMEM accesses, also when a
    // wait gives up
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {       // no lane goes on alone
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, &abort_flag)) != 0;
    };

#pragma unroll 1
    for (int j = 0; j < my_nb && ok; ++j) {
      const int key0 = (b_lo + j) * KB;
      ok = wait_all(&s_full[t], j & 1u);
      tc_fence_after();
      if (!ok) break;
      float v[KB];
#pragma unroll
      for (int ch = 0; ch < KB / 32; ++ch) tc_ld32(s_addr + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[ch * 32]));
      tc_wait_ld();
      if (C::SEP_P) {                      // S_t is in registers: the MMA warp may compute the next one
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[t]);
      }
      // keys this row may see: [key_min, pos]; blocks wholly inside need no per-element test
      const int key_min = p.window > 0 ? pos - p.window + 1 : -(1 << 30);
      const bool need_mask = __any_sync(0xffffffffu, key0 + KB - 1 > pos || key0 < key_min);
      if (need_mask) {
        const int hi = pos - key0, lo = key_min - key0;
#pragma unroll
        for (int i = 0; i < KB; ++i) v[i] = (i <= hi && i >= lo) ? v[i] : -INFINITY;
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < KB; i += 8) {
        mx[0] = max3(mx[0], v[i], v[i + 1]);
        mx[1] = max3(mx[1], v[i + 2], v[i + 3]);
        mx[2] = max3(mx[2], v[i + 4], v[i + 5]);
        mx[3] = max3(mx[3], v[i + 6], v[i + 7]);
      }
      const float m_new = fmaxf(max3(mx[0], mx[1], mx[2]), fmaxf(mx[3], m_run));
      // move the maximum only when it grew by more than 2^RESCALE_LOG2 (always from -inf)
      const bool grow = (m_new - m_run) * c_log2 > RESCALE_LOG2;
      bool o_waited = false;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2((m_run - m_use) * c_log2);       // 0 from -inf
        m_run = m_new;
        l_run *= alpha;
        if (j > 0) {                                   // O_t holds the blocks before this one: rescale its rows
          ok = wait_all(&o_done[t], (j - 1) & 1u);
          tc_fence_after();
          if (!ok) break;
          o_waited = true;
#pragma unroll
          for (int ch = 0; ch < HD / 32; ++ch) {
            uint32_t o[32];
            tc_ld32(o_addr + ch * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tc_st32(o_addr + ch * 32, o);
          }
        }
      }
      if (C::SEP_P && j > 0 && !o_waited) {            // the MMA that read the last P_t must be through with it
        ok = wait_all(&o_done[t], (j - 1) & 1u);
        tc_fence_after();
        if (!ok) break;
      }
      if (j < nb_turns) {
        ok = wait_all(&turn[t], j & 1u);
        if (!ok) break;
      }
      const float neg_mc = m_run == -INFINITY ? 0.f : -m_run * c_log2;
      const float2 c2 = make_float2(c_log2, c_log2), n2 = make_float2(neg_mc, neg_mc);
      float2 ls[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int ch = 0; ch < KB / 64; ++ch) {             // 64 keys = 32 columns of packed bf16 per store
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float2 x = fma2(make_float2(v[ch * 64 + i], v[ch * 64 + i + 1]), c2, n2);
          const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          ls[(i >> 1) & 1] = add2(ls[(i >> 1) & 1], e);
          __nv_bfloat162 b = __floats2bfloat162_rn(e.x, e.y);
          packed[i / 2] = *reinterpret_cast<uint32_t*>(&b);
        }
        tc_st32(p_addr + ch * 32, packed);
      }
      l_run += (ls[0].x + ls[0].y) + (ls[1].x + ls[1].y);
      if (j < nb_turns) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&turn[NT - 1 - t]);
      }
      // P (and a rescaled O) must have landed in tensor memory before the MMA is told
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }

    if (ok && my_nb > 0) {
      ok = wait_all(&o_done[t], (my_nb - 1) & 1u);
      tc_fence_after();
    }
    if (ok && my_nb > 0) {
      const int tk = t_first[t] + row / p.group, head = kvh * p.group + row % p.group;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = p.out + (long long)(tok0 + tk) * p.ld_o + (long long)head * HD;
#pragma unroll
      for (int ch = 0; ch < HD / 32; ++ch) {
        uint32_t o[32];
        tc_ld32(o_addr + ch * 32, o);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
            uint4 w;
            __nv_bfloat162 b0 = __floats2bfloat162_rn(__uint_as_float(o[d]) * inv, __uint_as_float(o[d + 1]) * inv);
            __nv_bfloat162 b1 = __floats2bfloat162_rn(__uint_as_float(o[d + 2]) * inv, __uint_as_float(o[d + 3]) * inv);
            __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(o[d + 4]) * inv, __uint_as_float(o[d + 5]) * inv);
            __nv_bfloat162 b3 = __floats2bfloat162_rn(__uint_as_float(o[d + 6]) * inv, __uint_as_float(o[d + 7]) * inv);
            w.x = *reinterpret_cast<uint32_t*>(&b0); w.y = *reinterpret_cast<uint32_t*>(&b1);
            w.z = *reinterpret_cast<uint32_t*>(&b2); w.w = *reinterpret_cast<uint32_t*>(&b3);
            *reinterpret_cast<uint4*>(dst + ch * 32 + d) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 400; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 2);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
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

template <int HD, int NT>
int launch_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, TcAttnParams p, int kv_heads,
              int requests, int* status, cudaStream_t stream) {
  using C = TcCfg<HD, NT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tc_kernel<HD, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
    if (e != cudaSuccess)
      return hfee_fail(HFEE_ERR_CUDA, "attention_tc: cannot get %d bytes of shared memory: %s", C::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  p.q_groups = (p.q_tiles + NT - 1) / NT;
  dim3 grid((unsigned)kv_heads, (unsigned)p.q_groups, (unsigned)requests);
  hfee_launch(attention_tc_kernel<HD, NT>, grid, dim3(C::THREADS), C::SMEM, stream, mq, mk, mv, p, status);
  return hfee_check_launch("attention_tc");
}

}  // namespace

// 1 if hfee_attention_tc takes this shape (bfloat16 is implied).
HFEE_API int hfee_attention_tc_supports(int heads, int kv_heads, int head_dim, int page_size) {
  if ((head_dim != 64 && head_dim != 128) || kv_heads <= 0 || heads % kv_heads != 0) return 0;
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
               "attention_tc: needs head_dim 64 or 128, at most 128 query heads per kv head and power-of-two pages "
               ">= 64 (got head_dim %d, heads %d/%d, page_size %d)", head_dim, heads, kv_heads, page_size);
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
  p.q_groups = 0;

  CUtensorMap mq, mk, mv;
  {
    // q as [token][kv head][head of group][d]; a box is (tokens_per_tile x group) rows of 64 d
    const cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)group, (cuuint64_t)kv_heads, (cuuint64_t)n_tokens};
    const cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)group * head_dim * 2, (cuuint64_t)ld_q * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)group, 1, (cuuint32_t)p.tokens_per_tile};
    int rc = make_map_4d(&mq, q, dims, strides, box);
    if (rc != HFEE_OK) return rc;
  }
  {
    const cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2,
                                   (cuuint64_t)kv_heads * page_size * head_dim * 2};
    const cuuint32_t box[4] = {64, 64, 1, 1};
    int rc = make_map_4d(&mk, k_pool, dims, strides, box);
    if (rc != HFEE_OK) return rc;
    rc = make_map_4d(&mv, v_pool, dims, strides, box);
    if (rc != HFEE_OK) return rc;
  }
  if (head_dim == 64) return launch_tc<64, 2>(mq, mk, mv, p, kv_heads, requests, status, stream);
  return launch_tc<128, 2>(mq, mk, mv, p, kv_heads, requests, status, stream);
}
