// out[M,N] (+)= A[M,K] . W[N,K]^T on the 5th-generation tensor cores: bfloat16 operands
// staged in shared memory by TMA (128-byte swizzle, no multicast), tcgen05.mma issued by
// one thread with the float32 accumulator in tensor memory, tcgen05.ld for the epilogue.
//
// The grid is persistent: CTA b computes the 128 x BN tiles (BN = 128, 192 or 256) b, b + gridDim.x,
// ... (M tiles fastest, so CTAs running together share a W tile in L2), K in blocks of 64, with
// two accumulators in tensor memory so that a tile's epilogue overlaps the next tile's MMAs:
//   warp 0     TMA producer   waits empty[s], arms full[s] with the stage's bytes, issues 2 loads
//   warp 1     MMA issuer     allocates TMEM; per tile waits tmem_empty[buf]; per K block waits
//                             full[s], issues 4 MMAs (K = 16 each), commits to empty[s]; after
//                             the tile's last block commits to tmem_full[buf]
//   warps 2-9  epilogue       wait tmem_full[buf]; warp w reads TMEM lanes 32*(w%4).. of one half
//                             of the columns, writes C, arrives on tmem_empty[buf]
// Tiles at the edges rely on TMA's zero fill for loads and on predicates for stores; K may
// be any multiple of 8 (16-byte row pitch), its tail is zero-filled too.
//
// When there are tiles for fewer than half of the SMs (prompt portions of a few hundred tokens)
// the launch splits the work by K blocks: the (tile, K block) pairs in tile order are cut into one
// contiguous range per CTA, equal to within one block, a whole number of ranges per tile.  A range
// that starts inside a tile computes that tile's remaining K blocks first, writes the float32 partial
// tile to its own slot of a workspace and raises the slot's flag; the CTA whose range holds the tile's
// first K block computes that part last, adds the partial tiles of the following CTAs in CTA order (a
// fixed order) and runs the epilogue.  Contributions are therefore written at the start of a CTA's
// work and consumed at the end of another's; the consumer's wait on the flag is bounded like every
// other wait, and the last consumer warp clears the flag for the next launch.
//
// Every mbarrier wait is bounded: a wait that runs out sets an abort flag that ends all
// other waits of the CTA, records a code in `status` and lets the CTA free its tensor
// memory and return.
// Reference: out[t*Rows+r] = Dot(W[r,:], x[t,:]), hostfog/hfee internal/ggml/ops.go:54-70.
#include "tcgen05.cuh"
#include "rope_epilogue.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int TC_THREADS = 320;       // 1 TMA warp, 1 MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int ACC_STAGES = 2;
constexpr int SK_MAX_PIECES = 4;      // a tile is cut into at most this many ranges of K blocks

enum Epilogue { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_ROPE = 3 };

template <int BN> struct TileCfg {
  static constexpr int STAGES = BN == 128 ? 6 : 4;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int W_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
  static constexpr int EPI_BYTES = EPI_WARPS * 32 * 128;        // accumulate epilogue: a 32 x 32 float chunk per warp
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + EPI_BYTES;      // + slack to align the base to 1024
};

template <int BN, int EPI, typename TOut>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_c, int reduce_by_tma,
               TOut* __restrict__ C, long long ldc, int M, int N, int K, int* __restrict__ status,
               float* __restrict__ sk_parts, int* __restrict__ sk_flags, const RopeEpi rope) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t TMEM_COLS = ACC_STAGES * BN <= 256 ? 256 : 512;      // a power of two
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[ACC_STAGES];
  __shared__ __align__(8) uint64_t tmem_empty_bar[ACC_STAGES];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* epi_stage = tiles + STAGES * Cfg::STAGE_BYTES;      // 1024-aligned: the tiles are whole KBs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + BK - 1) / BK;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  // This CTA's work as a sequence of segments (tile, first K block, end K block): whole tiles
  // b, b + gridDim.x, ... or, split by K blocks, the range [u_begin, u_end) of (tile, K block) pairs.
  const bool stream_k = sk_parts != nullptr;
  const long long total_units = (long long)total_tiles * k_blocks;
  auto range_begin = [&](long long cta) { return cta * total_units / (long long)gridDim.x; };
  struct Walk { long long u, u_end; int t, stride, tiles, k_blocks; bool stream_k; };
  auto walk_start = [&]() {
    Walk w;
    w.stream_k = stream_k; w.k_blocks = k_blocks; w.tiles = total_tiles; w.stride = gridDim.x; w.t = blockIdx.x;
    w.u = stream_k ? range_begin(blockIdx.x) : 0;
    w.u_end = stream_k ? range_begin((long long)blockIdx.x + 1) : 0;
    return w;
  };
  auto walk_next = [](Walk& w, int& t, int& kb0, int& kb1) {
    if (w.stream_k) {
      if (w.u >= w.u_end) return false;
      t = (int)(w.u / w.k_blocks);
      kb0 = (int)(w.u - (long long)t * w.k_blocks);
      const long long left = w.u_end - w.u;
      kb1 = (long long)(w.k_blocks - kb0) <= left ? w.k_blocks : kb0 + (int)left;
      w.u += kb1 - kb0;
      return true;
    }
    if (w.t >= w.tiles) return false;
    t = w.t; kb0 = 0; kb1 = w.k_blocks;
    w.t += w.stride;
    return true;
  };

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], EPI_WARPS); }
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
  // barriers and tensor memory are set up while the previous kernel may still run; its output
  // (A, and C when accumulating) is touched only from here on
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // Producer and MMA warps walk their loops as whole warps: control flow stays warp-uniform, so
    // addresses and descriptors can be kept in uniform registers, and one elected lane issues.
    uint32_t it = 0;                           // K blocks issued so far, over all segments
    bool ok = true;
    Walk w = walk_start();
    int t, kb0, kb1;
    while (ok && walk_next(w, t, kb0, kb1)) {
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, &abort_flag));
        if (!ok) break;
        if (elect_one()) {
          unsigned char* a_dst = tiles + s * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, kb * BK, m0, &full_bar[s]);
          tma_load_2d(a_dst + Cfg::A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc = make_idesc(BM, BN);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    Walk w = walk_start();
    int t, kb0, kb1;
    const uint64_t desc0 = make_desc(smem_u32(tiles));
    for (; ok && walk_next(w, t, kb0, kb1); ++acc_it) {
      const uint32_t buf = acc_it & 1u;
      // the epilogue has drained this accumulator
      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty_bar[buf], ((acc_it >> 1) & 1u) ^ 1u, &abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + buf * BN;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], (it / STAGES) & 1u, &abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          // descriptor addresses count 16-byte units
          const uint64_t da = desc0 + (uint64_t)(s * (Cfg::STAGE_BYTES >> 4)), dw = da + (uint64_t)(Cfg::A_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)       // 16 bf16 = 32 bytes further along K: +2 in 16-byte units
            tc_mma(tmem_d, da + 2 * k, dw + 2 * k, idesc, kb > kb0 || k != 0);
          tc_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (ok && elect_one()) tc_commit(&tmem_full_bar[buf]);
      __syncwarp();
    }
  } else {
    // epilogue warp w may read TMEM lanes 32*(w%4) .. +31 (= tile rows of the same numbers); the
    // two warps that share a lane quadrant take one half of the columns each
    const int quad = warp & 3, half = (warp - 2) >> 2;
    constexpr int CHUNKS = BN / 32 / 2;          // 32-column chunks per warp
    uint32_t acc_it = 0;
    bool ok = true;
    Walk w = walk_start();
    int t, kb0, kb1;
    for (; ok && walk_next(w, t, kb0, kb1); ++acc_it) {
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      const uint32_t buf = acc_it & 1u;
      ok = mbar_wait(&tmem_full_bar[buf], (acc_it >> 1) & 1u, &abort_flag);
      tc_fence_after();
      if (!ok) break;
      const int row = m0 + quad * 32 + lane;
      // split by K blocks: a segment that lacks the tile's first K block hands its partial tile over;
      // one that has it but not the last adds the partial tiles of the CTAs after this one
      const bool contribute = kb0 > 0;
      int parts = 0;
      if (kb0 == 0 && kb1 < k_blocks) {
        const long long tile_end = (long long)(t + 1) * k_blocks;
        while (parts < SK_MAX_PIECES - 1 && blockIdx.x + parts + 1 < gridDim.x &&
               range_begin((long long)blockIdx.x + parts + 1) < tile_end) ++parts;
        for (int pi = 1; pi <= parts && ok; ++pi) {
          int ready = 0;
          if (lane == 0) {
            const volatile int* flag = sk_flags + 2 * (blockIdx.x + pi);
            for (int spin = 0; spin < (1 << 20) && !ready && !*(volatile int*)&abort_flag; ++spin) {
              ready = *flag >= EPI_WARPS;
              if (!ready) __nanosleep(200);
            }
            if (!ready) abort_flag = 1;
          }
          ok = __shfl_sync(0xffffffffu, ready, 0) != 0;
        }
        __threadfence();                          // the partial tiles were written before their flags
        if (!ok) break;
      }
      // partial tiles are stored column by column (element (row, col) at col * 128 + row): a warp's
      // 32 rows of one column are 128 contiguous bytes
      float* my_part = contribute ? sk_parts + (long long)blockIdx.x * (BM * BN) + (quad * 32 + lane) : nullptr;
      if constexpr (EPI == EPI_ROPE) {
        rope_epilogue<BN>(rope, tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16), half, row, M, N, n0);
      } else {
#pragma unroll 1
      for (int cc = 0; cc < CHUNKS; ++cc) {
        const int ch = half * CHUNKS + cc;
        uint32_t v[32];
        tc_ld32(tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ch * 32), v);
        tc_wait_ld();
        if (contribute) {
#pragma unroll
          for (int j = 0; j < 32; ++j) my_part[(ch * 32 + j) * BM] = __uint_as_float(v[j]);
          continue;
        }
        if (parts > 0) {
          // all the partial tiles' values of this chunk are requested before the first is added
          const float* src = sk_parts + (long long)(blockIdx.x + 1) * (BM * BN) + (long long)(ch * 32) * BM + (quad * 32 + lane);
          float x[SK_MAX_PIECES - 1][32];
#pragma unroll
          for (int pi = 0; pi < SK_MAX_PIECES - 1; ++pi)
            if (pi < parts) {
#pragma unroll
              for (int j = 0; j < 32; ++j) x[pi][j] = __ldcg(src + (long long)pi * (BM * BN) + j * BM);
            }
#pragma unroll
          for (int pi = 0; pi < SK_MAX_PIECES - 1; ++pi)
            if (pi < parts) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + x[pi][j]);
            }
        }
        const int col0 = n0 + ch * 32;
        if constexpr (EPI == EPI_ACCUM) {
          if (reduce_by_tma) {
            // The chunk goes to shared memory (thread = row, 128 bytes, in the 128-byte swizzle the
            // tensor map of C expects) and from there into C by a bulk tensor reduction: the addition
            // happens in the memory system, nothing of C is read here, and rows or columns beyond the
            // matrix are clipped by the copy.
            const int row0 = m0 + quad * 32;
            if (row0 >= M || col0 >= N) continue;                      // the same for the whole warp
            unsigned char* cs = epi_stage + (warp - 2) * 4096;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous chunk has left the buffer
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(cs + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                  make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(reinterpret_cast<uint64_t>(&map_c)), "r"(col0), "r"(row0), "r"(smem_u32(cs)) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            continue;
          }
        }
        if (row >= M || col0 >= N) continue;
        if constexpr (EPI == EPI_SWIGLU) {
          // columns in groups of 8 = [4 gate | 4 up] -> 4 outputs per group at column col/2
          TOut* dst = C + (long long)row * ldc + col0 / 2;
          float o[16];
#pragma unroll
          for (int gq = 0; gq < 4; ++gq)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float gate = __uint_as_float(v[gq * 8 + i]), up = __uint_as_float(v[gq * 8 + 4 + i]);
              o[gq * 4 + i] = __fdividef(gate, 1.f + __expf(-gate)) * up;
            }
          if (col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              uint4 pk;
              __nv_bfloat162 p0 = __floats2bfloat162_rn(o[j], o[j + 1]), p1 = __floats2bfloat162_rn(o[j + 2], o[j + 3]);
              __nv_bfloat162 p2 = __floats2bfloat162_rn(o[j + 4], o[j + 5]), p3 = __floats2bfloat162_rn(o[j + 6], o[j + 7]);
              pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
              pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst) + j) = pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (col0 + (j / 4) * 8 + (j % 4) + 4 < N) dst[j] = from_f32<TOut>(o[j]);
          }
        } else {
          TOut* dst = C + (long long)row * ldc + col0;
          const bool full = col0 + 32 <= N && (((uintptr_t)dst) & 15) == 0;
          if (full) {
            if constexpr (sizeof(TOut) == 4) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                       __uint_as_float(v[j + 3]));
                if constexpr (EPI == EPI_ACCUM) {
                  float4 c = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(dst) + j);
                  o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                }
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + j) = o;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
                o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst) + j) = o;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j >= N) continue;
              float o = __uint_as_float(v[j]);
              if constexpr (EPI == EPI_ACCUM) o += to_f32<TOut>(dst[j]);
              dst[j] = from_f32<TOut>(o);
            }
          }
        }
      }
      }
      // this warp's reads of the accumulator are complete: hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
      if (contribute) {
        __threadfence();                          // this warp's part of the partial tile before its flag
        __syncwarp();
        if (lane == 0) atomicAdd(sk_flags + 2 * blockIdx.x, 1);
      } else if (parts > 0) {
        __syncwarp();
        if (lane == 0) {
          for (int pi = 1; pi <= parts; ++pi) {
            int* flag = sk_flags + 2 * (blockIdx.x + pi);
            if (atomicAdd(flag + 1, 1) == EPI_WARPS - 1) {          // the last warp to have read it clears the slot
              flag[0] = 0;
              flag[1] = 0;
            }
          }
        }
      }
    }
  }

  if constexpr (EPI == EPI_ACCUM) {
    // bulk reductions of this thread are complete (not merely read out of shared memory) before the CTA ends
    if (reduce_by_tma && warp >= 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // loads that were issued may still be landing in this CTA's shared memory: give them time
#pragma unroll 1
    for (int i = 0; i < 400; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------- host
// Whether to split by K blocks, and over how many CTAs.  Only when whole tiles would leave at
// least half of the SMs idle: CTAs that work on one panel of A or W at different K positions lose
// the sharing of those loads in L2 (measured: with 148 staggered ranges a K block took three times
// as long), so every tile is cut into the same number of (nearly) equal pieces, which keeps the
// CTAs of one piece index in step, and tiles that fill most SMs are left whole.
int plan_stream_k(long long tiles, int k_blocks, int sms, long long workspace_floats, int bn) {
  if (tiles * 2 > sms || k_blocks < 64) return 0;            // a short K gains less than the hand-over costs
  long long pieces = sms / tiles < SK_MAX_PIECES ? sms / tiles : SK_MAX_PIECES;
  while (pieces > 1 && k_blocks / pieces < 8) --pieces;       // at least 8 K blocks per piece
  const long long ctas = tiles * pieces;
  if (pieces < 2 || workspace_floats < ctas * (long long)BM * bn) return 0;
  return (int)ctas;
}

// Tensor map of the float32 output for the bulk reduction of 32 x 32 chunks (128-byte rows, swizzled).
int make_map_c(CUtensorMap* map, void* base, long long rows, long long cols, long long ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05: cuTensorMapEncodeTiled (output) failed with %d", (int)r);
  return HFEE_OK;
}

template <int BN, int EPI, typename TOut>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, long long ldc, int M, int N, int K, int* status,
           float* workspace, long long workspace_floats, int* flags, cudaStream_t stream, const RopeEpi& rope = RopeEpi{}) {
  using Cfg = TileCfg<BN>;
  // accumulate: by bulk tensor reduction when C can have a tensor map (16-byte aligned base and pitch)
  CUtensorMap mc = ma;
  int reduce_by_tma = 0;
  if (EPI == EPI_ACCUM && (uintptr_t)C % 16 == 0 && ldc % 4 == 0) {
    int rc = make_map_c(&mc, C, M, N, ldc);
    if (rc != HFEE_OK) return rc;
    reduce_by_tma = 1;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05: cannot get %d bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const int sms = hfee_sm_count();
  if (sms <= 0) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05: cannot ask the device for its number of SMs");
  long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int sk_ctas = (workspace && flags) ? plan_stream_k(tiles, (K + BK - 1) / BK, sms, workspace_floats, BN) : 0;
  dim3 grid((unsigned)(sk_ctas ? sk_ctas : (tiles < sms ? tiles : sms)));          // one CTA per SM
  hfee_launch(gemm_tc_kernel<BN, EPI, TOut>, dim3(grid), dim3(TC_THREADS), Cfg::SMEM, stream, ma, mw, mc, reduce_by_tma, (TOut*)C, ldc, M, N, K, status,
              sk_ctas ? workspace : (float*)nullptr, sk_ctas ? flags : (int*)nullptr, rope);
  return hfee_check_launch("gemm_tcgen05");
}

template <int BN>
int dispatch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, long long ldc, int out_dtype, int epilogue, int M,
             int N, int K, int* status, float* ws, long long ws_floats, int* flags, cudaStream_t stream) {
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_tcgen05: accumulate needs a float32 output");
    return launch<BN, EPI_ACCUM, float>(ma, mw, C, ldc, M, N, K, status, ws, ws_floats, flags, stream);
  }
  if (epilogue == EPI_SWIGLU) {
    if (out_dtype != HFEE_BF16) return hfee_fail(HFEE_ERR_ARG, "gemm_tcgen05: the SwiGLU epilogue writes bfloat16");
    return launch<BN, EPI_SWIGLU, __nv_bfloat16>(ma, mw, C, ldc, M, N, K, status, ws, ws_floats, flags, stream);
  }
  if (out_dtype == HFEE_BF16) return launch<BN, EPI_STORE, __nv_bfloat16>(ma, mw, C, ldc, M, N, K, status, ws, ws_floats, flags, stream);
  return launch<BN, EPI_STORE, float>(ma, mw, C, ldc, M, N, K, status, ws, ws_floats, flags, stream);
}

}  // namespace

// A, W: bfloat16, 16-byte aligned, leading dimensions multiples of 8.  epilogue: 0 store, 1 accumulate
// into float32 C, 2 SwiGLU over W rows interleaved [4 gate | 4 up] (C is [M, N/2] bfloat16).
// `status` (device int, may be null) is set to 1 if a CTA gave up waiting.  block_n: 128, 192 or 256.
// `workspace` (float32, 16-byte aligned, may be null) and `flags` (2 ints per SM, zero before the
// first use; every launch leaves them zero) allow the split by K blocks: it is used when it pays and
// the workspace holds one 128 x block_n tile per CTA.
HFEE_API int hfee_gemm_tcgen05(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                               int out_dtype, int epilogue, int M, int N, int K, int block_n, int* status,
                               float* workspace, long long workspace_floats, int* flags, cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "gemm_tcgen05: K=%d must be a positive multiple of 8", K);
  HFEE_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K,
               "gemm_tcgen05: leading dimensions (%lld, %lld) must be multiples of 8 and at least K", lda, ldw);
  HFEE_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tcgen05: operands must be 16-byte aligned");
  HFEE_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05: unknown epilogue %d", epilogue);
  HFEE_REQUIRE(epilogue != EPI_SWIGLU || N % 8 == 0, "gemm_tcgen05: SwiGLU needs N %% 8 == 0, got %d", N);
  HFEE_REQUIRE(ldc >= (epilogue == EPI_SWIGLU ? N / 2 : N), "gemm_tcgen05: ldc=%lld is too small", ldc);
  HFEE_REQUIRE(block_n == 128 || block_n == 192 || block_n == 256, "gemm_tcgen05: block_n must be 128, 192 or 256");
  HFEE_REQUIRE((long long)((M + BM - 1) / BM) * ((N + block_n - 1) / block_n) < (1ll << 31), "gemm_tcgen05: too many tiles");
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc != HFEE_OK) return rc;
  rc = make_map(&mw, W, N, K, ldw, block_n);
  if (rc != HFEE_OK) return rc;
  HFEE_REQUIRE((uintptr_t)workspace % 16 == 0, "gemm_tcgen05: the workspace must be 16-byte aligned");
  if (block_n == 256) return dispatch<256>(ma, mw, C, ldc, out_dtype, epilogue, M, N, K, status, workspace, workspace_floats, flags, stream);
  if (block_n == 192) return dispatch<192>(ma, mw, C, ldc, out_dtype, epilogue, M, N, K, status, workspace, workspace_floats, flags, stream);
  return dispatch<128>(ma, mw, C, ldc, out_dtype, epilogue, M, N, K, status, workspace, workspace_floats, flags, stream);
}

// How many CTAs hfee_gemm_tcgen05 would split this shape's K blocks among (0: whole tiles per CTA).
HFEE_API int hfee_gemm_tcgen05_stream_k(int M, int N, int K, int block_n, long long workspace_floats) {
  const int sms = hfee_sm_count();
  if (sms <= 0) return 0;
  long long tiles = (long long)((M + BM - 1) / BM) * ((N + block_n - 1) / block_n);
  return plan_stream_k(tiles, (K + BK - 1) / BK, sms, workspace_floats, block_n);
}

int hfee_gemm_pair_rope(const void* A, long long lda, const void* W, long long ldw, int M, int N, int K,
                        const tc::RopeEpi& rope, int block_n, int* status, cudaStream_t stream);      // gemm_tcgen05_pair.cu

// 1 if hfee_gemm_tcgen05_rope takes these head sizes (bfloat16 implied): heads of 64 or 128 dims, all
// of them rotated.
HFEE_API int hfee_gemm_tcgen05_rope_supports(int head_dim, int rope_dim) {
  return (head_dim == 64 || head_dim == 128) && rope_dim == head_dim ? 1 : 0;
}

// The q/k/v projection of prompt tokens with rotation and cache write in its epilogue (see RopeEpi):
// A [M, K] tokens, W [N, K] with N = (heads + 2 kv_heads) * head_dim rows [q heads | k heads | v heads],
// or N = heads * head_dim and null pools for a run that reads another run's cache.  cs [M, head_dim/2]
// (cos, sin) pairs or null; queries go to q_out [M, ld_q], keys and values to the pages of
// (slot_of_token, positions).
HFEE_API int hfee_gemm_tcgen05_rope(const void* A, long long lda, const void* W, long long ldw, int M, int N, int K,
                                    const float* cs, const int* positions, const int* slot_of_token, void* q_out,
                                    long long ld_q, void* k_pool, void* v_pool, const int* block_table, int max_pages,
                                    int page_size, int heads, int kv_heads, int head_dim, int interleaved, int* status,
                                    cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(hfee_gemm_tcgen05_rope_supports(head_dim, head_dim), "gemm_tcgen05_rope: head_dim %d is not 64 or 128", head_dim);
  HFEE_REQUIRE(M > 0 && K > 0 && K % 8 == 0, "gemm_tcgen05_rope: K=%d must be a positive multiple of 8", K);
  HFEE_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0,
               "gemm_tcgen05_rope: operands must be 16-byte aligned with leading dimensions that are multiples of 8 and at least K");
  HFEE_REQUIRE((k_pool == nullptr) == (v_pool == nullptr), "gemm_tcgen05_rope: key and value pools go together");
  HFEE_REQUIRE(N == (heads + (k_pool ? 2 * kv_heads : 0)) * head_dim, "gemm_tcgen05_rope: N=%d is not the width of the heads", N);
  HFEE_REQUIRE(ld_q % 8 == 0 && ld_q >= (long long)heads * head_dim && (uintptr_t)q_out % 16 == 0 &&
               (uintptr_t)k_pool % 16 == 0 && (uintptr_t)v_pool % 16 == 0 && (uintptr_t)cs % 16 == 0,
               "gemm_tcgen05_rope: outputs and the table must be 16-byte aligned");
  RopeEpi rope;
  rope.cs = (const float2*)cs; rope.positions = positions; rope.slot_of_token = slot_of_token;
  rope.q_out = (__nv_bfloat16*)q_out; rope.ld_q = ld_q;
  rope.k_pool = (__nv_bfloat16*)k_pool; rope.v_pool = (__nv_bfloat16*)v_pool;
  HFEE_REQUIRE(make_paged_cache(&rope.cache, block_table, max_pages, page_size, kv_heads, head_dim),
               "gemm_tcgen05_rope: page_size %d must be a power of two", page_size);
  rope.heads = heads; rope.kv_heads = kv_heads; rope.head_dim = head_dim; rope.interleaved = interleaved;
  // tiles of whole heads: 256 columns, or 128 where those fill the SMs better
  const int sms = hfee_sm_count();
  const long long tiles_256 = (long long)((M + BM - 1) / BM) * ((N + 255) / 256);
  // pairs of CTAs on tiles of 256 x 256 where those make two rounds or more (the q/k/v product of the
  // benchmark model at 2,048 tokens has 96 of them for 74 pairs: the single-CTA tiles fill the SMs better)
  if (sms > 0 && M > BM && (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256) >= 2 * (sms / 2))
    return hfee_gemm_pair_rope(A, lda, W, ldw, M, N, K, rope, 256, status, stream);
  if (sms > 0 && M > BM && head_dim == 64 && N % 192 == 0) {
    // pairs on tiles of 256 x 192 (three heads) where those fill their rounds to four fifths or more: the
    // q/k/v product of the benchmark model at 2,048 tokens has 128 of them for 74 pairs (prompt pass 3.76 -> 3.69 ms)
    const long long pairs = sms / 2, tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * (N / 192);
    const long long rounds = (tiles + pairs - 1) / pairs;
    if (tiles * 5 >= rounds * pairs * 4) return hfee_gemm_pair_rope(A, lda, W, ldw, M, N, K, rope, 192, status, stream);
  }
  int bn = tiles_256 >= 96 || sms <= 0 ? 256 : 128;
  if (bn == 256 && head_dim == 64 && sms > 0) {
    // three heads wide where that saves a round of tiles (16 x 12 tiles of 256 are two rounds on 148 SMs
    // with the second a third full; 16 x 16 tiles of 192 are two rounds of three quarters the work)
    const long long m_tiles = (M + BM - 1) / BM;
    const long long rounds_192 = (m_tiles * ((N + 191) / 192) + sms - 1) / sms, rounds_256 = (tiles_256 + sms - 1) / sms;
    if (rounds_192 * 192 * 105 < rounds_256 * 256 * 100) bn = 192;
  }
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc != HFEE_OK) return rc;
  rc = make_map(&mw, W, N, K, ldw, bn);
  if (rc != HFEE_OK) return rc;
  if (bn == 256) return launch<256, EPI_ROPE, __nv_bfloat16>(ma, mw, nullptr, 0, M, N, K, status, nullptr, 0, nullptr, stream, rope);
  if (bn == 192) return launch<192, EPI_ROPE, __nv_bfloat16>(ma, mw, nullptr, 0, M, N, K, status, nullptr, 0, nullptr, stream, rope);
  return launch<128, EPI_ROPE, __nv_bfloat16>(ma, mw, nullptr, 0, M, N, K, status, nullptr, 0, nullptr, stream, rope);
}
