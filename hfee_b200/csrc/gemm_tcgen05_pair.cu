// out (+)= A . W^T for prompt-sized A on tcgen05 with two CTAs on one tile (`cta_group::2`).
//
// Reference math: hostfog/hfee internal/ggml/ops.go:125-134 (the product), 160-165 (SwiGLU).
//
// A 128 x 256 tile per CTA (gemm_tcgen05.cu) needs 48 KB of operands for every 512 cycles of its
// tensor core, 96 B/clk, and the four stages that fit beside the epilogue's buffer hold less than the
// L2's latency asks for at that rate: the tensor pipe idled a quarter of the time.  Here the two CTAs
// of a cluster compute one 256 x 256 tile: each loads its own 128 rows of A and its own HALF of the
// 256 rows of W (32 KB per K block, 64 B/clk, six stages), one thread of the even CTA issues MMAs that
// read both CTAs' shared memory, and each CTA's tensor memory receives its own 128 rows of the result.
// No load is multicast: every CTA fetches what it needs itself.
//
//   warp 0      both CTAs: TMA producer.  The loads of both CTAs count on the even CTA's barrier.
//   warp 1      tensor-memory allocation in both CTAs; in the even CTA the MMA issuer, whose commits
//               arrive at the barriers of both CTAs
//   warps 2-9   both CTAs: epilogue of the CTA's own rows; they hand the accumulator back on the
//               even CTA's barrier
//
// Every wait has a time limit; a wait that runs out sets the status word, and the CTAs of a pair
// meet once more before they free tensor memory and leave.
#include "tcgen05.cuh"
#include "rope_epilogue.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;               // rows of A per CTA; a pair covers 256
// columns of a tile: 256, or 192 for the q/k/v product of 64-dim heads where three heads per tile save a round
constexpr int THREADS = 320;
constexpr int EPI_WARPS = 8;
constexpr int ACC_STAGES = 2;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int EPI_BYTES = EPI_WARPS * 32 * 128;
template <int BN> struct PairCfg {
  static constexpr int BNH = BN / 2;                    // rows of W each CTA loads
  static constexpr int W_BYTES = BNH * BK * 2;          // 16 KB (12 KB)
  static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + EPI_BYTES;
};

enum Epilogue { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2, EPI_ROPE = 3 };

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared-memory window, of what `local` is in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A tile into this CTA's shared memory whose bytes count on a barrier given by its address in the
// cluster's window (the even CTA's barrier, from either CTA).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// All MMAs issued so far: when they are complete, arrive at the barrier at this offset in both CTAs.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}

template <int BN, int EPI, typename TOut>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_c, int reduce_by_tma,
                 TOut* __restrict__ C, long long ldc, int M, int N, int K, int* __restrict__ status, const RopeEpi rope) {
  constexpr int BNH = PairCfg<BN>::BNH, STAGE_BYTES = PairCfg<BN>::STAGE_BYTES;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];         // used in the even CTA: both CTAs' loads of a stage
  __shared__ __align__(8) uint64_t empty_bar[STAGES];        // in each CTA: the MMAs that read the stage are done
  __shared__ __align__(8) uint64_t tmem_full_bar[ACC_STAGES];    // in each CTA: a tile's MMAs are done
  __shared__ __align__(8) uint64_t tmem_empty_bar[ACC_STAGES];   // used in the even CTA: both epilogues have read it
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  unsigned char* epi_stage = tiles + STAGES * STAGE_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                      // 0: the even CTA, which issues the MMAs
  const int k_blocks = (K + BK - 1) / BK;
  const int pair_m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
  const int total_tiles = pair_m_tiles * n_tiles;
  const int pairs = gridDim.x / 2, pair = blockIdx.x / 2;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&tmem_full_bar[a], 1); mbar_init(&tmem_empty_bar[a], 2 * EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    // one warp of each CTA of the pair: the same columns in both tensor memories
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();                 // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---- producer: this CTA's rows of A and its half of the rows of W
    uint32_t it = 0;
    bool ok = true;
    for (int t = pair; t < total_tiles && ok; t += pairs) {
      const int m0 = ((t % pair_m_tiles) * 2 + (int)rank) * BM;
      const int n0 = (t / pair_m_tiles) * BN + (int)rank * BNH;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, &abort_flag));
        if (!ok) break;
        if (elect_one()) {
          unsigned char* a_dst = tiles + s * STAGE_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, bar);
          tma_load_2d_pair(a_dst + A_BYTES, &map_w, kb * BK, n0, bar);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ---- MMA issuer of the pair: 256 x 256 x 16 per instruction, operands from both CTAs
      constexpr uint32_t idesc = make_idesc(2 * BM, BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      const uint64_t desc0 = make_desc(smem_u32(tiles));
      for (int t = pair; t < total_tiles && ok; t += pairs, ++acc_it) {
        const uint32_t buf = acc_it & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty_bar[buf], ((acc_it >> 1) & 1u) ^ 1u, &abort_flag));
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], (it / STAGES) & 1u, &abort_flag));
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            const uint64_t da = desc0 + (uint64_t)(s * (STAGE_BYTES >> 4)), dw = da + (uint64_t)(A_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc_mma_pair(tmem_d, da + 2 * k, dw + 2 * k, idesc, kb > 0 || k != 0);
            tc_commit_pair(&empty_bar[s]);
          }
          __syncwarp();
        }
        if (ok && elect_one()) tc_commit_pair(&tmem_full_bar[buf]);
        __syncwarp();
      }
    }
  } else {
    // ---- epilogue of this CTA's 128 rows: warp w reads TMEM lanes 32 (w % 4) .. + 31; the two warps
    // that share a lane quadrant take one half of the 256 columns each
    const int quad = warp & 3, half = (warp - 2) >> 2;
    constexpr int CHUNKS = BN / 32 / 2;
    const uint32_t empty_remote = map_to_cta(smem_u32(&tmem_empty_bar[0]), 0);
    uint32_t acc_it = 0;
    bool ok = true;
    for (int t = pair; t < total_tiles && ok; t += pairs, ++acc_it) {
      const int m0 = ((t % pair_m_tiles) * 2 + (int)rank) * BM, n0 = (t / pair_m_tiles) * BN;
      const uint32_t buf = acc_it & 1u;
      ok = mbar_wait(&tmem_full_bar[buf], (acc_it >> 1) & 1u, &abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      if (!ok) break;
      const int row = m0 + quad * 32 + lane;
      if constexpr (EPI == EPI_ROPE) {
        rope_epilogue<BN>(rope, tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16), half, row, M, N, n0);
      } else {
#pragma unroll 1
      for (int cc = 0; cc < CHUNKS; ++cc) {
        const int ch = half * CHUNKS + cc;
        uint32_t v[32];
        tc_ld32(tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ch * 32), v);
        tc_wait_ld();
        const int col0 = n0 + ch * 32;
        if constexpr (EPI == EPI_ACCUM) {
          if (reduce_by_tma) {
            // the chunk goes to shared memory (thread = row, 128 bytes, in the swizzle the tensor map of C
            // expects) and from there into C by a bulk tensor reduction, which clips at the matrix's edges
            const int row0 = m0 + quad * 32;
            if (row0 >= M || col0 >= N) continue;                      // the same for the whole warp
            unsigned char* cs = epi_stage + (warp - 2) * 4096;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
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
          // columns in groups of 8 = [4 gate | 4 up] -> 4 outputs per group at column col / 2
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
          if (full && sizeof(TOut) == 4) {
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
          } else if (full) {
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
      // this warp's reads of the accumulator are complete: tell the even CTA's MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(empty_remote + buf * 8);
    }
  }

  if constexpr (EPI == EPI_ACCUM) {
    // bulk reductions of this thread are complete (not merely read out of shared memory) before the CTA ends
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  // Neither CTA leaves, or frees tensor memory, while the other may still signal its barriers or its
  // MMAs read this CTA's shared memory.
  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 400; ++i) __nanosleep(1000);          // copies that may still be in flight
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 4);
  }
  cluster_sync_all();
  tc_fence_after();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

int make_map_c(CUtensorMap* map, void* base, long long rows, long long cols, long long ld) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05_pair: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05_pair: cuTensorMapEncodeTiled (output) failed with %d", (int)r);
  return HFEE_OK;
}

template <int BN, int EPI, typename TOut>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, void* C, long long ldc, int M, int N, int K, int* status,
                cudaStream_t stream, const RopeEpi& rope = RopeEpi{}) {
  CUtensorMap mc = ma;
  int reduce_by_tma = 0;
  if (EPI == EPI_ACCUM && (uintptr_t)C % 16 == 0 && ldc % 4 == 0) {
    int rc = make_map_c(&mc, C, M, N, ldc);
    if (rc != HFEE_OK) return rc;
    reduce_by_tma = 1;
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<BN>::SMEM);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05_pair: cannot get %d bytes of shared memory: %s", PairCfg<BN>::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const int sms = hfee_sm_count();
  if (sms < 2) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05_pair: cannot ask the device for its number of SMs");
  const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
  const long long pairs = tiles < sms / 2 ? tiles : sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = PairCfg<BN>::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[3];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = hfee_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const int carve = hfee_carveout();
  if (carve >= 0) {
    attr[2].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
    attr[2].val.sharedMemCarveout = (unsigned int)carve;
    cfg.numAttrs = 3;
  }
  cudaLaunchKernelEx(&cfg, gemm_pair_kernel<BN, EPI, TOut>, ma, mw, mc, reduce_by_tma, (TOut*)C, ldc, M, N, K, status, rope);
  return hfee_check_launch("gemm_tcgen05_pair");
}

}  // namespace

// As hfee_gemm_tcgen05 (A, W bfloat16, 16-byte aligned, leading dimensions multiples of 8; epilogue 0
// store, 1 accumulate into float32 C, 2 SwiGLU with a bfloat16 C of N/2 columns) with pairs of CTAs on
// tiles of 256 x 256.  `status` (device int, may be null) is set to 4 if a CTA gave up waiting.
HFEE_API int hfee_gemm_tcgen05_pair(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                                    int out_dtype, int epilogue, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "gemm_tcgen05_pair: K=%d must be a positive multiple of 8", K);
  HFEE_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K,
               "gemm_tcgen05_pair: leading dimensions (%lld, %lld) must be multiples of 8 and at least K", lda, ldw);
  HFEE_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tcgen05_pair: operands must be 16-byte aligned");
  HFEE_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05_pair: unknown epilogue %d", epilogue);
  HFEE_REQUIRE(epilogue != EPI_SWIGLU || N % 8 == 0, "gemm_tcgen05_pair: SwiGLU needs N %% 8 == 0, got %d", N);
  HFEE_REQUIRE(ldc >= (epilogue == EPI_SWIGLU ? N / 2 : N), "gemm_tcgen05_pair: ldc=%lld is too small", ldc);
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc != HFEE_OK) return rc;
  rc = make_map(&mw, W, N, K, ldw, 128);
  if (rc != HFEE_OK) return rc;
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_tcgen05_pair: accumulate needs a float32 output");
    return launch_pair<256, EPI_ACCUM, float>(ma, mw, C, ldc, M, N, K, status, stream);
  }
  if (epilogue == EPI_SWIGLU) {
    if (out_dtype != HFEE_BF16) return hfee_fail(HFEE_ERR_ARG, "gemm_tcgen05_pair: the SwiGLU epilogue writes bfloat16");
    return launch_pair<256, EPI_SWIGLU, __nv_bfloat16>(ma, mw, C, ldc, M, N, K, status, stream);
  }
  if (out_dtype == HFEE_BF16) return launch_pair<256, EPI_STORE, __nv_bfloat16>(ma, mw, C, ldc, M, N, K, status, stream);
  return launch_pair<256, EPI_STORE, float>(ma, mw, C, ldc, M, N, K, status, stream);
}

// The q/k/v product with rotation and cache write in its epilogue (hfee_gemm_tcgen05_rope) on pairs of
// CTAs; called by that entry point, which has checked the arguments, for shapes with at least two
// rounds of 256 x 256 tiles, or with tiles of 256 x 192 (block_n = 192, heads of 64 dims).
int hfee_gemm_pair_rope(const void* A, long long lda, const void* W, long long ldw, int M, int N, int K,
                        const tc::RopeEpi& rope, int block_n, int* status, cudaStream_t stream) {
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc != HFEE_OK) return rc;
  rc = make_map(&mw, W, N, K, ldw, block_n / 2);
  if (rc != HFEE_OK) return rc;
  if (block_n == 192) return launch_pair<192, EPI_ROPE, __nv_bfloat16>(ma, mw, nullptr, 0, M, N, K, status, stream, rope);
  return launch_pair<256, EPI_ROPE, __nv_bfloat16>(ma, mw, nullptr, 0, M, N, K, status, stream, rope);
}
