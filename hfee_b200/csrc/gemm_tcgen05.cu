// out[M,N] (+)= A[M,K] . W[N,K]^T on the 5th-generation tensor cores: bfloat16 operands
// staged in shared memory by TMA (128-byte swizzle, no multicast), tcgen05.mma issued by
// one thread with the float32 accumulator in tensor memory, tcgen05.ld for the epilogue.
//
// The grid is persistent: CTA b computes the 128 x BN tiles (BN = 128 or 256) b, b + gridDim.x,
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
// Every mbarrier wait is bounded: a wait that runs out sets an abort flag that ends all
// other waits of the CTA, records a code in `status` and lets the CTA free its tensor
// memory and return.
// Reference: out[t*Rows+r] = Dot(W[r,:], x[t,:]), hostfog/hfee internal/ggml/ops.go:54-70.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int TC_THREADS = 320;       // 1 TMA warp, 1 MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int ACC_STAGES = 2;

enum Epilogue { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };

template <int BN> struct TileCfg {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int W_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;      // + slack to align the base to 1024
};

template <int BN, int EPI, typename TOut>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               TOut* __restrict__ C, long long ldc, int M, int N, int K, int* __restrict__ status) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr uint32_t TMEM_COLS = ACC_STAGES * BN;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[ACC_STAGES];
  __shared__ __align__(8) uint64_t tmem_empty_bar[ACC_STAGES];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + BK - 1) / BK;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;

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
    if (lane == 0) {
      uint32_t it = 0;                           // K blocks issued so far, over all tiles
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, &abort_flag);
          if (!ok) break;
          unsigned char* a_dst = tiles + s * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, kb * BK, m0, &full_bar[s]);
          tma_load_2d(a_dst + Cfg::A_BYTES, &map_w, kb * BK, n0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++acc_it) {
        const uint32_t buf = acc_it & 1u;
        ok = mbar_wait(&tmem_empty_bar[buf], ((acc_it >> 1) & 1u) ^ 1u, &abort_flag);   // epilogue has drained it
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1u, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * Cfg::STAGE_BYTES);
          const uint64_t da = make_desc(a_addr), dw = make_desc(a_addr + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)       // 16 bf16 = 32 bytes further along K: +2 in 16-byte units
            tc_mma(tmem_d, da + 2 * k, dw + 2 * k, idesc, (kb | k) != 0);
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tmem_full_bar[buf]);
      }
    }
  } else {
    // epilogue warp w may read TMEM lanes 32*(w%4) .. +31 (= tile rows of the same numbers); the
    // two warps that share a lane quadrant take one half of the columns each
    const int quad = warp & 3, half = (warp - 2) >> 2;
    constexpr int CHUNKS = BN / 32 / 2;          // 32-column chunks per warp
    uint32_t acc_it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++acc_it) {
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      const uint32_t buf = acc_it & 1u;
      ok = mbar_wait(&tmem_full_bar[buf], (acc_it >> 1) & 1u, &abort_flag);
      tc_fence_after();
      if (!ok) break;
      const int row = m0 + quad * 32 + lane;
#pragma unroll 1
      for (int cc = 0; cc < CHUNKS; ++cc) {
        const int ch = half * CHUNKS + cc;
        uint32_t v[32];
        tc_ld32(tmem_base + buf * BN + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ch * 32), v);
        tc_wait_ld();
        const int col0 = n0 + ch * 32;
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
      // this warp's reads of the accumulator are complete: hand the buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
    // loads that were issued may still be landing in this CTA's shared memory: give them time
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
template <int BN, int EPI, typename TOut>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, long long ldc, int M, int N, int K, int* status,
           cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "gemm_tcgen05: cannot get %d bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  dim3 grid((unsigned)(tiles < sms ? tiles : sms));          // one CTA per SM walks the tiles
  hfee_launch(gemm_tc_kernel<BN, EPI, TOut>, dim3(grid), dim3(TC_THREADS), Cfg::SMEM, stream, ma, mw, (TOut*)C, ldc, M, N, K, status);
  return hfee_check_launch("gemm_tcgen05");
}

template <int BN>
int dispatch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, long long ldc, int out_dtype, int epilogue, int M,
             int N, int K, int* status, cudaStream_t stream) {
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_tcgen05: accumulate needs a float32 output");
    return launch<BN, EPI_ACCUM, float>(ma, mw, C, ldc, M, N, K, status, stream);
  }
  if (epilogue == EPI_SWIGLU) {
    if (out_dtype != HFEE_BF16) return hfee_fail(HFEE_ERR_ARG, "gemm_tcgen05: the SwiGLU epilogue writes bfloat16");
    return launch<BN, EPI_SWIGLU, __nv_bfloat16>(ma, mw, C, ldc, M, N, K, status, stream);
  }
  if (out_dtype == HFEE_BF16) return launch<BN, EPI_STORE, __nv_bfloat16>(ma, mw, C, ldc, M, N, K, status, stream);
  return launch<BN, EPI_STORE, float>(ma, mw, C, ldc, M, N, K, status, stream);
}

}  // namespace

// A, W: bfloat16, 16-byte aligned, leading dimensions multiples of 8.  epilogue: 0 store, 1 accumulate
// into float32 C, 2 SwiGLU over W rows interleaved [4 gate | 4 up] (C is [M, N/2] bfloat16).
// `status` (device int, may be null) is set to 1 if a CTA gave up waiting.  block_n: 128 or 256.
HFEE_API int hfee_gemm_tcgen05(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                               int out_dtype, int epilogue, int M, int N, int K, int block_n, int* status,
                               cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && N > 0 && K > 0 && K % 8 == 0, "gemm_tcgen05: K=%d must be a positive multiple of 8", K);
  HFEE_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K,
               "gemm_tcgen05: leading dimensions (%lld, %lld) must be multiples of 8 and at least K", lda, ldw);
  HFEE_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_tcgen05: operands must be 16-byte aligned");
  HFEE_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_tcgen05: unknown epilogue %d", epilogue);
  HFEE_REQUIRE(epilogue != EPI_SWIGLU || N % 8 == 0, "gemm_tcgen05: SwiGLU needs N %% 8 == 0, got %d", N);
  HFEE_REQUIRE(ldc >= (epilogue == EPI_SWIGLU ? N / 2 : N), "gemm_tcgen05: ldc=%lld is too small", ldc);
  HFEE_REQUIRE(block_n == 128 || block_n == 256, "gemm_tcgen05: block_n must be 128 or 256");
  HFEE_REQUIRE((long long)((M + BM - 1) / BM) * ((N + block_n - 1) / block_n) < (1ll << 31), "gemm_tcgen05: too many tiles");
  CUtensorMap ma, mw;
  int rc = make_map(&ma, A, M, K, lda, BM);
  if (rc != HFEE_OK) return rc;
  rc = make_map(&mw, W, N, K, ldw, block_n);
  if (rc != HFEE_OK) return rc;
  if (block_n == 256) return dispatch<256>(ma, mw, C, ldc, out_dtype, epilogue, M, N, K, status, stream);
  return dispatch<128>(ma, mw, C, ldc, out_dtype, epilogue, M, N, K, status, stream);
}
