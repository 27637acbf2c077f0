// out[M,N] (+)= A[M,K] . W[N,K]^T for few tokens (M <= 64) on tcgen05 with the operands swapped:
// 128 weight rows are the M side of the MMA, the tokens its N side (16, 32 or 64 columns).
//
// What bounds this product is reading W once from HBM, so the point of the kernel is to keep many
// bytes in flight: a TMA warp streams 128 x 64 weight tiles (and the small token tile) through a
// ring of 8-10 shared-memory stages, far more than registers could hold, while one thread issues
// the MMAs into tensor memory.  The grid is persistent over work items (weight tile, K split);
// K is split among CTAs when there are fewer weight tiles than SMs.  A split writes its partial
// tile to a float32 workspace and a second kernel adds the splits in split order, so the sum
// order is fixed; without a split the epilogue writes C directly (transposed: a thread holds one
// weight row for all tokens).  Epilogues: store, accumulate into float32 C, SwiGLU over rows
// interleaved [4 gate | 4 up].  Every barrier wait is bounded (see tcgen05.cuh).
// Reference: out[t*Rows+r] = Dot(W[r,:], x[t,:]), hostfog/hfee internal/ggml/ops.go:54-70
// ("each row is read once for all n inputs").
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int WM = 128;                 // weight rows per tile
constexpr int SK_THREADS = 192;         // 1 TMA warp, 1 MMA warp, 4 epilogue warps
constexpr int ACC_STAGES = 2;

enum Epilogue { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };

template <int TN> struct SkinnyCfg {
  static constexpr int W_BYTES = WM * BK * 2;
  static constexpr int A_BYTES = TN * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES > 10 ? 10 : (192 * 1024) / STAGE_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;
  static constexpr uint32_t TMEM_COLS = ACC_STAGES * TN < 32 ? 32 : ACC_STAGES * TN;
};

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr) : "memory");
}

struct SkinnyArgs {
  int M, N, K;
  int w_tiles, splits, kb_per_split, k_blocks;
  long long ldc;
  float* workspace;        // [splits][M][N] float32 partial tiles (splits > 1)
};

// One 16-token column group of a thread's weight row: direct epilogue or partial write.
template <int EPI, typename TOut, int COLS>
__device__ __forceinline__ void write_columns(const uint32_t (&v)[COLS], int tok0, int w_row, int lane, int split,
                                              TOut* __restrict__ C, const SkinnyArgs& a) {
  const bool row_ok = w_row < a.N;
  if (a.splits > 1) {
    if (row_ok) {
#pragma unroll
      for (int j = 0; j < COLS; ++j)
        if (tok0 + j < a.M) a.workspace[((long long)split * a.M + tok0 + j) * a.N + w_row] = __uint_as_float(v[j]);
    }
    return;
  }
  if constexpr (EPI == EPI_SWIGLU) {
    // weight rows come in groups of 8 = [4 gate | 4 up]: the up partner of this lane's row is 4 lanes on
    const bool writer = (lane & 7) < 4 && w_row + 4 < a.N;
    const long long col = (long long)(w_row >> 3) * 4 + (lane & 3);
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      float gate = __uint_as_float(v[j]);
      float up = __shfl_down_sync(0xffffffffu, gate, 4);
      if (writer && tok0 + j < a.M) {
        // a bfloat16 result does not need the exact exponential and division (the large-tile kernel
        // computes it the same way)
        float h;
        if constexpr (sizeof(TOut) == 2) h = __fdividef(gate, 1.f + __expf(-gate)) * up;
        else h = gate / (1.f + expf(-gate)) * up;
        C[(long long)(tok0 + j) * a.ldc + col] = from_f32<TOut>(h);
      }
    }
  } else {
    if (!row_ok) return;
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      if (tok0 + j >= a.M) continue;
      const long long o = (long long)(tok0 + j) * a.ldc + w_row;
      float x = __uint_as_float(v[j]);
      if constexpr (EPI == EPI_ACCUM) x += to_f32<TOut>(C[o]);
      C[o] = from_f32<TOut>(x);
    }
  }
}

template <int TN, int EPI, typename TOut>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   TOut* __restrict__ C, SkinnyArgs a, int* __restrict__ status) {
  using Cfg = SkinnyCfg<TN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[ACC_STAGES];
  __shared__ __align__(8) uint64_t tmem_empty_bar[ACC_STAGES];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int items = a.w_tiles * a.splits;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < ACC_STAGES; ++b) { mbar_init(&tmem_full_bar[b], 1); mbar_init(&tmem_empty_bar[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(Cfg::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    if (lane == 0) {
      // The weights are not the previous kernel's output: the weight tiles of the first round of the
      // ring (all stages are free) are requested before the wait, their token tiles after it.
      uint32_t pre = 0;
      for (int i = blockIdx.x; i < items && pre < (uint32_t)STAGES; i += gridDim.x) {
        const int n0 = (i % a.w_tiles) * WM, split = i / a.w_tiles;
        const int kb0 = split * a.kb_per_split, kb1 = min(a.k_blocks, kb0 + a.kb_per_split);
        for (int kb = kb0; kb < kb1 && pre < (uint32_t)STAGES; ++kb, ++pre) {
          mbar_expect_tx(&full_bar[pre], Cfg::STAGE_BYTES);
          tma_load_2d(tiles + pre * Cfg::STAGE_BYTES, &map_w, kb * BK, n0, &full_bar[pre]);
        }
      }
      pdl_wait();            // the token tiles are the previous kernel's output
      uint32_t it = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < items && ok; i += gridDim.x) {
        const int n0 = (i % a.w_tiles) * WM, split = i / a.w_tiles;
        const int kb0 = split * a.kb_per_split, kb1 = min(a.k_blocks, kb0 + a.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          unsigned char* w_dst = tiles + s * Cfg::STAGE_BYTES;
          if (it >= pre) {
            ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1u) ^ 1u, &abort_flag);
            if (!ok) break;
            mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
            tma_load_2d(w_dst, &map_w, kb * BK, n0, &full_bar[s]);
          }
          tma_load_2d(w_dst + Cfg::W_BYTES, &map_a, kb * BK, 0, &full_bar[s]);
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop (warp-uniform control flow keeps addresses and descriptors in
    // uniform registers); one elected lane issues the MMAs and commits.
    constexpr uint32_t idesc = make_idesc(WM, TN);
    uint32_t it = 0, acc_it = 0;
    bool ok = true;
    const uint64_t desc0 = make_desc(smem_u32(tiles));
    for (int i = blockIdx.x; i < items && ok; i += gridDim.x, ++acc_it) {
      const int split = i / a.w_tiles;
      const int kb0 = split * a.kb_per_split, kb1 = min(a.k_blocks, kb0 + a.kb_per_split);
      const uint32_t buf = acc_it & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty_bar[buf], ((acc_it >> 1) & 1u) ^ 1u, &abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + buf * TN;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[s], (it / STAGES) & 1u, &abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          // descriptor addresses count 16-byte units
          const uint64_t dw = desc0 + (uint64_t)(s * (Cfg::STAGE_BYTES >> 4)), da = dw + (uint64_t)(Cfg::W_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma(tmem_d, dw + 2 * k, da + 2 * k, idesc, (kb > kb0) || k != 0);
          tc_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (ok && elect_one()) tc_commit(&tmem_full_bar[buf]);
      __syncwarp();
    }
  } else {
    pdl_wait();            // C (when accumulating) is the previous kernel's output
    const int quad = warp & 3;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int i = blockIdx.x; i < items && ok; i += gridDim.x, ++acc_it) {
      const int n0 = (i % a.w_tiles) * WM, split = i / a.w_tiles;
      const uint32_t buf = acc_it & 1u;
      ok = mbar_wait(&tmem_full_bar[buf], (acc_it >> 1) & 1u, &abort_flag);
      tc_fence_after();
      if (!ok) break;
      const int w_row = n0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + buf * TN + ((uint32_t)(quad * 32) << 16);
#pragma unroll
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t v[16];
        tc_ld16(taddr + (uint32_t)c0, v);
        tc_wait_ld();
        write_columns<EPI, TOut, 16>(v, c0, w_row, lane, split, C, a);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
    }
  }
  pdl_launch_dependents();

  tc_fence_before();
  __syncthreads();
  if (abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 400; ++i) __nanosleep(1000);
    if (threadIdx.x == 0 && status != nullptr) atomicExch(status, 1);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

// C (+)= sum over splits (in split order) of the partial tiles, with the epilogue applied.  The
// partial values of up to eight splits are requested together and then added in split order.
constexpr int RED_BATCH = 8;

template <int EPI, typename TOut>
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, TOut* __restrict__ C, long long ldc, int M, int N,
                                     int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int out_cols = EPI == EPI_SWIGLU ? N / 2 : N;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * out_cols) return;
  const int t = (int)(idx / out_cols), c = (int)(idx % out_cols);
  const long long split_pitch = (long long)M * N;
  if constexpr (EPI == EPI_SWIGLU) {
    const float* p = ws + (long long)t * N + (c >> 2) * 8 + (c & 3);
    float gate = 0.f, up = 0.f;
    for (int s0 = 0; s0 < splits; s0 += RED_BATCH) {
      float g[RED_BATCH], u[RED_BATCH];
#pragma unroll
      for (int j = 0; j < RED_BATCH; ++j) {
        const bool ok = s0 + j < splits;
        g[j] = ok ? p[(s0 + j) * split_pitch] : 0.f;
        u[j] = ok ? p[(s0 + j) * split_pitch + 4] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < RED_BATCH; ++j) { gate += g[j]; up += u[j]; }
    }
    C[(long long)t * ldc + c] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
  } else {
    const float* p = ws + (long long)t * N + c;
    const long long o = (long long)t * ldc + c;
    float old = 0.f;
    if constexpr (EPI == EPI_ACCUM) old = to_f32<TOut>(C[o]);
    float v = 0.f;
    for (int s0 = 0; s0 < splits; s0 += RED_BATCH) {
      float part[RED_BATCH];
#pragma unroll
      for (int j = 0; j < RED_BATCH; ++j) part[j] = s0 + j < splits ? p[(s0 + j) * split_pitch] : 0.f;
#pragma unroll
      for (int j = 0; j < RED_BATCH; ++j) v += part[j];
    }
    C[o] = from_f32<TOut>(v + old);
  }
}

int device_sms() { return hfee_sm_count(); }

// K split for N weight rows and K: as many CTAs as SMs, at least 4 K blocks each.
void plan_split(int N, int K, int M, long long workspace_floats, int* splits, int* kb_per_split) {
  const int w_tiles = (N + WM - 1) / WM, k_blocks = (K + BK - 1) / BK;
  int want = device_sms() / w_tiles;
  if (want < 1) want = 1;
  int kbs = (k_blocks + want - 1) / want;
  if (kbs < 4) kbs = 4;
  if (kbs > k_blocks) kbs = k_blocks;
  int s = (k_blocks + kbs - 1) / kbs;
  while (s > 1 && (long long)s * M * N > workspace_floats) {     // shrink to what the workspace holds
    ++kbs;
    s = (k_blocks + kbs - 1) / kbs;
  }
  *splits = s;
  *kb_per_split = kbs;
}

template <int TN, int EPI, typename TOut>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, void* C, const SkinnyArgs& a, int* status, cudaStream_t stream) {
  using Cfg = SkinnyCfg<TN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<TN, EPI, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "gemm_skinny: cannot get %d bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e));
    configured = true;
  }
  const int items = a.w_tiles * a.splits;
  const int sms = device_sms();
  hfee_launch(gemm_skinny_kernel<TN, EPI, TOut>, dim3((unsigned)(items < sms ? items : sms)), dim3(SK_THREADS), Cfg::SMEM,
              stream, mw, ma, (TOut*)C, a, status);
  int rc = hfee_check_launch("gemm_skinny");
  if (rc != HFEE_OK || a.splits == 1) return rc;
  const long long outs = (long long)a.M * (EPI == EPI_SWIGLU ? a.N / 2 : a.N);
  hfee_launch(splitk_reduce_kernel<EPI, TOut>, dim3((unsigned)((outs + 255) / 256)), dim3(256), 0, stream,
              (const float*)a.workspace, (TOut*)C, a.ldc, a.M, a.N, a.splits);
  return hfee_check_launch("splitk_reduce");
}

template <int TN>
int dispatch(const CUtensorMap& mw, const CUtensorMap& ma, void* C, int out_dtype, int epilogue, const SkinnyArgs& a,
             int* status, cudaStream_t stream) {
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_skinny: accumulate needs a float32 output");
    return launch<TN, EPI_ACCUM, float>(mw, ma, C, a, status, stream);
  }
  if (epilogue == EPI_SWIGLU) {
    if (out_dtype == HFEE_BF16) return launch<TN, EPI_SWIGLU, __nv_bfloat16>(mw, ma, C, a, status, stream);
    return launch<TN, EPI_SWIGLU, float>(mw, ma, C, a, status, stream);
  }
  if (out_dtype == HFEE_BF16) return launch<TN, EPI_STORE, __nv_bfloat16>(mw, ma, C, a, status, stream);
  return launch<TN, EPI_STORE, float>(mw, ma, C, a, status, stream);
}

}  // namespace

// How many K splits hfee_gemm_skinny uses for this shape given `workspace_floats` of workspace
// (1 = none, no workspace needed, one launch; otherwise two launches).
HFEE_API int hfee_gemm_skinny_splits(int M, int N, int K, long long workspace_floats) {
  int s = 1, kbs = 1;
  plan_split(N, K, M, workspace_floats, &s, &kbs);
  return s;
}

// A [M,K], W [N,K]: bfloat16, 16-byte aligned, leading dimensions multiples of 8; M <= 64.
// `workspace` holds splits*M*N floats when the shape is split along K (may be null: no split).
HFEE_API int hfee_gemm_skinny(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                              int out_dtype, int epilogue, int M, int N, int K, float* workspace,
                              long long workspace_floats, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && M <= 64, "gemm_skinny: M=%d is outside 1..64", M);
  HFEE_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gemm_skinny: K=%d must be a positive multiple of 8", K);
  HFEE_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && lda >= K && ldw >= K,
               "gemm_skinny: leading dimensions (%lld, %lld) must be multiples of 8 and at least K", lda, ldw);
  HFEE_REQUIRE(((uintptr_t)A % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemm_skinny: operands must be 16-byte aligned");
  HFEE_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_skinny: unknown epilogue %d", epilogue);
  HFEE_REQUIRE(epilogue != EPI_SWIGLU || N % 8 == 0, "gemm_skinny: SwiGLU needs N %% 8 == 0, got %d", N);
  HFEE_REQUIRE(ldc >= (epilogue == EPI_SWIGLU ? N / 2 : N), "gemm_skinny: ldc=%lld is too small", ldc);
  SkinnyArgs a;
  a.M = M; a.N = N; a.K = K;
  a.w_tiles = (N + WM - 1) / WM;
  a.k_blocks = (K + BK - 1) / BK;
  plan_split(N, K, M, workspace ? workspace_floats : 0, &a.splits, &a.kb_per_split);
  a.ldc = ldc;
  a.workspace = workspace;
  const int tn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  CUtensorMap mw, ma;
  int rc = make_map(&mw, W, N, K, ldw, WM);
  if (rc != HFEE_OK) return rc;
  rc = make_map(&ma, A, M, K, lda, tn);
  if (rc != HFEE_OK) return rc;
  if (tn == 16) return dispatch<16>(mw, ma, C, out_dtype, epilogue, a, status, stream);
  if (tn == 32) return dispatch<32>(mw, ma, C, out_dtype, epilogue, a, status, stream);
  return dispatch<64>(mw, ma, C, out_dtype, epilogue, a, status, stream);
}
