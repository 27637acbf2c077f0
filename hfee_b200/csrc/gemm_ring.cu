// out (+)= tokens . W^T for a decode step of at most 8 tokens: the weights stream once through a
// ring of shared-memory stages that the copy engine fills, one TMA box per stage.
//
// Reference math: hostfog/hfee internal/ggml/ops.go:125-134 (the product), 160-165 (SwiGLU).
//
// Such a product computes almost nothing; its time is the time to read W.  The kernel that keeps
// the stream in registers (gemm_stream.cu) needs many warps per SM, each with a few 16-byte loads in
// flight, and ramps up slowly; here one CTA per SM owns a contiguous share of the rows of W and a
// producer warp requests it as boxes [8 slabs of 64 k][up to 16 rows] in the 128-byte swizzle, which
// `ldmatrix` reads without bank conflicts (one `cp.async.bulk` per weight row, 1 KB each, reached
// only 2.5 TB/s: the copy engine wants few, large requests; boxes of 16 KB reach 6 TB/s with five in
// flight per SM).  W is nobody's output, so its stream starts before the previous kernel has ended
// (programmatic dependent launch); the tokens, which are, come through a second producer warp that
// waits for them: all of them once when they fit beside the ring, else a chunk per stage.  Eight
// consumer warps take every eighth 16-wide k step of a stage (`mma.sync.m16n8k16`: 16 weight rows x
// 8 tokens), add their partial tiles through shared memory in warp order and apply the epilogue.
//
// Every wait has a time limit; a wait that runs out sets the status word.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int KC = 512;                          // k elements of a stage: 8 slabs of 64
constexpr int SLABS = KC / 64;
constexpr int TILE_ROWS = 16;                    // most weight rows of a stage: one MMA tile
constexpr int MAX_TOKENS = 8;
constexpr int CONSUMER_WARPS = 8;
constexpr int THREADS = 32 * (2 + CONSUMER_WARPS);
constexpr int W_BYTES = SLABS * TILE_ROWS * 128;         // 16 KB: a stage of weights, [slab][row][64 k]
constexpr int T_BYTES = SLABS * MAX_TOKENS * 128;        // 8 KB:  a box of tokens,    [slab][token][64 k]
constexpr int T_STAGES = 4;
constexpr int RESIDENT_MAX = 32 * 1024;                  // tokens that stay: K <= 2048
constexpr int RED_BYTES = CONSUMER_WARPS * TILE_ROWS * MAX_TOKENS * 4;
constexpr int MAX_STAGES = 4;
constexpr int BAR_BYTES = (2 * MAX_STAGES + 2 * T_STAGES + 1) * 8 + 16;
constexpr int EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2;
static_assert(W_BYTES % 1024 == 0 && T_BYTES % 1024 == 0, "the swizzle needs 1024-byte aligned tiles");

struct RingArgs {
  void* C; long long ldc;
  int M, N, K;
  int unit;                                        // rows that stay together: 8 for SwiGLU (4 gate, 4 up), else 1
  int tile;                                        // weight rows per stage (the TMA box's height)
  int stages;
  int resident;                                    // 1: all tokens are loaded once and stay in shared memory
  int token_bytes;                                 // size of the token region
  int* status;
};

// A box [8 slabs][rows][64 k] of a matrix seen as (k in slab, row, slab): coordinates (0, row, slab).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_16x8x16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory"); }

template <typename T> __device__ __forceinline__ T to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <int EPI, typename OutT>
__global__ void __launch_bounds__(THREADS, 1)
gemm_ring_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, RingArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* ring = smem;                                          // 1024-byte aligned (checked below)
  unsigned char* tokens = ring + a.stages * W_BYTES;                   // all tokens, or a ring of chunks
  float* red = reinterpret_cast<float*>(tokens + a.token_bytes);
  uint64_t* w_full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(red) + RED_BYTES);
  uint64_t* w_empty = w_full + MAX_STAGES;
  uint64_t* t_full = w_empty + MAX_STAGES;
  uint64_t* t_empty = t_full + T_STAGES;
  uint64_t* a_full = t_empty + T_STAGES;                               // the resident tokens have landed
  int& abort_flag = *reinterpret_cast<int*>(a_full + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = a.stages;
  // this CTA's rows: whole units, shared out evenly
  const int units = a.N / a.unit;
  const int r0 = a.unit * (int)((long long)blockIdx.x * units / gridDim.x);
  const int r1 = a.unit * (int)((long long)(blockIdx.x + 1) * units / gridDim.x);

  if (threadIdx.x == 0) {
    abort_flag = (smem_u32(ring) & 1023u) != 0 ? 1 : 0;       // misaligned tiles would corrupt the swizzle
    for (int s = 0; s < S; ++s) { mbar_init(&w_full[s], 1); mbar_init(&w_empty[s], CONSUMER_WARPS); }
    for (int s = 0; s < T_STAGES; ++s) { mbar_init(&t_full[s], 1); mbar_init(&t_empty[s], CONSUMER_WARPS); }
    mbar_init(a_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The next kernel may start at once.  Whatever of it finds room on the SMs beside this one requests
  // its own first weights now and has them when this kernel ends.
  pdl_launch_dependents();

  if (warp == 0) {
    // ---- weights: free-running, held back only by the ring
    uint32_t it = 0;
    bool ok = true;
    for (int row0 = r0; row0 < r1 && ok; row0 += a.tile) {
      for (int k0 = 0; k0 < a.K; k0 += KC, ++it) {
        const int s = it % S;
        ok = __all_sync(0xffffffffu, mbar_wait(&w_empty[s], ((it / S) & 1u) ^ 1u, &abort_flag));
        if (!ok) break;
        if (elect_one()) {
          // the box is always whole: rows behind the matrix and slabs behind K arrive as zeros
          mbar_expect_tx(&w_full[s], (uint32_t)(SLABS * a.tile * 128));
          tma_load_3d(ring + s * W_BYTES, &map_w, 0, row0, k0 / 64, &w_full[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---- tokens: the previous kernel's output
    pdl_wait();
    if (r0 < r1) {
      if (a.resident) {
        if (elect_one()) {
          const int boxes = (a.K + KC - 1) / KC;
          mbar_expect_tx(a_full, (uint32_t)(boxes * T_BYTES));
          for (int b = 0; b < boxes; ++b) tma_load_3d(tokens + b * T_BYTES, &map_a, 0, 0, b * SLABS, a_full);
        }
        __syncwarp();
      } else {
        uint32_t it = 0;
        bool ok = true;
        for (int row0 = r0; row0 < r1 && ok; row0 += a.tile) {
          for (int k0 = 0; k0 < a.K; k0 += KC, ++it) {
            const int s = it % T_STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&t_empty[s], ((it / T_STAGES) & 1u) ^ 1u, &abort_flag));
            if (!ok) break;
            if (elect_one()) {
              mbar_expect_tx(&t_full[s], (uint32_t)T_BYTES);
              tma_load_3d(tokens + s * T_BYTES, &map_a, 0, 0, k0 / 64, &t_full[s]);
            }
            __syncwarp();
          }
        }
      }
    }
  } else {
    // ---- consumers
    const int cw = warp - 2, ct = threadIdx.x - 64;                 // consumer warp and thread
    const int g = lane >> 2, c = lane & 3;
    uint32_t it = 0;
    bool ok = true;
    OutT* C = reinterpret_cast<OutT*>(a.C);
    if (EPI == EPI_ACCUM) pdl_wait();                               // what is added to is an earlier kernel's output
    if (a.resident && r0 < r1) ok = __all_sync(0xffffffffu, mbar_wait(a_full, 0, &abort_flag));

    for (int row0 = r0; row0 < r1 && ok; row0 += a.tile) {
      const int rows = min(a.tile, r1 - row0);
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
      // the epilogue's thread (row, token); what it will add to is requested now, a tile of weights
      // ahead of its use
      const int e_row = ct / MAX_TOKENS, e_m = ct % MAX_TOKENS;
      const bool e_mine = ct < TILE_ROWS * MAX_TOKENS && e_m < a.M && e_row < rows;
      float old = 0.f;
      if (EPI == EPI_ACCUM && e_mine) old = __ldcg(reinterpret_cast<const float*>(a.C) + (long long)e_m * a.ldc + row0 + e_row);
      for (int k0 = 0; k0 < a.K; k0 += KC, ++it) {
        const int s = it % S, ts = it % T_STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(&w_full[s], (it / S) & 1u, &abort_flag));
        if (ok && !a.resident) ok = __all_sync(0xffffffffu, mbar_wait(&t_full[ts], (it / T_STAGES) & 1u, &abort_flag));
        if (!ok) break;
        // weights: slab j of the stage holds rows 0 .. tile-1 of k 64 j .. 64 j + 63, a row 128 bytes,
        // its 16-byte piece p at position p ^ (128-byte line number mod 8)
        const uint32_t stage = smem_u32(ring + s * W_BYTES);
        const uint32_t tbase = a.resident ? smem_u32(tokens) + (uint32_t)(k0 / 64) * (MAX_TOKENS * 128)
                                          : smem_u32(tokens + ts * T_BYTES);
        const int w_row = min(lane & 15, a.tile - 1);               // rows the box does not have are never stored
        const int steps = min(KC, a.K - k0) / 16;
        // this warp's k steps of the stage (at most KC / 16 / CONSUMER_WARPS = 4): all fragments are
        // requested before the first MMA, and the MMAs alternate between two accumulators
        constexpr int MINE = KC / 16 / CONSUMER_WARPS;
        uint32_t wa[MINE][4], tb[MINE][2];
#pragma unroll
        for (int j = 0; j < MINE; ++j) {
          const int ks = cw + j * CONSUMER_WARPS;
          if (ks < steps) {
            const int slab = ks >> 2, piece = (ks & 3) * 2;
            const int w_line = slab * a.tile + w_row;
            ldmatrix_x4(wa[j], stage + w_line * 128 + (((piece + (lane >> 4)) ^ (w_line & 7)) << 4));
            // tokens: slab after slab, 8 lines of 128 bytes each (the region starts 1024-byte aligned,
            // so the line number within the region gives the swizzle)
            const int t_line = slab * MAX_TOKENS + (lane & 7);
            ldmatrix_x2(tb[j], tbase + t_line * 128 + (((piece + ((lane >> 3) & 1)) ^ (t_line & 7)) << 4));
          }
        }
#pragma unroll
        for (int j = 0; j < MINE; ++j)
          if (cw + j * CONSUMER_WARPS < steps) mma_16x8x16(j & 1 ? acc2 : acc, wa[j], tb[j]);
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&w_empty[s]);
          if (!a.resident) mbar_arrive(&t_empty[ts]);
        }
      }
      if (!ok) break;
      // ---- the warps' partial tiles meet in shared memory and are added in warp order
      float* mine = red + cw * (TILE_ROWS * MAX_TOKENS);
      *reinterpret_cast<float2*>(mine + g * MAX_TOKENS + 2 * c) = make_float2(acc[0] + acc2[0], acc[1] + acc2[1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * MAX_TOKENS + 2 * c) = make_float2(acc[2] + acc2[2], acc[3] + acc2[3]);
      consumer_sync();
      if (e_mine) {
        const int row = e_row, m = e_m;
        auto total = [&](int r) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[w * (TILE_ROWS * MAX_TOKENS) + r * MAX_TOKENS + m];
          return v;
        };
        if (EPI == EPI_STORE) {
          C[(long long)m * a.ldc + row0 + row] = to_out<OutT>(total(row));
        } else if (EPI == EPI_ACCUM) {
          C[(long long)m * a.ldc + row0 + row] = to_out<OutT>(old + total(row));
        } else if ((row & 7) < 4) {
          // rows 8u .. 8u+3 are gate rows, 8u+4 .. 8u+7 the up rows of the same four outputs
          const float gate = total(row), up = total(row + 4);
          const long long col = (long long)((row0 + row) >> 3) * 4 + (row & 3);
          C[(long long)m * a.ldc + col] = to_out<OutT>(__fdividef(gate, 1.f + __expf(-gate)) * up);
        }
      }
      consumer_sync();
    }
  }

  __syncthreads();
  if (abort_flag) {                    // a wait ran out: give copies that may still be in flight time to land
#pragma unroll 1
    for (int i = 0; i < 400; ++i) __nanosleep(1000);
    __syncthreads();
    if (threadIdx.x == 0 && a.status != nullptr) atomicExch(a.status, 3);
  }
}

int token_region_bytes(int K) {
  const int all = (K + KC - 1) / KC * T_BYTES;
  return all <= RESIDENT_MAX ? all : T_STAGES * T_BYTES;
}

// Stages of the weight ring.  With four (64 KB) and the tokens beside them the kernel stays below half
// of an SM's shared memory: the CTAs of the next such kernel find room beside this one's, and their
// first four boxes are there when this one ends (measured, down projection of the benchmark model at
// 8 tokens: 8.47 us with four stages, 8.82 with five, 9.23 with three).  More shared memory than
// needed is not free either: the SM's carve-out between shared memory and L1 follows the resident
// kernel, and behind a kernel with 213 KB a product that streams through L1 took twice as long.
constexpr int RING_STAGES = 4;

// Weight rows per stage for `rows` rows a CTA owns at most: as few stages as 16-row tiles allow, of equal height.
int tile_height(int rows, int unit) {
  if (rows <= 0) return unit;
  const int tiles = (rows + TILE_ROWS - 1) / TILE_ROWS;
  int h = (rows + tiles - 1) / tiles;
  h = (h + unit - 1) / unit * unit;
  return h > TILE_ROWS ? TILE_ROWS : h;
}

// Tensor map of a row-major bf16 matrix [rows, cols] (cols a multiple of 64) seen as (k within a slab of
// 64, row, slab): a box [8 slabs][box_rows][64] lands as 8 consecutive 128-byte-swizzled tiles.
int make_slab_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return hfee_fail(HFEE_ERR_CUDA, "gemm_ring: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)SLABS};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return hfee_fail(HFEE_ERR_CUDA, "gemm_ring: cuTensorMapEncodeTiled failed with %d", (int)r);
  return HFEE_OK;
}

template <int EPI, typename OutT>
int launch_ring(const CUtensorMap& mw, const CUtensorMap& ma, const RingArgs& a, int grid, size_t smem, cudaStream_t stream) {
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_ring_kernel<EPI, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "gemm_ring: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  hfee_launch(gemm_ring_kernel<EPI, OutT>, dim3((unsigned)grid), dim3(THREADS), smem, stream, mw, ma, a);
  return hfee_check_launch("gemm_ring");
}

}  // namespace

// 1 if hfee_gemm_ring takes this product (bfloat16 tokens and weights are implied).
HFEE_API int hfee_gemm_ring_supports(int M, int N, int K, int epilogue) {
  if (M < 1 || M > MAX_TOKENS || N < 1) return 0;
  if (K < 64 || K % 64) return 0;                         // whole 64-wide slabs of k
  if (epilogue < 0 || epilogue > 2) return 0;
  if (epilogue == EPI_SWIGLU && N % 8) return 0;
  return 1;
}

// epilogue: 0 store, 1 accumulate into float32 C, 2 SwiGLU (C is [M, N/2]; rows of W in groups of
// 4 gate rows and 4 up rows).  out_dtype: 0 float32, 1 bfloat16.
HFEE_API int hfee_gemm_ring(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                            int out_dtype, int epilogue, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  HFEE_REQUIRE(hfee_gemm_ring_supports(M, N, K, epilogue),
               "gemm_ring: takes 1..%d tokens, K a multiple of 64 and, for SwiGLU, N a multiple of 8 (got M=%d N=%d K=%d epilogue=%d)",
               MAX_TOKENS, M, N, K, epilogue);
  HFEE_REQUIRE(lda % 8 == 0 && lda >= K && ldw % 8 == 0 && ldw >= K && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0,
               "gemm_ring: rows of the tokens and of the weights must start on 16-byte boundaries");
  HFEE_REQUIRE(ldc >= (epilogue == EPI_SWIGLU ? N / 2 : N), "gemm_ring: ldc=%lld is too small", ldc);
  HFEE_REQUIRE(out_dtype == HFEE_F32 || out_dtype == HFEE_BF16, "gemm_ring: unknown output dtype %d", out_dtype);
  HFEE_REQUIRE(epilogue != EPI_ACCUM || out_dtype == HFEE_F32, "gemm_ring: accumulation wants a float32 output");
  const int sms = hfee_sm_count();
  if (sms <= 0) return hfee_fail(HFEE_ERR_CUDA, "gemm_ring: cannot ask the device for its number of SMs");
  RingArgs a;
  a.C = C; a.ldc = ldc; a.M = M; a.N = N; a.K = K;
  a.unit = epilogue == EPI_SWIGLU ? 8 : 1;
  const int units = N / a.unit;
  const int grid = units < sms ? units : sms;
  a.tile = tile_height(a.unit * ((units + grid - 1) / grid), a.unit);
  a.stages = RING_STAGES;
  a.token_bytes = token_region_bytes(K);
  a.resident = (K + KC - 1) / KC * T_BYTES <= RESIDENT_MAX ? 1 : 0;
  a.status = status;
  CUtensorMap mw, ma;
  int rc;
  if ((rc = make_slab_map(&mw, W, N, K, ldw, a.tile)) != HFEE_OK) return rc;
  if ((rc = make_slab_map(&ma, A, M, K, lda, MAX_TOKENS)) != HFEE_OK) return rc;
  const size_t smem = (size_t)a.stages * W_BYTES + a.token_bytes + RED_BYTES + BAR_BYTES;
#define HFEE_RING(EPI, T) return launch_ring<EPI, T>(mw, ma, a, grid, smem, stream)
  if (epilogue == EPI_ACCUM) HFEE_RING(EPI_ACCUM, float);
  if (epilogue == EPI_STORE) { if (out_dtype == HFEE_F32) HFEE_RING(EPI_STORE, float); HFEE_RING(EPI_STORE, __nv_bfloat16); }
  if (out_dtype == HFEE_F32) HFEE_RING(EPI_SWIGLU, float);
  HFEE_RING(EPI_SWIGLU, __nv_bfloat16);
#undef HFEE_RING
}
