// out[M,N] (+)= A[M,K] . W[N,K]^T for few tokens (M <= 64), bfloat16 inputs, float32
// accumulation: the decode-step matrix product, bound by reading W once from HBM.
//
// A CTA owns ROWS = 8*NT consecutive weight rows and all M tokens; its warps split K
// in interleaved blocks of 32.  Weights are the B operand of mma.sync.m16n8k16 (8
// weight rows per tile), tokens the A operand (16 per tile), so a lane's 16-byte
// load of a weight row feeds two MMAs directly from registers: the k order inside
// a block is permuted identically for both operands, which leaves the dot product
// unchanged.  Partial sums of the warps are added in warp order, so every output is
// summed in one fixed order whatever M is.
//
// Three kernels share the operand trick: this K-split one, a warp-per-tile one for many weight
// rows, and, for at most 8 tokens, one that keeps the tokens in registers (see further down).
//
// Epilogues: store (bf16 or f32), accumulate into a float32 output (the residual
// add), or SwiGLU over rows interleaved as [4 gate rows | 4 up rows] per group of 8.
// Reference: out[t*Rows+r] = Dot(W[r,:], x[t,:]), hostfog/hfee internal/ggml/ops.go:54-70
// ("each row is read once for all n inputs").
#include "common.cuh"

namespace {

constexpr int LOADS_IN_FLIGHT = 4;   // 16-byte weight loads per lane in one batch; two batches are in flight

enum Epilogue { EPI_STORE = 0, EPI_ACCUM = 1, EPI_SWIGLU = 2 };

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// MT: token tiles of 16; NT: weight-row tiles of 8; NW: warps per CTA (they split K, so the
// fewer tokens there are, the more warps keep loads in flight).  The grid is persistent: CTA b
// owns row tiles b, b + gridDim.x, ...; a warp's work is a sequence of load batches that runs
// across tile boundaries, so the next tile's weights are already in flight while this tile is
// reduced and written.  The first batch is issued before the wait on the previous kernel:
// weights do not depend on it.
//
// The kernel for at most 8 tokens further down can make the token operand on the fly from float32
// rows X (optionally gathered through `rows`): a[t, k] = bf16(X[t, k] * rsqrt(mean(X[t,:]^2) + eps) * nw[k]),
// the RMS norm of hostfog/hfee internal/ggml/ops.go:125-134 fused into the product that follows it.
struct NormArgs {
  const float* x;        // [*, ldx] float32 rows (A is unused)
  long long ldx;
  const int* rows;       // optional gather: token t reads row rows[t]
  const float* weight;   // [K]
  float eps;
  int add_unit;          // scale by 1 + weight
};

template <int MT, int NT, int NW, int EPI, typename TOut>
__global__ void __launch_bounds__(NW * 32, 2048 / (NW * 32) >= 4 ? 2 : 1)
gemm_stream_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ W,
                   long long ldw, TOut* __restrict__ C, long long ldc, int M, int N, int K) {
  constexpr int ROWS = 8 * NT;
  constexpr int UNROLL = LOADS_IN_FLIGHT / NT;     // k32-steps per batch of loads
  constexpr int STRIDE = NW * UNROLL;              // k32-steps all warps cover per batch
  __shared__ float red[NW][MT * 16][ROWS + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;

  const int steps = (K + 31) / 32;                 // k32 blocks in all; warp w takes w, w+NW, ...
  const int n_tiles = (N + ROWS - 1) / ROWS;
  const int bpt = (steps + STRIDE - 1) / STRIDE;   // batches per tile
  const int my_tiles = ((int)blockIdx.x < n_tiles) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total = my_tiles * bpt;

  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

  const __nv_bfloat16* arow[MT][2];
  bool aok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int t = mt * 16 + h * 8 + g;
      aok[mt][h] = t < M;
      arow[mt][h] = A + (long long)(aok[mt][h] ? t : 0) * lda;
    }

  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 wv[2][UNROLL][NT];

  // batch j of this CTA = batch (j % bpt) of its tile number (j / bpt); the loop below keeps
  // those two as counters instead of dividing
  auto load_batch = [&](int j, int tile_no, int in_tile, uint4 (&dst)[UNROLL][NT]) {
    const int n0 = ((int)blockIdx.x + tile_no * (int)gridDim.x) * ROWS;
    const int s0 = warp + in_tile * STRIDE;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int r = n0 + nt * 8 + g;
      const bool rok = j < total && r < N;
      const __nv_bfloat16* wrow = W + (long long)(rok ? r : 0) * ldw;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = (s0 + u * NW) * 32 + c * 8;
        dst[u][nt] = (rok && k < K) ? ld_stream(wrow + k) : zero;
      }
    }
  };
  auto compute_batch = [&](int in_tile, const uint4 (&src)[UNROLL][NT]) {
    const int s0 = warp + in_tile * STRIDE;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s0 + u * NW) * 32 + c * 8;
      const bool kok = k < K;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const uint4 lo = (kok && aok[mt][0]) ? __ldg((const uint4*)(arow[mt][0] + k)) : zero;
        const uint4 hi = (kok && aok[mt][1]) ? __ldg((const uint4*)(arow[mt][1] + k)) : zero;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma_bf16(acc[mt][nt], lo.x, hi.x, lo.y, hi.y, src[u][nt].x, src[u][nt].y);
          mma_bf16(acc[mt][nt], lo.z, hi.z, lo.w, hi.w, src[u][nt].z, src[u][nt].w);
        }
      }
    }
  };
  // After a tile's last batch: add the warps' partial sums in warp order and write the tile.
  auto finish_tile = [&](int tile_no) {
    const int n0 = ((int)blockIdx.x + tile_no * (int)gridDim.x) * ROWS;
    // fragment -> shared: c0,c1 = (token g, rows 2c,2c+1); c2,c3 = (token g+8, same rows)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        red[warp][mt * 16 + g][nt * 8 + 2 * c] = acc[mt][nt][0];
        red[warp][mt * 16 + g][nt * 8 + 2 * c + 1] = acc[mt][nt][1];
        red[warp][mt * 16 + g + 8][nt * 8 + 2 * c] = acc[mt][nt][2];
        red[warp][mt * 16 + g + 8][nt * 8 + 2 * c + 1] = acc[mt][nt][3];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;
      }
    __syncthreads();
    if constexpr (EPI == EPI_SWIGLU) {
      // rows of a group of 8: [gate x4 | up x4] -> 4 outputs at columns (n0/2 + group*4 ..)
      constexpr int OUTS = ROWS / 2;
      for (int idx = threadIdx.x; idx < MT * 16 * OUTS; idx += NW * 32) {
        int t = idx / OUTS, o = idx % OUTS;
        int col = n0 / 2 + o;
        if (t >= M || col >= N / 2) continue;
        int gr = (o / 4) * 8 + (o % 4);
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) { gate += red[w][t][gr]; up += red[w][t][gr + 4]; }
        C[(long long)t * ldc + col] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
      }
    } else {
      for (int idx = threadIdx.x; idx < MT * 16 * ROWS; idx += NW * 32) {
        int t = idx / ROWS, r = idx % ROWS;
        if (t >= M || n0 + r >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) v += red[w][t][r];
        long long o = (long long)t * ldc + n0 + r;
        if constexpr (EPI == EPI_ACCUM) C[o] = to_f32<TOut>(C[o]) + v;
        else C[o] = from_f32<TOut>(v);
      }
    }
    __syncthreads();
  };

  load_batch(0, 0, 0, wv[0]);
  pdl_wait();
  pdl_launch_dependents();
  int tile_no = 0, in_tile = 0;                 // of the batch being computed
  auto next = [&](int& t, int& b) { if (++b == bpt) { b = 0; ++t; } };
  for (int j = 0; j < total; j += 2) {
    int t1 = tile_no, b1 = in_tile;
    next(t1, b1);
    load_batch(j + 1, t1, b1, wv[1]);
    compute_batch(in_tile, wv[0]);
    if (in_tile == bpt - 1) finish_tile(tile_no);
    if (j + 1 < total) {
      int t2 = t1, b2 = b1;
      next(t2, b2);
      load_batch(j + 2, t2, b2, wv[0]);
      compute_batch(b1, wv[1]);
      if (b1 == bpt - 1) finish_tile(t1);
      tile_no = t2;
      in_tile = b2;
    }
  }
}

// The same product with one warp per tile of 8 weight rows over the whole of K: no partial sums
// to add across warps, no barriers, for shapes with enough tiles to occupy every warp of the GPU
// (gate/up and output-head projections).  Warp w of the grid owns tiles w, w + warps, ...; its
// loads run two batches ahead across tile boundaries.
constexpr int ROWS_WARPS = 8;                    // warps per CTA
constexpr int ROWS_UNROLL = 8;                   // 16-byte weight loads per lane in one batch

template <int MT, int EPI, typename TOut>
__global__ void __launch_bounds__(ROWS_WARPS * 32, 2)
gemm_stream_rows_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ W,
                        long long ldw, TOut* __restrict__ C, long long ldc, int M, int N, int K) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int warps = (int)gridDim.x * ROWS_WARPS;
  const int first = (int)blockIdx.x * ROWS_WARPS + (threadIdx.x >> 5);
  const int n_tiles = (N + 7) / 8;
  const int steps = (K + 31) / 32;
  const int bpt = (steps + ROWS_UNROLL - 1) / ROWS_UNROLL;
  const int my_tiles = first < n_tiles ? (n_tiles - 1 - first) / warps + 1 : 0;
  const int total = my_tiles * bpt;

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
  const __nv_bfloat16* arow[MT][2];
  bool aok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int t = mt * 16 + h * 8 + g;
      aok[mt][h] = t < M;
      arow[mt][h] = A + (long long)(aok[mt][h] ? t : 0) * lda;
    }
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 wv[2][ROWS_UNROLL];

  auto load_batch = [&](int j, int tile_no, int in_tile, uint4 (&dst)[ROWS_UNROLL]) {
    const int r = (first + tile_no * warps) * 8 + g;
    const bool rok = j < total && r < N;
    const __nv_bfloat16* wrow = W + (long long)(rok ? r : 0) * ldw;
#pragma unroll
    for (int u = 0; u < ROWS_UNROLL; ++u) {
      const int k = (in_tile * ROWS_UNROLL + u) * 32 + c * 8;
      dst[u] = (rok && k < K) ? ld_stream(wrow + k) : zero;
    }
  };
  auto compute_batch = [&](int in_tile, const uint4 (&src)[ROWS_UNROLL]) {
#pragma unroll
    for (int u = 0; u < ROWS_UNROLL; ++u) {
      const int k = (in_tile * ROWS_UNROLL + u) * 32 + c * 8;
      const bool kok = k < K;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        uint4 lo = (kok && aok[mt][0]) ? __ldg((const uint4*)(arow[mt][0] + k)) : zero;
        uint4 hi = (kok && aok[mt][1]) ? __ldg((const uint4*)(arow[mt][1] + k)) : zero;
        mma_bf16(acc[mt], lo.x, hi.x, lo.y, hi.y, src[u].x, src[u].y);
        mma_bf16(acc[mt], lo.z, hi.z, lo.w, hi.w, src[u].z, src[u].w);
      }
    }
  };
  // acc[mt] = {(token g, rows 2c, 2c+1), (token g+8, rows 2c, 2c+1)} of the tile
  auto finish_tile = [&](int tile_no) {
    const int n0 = (first + tile_no * warps) * 8;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if constexpr (EPI == EPI_SWIGLU) {
        // rows 0-3 gate, 4-7 up: lanes c = 0,1 hold gate, c = 2,3 the matching up values
        float u0 = __shfl_xor_sync(0xffffffffu, acc[mt][0], 2), u1 = __shfl_xor_sync(0xffffffffu, acc[mt][1], 2);
        float u2 = __shfl_xor_sync(0xffffffffu, acc[mt][2], 2), u3 = __shfl_xor_sync(0xffffffffu, acc[mt][3], 2);
        if (c < 2) {
          const int col = n0 / 2 + 2 * c;
          const float gv[4] = {acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]};
          const float uv[4] = {u0, u1, u2, u3};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int t = mt * 16 + h * 8 + g;
            if (t >= M) continue;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              if (col + e >= N / 2) continue;
              float gate = gv[2 * h + e], up = uv[2 * h + e];
              C[(long long)t * ldc + col + e] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
            }
          }
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int t = mt * 16 + h * 8 + g;
          if (t >= M) continue;
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = n0 + 2 * c + e;
            if (col >= N) continue;
            const long long o = (long long)t * ldc + col;
            const float v = acc[mt][2 * h + e];
            if constexpr (EPI == EPI_ACCUM) C[o] = to_f32<TOut>(C[o]) + v;
            else C[o] = from_f32<TOut>(v);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][i] = 0.f;
    }
  };

  load_batch(0, 0, 0, wv[0]);
  pdl_wait();
  pdl_launch_dependents();
  int tile_no = 0, in_tile = 0;
  auto next = [&](int& t, int& b) { if (++b == bpt) { b = 0; ++t; } };
  for (int j = 0; j < total; j += 2) {
    int t1 = tile_no, b1 = in_tile;
    next(t1, b1);
    load_batch(j + 1, t1, b1, wv[1]);
    compute_batch(in_tile, wv[0]);
    if (in_tile == bpt - 1) finish_tile(tile_no);
    if (j + 1 < total) {
      int t2 = t1, b2 = b1;
      next(t2, b2);
      load_batch(j + 2, t2, b2, wv[0]);
      compute_batch(b1, wv[1]);
      if (b1 == bpt - 1) finish_tile(t1);
      tile_no = t2;
      in_tile = b2;
    }
  }
}

// The product for at most 8 tokens with the tokens held in registers.  In the two kernels above
// every 16-byte weight load is matched by a 16-byte load of token values from L1, which costs a
// quarter of the time of a large product.  Here warp w of a CTA owns the same 256 columns of
// every 2048-column pass over K, so its token fragments (8 tokens x 256 values, 32 registers per
// lane) are loaded once per pass and serve every weight row the CTA reads.  A CTA owns a
// contiguous range of 8-row tiles (the ranges differ by at most one tile, whatever N is); the
// warps' partial sums of a group of up to 8 tiles meet in shared memory (pass after pass in pass
// order, then added in warp order: one fixed order whatever M is) and are written 64 columns wide.
// NORM (K of at most one pass) makes the token fragments from float32 rows: the RMS norm fused in
// front, computed once per CTA from the very loads that fill the fragments.
constexpr int SL_WARPS = 8;
constexpr int SL_STEPS = 8;                              // k32 steps per warp and pass
constexpr int SL_SLICE = SL_STEPS * 32;                  // 256 columns per warp and pass
constexpr int SL_PASS = SL_WARPS * SL_SLICE;             // 2048 columns per pass
constexpr int SL_GROUP = 8;                              // row tiles whose sums are added together
constexpr int SL_TOKEN_PITCH = SL_GROUP * 8 + 8;         // floats per token row of the partial sums (padded)

template <int EPI, bool NORM, typename TOut>
__global__ void __launch_bounds__(SL_WARPS * 32, 2)
gemm_stream_slices_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ W,
                          long long ldw, TOut* __restrict__ C, long long ldc, int M, int N, int K, NormArgs norm) {
  __shared__ __align__(16) float red[2][SL_WARPS][8][SL_TOKEN_PITCH];
  __shared__ __align__(16) float norm_w[NORM ? SL_PASS : 4];       // NORM: the scales of this pass, staged before the wait
  __shared__ float sq_part[SL_WARPS][8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int n_tiles = (N + 7) / 8;
  const int t_begin = (int)((long long)blockIdx.x * n_tiles / gridDim.x);
  const int my_tiles = (int)((long long)(blockIdx.x + 1) * n_tiles / gridDim.x) - t_begin;
  const int passes = (K + SL_PASS - 1) / SL_PASS;
  const int total = my_tiles * passes;                   // (tile, pass) units of this warp

  struct Unit { int grp, pass, tig; };                   // group of tiles, pass over K, tile in the group
  auto group_size = [&](int grp) { return min(SL_GROUP, my_tiles - grp * SL_GROUP); };
  auto advance = [&](Unit& s) {
    if (++s.tig == group_size(s.grp)) {
      s.tig = 0;
      if (++s.pass == passes) { s.pass = 0; ++s.grp; }
    }
  };
  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 wv[2][SL_STEPS];
  auto load_unit = [&](bool valid, const Unit& s, uint4 (&dst)[SL_STEPS]) {
    const int r = (t_begin + s.grp * SL_GROUP + s.tig) * 8 + g;
    const bool rok = valid && r < N;
    const __nv_bfloat16* wrow = W + (long long)(rok ? r : 0) * ldw + s.pass * SL_PASS + warp * SL_SLICE + c * 8;
    const int k0 = s.pass * SL_PASS + warp * SL_SLICE + c * 8;
#pragma unroll
    for (int u = 0; u < SL_STEPS; ++u) dst[u] = (rok && k0 + u * 32 < K) ? ld_stream(wrow + u * 32) : zero;
  };

  Unit cur{0, 0, 0};
  load_unit(total > 0, cur, wv[0]);
  const bool tok_ok = g < M;            // this lane's token: row g of the MMA's A tile; rows 8-15 stay zero
  const float* xrow = nullptr;
  if constexpr (NORM) {
    // NORM covers K <= one pass.  The scales do not come from the previous kernel: warp w stages the
    // 256 of its columns before the wait.
#pragma unroll
    for (int i = 0; i < SL_SLICE / 128; ++i) {
      const int k = warp * SL_SLICE + (lane + i * 32) * 4;
      float4 v = k < K ? __ldg((const float4*)(norm.weight + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (norm.add_unit) { v.x += 1.f; v.y += 1.f; v.z += 1.f; v.w += 1.f; }
      *reinterpret_cast<float4*>(&norm_w[k]) = v;
    }
    if (tok_ok) xrow = norm.x + (long long)(norm.rows ? norm.rows[g] : g) * norm.ldx;     // host-written gather
  }
  pdl_wait();
  pdl_launch_dependents();

  const __nv_bfloat16* arow = A + (long long)(tok_ok ? g : 0) * lda;
  uint4 a_lo[SL_STEPS];
  int a_pass = -1;
  if constexpr (NORM) {
    // This lane's 64 values of token g (all requested at once), their squares summed over the quad,
    // the warps' sums added in warp order: one fixed order whatever the batch is.  Then
    // a = bf16(x * rsqrt(mean(x^2) + eps) * w), as the norm kernel computes it.
    const int k0 = warp * SL_SLICE + c * 8;
    float4 xv[2 * SL_STEPS];
#pragma unroll
    for (int u = 0; u < SL_STEPS; ++u) {
      const int k = k0 + u * 32;
      const bool ok = tok_ok && k < K;
      xv[2 * u] = ok ? __ldg((const float4*)(xrow + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
      xv[2 * u + 1] = ok ? __ldg((const float4*)(xrow + k + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 2 * SL_STEPS; ++i) {
      ss = fmaf(xv[i].x, xv[i].x, ss); ss = fmaf(xv[i].y, xv[i].y, ss);
      ss = fmaf(xv[i].z, xv[i].z, ss); ss = fmaf(xv[i].w, xv[i].w, ss);
    }
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    if (c == 0) sq_part[warp][g] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < SL_WARPS; ++w) tot += sq_part[w][g];
    const float scale = 1.0f / sqrtf(tot / (float)K + norm.eps);
#pragma unroll
    for (int u = 0; u < SL_STEPS; ++u) {
      const int k = k0 + u * 32;
      if (!tok_ok || k >= K) { a_lo[u] = zero; continue; }
      const float4 n0 = *reinterpret_cast<const float4*>(&norm_w[k]), n1 = *reinterpret_cast<const float4*>(&norm_w[k + 4]);
      const float4 x0 = xv[2 * u], x1 = xv[2 * u + 1];
      a_lo[u].x = pack2(x0.x * scale * n0.x, x0.y * scale * n0.y);
      a_lo[u].y = pack2(x0.z * scale * n0.z, x0.w * scale * n0.w);
      a_lo[u].z = pack2(x1.x * scale * n1.x, x1.y * scale * n1.y);
      a_lo[u].w = pack2(x1.z * scale * n1.z, x1.w * scale * n1.w);
    }
    a_pass = 0;
  }
  auto load_tokens = [&](int pass) {
    const int k0 = pass * SL_PASS + warp * SL_SLICE + c * 8;
#pragma unroll
    for (int u = 0; u < SL_STEPS; ++u) {
      const int k = k0 + u * 32;
      a_lo[u] = (tok_ok && k < K) ? __ldg((const uint4*)(arow + k)) : zero;
    }
    a_pass = pass;
  };

  // sums of a finished group: warps in warp order, then the epilogue, 64 (SwiGLU: 32) columns per token
  auto finish_group = [&](int grp) {
    const int gs = group_size(grp);
    const int t0 = t_begin + grp * SL_GROUP;
    const float (*part)[8][SL_TOKEN_PITCH] = red[grp & 1];
    if constexpr (EPI == EPI_SWIGLU) {
      // rows of a tile: [gate x4 | up x4] -> 4 outputs at columns tile*4 ..
      const int t = threadIdx.x >> 5, o = threadIdx.x & 31;
      const int tile = o >> 2, i = o & 3;
      const long long col = (long long)(t0 + tile) * 4 + i;
      if (t < M && tile < gs && col < N / 2) {
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < SL_WARPS; ++w) { gate += part[w][t][tile * 8 + i]; up += part[w][t][tile * 8 + 4 + i]; }
        C[(long long)t * ldc + col] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = (threadIdx.x >> 6) + h * 4, o = threadIdx.x & 63;
        const long long col = (long long)t0 * 8 + o;
        if (t < M && o < gs * 8 && col < N) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < SL_WARPS; ++w) v += part[w][t][o];
          const long long at = (long long)t * ldc + col;
          if constexpr (EPI == EPI_ACCUM) C[at] = to_f32<TOut>(C[at]) + v;
          else C[at] = from_f32<TOut>(v);
        }
      }
    }
  };

  auto process = [&](const Unit& s, const uint4 (&src)[SL_STEPS]) {
    if (s.pass != a_pass) load_tokens(s.pass);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < SL_STEPS; ++u) {
      mma_bf16(acc, a_lo[u].x, 0u, a_lo[u].y, 0u, src[u].x, src[u].y);
      mma_bf16(acc, a_lo[u].z, 0u, a_lo[u].w, 0u, src[u].z, src[u].w);
    }
    // acc[0], acc[1] = (token g, rows 2c, 2c+1) of the tile over this warp's columns of this pass
    float2* dst = reinterpret_cast<float2*>(&red[s.grp & 1][warp][g][s.tig * 8 + 2 * c]);
    if (s.pass == 0) *dst = make_float2(acc[0], acc[1]);
    else { float2 old = *dst; *dst = make_float2(old.x + acc[0], old.y + acc[1]); }
    if (s.pass == passes - 1 && s.tig == group_size(s.grp) - 1) {
      // the other buffer is free again once every warp has passed this barrier: its sums were
      // read before the barrier of the group before
      __syncthreads();
      finish_group(s.grp);
    }
  };

  for (int j = 0; j < total; j += 2) {
    Unit n1 = cur;
    advance(n1);
    load_unit(j + 1 < total, n1, wv[1]);
    process(cur, wv[0]);
    if (j + 1 < total) {
      Unit n2 = n1;
      advance(n2);
      load_unit(j + 2 < total, n2, wv[0]);
      process(n1, wv[1]);
      cur = n2;
    }
  }
}

// 9 to 16 tokens, K of at most 2,048: one CTA of 16 warps per SM; warp w owns columns [128 w, 128 w + 128)
// and keeps both halves of the MMA's token tile for them in registers (32 registers), with four batches
// of four weight loads in flight.  Half as many CTAs as above read the tokens, so the token traffic (every
// CTA reads all of it) stays what it is for 8 tokens.
constexpr int WD_WARPS = 16;
constexpr int WD_STEPS = 4;
constexpr int WD_SLICE = WD_STEPS * 32;                  // 128 columns per warp
constexpr int WD_DEPTH = 4;

template <int EPI, typename TOut>
__global__ void __launch_bounds__(WD_WARPS * 32, 1)
gemm_stream_wide_kernel(const __nv_bfloat16* __restrict__ A, long long lda, const __nv_bfloat16* __restrict__ W,
                        long long ldw, TOut* __restrict__ C, long long ldc, int M, int N, int K) {
  extern __shared__ __align__(16) float red_raw[];       // [WD_WARPS][16][SL_TOKEN_PITCH]
  float (*red)[16][SL_TOKEN_PITCH] = reinterpret_cast<float (*)[16][SL_TOKEN_PITCH]>(red_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int n_tiles = (N + 7) / 8;
  const int t_begin = (int)((long long)blockIdx.x * n_tiles / gridDim.x);
  const int total = (int)((long long)(blockIdx.x + 1) * n_tiles / gridDim.x) - t_begin;      // one pass: a unit is a tile

  const uint4 zero = make_uint4(0, 0, 0, 0);
  uint4 wv[WD_DEPTH][WD_STEPS];
  const int k0 = warp * WD_SLICE + c * 8;
  auto load_unit = [&](int unit, uint4 (&dst)[WD_STEPS]) {
    const int r = (t_begin + unit) * 8 + g;
    const bool rok = unit < total && r < N;
    const __nv_bfloat16* wrow = W + (long long)(rok ? r : 0) * ldw + k0;
#pragma unroll
    for (int u = 0; u < WD_STEPS; ++u) dst[u] = (rok && k0 + u * 32 < K) ? ld_stream(wrow + u * 32) : zero;
  };
#pragma unroll
  for (int d = 0; d < WD_DEPTH - 1; ++d) load_unit(d, wv[d]);
  pdl_wait();
  pdl_launch_dependents();

  uint4 a_lo[WD_STEPS], a_hi[WD_STEPS];
  {
    const bool lo_ok = g < M, hi_ok = g + 8 < M;
    const __nv_bfloat16* row_lo = A + (long long)(lo_ok ? g : 0) * lda + k0;
    const __nv_bfloat16* row_hi = A + (long long)(hi_ok ? g + 8 : 0) * lda + k0;
#pragma unroll
    for (int u = 0; u < WD_STEPS; ++u) {
      a_lo[u] = (lo_ok && k0 + u * 32 < K) ? __ldg((const uint4*)(row_lo + u * 32)) : zero;
      a_hi[u] = (hi_ok && k0 + u * 32 < K) ? __ldg((const uint4*)(row_hi + u * 32)) : zero;
    }
  }

  auto group_size = [&](int grp) { return min(SL_GROUP, total - grp * SL_GROUP); };
  auto finish_group = [&](int grp) {
    const int gs = group_size(grp);
    const int t0 = t_begin + grp * SL_GROUP;
    if constexpr (EPI == EPI_SWIGLU) {
      const int t = threadIdx.x >> 5, o = threadIdx.x & 31;             // 16 tokens x 32 outputs = 512 threads
      const int tile = o >> 2, i = o & 3;
      const long long col = (long long)(t0 + tile) * 4 + i;
      if (t < M && tile < gs && col < N / 2) {
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < WD_WARPS; ++w) { gate += red[w][t][tile * 8 + i]; up += red[w][t][tile * 8 + 4 + i]; }
        C[(long long)t * ldc + col] = from_f32<TOut>(gate / (1.f + expf(-gate)) * up);
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int t = (threadIdx.x >> 6) + h * 8, o = threadIdx.x & 63;  // 16 tokens x 64 columns = 2 x 512
        const long long col = (long long)t0 * 8 + o;
        if (t < M && o < gs * 8 && col < N) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < WD_WARPS; ++w) v += red[w][t][o];
          const long long at = (long long)t * ldc + col;
          if constexpr (EPI == EPI_ACCUM) C[at] = to_f32<TOut>(C[at]) + v;
          else C[at] = from_f32<TOut>(v);
        }
      }
    }
  };
  auto process = [&](int unit, const uint4 (&src)[WD_STEPS]) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int u = 0; u < WD_STEPS; ++u) {
      mma_bf16(acc, a_lo[u].x, a_hi[u].x, a_lo[u].y, a_hi[u].y, src[u].x, src[u].y);
      mma_bf16(acc, a_lo[u].z, a_hi[u].z, a_lo[u].w, a_hi[u].w, src[u].z, src[u].w);
    }
    const int tig = unit % SL_GROUP, grp = unit / SL_GROUP;
    *reinterpret_cast<float2*>(&red[warp][g][tig * 8 + 2 * c]) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2*>(&red[warp][g + 8][tig * 8 + 2 * c]) = make_float2(acc[2], acc[3]);
    if (tig == group_size(grp) - 1) {
      __syncthreads();
      finish_group(grp);
      __syncthreads();                                   // the sums have been read: the next group may overwrite them
    }
  };

  for (int j = 0; j < total; j += WD_DEPTH) {
#pragma unroll
    for (int d = 0; d < WD_DEPTH; ++d) {
      if (j + d < total) {
        load_unit(j + d + WD_DEPTH - 1, wv[(d + WD_DEPTH - 1) % WD_DEPTH]);
        process(j + d, wv[d]);
      }
    }
  }
}

int launch_wide(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int out_dtype,
                int epilogue, int M, int N, int K, cudaStream_t stream) {
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  const int sms = hfee_sm_count();
  if (sms <= 0) return hfee_fail(HFEE_ERR_CUDA, "gemm_stream: cannot ask the device for its number of SMs");
  const int n_tiles = (N + 7) / 8;
  unsigned grid = (unsigned)(n_tiles < sms ? n_tiles : sms);
  constexpr int RED_BYTES = WD_WARPS * 16 * SL_TOKEN_PITCH * 4;
#define HFEE_GO(EPI, T)                                                                                                   \
  do {                                                                                                                    \
    static bool configured = false;                                                                                       \
    if (!configured) {                                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(gemm_stream_wide_kernel<EPI, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, RED_BYTES); \
      if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "gemm_stream: cannot get shared memory: %s", cudaGetErrorString(e)); \
      configured = true;                                                                                                  \
    }                                                                                                                     \
    hfee_launch(gemm_stream_wide_kernel<EPI, T>, dim3(grid), dim3(WD_WARPS * 32), RED_BYTES, stream, a, lda, w, ldw, (T*)C, ldc, M, N, K); \
  } while (0)
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_stream: accumulate needs a float32 output");
    HFEE_GO(EPI_ACCUM, float);
  } else if (epilogue == EPI_SWIGLU) {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_SWIGLU, __nv_bfloat16); else HFEE_GO(EPI_SWIGLU, float);
  } else {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_STORE, __nv_bfloat16); else HFEE_GO(EPI_STORE, float);
  }
#undef HFEE_GO
  return hfee_check_launch("gemm_stream_wide");
}

template <bool NORM>
int launch_slices(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int out_dtype,
                  int epilogue, int M, int N, int K, const NormArgs& norm, cudaStream_t stream) {
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  const int resident = 2 * hfee_sm_count();
  if (resident <= 0) return hfee_fail(HFEE_ERR_CUDA, "gemm_stream: cannot ask the device for its number of SMs");
  const int n_tiles = (N + 7) / 8;
  unsigned grid = (unsigned)(n_tiles < resident ? n_tiles : resident);
#define HFEE_GO(EPI, T) hfee_launch(gemm_stream_slices_kernel<EPI, NORM, T>, dim3(grid), dim3(SL_WARPS * 32), 0, stream, a, lda, w, ldw, (T*)C, ldc, M, N, K, norm)
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_stream: accumulate needs a float32 output");
    HFEE_GO(EPI_ACCUM, float);
  } else if (epilogue == EPI_SWIGLU) {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_SWIGLU, __nv_bfloat16); else HFEE_GO(EPI_SWIGLU, float);
  } else {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_STORE, __nv_bfloat16); else HFEE_GO(EPI_STORE, float);
  }
#undef HFEE_GO
  return hfee_check_launch("gemm_stream_slices");
}

template <int MT, int NT, int NW>
int launch(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int out_dtype,
           int epilogue, int M, int N, int K, cudaStream_t stream) {
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  static int resident = 0;                       // CTAs of this instantiation the whole GPU holds at once
  if (resident == 0) {
    int per_sm = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_stream_kernel<MT, NT, NW, EPI_STORE, float>, NW * 32, 0);
    resident = hfee_sm_count() * (per_sm > 0 ? per_sm : 1);
    if (resident <= 0) return hfee_fail(HFEE_ERR_CUDA, "gemm_stream: cannot ask the device for its number of SMs");
  }
  int n_tiles = (N + 8 * NT - 1) / (8 * NT);
  unsigned grid = (unsigned)(n_tiles < resident ? n_tiles : resident);
#define HFEE_GO(EPI, T) hfee_launch(gemm_stream_kernel<MT, NT, NW, EPI, T>, dim3(grid), dim3(NW * 32), 0, stream, a, lda, w, ldw, (T*)C, ldc, M, N, K)
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_stream: accumulate needs a float32 output");
    HFEE_GO(EPI_ACCUM, float);
  } else if (epilogue == EPI_SWIGLU) {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_SWIGLU, __nv_bfloat16); else HFEE_GO(EPI_SWIGLU, float);
  } else {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_STORE, __nv_bfloat16); else HFEE_GO(EPI_STORE, float);
  }
#undef HFEE_GO
  return hfee_check_launch("gemm_stream");
}

}  // namespace

namespace {
template <int MT>
int launch_rows(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int out_dtype,
                int epilogue, int M, int N, int K, cudaStream_t stream) {
  const __nv_bfloat16* a = (const __nv_bfloat16*)A;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  int n_tiles = (N + 7) / 8;
  int ctas = (n_tiles + ROWS_WARPS - 1) / ROWS_WARPS;
  const int resident = 2 * hfee_sm_count();              // two CTAs of this kernel share an SM
  if (resident <= 0) return hfee_fail(HFEE_ERR_CUDA, "gemm_stream: cannot ask the device for its number of SMs");
  unsigned grid = (unsigned)(ctas < resident ? ctas : resident);
#define HFEE_GO(EPI, T) hfee_launch(gemm_stream_rows_kernel<MT, EPI, T>, dim3(grid), dim3(ROWS_WARPS * 32), 0, stream, a, lda, w, ldw, (T*)C, ldc, M, N, K)
  if (epilogue == EPI_ACCUM) {
    if (out_dtype != HFEE_F32) return hfee_fail(HFEE_ERR_ARG, "gemm_stream: accumulate needs a float32 output");
    HFEE_GO(EPI_ACCUM, float);
  } else if (epilogue == EPI_SWIGLU) {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_SWIGLU, __nv_bfloat16); else HFEE_GO(EPI_SWIGLU, float);
  } else {
    if (out_dtype == HFEE_BF16) HFEE_GO(EPI_STORE, __nv_bfloat16); else HFEE_GO(EPI_STORE, float);
  }
#undef HFEE_GO
  return hfee_check_launch("gemm_stream_rows");
}

// Enough 8-row tiles to give every resident warp (148 SMs x 16) about one: a warp per tile.
constexpr int ROWS_MIN_TILES = 1536;

int by_tokens(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc, int out_dtype,
              int epilogue, int M, int N, int K, cudaStream_t stream) {
  if (M <= 16) return launch<1, 1, 16>(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
  if (M <= 32) return launch<2, 2, 8>(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
  return launch<4, 4, 4>(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
}

int check_common(const void* W, long long ldw, long long ldc, int epilogue, int M, int N, int K) {
  HFEE_REQUIRE(M > 0 && M <= 64, "gemm_stream: M=%d is outside 1..64", M);
  HFEE_REQUIRE(N > 0 && K > 0 && K % 8 == 0, "gemm_stream: K=%d must be a positive multiple of 8", K);
  HFEE_REQUIRE(ldw % 8 == 0 && ldw >= K, "gemm_stream: the weights' leading dimension %lld must be a multiple of 8 and at least K", ldw);
  HFEE_REQUIRE((uintptr_t)W % 16 == 0, "gemm_stream: weights must be 16-byte aligned");
  HFEE_REQUIRE(epilogue >= 0 && epilogue <= 2, "gemm_stream: unknown epilogue %d", epilogue);
  HFEE_REQUIRE(epilogue != EPI_SWIGLU || N % 8 == 0, "gemm_stream: SwiGLU needs N %% 8 == 0, got %d", N);
  HFEE_REQUIRE(ldc >= (epilogue == EPI_SWIGLU ? N / 2 : N), "gemm_stream: ldc=%lld is too small", ldc);
  return HFEE_OK;
}
}  // namespace

// epilogue: 0 store, 1 accumulate into float32 C, 2 SwiGLU (C is [M, N/2]; N % 8 == 0).
HFEE_API int hfee_gemm_stream(const void* A, long long lda, const void* W, long long ldw, void* C, long long ldc,
                              int out_dtype, int epilogue, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  int rc = check_common(W, ldw, ldc, epilogue, M, N, K);
  if (rc != HFEE_OK) return rc;
  HFEE_REQUIRE(lda % 8 == 0 && lda >= K && (uintptr_t)A % 16 == 0,
               "gemm_stream: the tokens' leading dimension %lld must be a multiple of 8, at least K, and 16-byte aligned", lda);
  NormArgs none{nullptr, 0, nullptr, nullptr, 0.f, 0};
  if (M <= 8) return launch_slices<false>(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, none, stream);
  if (M <= 16 && K <= WD_WARPS * WD_SLICE) return launch_wide(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
  if ((N + 7) / 8 >= ROWS_MIN_TILES && M <= 32) {
    if (M <= 16) return launch_rows<1>(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
    return launch_rows<2>(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
  }
  return by_tokens(A, lda, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, stream);
}

// The same with the RMS norm of float32 rows X fused in front: tokens = bf16(norm(X[rows])).  For at
// most 8 tokens and K <= 2048 (the kernel that keeps the tokens in registers); other shapes are
// refused: run the norm kernel and hfee_gemm_stream instead.
HFEE_API int hfee_gemm_stream_norm(const float* X, long long ldx, const int* rows, const float* norm_weight,
                                   float eps, int add_unit, const void* W, long long ldw, void* C, long long ldc,
                                   int out_dtype, int epilogue, int M, int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return HFEE_OK;
  int rc = check_common(W, ldw, ldc, epilogue, M, N, K);
  if (rc != HFEE_OK) return rc;
  HFEE_REQUIRE(M <= 8 && K <= SL_PASS, "gemm_stream_norm: the fused norm takes at most 8 tokens and K <= %d (got M=%d, K=%d)", SL_PASS, M, K);
  HFEE_REQUIRE(ldx % 4 == 0 && ldx >= K && (uintptr_t)X % 16 == 0 && (uintptr_t)norm_weight % 16 == 0,
               "gemm_stream_norm: float32 rows need a leading dimension %% 4 == 0 and 16-byte alignment");
  NormArgs norm{X, ldx, rows, norm_weight, eps, add_unit};
  return launch_slices<true>(nullptr, 0, W, ldw, C, ldc, out_dtype, epilogue, M, N, K, norm, stream);
}
