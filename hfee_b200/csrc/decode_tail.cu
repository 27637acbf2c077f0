// The tail of a decoder layer for a decode step of at most 8 tokens, as ONE persistent kernel:
//
//   phase A   residual += att . W_o^T                          (output projection of the mixer)
//   phase B   h = silu(g) * u,  (g, u) = rmsnorm(residual) . W_gate_up^T
//   phase C   residual += h . W_down^T
//
// Reference math: hostfog/hfee internal/llm/forward.go:106-114, internal/ggml/ops.go:125-134,160-165.
//
// A decode step of a few tokens reads every weight once and computes almost nothing, so its time
// is the time to stream the weights plus whatever latency is exposed between dependent products.
// As separate kernels each product pays a launch boundary and ramps its loads up from nothing.
// Here one CTA per SM owns a fixed share of the rows of all three matrices; a producer warp
// streams that share, in the order it will be used, through one ring of shared-memory stages, one
// TMA box per stage: [8 slabs of 64 k][up to 16 rows] in the 128-byte swizzle, which `ldmatrix`
// reads without bank conflicts (a copy per weight row, `cp.async.bulk` of 1 KB each, reached only
// 2.5 TB/s: the copy engine wants few, large requests).  The weight stream does not depend on any activation: it
// starts before the previous kernel has finished (programmatic dependent launch) and runs on
// across the two grid-wide barriers that separate the phases, so HBM stays busy while the CTAs
// wait for each other.  Eight consumer warps take every eighth 16-wide k step of a stage
// (`mma.sync.m16n8k16`: 16 weight rows x 8 tokens), sum their partial tiles through shared
// memory in warp order and apply the epilogue.  Tokens: phases A and C get theirs (att, h) in
// chunks, a stage at a time, from a second producer warp, which waits for what they depend on.
// The norm between A and B is split so that no CTA reads the whole float32 residual (148 SMs
// reading the same 64 KB at the same moment took 5 us): the CTA that owns a column in phase A also
// writes y = bf16(x * w_norm) for it and adds x^2 to its own partial sums; after the barrier every
// CTA adds the partial sums in CTA order, fetches y (bfloat16, half the bytes, by TMA) and applies
// the rows' scales 1/sqrt(mean x^2 + eps) to its gate/up sums after the MMAs.
//
// Everything a CTA waits for has a time limit; a wait that runs out sets the status word.
#include "tcgen05.cuh"
#include <stdlib.h>

namespace {

using namespace tc;

constexpr int KC = 512;                          // k elements of a stage: 8 slabs of 64
constexpr int SLABS = KC / 64;
constexpr int TILE_ROWS = 16;                    // most weight rows of a stage: one MMA tile
constexpr int MAX_TOKENS = 8;
constexpr int CONSUMER_WARPS = 8;
constexpr int THREADS = 32 * (2 + CONSUMER_WARPS);
constexpr int W_BYTES = SLABS * TILE_ROWS * 128;         // 16 KB: a stage of weights, [slab][row][64 k]
constexpr int T_BYTES = SLABS * MAX_TOKENS * 128;        // 8 KB:  a stage of tokens,  [slab][token][64 k]
constexpr int T_STAGES = 4;
constexpr int RED_BYTES = CONSUMER_WARPS * TILE_ROWS * MAX_TOKENS * 4;
constexpr int MAX_STAGES = 12;
constexpr int SMALL_BYTES = (TILE_ROWS * MAX_TOKENS + 2 * MAX_TOKENS) * 4;      // squares of a tile, scales, sums
constexpr int BAR_BYTES = (2 * MAX_STAGES + 2 * T_STAGES + 4) * 8 + 16;
static_assert(W_BYTES % 1024 == 0 && T_BYTES % 1024 == 0, "the swizzle needs 1024-byte aligned tiles");

// Shared memory: the ring of weight stages; one region that holds the token stages of phases A and C
// and, between them, the whole input of phase B; the warps' partial tiles; small arrays; the barriers.
__host__ __device__ inline long long token_region_bytes(int D) {
  long long y = (long long)((D + KC - 1) / KC) * T_BYTES;          // all of y, in boxes of 8 slabs
  return y > T_STAGES * T_BYTES ? y : T_STAGES * T_BYTES;
}

struct TailArgs {
  float* residual; long long ld_res;               // [M, D]
  const float* norm_w; float eps; int add_unit;    // [D]
  __nv_bfloat16* h; long long ld_h;                // [M, I]
  __nv_bfloat16* y; long long ld_y;                // [M, D]: x * w_norm, the un-scaled input of phase B
  float* ssq;                                      // [CTAs, 8]: each CTA's share of the rows' sums of squares
  int M, D, Q, I;
  int tile_rows[3];                                // weight rows per stage in each phase (the TMA boxes' height)
  int stages;
  unsigned int* sync;                              // [0] arrivals at the grid barriers, [1] CTAs that have left
  int* status;
};

struct Phase {
  bool streamed_tokens;                            // false: the tokens are in shared memory (phase B)
  int K, r0, r1, tile;
};

__device__ __forceinline__ Phase phase_of(const TailArgs& a, int which, int cta, int ctas) {
  Phase p;
  p.tile = a.tile_rows[which];
  if (which == 1) {
    const int units = a.I / 4;                     // 8 rows each: 4 gate, 4 up -> 4 outputs
    p.streamed_tokens = false; p.K = a.D;
    p.r0 = 8 * (int)((long long)cta * units / ctas); p.r1 = 8 * (int)((long long)(cta + 1) * units / ctas);
  } else {
    p.streamed_tokens = true; p.K = which == 0 ? a.Q : a.I;
    p.r0 = (int)((long long)cta * a.D / ctas); p.r1 = (int)((long long)(cta + 1) * a.D / ctas);
  }
  return p;
}

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

__device__ __forceinline__ unsigned int load_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

#ifdef DT_TRACE
__device__ long long dt_trace[4 * 256];
#define DTRACE(row, i) do { if (blockIdx.x == DT_TRACE && (i) < 256) dt_trace[(row) * 256 + (i)] = clock64(); } while (0)
#else
#define DTRACE(row, i) do {} while (0)
#endif

__global__ void __launch_bounds__(THREADS, 1)
decode_tail_kernel(const __grid_constant__ CUtensorMap map_wo, const __grid_constant__ CUtensorMap map_wgu,
                   const __grid_constant__ CUtensorMap map_wdown, const __grid_constant__ CUtensorMap map_att,
                   const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_y, TailArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* ring = smem;                                          // 1024-byte aligned (checked below)
  unsigned char* tokens = ring + a.stages * W_BYTES;                   // token stages (A, C) / all of y (B)
  float* red = reinterpret_cast<float*>(tokens + token_region_bytes(a.D));
  float* squares = red + CONSUMER_WARPS * TILE_ROWS * MAX_TOKENS;      // [16 rows][8 tokens] of the tile in hand
  float* scale_s = squares + TILE_ROWS * MAX_TOKENS;                   // [8] 1/sqrt(mean x^2 + eps) per token
  uint64_t* w_full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(red) + RED_BYTES + SMALL_BYTES);
  uint64_t* w_empty = w_full + MAX_STAGES;
  uint64_t* t_full = w_empty + MAX_STAGES;
  uint64_t* t_empty = t_full + T_STAGES;
  uint64_t* y_ready = t_empty + T_STAGES;                              // the grid is past barrier 1: y is complete
  uint64_t* y_full = y_ready + 1;                                      // y has landed in shared memory
  uint64_t* h_ready = y_full + 1;                                      // the grid is past barrier 2: h is complete
  int& abort_flag = *reinterpret_cast<int*>(h_ready + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, ctas = gridDim.x, S = a.stages;

  if (threadIdx.x == 0) {
    abort_flag = (smem_u32(ring) & 1023u) != 0 ? 1 : 0;       // misaligned tiles would corrupt the swizzle
    for (int s = 0; s < S; ++s) { mbar_init(&w_full[s], 1); mbar_init(&w_empty[s], CONSUMER_WARPS); }
    for (int s = 0; s < T_STAGES; ++s) { mbar_init(&t_full[s], 1); mbar_init(&t_empty[s], CONSUMER_WARPS); }
    mbar_init(h_ready, 1); mbar_init(y_ready, 1); mbar_init(y_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    // ---- weights: free-running, held back only by the ring.  They are nobody's output, so the
    // stream starts while the previous kernel still runs.
    uint32_t it = 0;
    bool ok = true;
    for (int ph = 0; ph < 3 && ok; ++ph) {
      const Phase p = phase_of(a, ph, cta, ctas);
      const CUtensorMap* map = ph == 0 ? &map_wo : (ph == 1 ? &map_wgu : &map_wdown);
      for (int row0 = p.r0; row0 < p.r1 && ok; row0 += p.tile) {
        for (int k0 = 0; k0 < p.K; k0 += KC, ++it) {
          const int s = it % S;
          ok = __all_sync(0xffffffffu, mbar_wait(&w_empty[s], ((it / S) & 1u) ^ 1u, &abort_flag));
          if (!ok) break;
          if (elect_one()) {
            DTRACE(0, it);
            // the box is always whole: rows behind the matrix and slabs behind K arrive as zeros
            mbar_expect_tx(&w_full[s], (uint32_t)(SLABS * p.tile * 128));
            tma_load_3d(ring + s * W_BYTES, map, 0, row0, k0 / 64, &w_full[s]);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    // ---- tokens of phases A (att: the previous kernel's output) and C (h: complete once the grid
    // is past its second barrier), a chunk for each stage of weights, through a small ring of their own
    uint32_t it = 0;
    bool ok = true;
    pdl_wait();
    for (int ph = 0; ph < 3 && ok; ph += 2) {
      const Phase p = phase_of(a, ph, cta, ctas);
      if (ph == 2) {
        // between the phases: all of y, once the grid is past barrier 1 (phase A's token stages, whose
        // place it takes, have all been read by then)
        ok = __all_sync(0xffffffffu, mbar_wait(y_ready, 0, &abort_flag));
        asm volatile("fence.proxy.async;" ::: "memory");          // y was written with ordinary stores by other CTAs
        if (!ok) break;
        if (elect_one()) {
          const int boxes = (a.D + KC - 1) / KC;
          mbar_expect_tx(y_full, (uint32_t)(boxes * T_BYTES));
          for (int b = 0; b < boxes; ++b) tma_load_3d(tokens + b * T_BYTES, &map_y, 0, 0, b * SLABS, y_full);
        }
        __syncwarp();
        // past barrier 2 nobody reads y any more, whose place the stages of h take
        ok = __all_sync(0xffffffffu, mbar_wait(h_ready, 0, &abort_flag));
        asm volatile("fence.proxy.async;" ::: "memory");          // h was written with ordinary stores by other CTAs
        if (!ok) break;
      }
      const CUtensorMap* map = ph == 0 ? &map_att : &map_h;
      for (int row0 = p.r0; row0 < p.r1 && ok; row0 += p.tile) {
        for (int k0 = 0; k0 < p.K; k0 += KC, ++it) {
          const int s = it % T_STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(&t_empty[s], ((it / T_STAGES) & 1u) ^ 1u, &abort_flag));
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&t_full[s], (uint32_t)T_BYTES);
            tma_load_3d(tokens + s * T_BYTES, map, 0, 0, k0 / 64, &t_full[s]);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ---- consumers
    const int cw = warp - 2, ct = threadIdx.x - 64;                 // consumer warp and thread
    const int g = lane >> 2, c = lane & 3;
    uint32_t it = 0, tit = 0, barriers = 0;
    float ssq_mine = 0.f;                                           // thread m < 8: this CTA's share of sum x^2 of token m
    bool ok = true;
    pdl_wait();                                                     // the residual rows are earlier kernels' output

    // All CTAs of the grid meet; afterwards everything any of them wrote before is visible.
    auto grid_barrier = [&]() {
      if (ct == 0) DTRACE(3, barriers * 2);
      consumer_sync();
      ++barriers;
      if (ct == 0) {
        __threadfence();
        atomicAdd(&a.sync[0], 1u);
        const unsigned int target = barriers * (unsigned int)ctas;
        uint64_t t0 = 0;
        for (uint32_t i = 0; load_acquire(&a.sync[0]) < target; ++i) {
          if ((i & 63u) == 63u) {
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_NS || *reinterpret_cast<volatile int*>(&abort_flag)) { abort_flag = 1; break; }
          }
        }
      }
      consumer_sync();
      if (ct == 0) DTRACE(3, barriers * 2 - 1);
      return *reinterpret_cast<volatile int*>(&abort_flag) == 0;
    };

    for (int ph = 0; ph < 3 && ok; ++ph) {
      const Phase p = phase_of(a, ph, cta, ctas);
      if (ph == 1) {
        // every CTA has written its columns of y and its share of the sums of squares
        if (ct < MAX_TOKENS && ct < a.M) a.ssq[cta * MAX_TOKENS + ct] = ssq_mine;
        ok = grid_barrier();
        if (!ok) break;
        if (ct == 0) mbar_arrive(y_ready);
        if (cw < a.M) {                                          // warp m adds token m's shares in CTA order
          float v = 0.f;
          for (int c0 = 0; c0 < ctas; c0 += 32) {
            const float part = c0 + lane < ctas ? __ldcg(a.ssq + (c0 + lane) * MAX_TOKENS + cw) : 0.f;
            v += warp_sum(part);
          }
          if (lane == 0) scale_s[cw] = 1.0f / sqrtf(v / (float)a.D + a.eps);
        }
        consumer_sync();
        ok = __all_sync(0xffffffffu, mbar_wait(y_full, 0, &abort_flag));
        if (!ok) break;
      } else if (ph == 2) {
        ok = grid_barrier();                                        // h is complete
        if (!ok) break;
        if (ct == 0) mbar_arrive(h_ready);
      }
      for (int row0 = p.r0; row0 < p.r1 && ok; row0 += p.tile) {
        const int rows = min(p.tile, p.r1 - row0);
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
        // the epilogue's thread (row, token): what it will add to, and the column's norm weight, are
        // requested now, a whole tile of weights ahead of their use
        const int e_row = ct / MAX_TOKENS, e_m = ct % MAX_TOKENS;
        const bool e_mine = ct < TILE_ROWS * MAX_TOKENS && e_m < a.M && e_row < rows;
        float old = 0.f, wn = 0.f;
        if (e_mine && ph != 1) {
          old = __ldcg(a.residual + (long long)e_m * a.ld_res + row0 + e_row);
          if (ph == 0) wn = __ldg(a.norm_w + row0 + e_row) + (a.add_unit ? 1.f : 0.f);
        }
        for (int k0 = 0; k0 < p.K; k0 += KC, ++it) {
          const int s = it % S, ts = tit % T_STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(&w_full[s], (it / S) & 1u, &abort_flag));
          if (ok && p.streamed_tokens) ok = __all_sync(0xffffffffu, mbar_wait(&t_full[ts], (tit / T_STAGES) & 1u, &abort_flag));
          if (!ok) break;
          if (cw == 0 && lane == 0) DTRACE(1, it);
          // weights: slab j of the stage holds rows 0 .. tile-1 of k 64 j .. 64 j + 63, a row 128 bytes,
          // its 16-byte piece c at position c ^ (128-byte line number mod 8)
          const uint32_t stage = smem_u32(ring + s * W_BYTES), tstage = smem_u32(tokens + ts * T_BYTES);
          const int w_row = min(lane & 15, p.tile - 1);               // rows the box does not have are never stored
          const int steps = min(KC, p.K - k0) / 16;
          // this warp's k steps of the stage (at most KC / 16 / CONSUMER_WARPS = 4): all fragments are
          // requested before the first MMA, and the MMAs alternate between two accumulators
          constexpr int MINE = KC / 16 / CONSUMER_WARPS;
          uint32_t wa[MINE][4], tb[MINE][2];
#pragma unroll
          for (int j = 0; j < MINE; ++j) {
            const int ks = cw + j * CONSUMER_WARPS;
            if (ks < steps) {
              const int slab = ks >> 2, piece = (ks & 3) * 2;
              const int w_line = slab * p.tile + w_row;
              ldmatrix_x4(wa[j], stage + w_line * 128 + (((piece + (lane >> 4)) ^ (w_line & 7)) << 4));
              if (p.streamed_tokens) {
                const int t_line = slab * MAX_TOKENS + (lane & 7);
                ldmatrix_x2(tb[j], tstage + t_line * 128 + (((piece + ((lane >> 3) & 1)) ^ (t_line & 7)) << 4));
              } else {
                const int y_line = (k0 / 64 + slab) * MAX_TOKENS + (lane & 7);          // y: slab after slab, all of K
                ldmatrix_x2(tb[j], smem_u32(tokens) + y_line * 128 + (((piece + ((lane >> 3) & 1)) ^ (y_line & 7)) << 4));
              }
            }
          }
#pragma unroll
          for (int j = 0; j < MINE; ++j)
            if (cw + j * CONSUMER_WARPS < steps) mma_16x8x16(j & 1 ? acc2 : acc, wa[j], tb[j]);
          __syncwarp();
          if (cw == 0 && lane == 0) DTRACE(2, it);
          if (lane == 0) {
            mbar_arrive(&w_empty[s]);
            if (p.streamed_tokens) mbar_arrive(&t_empty[ts]);
          }
          if (p.streamed_tokens) ++tit;
        }
        if (!ok) break;
        // ---- the warps' partial tiles meet in shared memory and are added in warp order
        float* mine = red + cw * (TILE_ROWS * MAX_TOKENS);
        *reinterpret_cast<float2*>(mine + g * MAX_TOKENS + 2 * c) = make_float2(acc[0] + acc2[0], acc[1] + acc2[1]);
        *reinterpret_cast<float2*>(mine + (g + 8) * MAX_TOKENS + 2 * c) = make_float2(acc[2] + acc2[2], acc[3] + acc2[3]);
        consumer_sync();
        float sq = 0.f;
        if (e_mine) {
          const int row = e_row, m = e_m;
          auto total = [&](int r) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; ++w) v += red[w * (TILE_ROWS * MAX_TOKENS) + r * MAX_TOKENS + m];
            return v;
          };
          if (ph != 1) {
            const float x = old + total(row);
            a.residual[(long long)m * a.ld_res + row0 + row] = x;
            if (ph == 0) {                          // what the norm in front of phase B needs of this column
              a.y[(long long)m * a.ld_y + row0 + row] = __float2bfloat16_rn(x * wn);
              sq = x * x;
            }
          } else if ((row & 7) < 4) {
            // rows 8u .. 8u+3 are gate rows, 8u+4 .. 8u+7 the up rows of the same four outputs; the
            // norm's scale of the token comes in here, behind the sums
            const float gate = total(row) * scale_s[m], up = total(row + 4) * scale_s[m];
            const long long col = (long long)((row0 + row) >> 3) * 4 + (row & 3);
            a.h[(long long)m * a.ld_h + col] = __float2bfloat16_rn(__fdividef(gate, 1.f + __expf(-gate)) * up);
          }
        }
        if (ph == 0) {                              // this tile's squares, added row by row for each token
          if (ct < TILE_ROWS * MAX_TOKENS) squares[ct] = sq;
          consumer_sync();
          if (ct < MAX_TOKENS)
            for (int r = 0; r < rows; ++r) ssq_mine += squares[r * MAX_TOKENS + ct];
        }
        consumer_sync();
      }
    }
  }

  pdl_launch_dependents();
  __syncthreads();
  if (abort_flag) {                    // a wait ran out: give copies that may still be in flight time to land
#pragma unroll 1
    for (int i = 0; i < 400; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    DTRACE(3, 8);
    if (abort_flag && a.status != nullptr) atomicExch(a.status, 3);
    // the last CTA to leave puts the barrier words back for the next launch
    __threadfence();
    if (atomicAdd(&a.sync[1], 1u) == (unsigned int)ctas - 1u) {
      a.sync[0] = 0u;
      a.sync[1] = 0u;
      __threadfence();
    }
  }
}

// Stages of the weight ring.  More shared memory per CTA than the kernel needs is not free: the SM's
// carve-out between shared memory and L1 follows the resident kernel, and a kernel that starts right
// behind this one keeps the small L1 it finds (measured: with 213 KB here the streaming product that
// follows took twice as long, with 117 KB it did not, and this kernel was as fast with 5 stages as with
// 11).  So: the smallest of the carve-out steps that holds at least four stages.
int tail_stages(int D) {
  const long long fixed = token_region_bytes(D) + RED_BYTES + SMALL_BYTES + BAR_BYTES;
  const long long steps[] = {131LL * 1024, 163LL * 1024, 195LL * 1024, 227LL * 1024};     // 1 KB is the system's
  long long s = 0;
  for (long long step : steps) {
    s = (step - fixed) / W_BYTES;
    if (s >= 4) break;
  }
  if (const char* cap = getenv("HFEE_TAIL_STAGES")) { long long c = atoll(cap); if (c >= 3 && c < s) s = c; }
  return (int)(s > MAX_STAGES ? MAX_STAGES : s);
}

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
  if (!fn) return hfee_fail(HFEE_ERR_CUDA, "decode_tail: the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(cols / 64)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, 128};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)SLABS};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return hfee_fail(HFEE_ERR_CUDA, "decode_tail: cuTensorMapEncodeTiled failed with %d", (int)r);
  return HFEE_OK;
}

}  // namespace

#ifdef DT_TRACE
HFEE_API int hfee_dt_trace_read(long long* out) { return (int)cudaMemcpyFromSymbol(out, dt_trace, sizeof(dt_trace)); }
#endif

// 1 if hfee_decode_tail takes these sizes (bfloat16 weights and activations are implied).
HFEE_API int hfee_decode_tail_supports(int M, int D, int Q, int I) {
  if (M < 1 || M > MAX_TOKENS) return 0;
  if (D < 64 || Q < 64 || I < 64 || D % 64 || Q % 64 || I % 64) return 0;      // whole 64-wide slabs of k
  if (tail_stages(D) < 3) return 0;
  return 1;
}

// residual[M, D] (float32) += att[M, Q] . w_o[D, Q]^T;  h = swiglu(rmsnorm(residual) . w_gate_up[2 I, D]^T);
// residual += h . w_down[D, I]^T.  `h` [M, I] is scratch for the activations between the last two;
// `y` [M, D] (bfloat16) and `ssq` [number of SMs, 8] (float32) are scratch for the norm; `sync` are two
// zeroed 32-bit words the kernel leaves zeroed.  All matrices bfloat16, row-major.
HFEE_API int hfee_decode_tail(const void* att, long long ld_att, const void* w_o, long long ld_wo, float* residual,
                              long long ld_res, const float* norm_w, float eps, int add_unit, const void* w_gate_up,
                              long long ld_gu, const void* w_down, long long ld_down, void* h, long long ld_h, void* y,
                              long long ld_y, float* ssq, int M, int D, int Q, int I, unsigned int* sync, int* status,
                              cudaStream_t stream) {
  if (M == 0) return HFEE_OK;
  HFEE_REQUIRE(hfee_decode_tail_supports(M, D, Q, I),
               "decode_tail: takes 1..%d tokens and widths that are multiples of 64 (got M=%d D=%d Q=%d I=%d)",
               MAX_TOKENS, M, D, Q, I);
  HFEE_REQUIRE(ld_att % 8 == 0 && ld_wo % 8 == 0 && ld_gu % 8 == 0 && ld_down % 8 == 0 && ld_h % 8 == 0 && ld_res % 4 == 0 &&
               (uintptr_t)att % 16 == 0 && (uintptr_t)w_o % 16 == 0 && (uintptr_t)w_gate_up % 16 == 0 &&
               (uintptr_t)w_down % 16 == 0 && (uintptr_t)h % 16 == 0 && (uintptr_t)residual % 16 == 0 &&
               (uintptr_t)norm_w % 16 == 0 && (uintptr_t)y % 16 == 0 && ld_y % 8 == 0,
               "decode_tail: every row must start on a 16-byte boundary");
  const int sms = hfee_sm_count();
  if (sms <= 0) return hfee_fail(HFEE_ERR_CUDA, "decode_tail: cannot ask the device for its number of SMs");
  TailArgs a;
  a.residual = residual; a.ld_res = ld_res;
  a.norm_w = norm_w; a.eps = eps; a.add_unit = add_unit;
  a.h = (__nv_bfloat16*)h; a.ld_h = ld_h;
  a.y = (__nv_bfloat16*)y; a.ld_y = ld_y; a.ssq = ssq;
  a.M = M; a.D = D; a.Q = Q; a.I = I;
  a.tile_rows[0] = a.tile_rows[2] = tile_height((D + sms - 1) / sms, 1);
  a.tile_rows[1] = tile_height(8 * ((I / 4 + sms - 1) / sms), 8);
  a.stages = tail_stages(D);
  a.sync = sync; a.status = status;
  CUtensorMap m_wo, m_wgu, m_wdown, m_att, m_h, m_y;
  int rc;
  if ((rc = make_slab_map(&m_wo, w_o, D, Q, ld_wo, a.tile_rows[0])) != HFEE_OK) return rc;
  if ((rc = make_slab_map(&m_wgu, w_gate_up, 2LL * I, D, ld_gu, a.tile_rows[1])) != HFEE_OK) return rc;
  if ((rc = make_slab_map(&m_wdown, w_down, D, I, ld_down, a.tile_rows[2])) != HFEE_OK) return rc;
  if ((rc = make_slab_map(&m_att, att, M, Q, ld_att, MAX_TOKENS)) != HFEE_OK) return rc;
  if ((rc = make_slab_map(&m_h, h, M, I, ld_h, MAX_TOKENS)) != HFEE_OK) return rc;
  if ((rc = make_slab_map(&m_y, y, M, D, ld_y, MAX_TOKENS)) != HFEE_OK) return rc;
  const size_t smem = (size_t)a.stages * W_BYTES + token_region_bytes(D) + RED_BYTES + SMALL_BYTES + BAR_BYTES;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "decode_tail: cannot get %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  // one CTA per SM, all resident at once: the grid-wide barriers rely on it
  hfee_launch(decode_tail_kernel, dim3((unsigned)sms), dim3(THREADS), smem, stream, m_wo, m_wgu, m_wdown, m_att, m_h, m_y, a);
  return hfee_check_launch("decode_tail");
}
