// Next-token choice on the device over float32 logits [M, V]: argmax where a
// row's temperature is <= 0 (first maximum wins), else one draw from
// softmax(logits / T) by inverse CDF with the uniform number the host supplies
// for that row, walking the tokens in one fixed order (chunks of 2,048 ids; in a
// chunk the ids t, t + 256, ... of thread t = 0..255 in turn).
// Reference: hostfog/hfee internal/llm/sampler.go:76-84 (greedy, strict '>'),
// :88-95 (probabilities relative to the maximum, float64), :118-129 (draw).
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

// Greedy choice for many rows at once: each row's columns are divided among `chunks` blocks
// (stage 1), then one block per row picks among the chunk winners (stage 2).  Ties go to the
// lower index in both stages, so the result is the first maximum.
__global__ void __launch_bounds__(THREADS)
argmax_stage1_kernel(const float* __restrict__ logits, long long ld, int V, int chunks, float* __restrict__ part) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_val[THREADS];
  __shared__ int s_idx[THREADS];
  int r = blockIdx.y, ch = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (long long)r * ld;
  int per = (V + chunks - 1) / chunks;
  int begin = min(V, ch * per), end = min(V, begin + per);
  float best = -INFINITY;
  int best_i = V;
  // eight loads are requested before the first comparison needs one: a loop of load-then-compare
  // would pay one memory round trip per element
  for (int c0 = begin + tid; c0 < end; c0 += 8 * THREADS) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = c0 + j * THREADS < end ? row[c0 + j * THREADS] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + j * THREADS;
      if (c < end && (best_i == V || v[j] > best)) { best = v[j]; best_i = c; }      // ascending c: the first maximum stays
    }
  }
  s_val[tid] = best;
  s_idx[tid] = best_i;
  __syncthreads();
  for (int o = THREADS / 2; o > 0; o >>= 1) {
    if (tid < o) {
      float v2 = s_val[tid + o];
      int i2 = s_idx[tid + o];
      if (i2 < V && (s_idx[tid] == V || v2 > s_val[tid] || (v2 == s_val[tid] && i2 < s_idx[tid]))) {
        s_val[tid] = v2;
        s_idx[tid] = i2;
      }
    }
    __syncthreads();
  }
  if (tid == 0) {
    part[((long long)r * chunks + ch) * 2] = s_val[0];
    part[((long long)r * chunks + ch) * 2 + 1] = __int_as_float(s_idx[0]);
  }
}

__global__ void __launch_bounds__(32)
argmax_stage2_kernel(const float* __restrict__ part, int V, int chunks, int* __restrict__ out,
                     const int* __restrict__ slots, int* __restrict__ feedback) {
  pdl_wait();
  pdl_launch_dependents();
  // one warp per row: lane l takes chunks l, l+32, ... (four requested at a time), then the lanes'
  // winners are compared; the larger value wins, on a tie the lower index (= the earlier chunk)
  const int r = blockIdx.x, lane = threadIdx.x;
  const float2* row = reinterpret_cast<const float2*>(part) + (long long)r * chunks;
  float best = -INFINITY;
  int best_i = V;
  for (int c0 = lane; c0 < chunks; c0 += 4 * 32) {
    float2 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = c0 + j * 32 < chunks ? row[c0 + j * 32] : make_float2(0.f, __int_as_float(V));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = __float_as_int(v[j].y);
      if (i < V && (best_i == V || v[j].x > best)) { best = v[j].x; best_i = i; }   // chunks ascend: ties keep the first
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (i2 < V && (best_i == V || v2 > best || (v2 == best && i2 < best_i))) { best = v2; best_i = i2; }
  }
  if (lane != 0) return;
  out[r] = best_i;
  if (feedback) feedback[slots[r]] = best_i;      // kept on the device for the request's next step
}


// One round of "largest remaining value, lowest index on ties" over a block: every thread offers its
// best, the winner is broadcast.  An offer with index `none` never wins.  `s_val`/`s_idx` hold two
// sets of per-warp slots used in turn (`round` & 1), so one barrier per round is enough.
__device__ __forceinline__ void block_best(float& val, int& idx, int none, float* s_val, int* s_idx, int round = 0) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int WARPS = THREADS / 32;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, val, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
    if (i2 != none && (idx == none || v2 > val || (v2 == val && i2 < idx))) { val = v2; idx = i2; }
  }
  float* sv = s_val + (round & 1) * WARPS;
  int* si = s_idx + (round & 1) * WARPS;
  if (lane == 0) { sv[warp] = val; si[warp] = idx; }
  __syncthreads();
  val = sv[0]; idx = si[0];
#pragma unroll
  for (int w = 1; w < WARPS; ++w) {
    const float v2 = sv[w];
    const int i2 = si[w];
    if (i2 != none && (idx == none || v2 > val || (v2 == val && i2 < idx))) { val = v2; idx = i2; }
  }
}

// ---------------------------------------------------------------------------------------------
// Plain temperature sampling over all tokens in two stages.  Stage 1, one block per (row, chunk of
// 2,048 ids): the chunk's maximum with its first position, and the sum of exp((x - max) / T) in
// float64.  Stage 2, one block per row: the row maximum (greedy rows end here), the chunks' sums
// brought to that maximum, the chunk in which the running sum reaches U * total, then the thread and
// the element inside that chunk.  All sums are taken in fixed orders, so a row's draw does not depend
// on the batch.
struct ChunkStat { float max; int first; double sum; };

__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(THREADS)
temperature_stage1_kernel(const float* __restrict__ logits, long long ld, int V, int chunks,
                          const float* __restrict__ temperature, ChunkStat* __restrict__ stats) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_val[2 * THREADS / 32];
  __shared__ int s_idx[2 * THREADS / 32];
  __shared__ double s_sum[THREADS / 32];
  constexpr int NE = 2048 / THREADS;
  const int r = blockIdx.y, ch = blockIdx.x, tid = threadIdx.x;
  const float T = temperature ? temperature[r] : 0.f;
  const float* row = logits + (long long)r * ld;
  const int begin = ch * 2048;
  float v[NE];
  float bv = 0.f;
  int bi = V;
#pragma unroll
  for (int j = 0; j < NE; ++j) {
    const int c = begin + tid + j * THREADS;
    v[j] = c < V ? row[c] : 0.f;
    if (c < V && (bi == V || v[j] > bv)) { bv = v[j]; bi = c; }       // ascending ids: the first maximum stays
  }
  float m = bv;
  int first = bi;
  block_best(m, first, V, s_val, s_idx);
  double sum = 0.0;
  if (T > 0.f) {
#pragma unroll
    for (int j = 0; j < NE; ++j)
      if (begin + tid + j * THREADS < V) sum += exp((double)((v[j] - m) / T));
    sum = warp_sum_f64(sum);
    if ((tid & 31) == 0) s_sum[tid >> 5] = sum;
    __syncthreads();
    sum = 0.0;
    for (int w = 0; w < THREADS / 32; ++w) sum += s_sum[w];
  }
  if (tid == 0) stats[(long long)r * chunks + ch] = ChunkStat{m, first, sum};
}

__global__ void __launch_bounds__(THREADS)
temperature_stage2_kernel(const float* __restrict__ logits, long long ld, int V, int chunks,
                          const float* __restrict__ temperature, const double* __restrict__ uniform,
                          const ChunkStat* __restrict__ stats, int* __restrict__ out, const int* __restrict__ slots,
                          int* __restrict__ feedback) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ double part[THREADS];
  __shared__ int s_chunk, s_thread, s_greedy;
  __shared__ float s_max;
  __shared__ double s_left;
  constexpr int NE = 2048 / THREADS;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float T = temperature ? temperature[r] : 0.f;
  const ChunkStat* st = stats + (long long)r * chunks;
  if (tid == 0) {
    float M = st[0].max;
    int imax = st[0].first;
    for (int c = 1; c < chunks; ++c)
      if (st[c].first < V && (imax == V || st[c].max > M)) { M = st[c].max; imax = st[c].first; }      // chunks ascend: the first maximum stays
    s_greedy = imax;
    s_chunk = -1;
    if (T > 0.f) {
      double total = 0.0;
      for (int c = 0; c < chunks; ++c) total += st[c].sum * exp((double)((st[c].max - M) / T));
      const double target = uniform[r] * total;
      double run = 0.0;
      int pick = 0;
      double before = 0.0;
      for (int c = 0; c < chunks; ++c) {
        const double w = st[c].sum * exp((double)((st[c].max - M) / T));
        if (w > 0.0) { pick = c; before = run; }
        if (run + w >= target) break;
        run += w;
      }
      s_chunk = pick;
      s_max = st[pick].max;
      s_left = (target - before) / exp((double)((st[pick].max - M) / T));       // in the chunk's own scale
    }
  }
  __syncthreads();
  if (s_chunk < 0) {
    if (tid == 0) {
      out[r] = s_greedy;
      if (feedback) feedback[slots[r]] = s_greedy;
    }
    return;
  }
  const float* row = logits + (long long)r * ld;
  const int begin = s_chunk * 2048;
  double e[NE];
  double mine = 0.0;
#pragma unroll
  for (int j = 0; j < NE; ++j) {
    const int c = begin + tid + j * THREADS;
    e[j] = c < V ? exp((double)((row[c] - s_max) / T)) : 0.0;
    mine += e[j];
  }
  part[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    double run = 0.0, before = 0.0;
    int pick = 0;
    for (int t = 0; t < THREADS; ++t) {
      if (part[t] > 0.0) { pick = t; before = run; }
      if (run + part[t] >= s_left) break;
      run += part[t];
    }
    s_thread = pick;
    s_left -= before;
  }
  __syncthreads();
  if (tid != s_thread) return;
  double run = 0.0;
  int token = s_greedy;
#pragma unroll
  for (int j = 0; j < NE; ++j) {
    const int c = begin + tid + j * THREADS;
    if (c >= V) break;
    run += e[j];
    token = c;
    if (run >= s_left) break;
  }
  out[r] = token;
  if (feedback) feedback[slots[r]] = token;
}

// ---------------------------------------------------------------------------------------------
// The whole chain of hostfog/hfee internal/llm/sampler.go:54-130 on the device, for rows whose
// top-k is between 1 and CHAIN_MAX_K (a greedy row is the chain with k = 1): repeat penalty over the
// request's recent tokens (kept in a ring per request slot), the k largest logits in descending
// order (ties: lower id first), probabilities exp((l - l_max) / T) in float64, top-p and min-p cuts,
// and the draw r = U * total that walks the kept candidates.
//
// Per row eight doubles of parameters: temperature, top_k, top_p, min_p, repeat penalty,
// repeat_last_n, uniform number, unused.  top_p and min_p arrive rounded to float32, as the
// reference compares them.
constexpr int CHAIN_MAX_K = 64;
constexpr int CHAIN_CHUNK = 2048;          // vocabulary entries one stage-1 block looks at (8 per thread)
constexpr int CHAIN_PARAMS = 8;

// sampler.go:57-74: every distinct id among the last `repeat_last_n` tokens once; a positive logit
// is divided by the penalty, another multiplied.  In place.
__global__ void __launch_bounds__(THREADS)
chain_penalty_kernel(float* __restrict__ logits, long long ld, int V, const double* __restrict__ params,
                     const int* __restrict__ slots, const int* __restrict__ history, int cap,
                     const int* __restrict__ history_len) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int toks[THREADS];
  const int r = blockIdx.x, i = threadIdx.x;
  const float pen = (float)params[r * CHAIN_PARAMS + 4];
  const int last_n = (int)params[r * CHAIN_PARAMS + 5];
  if (pen == 1.f || last_n <= 0) return;                       // the same for the whole block
  const int slot = slots[r], len = history_len[slot];
  const int cnt = min(min(last_n, len), min(cap, THREADS));
  if (i < cnt) toks[i] = history[(long long)slot * cap + (len - 1 - i) % cap];
  __syncthreads();
  if (i >= cnt) return;
  const int tok = toks[i];
  for (int j = 0; j < i; ++j)
    if (toks[j] == tok) return;                                // a later copy of an id already handled
  if (tok < 0 || tok >= V) return;
  float* x = logits + (long long)r * ld + tok;
  *x = *x > 0.f ? *x / pen : *x * pen;
}

// Stage 1: the k largest of each chunk of a row, in descending order, to cand[(row, chunk)][CHAIN_MAX_K] as
// (value, id) pairs; unused places hold id V.
__global__ void __launch_bounds__(THREADS)
chain_stage1_kernel(const float* __restrict__ logits, long long ld, int V, int chunks, const double* __restrict__ params,
                    float2* __restrict__ cand) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_val[2 * THREADS / 32];
  __shared__ int s_idx[2 * THREADS / 32];
  constexpr int NE = CHAIN_CHUNK / THREADS;
  const int r = blockIdx.y, ch = blockIdx.x, tid = threadIdx.x;
  const double temp = params[r * CHAIN_PARAMS];
  const int k = temp > 0.0 ? min(max((int)params[r * CHAIN_PARAMS + 1], 1), CHAIN_MAX_K) : 1;
  const float* row = logits + (long long)r * ld;
  const int begin = ch * CHAIN_CHUNK;
  float v[NE];
  unsigned alive = 0;
#pragma unroll
  for (int j = 0; j < NE; ++j) {
    const int c = begin + tid + j * THREADS;
    v[j] = c < V ? row[c] : 0.f;
    if (c < V) alive |= 1u << j;
  }
  float2* dst = cand + ((long long)r * chunks + ch) * CHAIN_MAX_K;
  for (int round = 0; round < k; ++round) {
    float bv = 0.f;
    int bj = -1;
#pragma unroll
    for (int j = 0; j < NE; ++j)
      if (((alive >> j) & 1u) && (bj < 0 || v[j] > bv)) { bv = v[j]; bj = j; }      // ascending j = ascending id
    float val = bv;
    int idx = bj >= 0 ? begin + tid + bj * THREADS : V;
    const int mine = idx;
    block_best(val, idx, V, s_val, s_idx, round);
    if (idx != V && idx == mine) alive &= ~(1u << bj);
    if (tid == 0) dst[round] = make_float2(val, __int_as_float(idx));
  }
}

// Stage 2: the k largest of a row's candidates, then the chain.  The chunks' lists are sorted, so the
// next largest is always at the head of some list: one warp merges them (lane l owns the lists l,
// l + 32, ...; a round is a comparison of the lanes' best heads by shuffles, no barrier).  Appends
// the choice to the request's history ring (when there is one) and stores it in feedback[slot] for
// the next step's embedding.
__global__ void __launch_bounds__(THREADS)
chain_stage2_kernel(const float2* __restrict__ cand, int V, int chunks, const double* __restrict__ params,
                    const int* __restrict__ slots, int* __restrict__ history, int cap, int* __restrict__ history_len,
                    int* __restrict__ out, int* __restrict__ feedback) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float2 lists[];                             // [chunks][k]
  __shared__ float top_val[CHAIN_MAX_K];
  __shared__ int top_idx[CHAIN_MAX_K];
  __shared__ double prob[CHAIN_MAX_K];
  __shared__ double s_sum;
  __shared__ int s_n;
  const int r = blockIdx.x, tid = threadIdx.x;
  const double* pr = params + r * CHAIN_PARAMS;
  const double temp = pr[0];
  const int k = temp > 0.0 ? min(max((int)pr[1], 1), CHAIN_MAX_K) : 1;
  for (int e = tid; e < chunks * k; e += THREADS)
    lists[e] = cand[((long long)r * chunks + e / k) * CHAIN_MAX_K + e % k];
  __syncthreads();
  if (tid < 32) {
    constexpr int OWN = 4;                                      // up to 128 chunks over 32 lanes
    int pos[OWN];
#pragma unroll
    for (int j = 0; j < OWN; ++j) pos[j] = 0;
    for (int round = 0; round < k; ++round) {
      float bv = 0.f;
      int bi = V, bj = 0;
#pragma unroll
      for (int j = 0; j < OWN; ++j) {
        const int c = tid + j * 32;
        if (c < chunks && pos[j] < k) {
          const float2 h = lists[c * k + pos[j]];
          const int hi = __float_as_int(h.y);
          if (hi != V && (bi == V || h.x > bv || (h.x == bv && hi < bi))) { bv = h.x; bi = hi; bj = j; }
        }
      }
      float val = bv;
      int idx = bi;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, val, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (i2 != V && (idx == V || v2 > val || (v2 == val && i2 < idx))) { val = v2; idx = i2; }
      }
      if (idx != V && idx == bi) {
#pragma unroll
        for (int j = 0; j < OWN; ++j)
          if (j == bj) ++pos[j];
      }
      if (tid == 0) { top_val[round] = val; top_idx[round] = idx; }
    }
  }
  __syncthreads();
  if (temp > 0.0 && tid < k)
    prob[tid] = top_idx[tid] != V ? exp((double)((top_val[tid] - top_val[0]) / (float)temp)) : 0.0;
  __syncthreads();
  // probabilities p_i = prob_i / sum: the sum by one thread in candidate order, the divisions (slow in
  // float64) by the candidates' threads, so that the walk below only adds and compares
  if (tid == 0) {
    int n = 0;
    double sum = 0.0;
    while (n < k && top_idx[n] != V) sum += prob[n++];
    s_sum = sum;
    s_n = n;
  }
  __syncthreads();
  if (temp > 0.0 && tid < k) prob[tid] = prob[tid] / s_sum;
  __syncthreads();
  if (tid != 0) return;
  int token = top_idx[0];
  if (temp > 0.0) {
    const int n = s_n;
    const double top_p = pr[2], min_p = pr[3];
    int keep = n;
    if (top_p > 0.0 && top_p < 1.0) {
      double cum = 0.0;
      for (int i = 0; i < n; ++i) {
        cum += prob[i];
        if (cum >= top_p) { keep = i + 1; break; }
      }
    }
    if (min_p > 0.0) {
      const double floor_p = min_p * prob[0];
      for (int i = 1; i < keep; ++i)
        if (prob[i] < floor_p) { keep = i; break; }
    }
    double kept = 0.0;
    for (int i = 0; i < keep; ++i) kept += prob[i];
    double left = pr[6] * kept;
    token = top_idx[keep - 1];
    for (int i = 0; i < keep; ++i) {
      left -= prob[i];
      if (left <= 0.0) { token = top_idx[i]; break; }
    }
  }
  out[r] = token;
  if (slots != nullptr) {
    const int slot = slots[r];
    if (feedback != nullptr) feedback[slot] = token;
    if (history != nullptr) {
      const int len = history_len[slot];
      history[(long long)slot * cap + len % cap] = token;
      history_len[slot] = len + 1;
    }
  }
}

}  // namespace

// scratch: M * chunks * 2 floats.
// slots/feedback (optional): also store row r's choice in feedback[slots[r]].
HFEE_API int hfee_argmax(const float* logits, long long ld, int M, int V, int chunks, float* scratch, int* out,
                         const int* slots, int* feedback, cudaStream_t stream) {
  if (M == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && V > 0 && ld >= V && chunks > 0 && chunks <= 1024 && scratch != nullptr,
               "argmax: bad sizes M=%d V=%d chunks=%d", M, V, chunks);
  HFEE_REQUIRE(M <= 65535, "argmax: too many rows");
  hfee_launch(argmax_stage1_kernel, dim3(dim3((unsigned)chunks, (unsigned)M)), dim3(THREADS), 0, stream, logits, ld, V, chunks, scratch);
  hfee_launch(argmax_stage2_kernel, dim3(M), dim3(32), 0, stream, scratch, V, chunks, out, slots, feedback);
  return hfee_check_launch("argmax");
}

// scratch: M * ceil(V / 2048) * 2 doubles (16-byte aligned).
HFEE_API int hfee_sample(const float* logits, long long ld, int M, int V, const float* temperature,
                         const double* uniform, double* scratch, long long scratch_doubles, int* out, const int* slots,
                         int* feedback, cudaStream_t stream) {
  if (M == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && M <= 65535 && V > 0 && ld >= V, "sample: bad sizes M=%d V=%d ld=%lld", M, V, ld);
  HFEE_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: temperatures need uniform numbers");
  const int chunks = (V + 2047) / 2048;
  HFEE_REQUIRE(scratch != nullptr && scratch_doubles >= (long long)M * chunks * 2 && (uintptr_t)scratch % 16 == 0,
               "sample: the scratch must hold %lld doubles", (long long)M * chunks * 2);
  hfee_launch(temperature_stage1_kernel, dim3((unsigned)chunks, (unsigned)M), dim3(THREADS), 0, stream, logits, ld, V, chunks,
              temperature, (ChunkStat*)scratch);
  hfee_launch(temperature_stage2_kernel, dim3(M), dim3(THREADS), 0, stream, logits, ld, V, chunks, temperature, uniform,
              (const ChunkStat*)scratch, out, slots, feedback);
  return hfee_check_launch("sample");
}

// The sampling chain on the device for M rows (see chain_stage2_kernel).  `params`: M x 8 doubles.
// `logits` is changed in place where a row penalises.  `scratch`: M * ceil(V / 2048) * 64 * 2 floats.
// `history` [slots][cap] int32 with `history_len` [slots] (tokens appended so far): the rings of recent
// tokens, may be null when no row penalises; `slots` maps rows to request slots (needed with
// history or feedback).
HFEE_API int hfee_sample_chain(float* logits, long long ld, int M, int V, const double* params, const int* slots,
                               int* history, int history_cap, int* history_len, int penalise, float* scratch,
                               long long scratch_floats, int* out, int* feedback, cudaStream_t stream) {
  if (M == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && M <= 65535 && V > 0 && ld >= V && params != nullptr && out != nullptr, "sample_chain: bad sizes M=%d V=%d", M, V);
  const int chunks = (V + CHAIN_CHUNK - 1) / CHAIN_CHUNK;
  HFEE_REQUIRE(chunks <= 128, "sample_chain: a vocabulary of %d exceeds %d", V, 128 * CHAIN_CHUNK);
  HFEE_REQUIRE(scratch != nullptr && scratch_floats >= (long long)M * chunks * CHAIN_MAX_K * 2 && (uintptr_t)scratch % 8 == 0,
               "sample_chain: the scratch must hold %lld floats", (long long)M * chunks * CHAIN_MAX_K * 2);
  HFEE_REQUIRE((feedback == nullptr && history == nullptr) || slots != nullptr, "sample_chain: feedback and history need the rows' slots");
  HFEE_REQUIRE(!penalise || (history != nullptr && history_len != nullptr && history_cap > 0 && history_cap <= THREADS),
               "sample_chain: a repeat penalty needs the history rings (at most %d tokens each)", THREADS);
  if (penalise)
    hfee_launch(chain_penalty_kernel, dim3(M), dim3(THREADS), 0, stream, logits, ld, V, params, slots, (const int*)history,
                history_cap, (const int*)history_len);
  hfee_launch(chain_stage1_kernel, dim3((unsigned)chunks, (unsigned)M), dim3(THREADS), 0, stream, (const float*)logits, ld, V,
              chunks, params, (float2*)scratch);
  // the candidate lists of a row in shared memory: chunks * CHAIN_MAX_K pairs at most (64 KB at 128 chunks)
  const size_t list_bytes = (size_t)chunks * CHAIN_MAX_K * sizeof(float2);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(chain_stage2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * CHAIN_MAX_K * (int)sizeof(float2));
    if (e != cudaSuccess) return hfee_fail(HFEE_ERR_CUDA, "sample_chain: cannot get shared memory for the candidate lists: %s", cudaGetErrorString(e));
    configured = true;
  }
  hfee_launch(chain_stage2_kernel, dim3(M), dim3(THREADS), list_bytes, stream, (const float2*)scratch, V, chunks, params, slots,
              history, history_cap, history_len, out, feedback);
  return hfee_check_launch("sample_chain");
}
