// Next-token choice on the device over float32 logits [M, V]: argmax where a
// row's temperature is <= 0 (first maximum wins), else one draw from
// softmax(logits / T) by inverse CDF in index order with the uniform number the
// host supplies for that row.
// Reference: hostfog/hfee internal/llm/sampler.go:76-84 (greedy, strict '>'),
// :88-95 (probabilities relative to the maximum, float64), :118-129 (draw).
#include "common.cuh"

namespace {

constexpr int THREADS = 256;

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const double* __restrict__ uniform, int* __restrict__ out, const int* __restrict__ slots,
              int* __restrict__ feedback) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_val[THREADS];
  __shared__ int s_idx[THREADS];
  __shared__ double s_sum[THREADS];
  int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (long long)r * ld;

  // contiguous chunk per thread so that index order is kept
  int chunk = (V + THREADS - 1) / THREADS;
  int begin = min(V, tid * chunk), end = min(V, begin + chunk);

  float best = -INFINITY;
  int best_i = V;          // V = "none"
  for (int c = begin; c < end; ++c) {
    float v = row[c];
    if (best_i == V || v > best) { best = v; best_i = c; }
  }
  s_val[tid] = best;
  s_idx[tid] = best_i;
  __syncthreads();
  for (int o = THREADS / 2; o > 0; o >>= 1) {
    if (tid < o) {
      float v2 = s_val[tid + o];
      int i2 = s_idx[tid + o];
      // keep the lower index on ties; an empty chunk (index V) never wins
      if (i2 < V && (s_idx[tid] == V || v2 > s_val[tid] || (v2 == s_val[tid] && i2 < s_idx[tid]))) {
        s_val[tid] = v2;
        s_idx[tid] = i2;
      }
    }
    __syncthreads();
  }
  float vmax = s_val[0];
  int imax = s_idx[0];
  float T = temperature ? temperature[r] : 0.f;
  if (!(T > 0.f)) {
    if (tid == 0) {
      out[r] = imax;
      if (feedback) feedback[slots[r]] = imax;
    }
    return;
  }

  double local = 0.0;
  for (int c = begin; c < end; ++c) local += exp((double)((row[c] - vmax) / T));
  s_sum[tid] = local;
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int t = 0; t < THREADS; ++t) total += s_sum[t];
    double target = uniform[r] * total;
    // find the chunk, then the element, where the running sum first reaches the target
    int t = 0;
    double run = 0.0;
    while (t < THREADS - 1 && run + s_sum[t] < target) run += s_sum[t++];
    int b = min(V, t * chunk), e = min(V, b + chunk);
    int pick = imax;
    bool found = false;
    for (int c = b; c < e; ++c) {
      run += exp((double)((row[c] - vmax) / T));
      pick = c;
      if (run >= target) { found = true; break; }
    }
    if (!found && e == b) pick = imax;
    out[r] = pick;
    if (feedback) feedback[slots[r]] = pick;
  }
}

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

HFEE_API int hfee_sample(const float* logits, long long ld, int M, int V, const float* temperature,
                         const double* uniform, int* out, const int* slots, int* feedback, cudaStream_t stream) {
  if (M == 0) return HFEE_OK;
  HFEE_REQUIRE(M > 0 && V > 0 && ld >= V, "sample: bad sizes M=%d V=%d ld=%lld", M, V, ld);
  HFEE_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: temperatures need uniform numbers");
  hfee_launch(sample_kernel, dim3(M), dim3(THREADS), 0, stream, logits, ld, V, temperature, uniform, out, slots, feedback);
  return hfee_check_launch("sample");
}
