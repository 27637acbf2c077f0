// Causal grouped-query attention over the paged cache on the CUDA cores, float32
// arithmetic, for any head size: one warp per (token, query head).
//
// The keys a token sees are the positions lo..pos of its own request, lo = 0 or
// pos+1-window.  They are visited in blocks of 32 counted from lo with an online
// softmax, so the result at a position depends neither on how the tokens were cut
// into steps nor on which pages hold them.  This kernel is the attention of the
// true 32-bit path and the fallback of the bfloat16 path.
// Reference: hostfog/hfee internal/llm/forward.go:146-178 (scores scaled after the
// dot, softmax over 0..pos, weighted sum of values), internal/ggml/ops.go:136-150.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int ld_q, const T* __restrict__ k_pool,
                      const T* __restrict__ v_pool, PagedCache cache, const int* __restrict__ positions,
                      const int* __restrict__ slot_of_token, T* __restrict__ out, int ld_o, int n, int heads,
                      float scale, int window) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float q_s[WARPS][MAX_HD];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long task = (long long)blockIdx.x * WARPS + warp;
  if (task >= (long long)n * heads) return;
  int i = (int)(task / heads), h = (int)(task % heads);
  int hd = cache.head_dim;
  int kvh = h / (heads / cache.kv_heads);
  int pos = positions[i], slot = slot_of_token[i];
  int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;

  const T* qrow = q + (long long)i * ld_q + (long long)h * hd;
  for (int d = lane; d < hd; d += 32) q_s[warp][d] = to_f32<T>(qrow[d]);
  __syncwarp();

  constexpr int DPL = MAX_HD / 32;     // output dims per lane
  float o[DPL];
#pragma unroll
  for (int j = 0; j < DPL; ++j) o[j] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = lo; base <= pos; base += 32) {
    int key = base + lane;
    float s = -INFINITY;
    if (key <= pos) {
      const T* kr = k_pool + paged_offset(cache, slot, key, kvh);
      float acc = 0.f;
      for (int d = 0; d < hd; ++d) acc = fmaf(q_s[warp][d], to_f32<T>(kr[d]), acc);
      s = acc * scale;
    }
    float m_new = fmaxf(m, warp_max(s));
    float p = key <= pos ? expf(s - m_new) : 0.f;
    float alpha = expf(m - m_new);          // exp(-inf) = 0 on the first block
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int j = 0; j < DPL; ++j) o[j] *= alpha;
    int count = min(32, pos + 1 - base);
    for (int t = 0; t < count; ++t) {
      float pt = __shfl_sync(0xffffffffu, p, t);
      const T* vr = v_pool + paged_offset(cache, slot, base + t, kvh);
#pragma unroll
      for (int j = 0; j < DPL; ++j) {
        int d = lane + 32 * j;
        if (d < hd) o[j] = fmaf(pt, to_f32<T>(vr[d]), o[j]);
      }
    }
    m = m_new;
  }
  T* orow = out + (long long)i * ld_o + (long long)h * hd;
  float inv = 1.f / l;
#pragma unroll
  for (int j = 0; j < DPL; ++j) {
    int d = lane + 32 * j;
    if (d < hd) orow[d] = from_f32<T>(o[j] * inv);
  }
}

}  // namespace

HFEE_API int hfee_attention_simt(const void* q, int ld_q, const void* k_pool, const void* v_pool,
                                 const int* block_table, int max_pages, int page_size, const int* positions,
                                 const int* slot_of_token, void* out, int ld_o, int n, int heads, int kv_heads,
                                 int head_dim, float scale, int window, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(head_dim > 0 && head_dim <= MAX_HD, "attention_simt: head_dim %d is outside 1..%d", head_dim, MAX_HD);
  HFEE_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
               "attention_simt: heads %d must be a multiple of kv_heads %d", heads, kv_heads);
  HFEE_REQUIRE(page_size > 0 && max_pages > 0, "attention_simt: bad cache sizes");
  PagedCache c;
  HFEE_REQUIRE(make_paged_cache(&c, block_table, max_pages, page_size, kv_heads, head_dim),
               "page_size %d must be a power of two", page_size);
  long long tasks = (long long)n * heads;
  unsigned blocks = (unsigned)((tasks + WARPS - 1) / WARPS);
  if (dtype == HFEE_F32)
    hfee_launch(attention_simt_kernel<float>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const float*)q, ld_q, (const float*)k_pool,
        (const float*)v_pool, c, positions, slot_of_token, (float*)out, ld_o, n, heads, scale, window);
  else if (dtype == HFEE_BF16)
    hfee_launch(attention_simt_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), 0, stream, (const __nv_bfloat16*)q, ld_q,
        (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, c, positions, slot_of_token,
        (__nv_bfloat16*)out, ld_o, n, heads, scale, window);
  else
    return hfee_fail(HFEE_ERR_ARG, "attention_simt: unknown dtype %d", dtype);
  return hfee_check_launch("attention_simt");
}
