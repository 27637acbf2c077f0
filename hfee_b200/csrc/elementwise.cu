// Embedding gather, RMSNorm, rotary table, rotary + cache write, SwiGLU.
// All arithmetic is float32 (the rotary table is built in float64); T is the
// storage type of activations, weights tables and cache pages.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[i,:] = table[token_i,:] as float32 (the residual stream is float32).
// Reference: x[i,:] = embed.Row(tokens[i]), hostfog/hfee internal/llm/forward.go:75-77.
// A negative token id means "the token last sampled on the device for this token's request":
// it is read from feedback[slot_of_token[i]], so a decode step can be launched before the host
// has seen the previous step's result.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             const int* __restrict__ slot_of_token, const int* __restrict__ feedback,
                             float* __restrict__ out, int width, int vocab) {
  pdl_wait();
  pdl_launch_dependents();
  int i = blockIdx.x;
  int tok = tokens[i];
  if (tok < 0 && feedback != nullptr) tok = feedback[slot_of_token[i]];
  bool ok = tok >= 0 && tok < vocab;
  const T* row = table + (long long)(ok ? tok : 0) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(long long)i * width + c] = ok ? to_f32<T>(row[c]) : 0.f;
}

// The same with 16-byte reads: one piece of the row per thread and trip, all of a thread's pieces
// requested before the first is converted.
template <typename T, int VEC>
__global__ void embed_vec_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                 const int* __restrict__ slot_of_token, const int* __restrict__ feedback,
                                 float* __restrict__ out, int width, int vocab) {
  struct alignas(16) Piece { T v[VEC]; };
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x;
  int tok = tokens[i];
  if (tok < 0 && feedback != nullptr) tok = feedback[slot_of_token[i]];
  const bool ok = tok >= 0 && tok < vocab;
  const T* row = table + (long long)(ok ? tok : 0) * width;
  float* dst = out + (long long)i * width;
  const int pieces = width / VEC;
  for (int p0 = threadIdx.x; p0 < pieces; p0 += 4 * blockDim.x) {
    Piece v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + j * blockDim.x;
      if (p < pieces && ok) v[j] = *reinterpret_cast<const Piece*>(row + p * VEC);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + j * blockDim.x;
      if (p >= pieces) continue;
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        float4 o = ok ? make_float4(to_f32<T>(v[j].v[e]), to_f32<T>(v[j].v[e + 1]), to_f32<T>(v[j].v[e + 2]), to_f32<T>(v[j].v[e + 3]))
                      : make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(dst + p * VEC + e) = o;
      }
    }
  }
}

HFEE_API int hfee_embed(const void* table, int dtype, const int* tokens, const int* slot_of_token,
                        const int* feedback, float* out, int n, int width, int vocab, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0 && vocab > 0, "embed: bad sizes n=%d width=%d vocab=%d", n, width, vocab);
  int threads = width >= 256 ? 256 : 64;
  const int vec = dtype == HFEE_F32 ? 4 : 8;
  const bool vector = width % vec == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)out % 16 == 0;
  if (dtype == HFEE_F32) {
    if (vector) hfee_launch(embed_vec_kernel<float, 4>, dim3(n), dim3(threads), 0, stream, (const float*)table, tokens, slot_of_token, feedback, out, width, vocab);
    else hfee_launch(embed_kernel<float>, dim3(n), dim3(threads), 0, stream, (const float*)table, tokens, slot_of_token, feedback, out, width, vocab);
  } else if (dtype == HFEE_BF16) {
    if (vector) hfee_launch(embed_vec_kernel<__nv_bfloat16, 8>, dim3(n), dim3(threads), 0, stream, (const __nv_bfloat16*)table, tokens, slot_of_token, feedback, out, width, vocab);
    else hfee_launch(embed_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, (const __nv_bfloat16*)table, tokens, slot_of_token, feedback, out, width, vocab);
  } else {
    return hfee_fail(HFEE_ERR_ARG, "embed: unknown dtype %d", dtype);
  }
  return hfee_check_launch("embed");
}

// ---------------------------------------------------------------- RMSNorm
// out[r,:] = x[row(r),:] * rsqrt(mean(x^2) + eps) * w, one block per row, float32 math
// with a fixed reduction order (so a row's result does not depend on the batch).
// `rows` (optional) gathers: row(r) = rows[r].  `add_unit` uses (1 + w).
// Reference: internal/ggml/ops.go:125-134 (order (x*scale)*w).
template <typename TOut, int THREADS>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               const int* __restrict__ rows, TOut* __restrict__ out, int width,
                               float eps, int add_unit) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float partial[THREADS / 32];
  int r = blockIdx.x;
  const float* xr = x + (long long)(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float v = xr[c];
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += partial[i];
  float scale = 1.0f / sqrtf(total / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += THREADS) {
    float wv = add_unit ? 1.f + w[c] : w[c];
    out[(long long)r * width + c] = from_f32<TOut>(xr[c] * scale * wv);
  }
}

// The same for widths that are multiples of 4 with 16-byte accesses.  A thread owns the pieces
// tid, tid + THREADS, ...; it requests NCH of them before it uses the first (a loop of load-then-use
// would pay one memory round trip per piece), the scales even before the wait on the previous
// kernel, and a row of at most THREADS * 4 * NCH values stays in registers between the two passes.
template <typename TOut, int THREADS, int NCH>
__global__ void __launch_bounds__(THREADS)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                   TOut* __restrict__ out, int width, float eps, int add_unit) {
  constexpr int SPAN = THREADS * 4 * NCH;
  __shared__ float partial[THREADS / 32];
  const int r = blockIdx.x, tid = threadIdx.x;
  const bool single = width <= SPAN;
  float4 wv[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    const int c = (tid + j * THREADS) * 4;
    wv[j] = c < width ? __ldg(reinterpret_cast<const float4*>(w + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int src_row = rows ? rows[r] : r;                 // host-written, like the batch layout
  pdl_wait();
  pdl_launch_dependents();
  const float* xr = x + (long long)src_row * width;
  float4 xv[NCH];
  float ss = 0.f;
  for (int base = 0; base < width; base += SPAN) {
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = base + (tid + j * THREADS) * 4;
      xv[j] = c < width ? *reinterpret_cast<const float4*>(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      ss = fmaf(xv[j].x, xv[j].x, ss); ss = fmaf(xv[j].y, xv[j].y, ss);
      ss = fmaf(xv[j].z, xv[j].z, ss); ss = fmaf(xv[j].w, xv[j].w, ss);
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) partial[tid >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += partial[i];
  const float scale = 1.0f / sqrtf(total / (float)width + eps);
  TOut* dst = out + (long long)r * width;
  for (int base = 0; base < width; base += SPAN) {
    if (!single) {
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int c = base + (tid + j * THREADS) * 4;
        xv[j] = c < width ? *reinterpret_cast<const float4*>(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        wv[j] = c < width ? __ldg(reinterpret_cast<const float4*>(w + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      const int c = base + (tid + j * THREADS) * 4;
      if (c >= width) continue;
      float4 g = wv[j];
      if (add_unit) { g.x += 1.f; g.y += 1.f; g.z += 1.f; g.w += 1.f; }
      const float o0 = xv[j].x * scale * g.x, o1 = xv[j].y * scale * g.y, o2 = xv[j].z * scale * g.z, o3 = xv[j].w * scale * g.w;
      if constexpr (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(dst + c) = make_float4(o0, o1, o2, o3);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(o0, o1), hi = __floats2bfloat162_rn(o2, o3);
        *reinterpret_cast<uint2*>(dst + c) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      }
    }
  }
}

// Many rows (a prompt portion), bfloat16 out: a warp per row and the whole row in registers, so a row
// costs one memory round trip and no block-wide barrier, and a CTA of 8 warps keeps 8 rows in flight.
// NV float4 per lane: rows of up to 128 * NV values.
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, const int* __restrict__ rows,
                    __nv_bfloat16* __restrict__ out, int n, int width, float eps, int add_unit) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (r >= n) return;
  const int src_row = rows ? rows[r] : r;                 // host-written, like the batch layout
  pdl_wait();
  pdl_launch_dependents();
  const float* xr = x + (long long)src_row * width;
  float4 xv[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = (lane + j * 32) * 4;
    xv[j] = c < width ? *reinterpret_cast<const float4*>(xr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    ss = fmaf(xv[j].x, xv[j].x, ss); ss = fmaf(xv[j].y, xv[j].y, ss);
    ss = fmaf(xv[j].z, xv[j].z, ss); ss = fmaf(xv[j].w, xv[j].w, ss);
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)width + eps);
  const float unit = add_unit ? 1.f : 0.f;
  __nv_bfloat16* dst = out + (long long)r * width;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = (lane + j * 32) * 4;
    if (c >= width) continue;
    const float4 g = __ldg(reinterpret_cast<const float4*>(w + c));
    __nv_bfloat162 lo = __floats2bfloat162_rn(xv[j].x * scale * (g.x + unit), xv[j].y * scale * (g.y + unit));
    __nv_bfloat162 hi = __floats2bfloat162_rn(xv[j].z * scale * (g.z + unit), xv[j].w * scale * (g.w + unit));
    *reinterpret_cast<uint2*>(dst + c) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
}

HFEE_API int hfee_rmsnorm(const float* x, const float* w, const int* rows, void* out, int out_dtype,
                          int n, int width, float eps, int add_unit, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && width > 0, "rmsnorm: bad sizes n=%d width=%d", n, width);
  const bool vector = width % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
  if (out_dtype == HFEE_F32) {
    if (vector) hfee_launch(rmsnorm_vec_kernel<float, 256, 4>, dim3(n), dim3(256), 0, stream, x, w, rows, (float*)out, width, eps, add_unit);
    else hfee_launch(rmsnorm_kernel<float, 256>, dim3(n), dim3(256), 0, stream, x, w, rows, (float*)out, width, eps, add_unit);
  } else if (out_dtype == HFEE_BF16 && vector && n >= 256 && width <= 128 * 32) {
    // enough rows to fill the GPU with a warp each
    const dim3 grid((unsigned)((n + 7) / 8));
    if (width <= 128 * 8) hfee_launch(rmsnorm_rows_kernel<8>, grid, dim3(256), 0, stream, x, w, rows, (__nv_bfloat16*)out, n, width, eps, add_unit);
    else if (width <= 128 * 16) hfee_launch(rmsnorm_rows_kernel<16>, grid, dim3(256), 0, stream, x, w, rows, (__nv_bfloat16*)out, n, width, eps, add_unit);
    else hfee_launch(rmsnorm_rows_kernel<32>, grid, dim3(256), 0, stream, x, w, rows, (__nv_bfloat16*)out, n, width, eps, add_unit);
  } else if (out_dtype == HFEE_BF16) {
    if (vector) hfee_launch(rmsnorm_vec_kernel<__nv_bfloat16, 256, 4>, dim3(n), dim3(256), 0, stream, x, w, rows, (__nv_bfloat16*)out, width, eps, add_unit);
    else hfee_launch(rmsnorm_kernel<__nv_bfloat16, 256>, dim3(n), dim3(256), 0, stream, x, w, rows, (__nv_bfloat16*)out, width, eps, add_unit);
  } else {
    return hfee_fail(HFEE_ERR_ARG, "rmsnorm: unknown dtype %d", out_dtype);
  }
  return hfee_check_launch("rmsnorm");
}

// ---------------------------------------------------------------- rotary table
// cs[i, j] = (cos, sin)(positions[i] * inv_freq[j]) evaluated in float64, stored
// as float32; built once per step and shared by every layer with the same
// rotary parameters.  Reference: math.Sincos(float64(pos) * invFreq[i]),
// internal/llm/forward.go:185-186.
__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int n, int half) {
  pdl_wait();
  pdl_launch_dependents();
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * half) return;
  int i = idx / half, j = idx % half;
  double s, c;
  sincos((double)positions[i] * inv_freq[j], &s, &c);
  cs[idx] = make_float2((float)c, (float)s);
}

HFEE_API int hfee_rope_table(const int* positions, const double* inv_freq, float* cs, int n, int half,
                             cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && half > 0, "rope_table: bad sizes n=%d half=%d", n, half);
  int total = n * half;
  hfee_launch(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, stream, positions, inv_freq, (float2*)cs, n, half);
  return hfee_check_launch("rope_table");
}

// ---------------------------------------------------------------- rotary + cache write
// Input rows hold [q heads | k heads | v heads] (the fused projection).  Rotates q
// into q_out and k into the cache page of (slot, position); copies v to its page.
// `cs` may be null (no rotation).  Pair (i, i+rope_dim/2) when `interleaved` is 0,
// (2i, 2i+1) otherwise; dims at or above rope_dim pass through.  k/v pools may be
// null when this layer reads another layer's cache (q only).
// Reference: internal/llm/forward.go:90-102,181-196.
// VEC: elements per 16-byte access (8 for bfloat16, 4 for float32).  A work item is one 16-byte piece
// of the first member of each pair together with the matching piece of the second member:
// half-split pairing pairs piece [a, a+VEC) with [a+half, a+half+VEC); interleaved pairing keeps both
// members in one piece.  Dims at or above rope_dim (and all of v) are copied piece by piece.
template <typename T, int VEC>
struct alignas(16) Piece { T v[VEC]; };

template <typename T, int VEC>
__global__ void rope_cache_kernel(const T* __restrict__ qkv, int ld_qkv, const float2* __restrict__ cs,
                                  const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                                  T* __restrict__ q_out, int ld_q, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  PagedCache cache, int heads, int rope_dim, int interleaved) {
  using P = Piece<T, VEC>;
  const int i = blockIdx.x;
  const int hd = cache.head_dim, kvh = cache.kv_heads;
  const int half = rope_dim / 2;
  const int per_block = (int)blockDim.x * gridDim.y;    // work items are spread over the blocks of grid.y
  const int pos = positions[i];                          // host-written: readable before the previous kernel ends
  const int slot = slot_of_token[i];
  const int page_warm = k_pool ? cache.block_table[(long long)slot * cache.max_pages + (pos >> cache.page_shift)] : 0;
  asm volatile("" ::"r"(page_warm));
  pdl_wait();
  pdl_launch_dependents();
  const T* row = qkv + (long long)i * ld_qkv;
  const int total_heads = k_pool ? heads + 2 * kvh : heads;   // q only when this run reads another run's cache
  const int pieces = hd / VEC;                                 // 16-byte pieces per head
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < total_heads * pieces; w += per_block) {
    const int h = w / pieces, a = (w % pieces) * VEC;          // first dim of this piece
    const T* src = row + (long long)h * hd;
    T* dst;
    if (h < heads) {
      dst = q_out + (long long)i * ld_q + (long long)h * hd;
    } else {
      const int kh = h < heads + kvh ? h - heads : h - heads - kvh;
      dst = (h < heads + kvh ? k_pool : v_pool) + paged_offset(cache, slot, pos, kh);
    }
    const bool rotate = cs != nullptr && h < heads + kvh && a < rope_dim;
    if (!rotate) {
      *reinterpret_cast<P*>(dst + a) = *reinterpret_cast<const P*>(src + a);
      continue;
    }
    const float2* t = cs + (long long)i * half;
    if (interleaved) {                                         // pairs (2p, 2p+1) inside the piece
      P x = *reinterpret_cast<const P*>(src + a), y;
      float2 cc[VEC / 2];                                    // the piece's table entries, 16 bytes at a time
#pragma unroll
      for (int e = 0; e < VEC / 2; e += 2) *reinterpret_cast<float4*>(&cc[e]) = *reinterpret_cast<const float4*>(t + a / 2 + e);
#pragma unroll
      for (int e = 0; e < VEC; e += 2) {
        const float2 c = cc[e / 2];
        const float x0 = to_f32<T>(x.v[e]), x1 = to_f32<T>(x.v[e + 1]);
        y.v[e] = from_f32<T>(x0 * c.x - x1 * c.y);
        y.v[e + 1] = from_f32<T>(x0 * c.y + x1 * c.x);
      }
      *reinterpret_cast<P*>(dst + a) = y;
    } else if (a < half) {                                     // pairs (a+e, a+e+half): this item does both pieces
      P x0 = *reinterpret_cast<const P*>(src + a), x1 = *reinterpret_cast<const P*>(src + a + half), y0, y1;
      float2 cc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; e += 2) *reinterpret_cast<float4*>(&cc[e]) = *reinterpret_cast<const float4*>(t + a + e);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float2 c = cc[e];
        const float u = to_f32<T>(x0.v[e]), v = to_f32<T>(x1.v[e]);
        y0.v[e] = from_f32<T>(u * c.x - v * c.y);
        y1.v[e] = from_f32<T>(u * c.y + v * c.x);
      }
      *reinterpret_cast<P*>(dst + a) = y0;
      *reinterpret_cast<P*>(dst + a + half) = y1;
    }                                                          // pieces in [half, rope_dim) were written by their partner
  }
}

// Element-pair version for shapes whose rows or rotary halves are not whole 16-byte pieces.
template <typename T>
__global__ void rope_cache_scalar_kernel(const T* __restrict__ qkv, int ld_qkv, const float2* __restrict__ cs,
                                  const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                                  T* __restrict__ q_out, int ld_q, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  PagedCache cache, int heads, int rope_dim, int interleaved) {
  int i = blockIdx.x;
  int hd = cache.head_dim, kvh = cache.kv_heads;
  int half = rope_dim / 2;
  int per_block = (int)blockDim.x * gridDim.y;    // work items are spread over the blocks of grid.y
  int pos = positions[i];                          // host-written: readable before the previous kernel ends
  int slot = slot_of_token[i];
  int page_warm = k_pool ? cache.block_table[(long long)slot * cache.max_pages + pos / cache.page_size] : 0;
  asm volatile("" ::"r"(page_warm));
  pdl_wait();
  pdl_launch_dependents();
  const T* row = qkv + (long long)i * ld_qkv;
  int total_heads = k_pool ? heads + 2 * kvh : heads;   // q only when this run reads another run's cache
  // one work item = (head, pair index within the head); hd/2 items per head
  int per_head = hd / 2;
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < total_heads * per_head; w += per_block) {
    int h = w / per_head, p = w % per_head;
    const T* src = row + (long long)h * hd;
    int a, b;
    bool rotate = cs != nullptr && h < heads + kvh;
    if (p < half) {
      a = interleaved ? 2 * p : p;
      b = interleaved ? 2 * p + 1 : p + half;
    } else {                       // unrotated tail of a partial rotary head
      a = rope_dim + 2 * (p - half);
      b = a + 1;
      rotate = false;
    }
    float x0 = to_f32<T>(src[a]), x1 = to_f32<T>(src[b]);
    float y0 = x0, y1 = x1;
    if (rotate) {
      float2 t = cs[(long long)i * half + p];
      y0 = x0 * t.x - x1 * t.y;
      y1 = x0 * t.y + x1 * t.x;
    }
    T* dst;
    if (h < heads) {
      dst = q_out + (long long)i * ld_q + (long long)h * hd;
    } else {
      if (k_pool == nullptr) continue;
      int kh = h < heads + kvh ? h - heads : h - heads - kvh;
      T* pool = h < heads + kvh ? k_pool : v_pool;
      dst = pool + paged_offset(cache, slot, pos, kh);
    }
    dst[a] = from_f32<T>(y0);
    dst[b] = from_f32<T>(y1);
  }
}

HFEE_API int hfee_rope_cache_write(const void* qkv, int ld_qkv, const float* cs, const int* positions,
                                   const int* slot_of_token, void* q_out, int ld_q, void* k_pool,
                                   void* v_pool, const int* block_table, int max_pages, int page_size,
                                   int n, int heads, int kv_heads, int head_dim, int rope_dim,
                                   int interleaved, int dtype, cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope: head_dim %d must be even", head_dim);
  HFEE_REQUIRE(rope_dim >= 0 && rope_dim <= head_dim && rope_dim % 2 == 0,
               "rope: rope_dim %d must be even and at most head_dim %d", rope_dim, head_dim);
  HFEE_REQUIRE(heads > 0 && kv_heads > 0 && page_size > 0 && max_pages > 0, "rope: bad sizes");
  const int vec = dtype == HFEE_F32 ? 4 : 8;                   // elements per 16 bytes
  // few tokens (decode): the element-pair kernel spreads the little work there is over more threads
  const bool vector = n >= 64 && head_dim % vec == 0 && (rope_dim / 2) % vec == 0 && ld_qkv % vec == 0 && ld_q % vec == 0 &&
                      (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)k_pool % 16 == 0 &&
                      (uintptr_t)v_pool % 16 == 0;
  PagedCache c;
  HFEE_REQUIRE(make_paged_cache(&c, block_table, max_pages, page_size, kv_heads, head_dim),
               "page_size %d must be a power of two", page_size);
  int items = (heads + 2 * kv_heads) * (vector ? head_dim / vec : head_dim / 2);
  int threads = 256;
  dim3 grid((unsigned)n, (unsigned)((items + threads - 1) / threads));
  if (grid.y > 64) grid.y = 64;
  if (!vector) {
    if (dtype == HFEE_F32)
      hfee_launch(rope_cache_scalar_kernel<float>, dim3(grid), dim3(threads), 0, stream, (const float*)qkv, ld_qkv,
                  (const float2*)cs, positions, slot_of_token, (float*)q_out, ld_q, (float*)k_pool, (float*)v_pool, c,
                  heads, rope_dim, interleaved);
    else if (dtype == HFEE_BF16)
      hfee_launch(rope_cache_scalar_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream,
                  (const __nv_bfloat16*)qkv, ld_qkv, (const float2*)cs, positions, slot_of_token, (__nv_bfloat16*)q_out,
                  ld_q, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, c, heads, rope_dim, interleaved);
    else
      return hfee_fail(HFEE_ERR_ARG, "rope: unknown dtype %d", dtype);
    return hfee_check_launch("rope_cache_write");
  }
  if (dtype == HFEE_F32)
    hfee_launch(rope_cache_kernel<float, 4>, dim3(grid), dim3(threads), 0, stream, (const float*)qkv, ld_qkv, (const float2*)cs, positions,
        slot_of_token, (float*)q_out, ld_q, (float*)k_pool, (float*)v_pool, c, heads, rope_dim, interleaved);
  else if (dtype == HFEE_BF16)
    hfee_launch(rope_cache_kernel<__nv_bfloat16, 8>, dim3(grid), dim3(threads), 0, stream, (const __nv_bfloat16*)qkv, ld_qkv, (const float2*)cs,
        positions, slot_of_token, (__nv_bfloat16*)q_out, ld_q, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, c,
        heads, rope_dim, interleaved);
  else
    return hfee_fail(HFEE_ERR_ARG, "rope: unknown dtype %d", dtype);
  return hfee_check_launch("rope_cache_write");
}

// ---------------------------------------------------------------- SwiGLU
// h[i, c] = silu(gate) * up in float32, g / (1 + exp(-g)) * u.  The fused projection's
// columns come in groups of `granule` gate columns followed by `granule` up columns:
// gate(c) = gu[i, (c / granule) * 2 * granule + c % granule], up(c) = gate(c) + granule
// (granule = inter: all gate columns, then all up columns).
// Reference: internal/ggml/ops.go:160-165.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, int ld_gu, T* __restrict__ h, int ld_h, int n, int inter,
                              int granule) {
  pdl_wait();
  pdl_launch_dependents();
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * inter) return;
  int i = (int)(idx / inter), c = (int)(idx % inter);
  long long gcol = (long long)(c / granule) * 2 * granule + c % granule;
  float g = to_f32<T>(gu[(long long)i * ld_gu + gcol]);
  float u = to_f32<T>(gu[(long long)i * ld_gu + gcol + granule]);
  h[(long long)i * ld_h + c] = from_f32<T>(g / (1.f + expf(-g)) * u);
}

HFEE_API int hfee_swiglu(const void* gu, int ld_gu, void* h, int ld_h, int n, int inter, int granule, int dtype,
                         cudaStream_t stream) {
  if (n == 0) return HFEE_OK;
  HFEE_REQUIRE(n > 0 && inter > 0 && ld_gu >= 2 * inter && ld_h >= inter, "swiglu: bad sizes");
  HFEE_REQUIRE(granule > 0 && inter % granule == 0, "swiglu: granule %d does not divide %d", granule, inter);
  long long total = (long long)n * inter;
  unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == HFEE_F32)
    hfee_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, ld_gu, (float*)h, ld_h, n, inter, granule);
  else if (dtype == HFEE_BF16)
    hfee_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, ld_gu, (__nv_bfloat16*)h, ld_h, n, inter, granule);
  else
    return hfee_fail(HFEE_ERR_ARG, "swiglu: unknown dtype %d", dtype);
  return hfee_check_launch("swiglu");
}
