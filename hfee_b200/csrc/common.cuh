// Shared declarations of the sm_100a kernel library.
//
// Every exported function is extern "C", takes raw device pointers, sizes and a
// cudaStream_t, launches on that stream and returns 0 or a negative error code
// (hfee_last_error() gives the text).  Nothing here allocates device memory.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define HFEE_API extern "C" __attribute__((visibility("default")))

enum HfeeDtype { HFEE_F32 = 0, HFEE_BF16 = 1 };

enum HfeeError {
  HFEE_OK = 0,
  HFEE_ERR_ARG = -1,       // a size or option the kernel does not take
  HFEE_ERR_CUDA = -2,      // a CUDA call failed
  HFEE_ERR_ALIGN = -3,     // a pointer or leading dimension breaks an alignment rule
};

// Sets the message returned by hfee_last_error() and returns `code`.
int hfee_fail(int code, const char* fmt, ...);
// Checks cudaGetLastError() after a launch.
int hfee_check_launch(const char* what);

#define HFEE_REQUIRE(cond, ...)                        \
  do {                                                  \
    if (!(cond)) return hfee_fail(HFEE_ERR_ARG, __VA_ARGS__); \
  } while (0)

// Programmatic dependent launch: every kernel is launched so that it may start while its
// predecessor in the stream is still running.  A kernel calls pdl_wait() before it touches
// anything the predecessor wrote (it returns once the predecessor has completed and its writes
// are visible) and pdl_launch_dependents() to let its own successor start early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming multiprocessors of the current device; 0 if the query fails (launchers then refuse).
extern "C" int hfee_sm_count();

// 0 when the environment variable HFEE_NO_PDL is set.
int hfee_pdl_enabled();
int hfee_carveout();

template <typename... KArgs, typename... Args>
cudaError_t hfee_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                        Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = hfee_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int carve = hfee_carveout();
  if (carve >= 0) {
    attr[1].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
    attr[1].val.sharedMemCarveout = (unsigned int)carve;
    cfg.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Paged cache addressing shared by every kernel that touches the cache.
// Pool layout of one layer: [num_pages][kv_heads][page_size][head_dim].
struct PagedCache {
  const int* block_table;   // [max_requests][max_pages] page ids, row = request slot
  int max_pages;            // row length of block_table
  int page_size;            // a power of two
  int page_shift;           // log2(page_size)
  int kv_heads;
  int head_dim;
  long long page_stride;    // elements per page = kv_heads*page_size*head_dim
};

// Fills a PagedCache; returns false if page_size is not a power of two.
inline bool make_paged_cache(PagedCache* c, const int* block_table, int max_pages, int page_size, int kv_heads,
                             int head_dim) {
  if (page_size <= 0 || (page_size & (page_size - 1)) != 0) return false;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  *c = PagedCache{block_table, max_pages, page_size, shift, kv_heads, head_dim,
                  (long long)kv_heads * page_size * head_dim};
  return true;
}

__device__ __forceinline__ long long paged_offset(const PagedCache& c, int slot, int pos, int kv_head) {
  int page = c.block_table[(long long)slot * c.max_pages + (pos >> c.page_shift)];
  return (long long)page * c.page_stride +
         ((long long)kv_head * c.page_size + (pos & (c.page_size - 1))) * c.head_dim;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Counter-based uniform in [0,1): splitmix64 of (seed, stream, counter).  The host
// sampler uses the same function so a draw does not depend on batching.
__host__ __device__ __forceinline__ uint64_t hfee_mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__host__ __device__ __forceinline__ double hfee_uniform(uint64_t seed, uint64_t stream, uint64_t counter) {
  uint64_t h = hfee_mix64(hfee_mix64(hfee_mix64(seed) ^ stream) ^ counter);
  return (double)(h >> 11) * (1.0 / 9007199254740992.0);
}
