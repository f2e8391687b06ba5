// Shared device helpers for every kernel file of the engine: element types, widening loads,
// rounding stores, warp and block reductions, and paged-cache addressing.
//
// Element type codes cross the C ABI as ints: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define DT_F32 0
#define DT_BF16 1

#define LLM_HOST_CHECK(cond, code) \
  do {                             \
    if (!(cond)) return (code);    \
  } while (0)

// Error codes returned by launchers (0 = launched; CUDA errors are returned as 1000 + code).
#define ERR_BAD_DTYPE 1
#define ERR_BAD_SIZE 2
#define ERR_BAD_ALIGN 3

// Programmatic dependent launch.  Every kernel of the engine is launched with the attribute that
// lets it start while the kernel before it in the stream is still running.  In return every
// kernel calls pdl_wait() before it touches global memory that another kernel may have written
// or may still read (it returns once all earlier kernels have finished and their writes are
// visible), and pdl_launch_dependents() at its start, which lets the next kernel begin its own
// preamble.  What runs before pdl_wait() may only touch shared memory, tensor memory, and global
// memory that no kernel writes (weights).  Set BARE_CUDA_B200_NO_PDL=1 to launch without it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* v = getenv("BARE_CUDA_B200_NO_PDL");
    enabled = (v && v[0] && v[0] != '0') ? 0 : 1;
  }
  return enabled == 1;
}

template <typename... KArgs, typename... Args>
static inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + static_cast<int>(e);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

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

// Sum over a block whose size is a multiple of 32 (at most 1024 threads); every thread gets the
// result.  `scratch` holds 32 floats.  The order of the additions depends on the block size only.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarp ? scratch[lane] : 0.0f;
  return warp_sum(r);
}

// Where the keys and values of one cache (one run of a layer) live.  A page of the pool holds,
// for every cache of its group, keys then values, each [kv_heads][page_tokens][head_dim].
// `k` and `v` already point at this cache's part of page 0.
struct PagedCache {
  void* k;
  void* v;
  const int32_t* block_table;  // [batch sequences][table_stride]: page of a request's n-th block, -1 if none
  long long page_stride;       // elements from one page to the next
  int table_stride;
  int page_tokens;
  int kv_heads;
  int head_dim;
};

// Element offset of (batch sequence, position, kv head) inside the pool, or -1 if the page is not held.
__device__ __forceinline__ long long cache_offset(const PagedCache& c, int seq, int pos, int kvh) {
  const int page = c.block_table[(long long)seq * c.table_stride + pos / c.page_tokens];
  if (page < 0) return -1;
  return (long long)page * c.page_stride +
         ((long long)kvh * c.page_tokens + (pos % c.page_tokens)) * c.head_dim;
}
