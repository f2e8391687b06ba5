// Shared device helpers for every kernel file of the engine: element types, widening loads,
// rounding stores, warp and block reductions, and paged-cache addressing.
//
// Element type codes cross the C ABI as ints: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

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
