// Plain kernels: one simple SIMT kernel per operation, every size a run-time argument, all
// arithmetic in float32.  They are the whole float32 path of the engine, the reference that
// each fast bfloat16 kernel is tested against, and the bfloat16 path's fallback for sizes the
// fast kernels refuse.
//
// The order in which any output element's sum is formed depends only on the operation's own
// sizes (hidden width, head size, absolute key position), never on how many rows a launch
// carries or where a row sits in the batch: cutting the same tokens into other steps gives the
// same bits.  (This holds for the float32 kernels.  The vector variants that only bfloat16 steps
// use - the norm for few and for many rows, the rotation for many tokens - pick their shape from
// the number of rows, so there a row's sum may be formed in another order in another step; the
// difference is float32 rounding under a bfloat16 result.)
//
// Formulas follow cuongvng/bare-cuda-4gib: embedding (engine/kernels/embedding_lookup.cu:22-30),
// RMSNorm (engine/kernels/rmsnorm.cu:26-40), matmul against [out, in] weights
// (engine/kernels/gemm_tiled.cuh:36-96), rotate_half RoPE (engine/kernels/rope.cu:44-53),
// causal attention (engine/kernels/attention_qk.cu:49-68, softmax.cu:28-42,
// attention_av.cu:24-44), SwiGLU (engine/kernels/swiglu.cu:22-23), argmax with the lowest index
// on ties (engine/kernels/logits_argmax.cu:36-64).  Unlike the reference, exp and sincos are the
// precise functions, softmax is computed online over key blocks (no [heads, T, T] buffer), and
// the residual add is fused with the norm that follows it.

#include "common.cuh"

#include <math.h>

// ------------------------------------------------------------------------------- embedding

template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int32_t* __restrict__ ids,
                                    float* __restrict__ out, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const TW* row = table + (long long)ids[t] * hidden;
  float* dst = out + (long long)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(row[i]);
}

extern "C" int llm_embed_gather(const void* table, int table_dtype, const int32_t* ids, float* out,
                                int n_tokens, int hidden, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (table_dtype == DT_F32) {
    launch_kernel(embed_gather_kernel<float>, n_tokens, 256, 0, stream, (const float*)table, ids, out, hidden);
  } else if (table_dtype == DT_BF16) {
    launch_kernel(embed_gather_kernel<__nv_bfloat16>, n_tokens, 256, 0, stream, (const __nv_bfloat16*)table, ids, out,
                  hidden);
  } else {
    return ERR_BAD_DTYPE;
  }
  return launch_status();
}

// --------------------------------------------------------------- residual add + RMSNorm

// One block per output row.  If `delta` is given, residual[row] += sum over `n_partials` partial
// results (added in index order) before the norm; the updated residual is written back.
// `row_index` (optional, distinct entries) picks which residual row each output row works on.
// Each element's sum and the order of the row's sum of squares depend on the block size only,
// which the launcher picks from `hidden`, never from the number of rows.
template <typename TD, typename TW, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   int n_partials, long long partial_stride,
                                   const TW* __restrict__ weight, TO* __restrict__ out,
                                   const int32_t* __restrict__ row_index, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_cache[];  // hidden floats + 32 scratch
  float* scratch = row_cache + hidden;
  const int r = blockIdx.x;
  const long long src = row_index ? row_index[r] : r;
  float* x = residual + src * hidden;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = x[i];
    if (delta) {
      for (int p = 0; p < n_partials; ++p) v += to_float(delta[p * partial_stride + src * hidden + i]);
      x[i] = v;
    }
    row_cache[i] = v;
    sq += v * v;
  }
  const float total = block_sum(sq, scratch);
  const float scale = 1.0f / sqrtf(total / (float)hidden + eps);
  if (out) {
    TO* dst = out + (long long)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      dst[i] = from_float<TO>(row_cache[i] * scale * to_float(weight[i]));
  }
}

// The same with 16-byte accesses: float32 delta, bfloat16 weight and output, hidden a multiple of 4.
// A thread keeps its elements in registers (at most 4 float4: hidden <= 16 * blockDim.x).
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                       int n_partials, long long partial_stride,
                                       const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
                                       const int32_t* __restrict__ row_index, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const long long src = row_index ? row_index[r] : r;
  float4* x = reinterpret_cast<float4*>(residual + src * hidden);
  const int n4 = hidden / 4;
  float4 v[4];
  float sq = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < n4) {
      float4 a = x[i];
      if (delta) {
        for (int p = 0; p < n_partials; ++p) {
          const float4 d = reinterpret_cast<const float4*>(delta + p * partial_stride + src * hidden)[i];
          a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
        }
        x[i] = a;
      }
      v[j] = a;
      sq += a.x * a.x;
      sq += a.y * a.y;
      sq += a.z * a.z;
      sq += a.w * a.w;
    }
  }
  const float total = block_sum(sq, scratch);
  const float scale = 1.0f / sqrtf(total / (float)hidden + eps);
  if (out) {
    uint2* dst = reinterpret_cast<uint2*>(out + (long long)r * hidden);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < n4) {
        const uint2 wraw = reinterpret_cast<const uint2*>(weight)[i];
        const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.x);
        const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.y);
        __nv_bfloat162 o01 = __floats2bfloat162_rn(v[j].x * scale * __low2float(w01), v[j].y * scale * __high2float(w01));
        __nv_bfloat162 o23 = __floats2bfloat162_rn(v[j].z * scale * __low2float(w23), v[j].w * scale * __high2float(w23));
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&o01);
        o.y = *reinterpret_cast<uint32_t*>(&o23);
        dst[i] = o;
      }
    }
  }
}

// The same for many rows (prompt portions): one warp per row, the row kept in registers between
// the sum of squares and the scaling, no block barrier, so that an SM has dozens of rows' loads
// in flight at once.  HOLD float4 values per lane: rows of up to 128 * HOLD values.
template <int HOLD>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ residual, const float* __restrict__ delta, int n_partials,
                        long long partial_stride, const __nv_bfloat16* __restrict__ weight,
                        __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ row_index, int rows, int hidden,
                        float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const long long src = row_index ? row_index[r] : r;
  float4* x = reinterpret_cast<float4*>(residual + src * hidden);
  const int n4 = hidden / 4;
  float4 v[HOLD];
#pragma unroll
  for (int j = 0; j < HOLD; ++j)
    if (lane + 32 * j < n4) v[j] = x[lane + 32 * j];
  if (delta) {
    for (int p = 0; p < n_partials; ++p) {
      const float4* d4 = reinterpret_cast<const float4*>(delta + p * partial_stride + src * hidden);
      float4 d[HOLD];
#pragma unroll
      for (int j = 0; j < HOLD; ++j)
        if (lane + 32 * j < n4) d[j] = d4[lane + 32 * j];
#pragma unroll
      for (int j = 0; j < HOLD; ++j)
        if (lane + 32 * j < n4) {
          v[j].x += d[j].x;
          v[j].y += d[j].y;
          v[j].z += d[j].z;
          v[j].w += d[j].w;
        }
    }
#pragma unroll
    for (int j = 0; j < HOLD; ++j)
      if (lane + 32 * j < n4) x[lane + 32 * j] = v[j];
  }
  float sq = 0.0f;
#pragma unroll
  for (int j = 0; j < HOLD; ++j)
    if (lane + 32 * j < n4) {
      sq += v[j].x * v[j].x;
      sq += v[j].y * v[j].y;
      sq += v[j].z * v[j].z;
      sq += v[j].w * v[j].w;
    }
  const float scale = 1.0f / sqrtf(warp_sum(sq) / (float)hidden + eps);
  if (out) {
    uint2* dst = reinterpret_cast<uint2*>(out + (long long)r * hidden);
#pragma unroll
    for (int j = 0; j < HOLD; ++j)
      if (lane + 32 * j < n4) {
        const uint2 wraw = reinterpret_cast<const uint2*>(weight)[lane + 32 * j];
        const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.x);
        const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.y);
        const __nv_bfloat162 o01 = __floats2bfloat162_rn(v[j].x * scale * __low2float(w01), v[j].y * scale * __high2float(w01));
        const __nv_bfloat162 o23 = __floats2bfloat162_rn(v[j].z * scale * __low2float(w23), v[j].w * scale * __high2float(w23));
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&o01);
        o.y = *reinterpret_cast<const uint32_t*>(&o23);
        dst[lane + 32 * j] = o;
      }
  }
}

template <typename TD, typename TW>
static int add_rmsnorm_out(float* residual, const void* delta, int n_partials,
                           long long partial_stride, const void* weight, void* out, int out_dtype,
                           const int32_t* row_index, int rows, int hidden, float eps,
                           cudaStream_t stream) {
  const size_t smem = (size_t)(hidden + 32) * sizeof(float);
  if (smem > 200 * 1024) return ERR_BAD_SIZE;
#define LAUNCH_NORM(TO)                                                                         \
  do {                                                                                          \
    auto kern = add_rmsnorm_kernel<TD, TW, TO>;                                                 \
    if (smem > 48 * 1024)                                                                       \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    launch_kernel(kern, rows, 256, smem, stream, residual, (const TD*)delta, n_partials,        \
                  partial_stride, (const TW*)weight, (TO*)out, row_index, hidden, eps);         \
  } while (0)
  if (out_dtype == DT_F32) LAUNCH_NORM(float);
  else if (out_dtype == DT_BF16) LAUNCH_NORM(__nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH_NORM
  return launch_status();
}

extern "C" int llm_add_rmsnorm(float* residual, const void* delta, int delta_dtype, int n_partials,
                               long long partial_stride, const void* weight, int weight_dtype,
                               void* out, int out_dtype, const int32_t* row_index, int rows,
                               int hidden, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  // the bfloat16 path's common case: vector accesses, block size from the width alone
  const auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (delta_dtype == DT_F32 && weight_dtype == DT_BF16 && (out == nullptr || out_dtype == DT_BF16) &&
      hidden % 4 == 0 && hidden <= 16 * 1024 && aligned16(residual) && aligned16(delta) &&
      (partial_stride % 4 == 0) && (reinterpret_cast<uintptr_t>(weight) & 7) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 7) == 0) {
    const int n4 = hidden / 4;
    if (rows >= 256 && n4 <= 32 * 32) {   // many rows (enough warps to fill the GPU): a warp per row
      const int blocks = (rows + 7) / 8;
      if (n4 <= 32 * 16)
        launch_kernel(add_rmsnorm_rows_kernel<16>, blocks, 256, 0, stream, residual, (const float*)delta, n_partials,
                      partial_stride, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, row_index, rows, hidden, eps);
      else
        launch_kernel(add_rmsnorm_rows_kernel<32>, blocks, 256, 0, stream, residual, (const float*)delta, n_partials,
                      partial_stride, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, row_index, rows, hidden, eps);
      return launch_status();
    }
    int threads = 128;
    while (threads < 1024 && threads * 2 <= n4) threads *= 2;   // <= 2 float4 per thread when wide
    while (threads * 4 < n4) threads *= 2;
    launch_kernel(add_rmsnorm_vec_kernel, rows, threads, 0, stream, residual, (const float*)delta, n_partials,
                  partial_stride, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out, row_index, hidden, eps);
    return launch_status();
  }
  if (delta_dtype == DT_F32 && weight_dtype == DT_F32)
    return add_rmsnorm_out<float, float>(residual, delta, n_partials, partial_stride, weight, out,
                                         out_dtype, row_index, rows, hidden, eps, stream);
  if (delta_dtype == DT_F32 && weight_dtype == DT_BF16)
    return add_rmsnorm_out<float, __nv_bfloat16>(residual, delta, n_partials, partial_stride, weight,
                                                 out, out_dtype, row_index, rows, hidden, eps, stream);
  if (delta_dtype == DT_BF16 && weight_dtype == DT_F32)
    return add_rmsnorm_out<__nv_bfloat16, float>(residual, delta, n_partials, partial_stride, weight,
                                                 out, out_dtype, row_index, rows, hidden, eps, stream);
  if (delta_dtype == DT_BF16 && weight_dtype == DT_BF16)
    return add_rmsnorm_out<__nv_bfloat16, __nv_bfloat16>(residual, delta, n_partials, partial_stride,
                                                         weight, out, out_dtype, row_index, rows,
                                                         hidden, eps, stream);
  return ERR_BAD_DTYPE;
}

// ------------------------------------------------------------------------------- matmul

// out[m, n] = sum_k a[m, k] * w[n, k].  64x64 output tile per block of 256 threads, 4x4 outputs
// per thread, K in slices of 16.  Each slice is summed on its own and then added to the running
// total, so the rounding error grows with K/16 + 16 rather than K.
constexpr int GT = 64, GK = 16;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
matmul_plain_kernel(const TA* __restrict__ a, const TW* __restrict__ w, TO* __restrict__ out, int M,
                    int N, int K, long long lda, long long ldo) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float as[GK][GT + 1];
  __shared__ float ws[GK][GT + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * GT, n0 = blockIdx.x * GT;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += GK) {
    for (int i = threadIdx.x; i < GT * GK; i += 256) {
      const int r = i / GK, c = i % GK;
      const int m = m0 + r, n = n0 + r, k = k0 + c;
      as[c][r] = (m < M && k < K) ? to_float(a[(long long)m * lda + k]) : 0.0f;
      ws[c][r] = (n < N && k < K) ? to_float(w[(long long)n * K + k]) : 0.0f;
    }
    __syncthreads();
    float part[4][4] = {};
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) part[i][j] = fmaf(av[i], wv[j], part[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(long long)m * ldo + n] = from_float<TO>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW>
static int matmul_plain_out(const void* a, const void* w, void* out, int out_dtype, int M, int N,
                            int K, long long lda, long long ldo, cudaStream_t stream) {
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  if (grid.y > 65535) return ERR_BAD_SIZE;
  if (out_dtype == DT_F32)
    launch_kernel(matmul_plain_kernel<TA, TW, float>, grid, 256, 0, stream, (const TA*)a, (const TW*)w, (float*)out,
                  M, N, K, lda, ldo);
  else if (out_dtype == DT_BF16)
    launch_kernel(matmul_plain_kernel<TA, TW, __nv_bfloat16>, grid, 256, 0, stream, (const TA*)a, (const TW*)w,
                  (__nv_bfloat16*)out, M, N, K, lda, ldo);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

extern "C" int llm_matmul_plain(const void* a, int a_dtype, const void* w, int w_dtype, void* out,
                                int out_dtype, int M, int N, int K, long long lda, long long ldo,
                                cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return ERR_BAD_SIZE;
  if (a_dtype == DT_F32 && w_dtype == DT_F32)
    return matmul_plain_out<float, float>(a, w, out, out_dtype, M, N, K, lda, ldo, stream);
  if (a_dtype == DT_F32 && w_dtype == DT_BF16)
    return matmul_plain_out<float, __nv_bfloat16>(a, w, out, out_dtype, M, N, K, lda, ldo, stream);
  if (a_dtype == DT_BF16 && w_dtype == DT_F32)
    return matmul_plain_out<__nv_bfloat16, float>(a, w, out, out_dtype, M, N, K, lda, ldo, stream);
  if (a_dtype == DT_BF16 && w_dtype == DT_BF16)
    return matmul_plain_out<__nv_bfloat16, __nv_bfloat16>(a, w, out, out_dtype, M, N, K, lda, ldo,
                                                          stream);
  return ERR_BAD_DTYPE;
}

// ------------------------------------------------------------- rotation + cache write

// One warp per (token, head) of the token's fused projection row [q heads | k heads | v heads]
// (optionally a sum of partial results): q and k heads are rotated by the token's position, q goes
// to q_out, k and v into the request's cache pages.  The angle is float(pos) * inv_freq[p], a
// float32 product; sin and cos are the precise functions.  inv_freq == nullptr means no rotation.
constexpr int ROPE_HEADS_PER_BLOCK = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(ROPE_HEADS_PER_BLOCK * 32)
rope_cache_write_kernel(const TI* __restrict__ qkv, int n_partials, long long partial_stride,
                        TO* __restrict__ q_out, PagedCache cache, const int32_t* __restrict__ positions,
                        const int32_t* __restrict__ row_seq, const float* __restrict__ inv_freq, int q_heads,
                        int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int h = blockIdx.y * ROPE_HEADS_PER_BLOCK + (threadIdx.x >> 5);
  const int d = cache.head_dim, half = d / 2;
  const int kvh_n = cache.kv_heads;
  const int n_heads = q_heads + 2 * kvh_n;
  if (h >= n_heads || (h >= q_heads && !write_cache)) return;
  const int pos = positions[t];
  const TI* row = qkv + (long long)t * n_heads * d + (long long)h * d;
  auto load = [&](int i) {
    float v = 0.0f;
    for (int p = 0; p < n_partials; ++p) v += to_float(row[p * partial_stride + i]);
    return v;
  };
  if (h < q_heads + kvh_n) {  // rotated: a q head or a k head
    TO* dst;
    if (h < q_heads) {
      dst = q_out + ((long long)t * q_heads + h) * d;
    } else {
      const long long off = cache_offset(cache, row_seq[t], pos, h - q_heads);
      if (off < 0) return;
      dst = (TO*)cache.k + off;
    }
    for (int p = lane; p < half; p += 32) {
      const float lo = load(p), hi = load(p + half);
      float c = 1.0f, s = 0.0f;
      if (inv_freq) sincosf((float)pos * inv_freq[p], &s, &c);
      dst[p] = from_float<TO>(lo * c - hi * s);
      dst[p + half] = from_float<TO>(hi * c + lo * s);
    }
  } else {
    const long long off = cache_offset(cache, row_seq[t], pos, h - q_heads - kvh_n);
    if (off < 0) return;
    TO* dst = (TO*)cache.v + off;
    for (int i = lane; i < d; i += 32) dst[i] = from_float<TO>(load(i));
  }
}

// The same for many tokens of a bfloat16 step (head sizes that are multiples of 16 up to 256, one
// finished input, no partials): one block per token.  A token's angles are the same for every
// head, so the block first computes its head_dim / 2 sines and cosines once into shared memory
// (the precise sincosf is what the kernel's time would otherwise go to: 36 heads would each repeat
// it), then each thread rotates eight neighbouring pairs with 16-byte loads and stores.
constexpr int ROPE_VEC_THREADS = 128;
__global__ void __launch_bounds__(ROPE_VEC_THREADS)
rope_cache_write_vec_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out, PagedCache cache,
                            const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq,
                            const float* __restrict__ inv_freq, int q_heads, int write_cache, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float cs[128], sn[128];
  const int d = cache.head_dim, half = d / 2;
  const int groups = half / 8;                         // 8-pair groups per rotated head
  const int n_heads = q_heads + 2 * cache.kv_heads;
  const int t = blockIdx.x;
  const int pos = positions[t];
  for (int p = threadIdx.x; p < half; p += ROPE_VEC_THREADS) {
    float c = 1.0f, s = 0.0f;
    if (inv_freq) sincosf((float)pos * inv_freq[p], &s, &c);
    cs[p] = c;
    sn[p] = s;
  }
  __syncthreads();
  const int rotated = (q_heads + cache.kv_heads) * groups;
  const int per_token = rotated + cache.kv_heads * (d / 8);
  const __nv_bfloat16* row = qkv + (long long)t * n_heads * d;
  const int seq = row_seq[t];
  for (int w = threadIdx.x; w < per_token; w += ROPE_VEC_THREADS) {
    if (w < rotated) {
      const int h = w / groups, p0 = (w % groups) * 8;
      __nv_bfloat16* dst;
      if (h < q_heads) {
        dst = q_out + ((long long)t * q_heads + h) * d;
      } else {
        if (!write_cache) continue;
        const long long off = cache_offset(cache, seq, pos, h - q_heads);
        if (off < 0) continue;
        dst = (__nv_bfloat16*)cache.k + off;
      }
      const uint4 lo_raw = *reinterpret_cast<const uint4*>(row + (long long)h * d + p0);
      const uint4 hi_raw = *reinterpret_cast<const uint4*>(row + (long long)h * d + half + p0);
      const __nv_bfloat16* lo = reinterpret_cast<const __nv_bfloat16*>(&lo_raw);
      const __nv_bfloat16* hi = reinterpret_cast<const __nv_bfloat16*>(&hi_raw);
      uint4 lo_out, hi_out;
      __nv_bfloat16* lo_o = reinterpret_cast<__nv_bfloat16*>(&lo_out);
      __nv_bfloat16* hi_o = reinterpret_cast<__nv_bfloat16*>(&hi_out);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cs[p0 + j], s = sn[p0 + j];
        const float a = __bfloat162float(lo[j]), b = __bfloat162float(hi[j]);
        lo_o[j] = __float2bfloat16_rn(a * c - b * s);
        hi_o[j] = __float2bfloat16_rn(b * c + a * s);
      }
      *reinterpret_cast<uint4*>(dst + p0) = lo_out;
      *reinterpret_cast<uint4*>(dst + half + p0) = hi_out;
    } else {
      if (!write_cache) continue;
      const int v = w - rotated;
      const int kvh = v / (d / 8), c0 = (v % (d / 8)) * 8;
      const long long off = cache_offset(cache, seq, pos, kvh);
      if (off < 0) continue;
      *reinterpret_cast<uint4*>((__nv_bfloat16*)cache.v + off + c0) =
          *reinterpret_cast<const uint4*>(row + (long long)(q_heads + cache.kv_heads + kvh) * d + c0);
    }
  }
}

extern "C" int llm_rope_cache_write(const void* qkv, int in_dtype, int n_partials,
                                    long long partial_stride, void* q_out, int out_dtype, void* k_base,
                                    void* v_base, const int32_t* block_table, long long page_stride,
                                    int table_stride, int page_tokens, int kv_heads, int head_dim,
                                    const int32_t* positions, const int32_t* row_seq,
                                    const float* inv_freq, int q_heads,
                                    int write_cache, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim % 2) return ERR_BAD_SIZE;
  PagedCache c{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  const int n_heads = q_heads + 2 * kv_heads;
  const auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (in_dtype == DT_BF16 && out_dtype == DT_BF16 && n_partials == 1 && head_dim % 16 == 0 && head_dim <= 256 && n_tokens >= 64 &&
      aligned16(qkv) && aligned16(q_out) && aligned16(k_base) && aligned16(v_base)) {
    launch_kernel(rope_cache_write_vec_kernel, n_tokens, ROPE_VEC_THREADS, 0, stream, (const __nv_bfloat16*)qkv,
                  (__nv_bfloat16*)q_out, c, positions, row_seq, inv_freq, q_heads, write_cache, n_tokens);
    return launch_status();
  }
  dim3 grid(n_tokens, (n_heads + ROPE_HEADS_PER_BLOCK - 1) / ROPE_HEADS_PER_BLOCK);
  if (grid.y > 65535) return ERR_BAD_SIZE;
#define LAUNCH_ROPE(TI, TO)                                                                   \
  launch_kernel(rope_cache_write_kernel<TI, TO>, grid, ROPE_HEADS_PER_BLOCK * 32, 0, stream,   \
                (const TI*)qkv, n_partials, partial_stride, (TO*)q_out, c, positions, row_seq,  \
                inv_freq, q_heads, write_cache)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) LAUNCH_ROPE(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) LAUNCH_ROPE(float, __nv_bfloat16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) LAUNCH_ROPE(__nv_bfloat16, __nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH_ROPE
  return launch_status();
}

// ------------------------------------------------------------------------------- attention

// One warp per (token, query head).  Keys are visited in blocks of 32 aligned to absolute
// positions; lane l scores key block*32 + l, the block's maximum and sum update the running
// softmax, and each lane accumulates the output channels l, l+32, ...  Scores are
// (q . k) * scale with the scale applied after the dot product.  A key j is visible to the
// query at position pos if first <= j <= pos, first = max(0, pos - window + 1) (window <= 0: all).
constexpr int ATT_WARPS = 4;
constexpr int ATT_MAX_CH = 8;  // head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_plain_kernel(const T* __restrict__ q, T* __restrict__ out, PagedCache cache,
                       const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq,
                       int q_heads, int n_tokens, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float q_smem[];  // ATT_WARPS * head_dim
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
  const int d = cache.head_dim;
  const bool active = item < (long long)n_tokens * q_heads;
  const int t = active ? (int)(item / q_heads) : 0;
  const int h = active ? (int)(item % q_heads) : 0;
  float* qs = q_smem + warp * d;
  if (active)
    for (int c = lane; c < d; c += 32) qs[c] = to_float(q[((long long)t * q_heads + h) * d + c]);
  __syncwarp();
  if (!active) return;

  const int pos = positions[t];
  const int slot = row_seq[t];
  const int kvh = h / (q_heads / cache.kv_heads);
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const T* kc = (const T*)cache.k;
  const T* vc = (const T*)cache.v;

  float m = -INFINITY, l = 0.0f;
  float acc[ATT_MAX_CH];
#pragma unroll
  for (int i = 0; i < ATT_MAX_CH; ++i) acc[i] = 0.0f;

  for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool visible = j >= first && j <= pos;
    float s = -INFINITY;
    long long off = -1;
    if (visible) {
      off = cache_offset(cache, slot, j, kvh);
      if (off >= 0) {
        float dot = 0.0f;
        for (int c = 0; c < d; ++c) dot = fmaf(qs[c], to_float(kc[off + c]), dot);
        s = dot * scale;
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAX_CH; ++i) acc[i] *= corr;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long offj = __shfl_sync(0xffffffffu, off, jj);
      if (pj == 0.0f || offj < 0) continue;
#pragma unroll
      for (int i = 0; i < ATT_MAX_CH; ++i) {
        const int c = lane + 32 * i;
        if (c < d) acc[i] = fmaf(pj, to_float(vc[offj + c]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
  for (int i = 0; i < ATT_MAX_CH; ++i) {
    const int c = lane + 32 * i;
    if (c < d) out[((long long)t * q_heads + h) * d + c] = from_float<T>(acc[i] * inv);
  }
}

extern "C" int llm_attention_plain(const void* q, void* out, int dtype, void* k_base, void* v_base,
                                   const int32_t* block_table, long long page_stride,
                                   int table_stride, int page_tokens, int kv_heads, int head_dim,
                                   const int32_t* positions, const int32_t* row_seq, int q_heads,
                                   int n_tokens, float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (head_dim > 32 * ATT_MAX_CH || q_heads % kv_heads) return ERR_BAD_SIZE;
  PagedCache c{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  const long long items = (long long)n_tokens * q_heads;
  const unsigned blocks = (unsigned)((items + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = (size_t)ATT_WARPS * head_dim * sizeof(float);
  if (dtype == DT_F32)
    launch_kernel(attention_plain_kernel<float>, blocks, ATT_WARPS * 32, smem, stream, (const float*)q, (float*)out,
                  c, positions, row_seq, q_heads, n_tokens, scale, window);
  else if (dtype == DT_BF16)
    launch_kernel(attention_plain_kernel<__nv_bfloat16>, blocks, ATT_WARPS * 32, smem, stream,
                  (const __nv_bfloat16*)q, (__nv_bfloat16*)out, c, positions, row_seq, q_heads, n_tokens, scale,
                  window);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------------- SwiGLU

// out[t, i] = silu(gate[t, i]) * up[t, i] with gate = in[t, i] and up = in[t, inter + i]; `in`
// may be a sum of partial results.
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ in, int n_partials, long long partial_stride,
                              TO* __restrict__ out, long long total, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / inter;
    const int c = (int)(i % inter);
    float g = 0.0f, u = 0.0f;
    for (int p = 0; p < n_partials; ++p) {
      g += to_float(in[p * partial_stride + t * 2 * inter + c]);
      u += to_float(in[p * partial_stride + t * 2 * inter + inter + c]);
    }
    out[i] = from_float<TO>(g / (1.0f + expf(-g)) * u);
  }
}

extern "C" int llm_swiglu(const void* in, int in_dtype, int n_partials, long long partial_stride,
                          void* out, int out_dtype, int n_tokens, int inter, cudaStream_t stream) {
  const long long total = (long long)n_tokens * inter;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define LAUNCH_SWIGLU(TI, TO)                                                                    \
  launch_kernel(swiglu_kernel<TI, TO>, blocks, 256, 0, stream, (const TI*)in, n_partials,        \
                partial_stride, (TO*)out, total, inter)
  if (in_dtype == DT_F32 && out_dtype == DT_F32) LAUNCH_SWIGLU(float, float);
  else if (in_dtype == DT_F32 && out_dtype == DT_BF16) LAUNCH_SWIGLU(float, __nv_bfloat16);
  else if (in_dtype == DT_BF16 && out_dtype == DT_BF16) LAUNCH_SWIGLU(__nv_bfloat16, __nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH_SWIGLU
  return launch_status();
}

// ------------------------------------------------------------------------------- sampling

// One block per row: the index of the largest logit; the lowest index wins a tie.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int32_t* __restrict__ out,
                                   int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const float* row = logits + (long long)blockIdx.x * vocab;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < vocab / 4; i += blockDim.x) {
      const float4 q = row4[i];
      const float v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v[j] > bv || (v[j] == bv && 4 * i + j < bi)) { bv = v[j]; bi = 4 * i + j; }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
  }
  auto better = [](float v, int i, float w, int j) { return v > w || (v == w && i < j); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nwarp = blockDim.x >> 5;
    bv = lane < nwarp ? best_v[lane] : -INFINITY;
    bi = lane < nwarp ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

extern "C" int llm_argmax_rows(const float* logits, int32_t* out, int rows, int vocab,
                               cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_kernel(argmax_rows_kernel, rows, 1024, 0, stream, logits, out, vocab);
  return launch_status();
}

// One block per row.  temperature[r] <= 0: argmax.  Otherwise weights exp((l - max) / T) and an
// inverse-CDF walk in id order: the first id whose running sum exceeds uniform[r] * total
// (cuongvng/bare-cuda-4gib engine/src/sampler.cpp:38-58).  Each thread owns a contiguous span of
// ids, so the walk order is the id order.
__global__ void sample_rows_kernel(const float* __restrict__ logits,
                                   const float* __restrict__ temperature,
                                   const float* __restrict__ uniform, int32_t* __restrict__ out,
                                   int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ float span_sum[256];
  __shared__ int chosen_thread;
  const int r = blockIdx.x;
  const float temp = temperature[r];
  if (!(temp > 0.0f)) return;  // greedy rows are filled by the argmax kernel
  const float* row = logits + (long long)r * vocab;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = scratch[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) mx = fmaxf(mx, scratch[w]);
  __syncthreads();

  const float inv_t = 1.0f / temp;
  const int span = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * span, hi = min(vocab, lo + span);
  float mine = 0.0f;
  for (int i = lo; i < hi; ++i) mine += expf((row[i] - mx) * inv_t);
  span_sum[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    double total = 0.0;
    for (int i = 0; i < blockDim.x; ++i) total += span_sum[i];
    double target = (double)uniform[r] * total;
    int pick = -1;
    for (int i = 0; i < blockDim.x; ++i) {
      if (target < (double)span_sum[i]) { pick = i; break; }
      target -= span_sum[i];
    }
    chosen_thread = pick;
    scratch[0] = (float)target;
  }
  __syncthreads();
  const int pick = chosen_thread;
  if (pick < 0) {
    // rounding left the sum short: the last id with any weight, as the host sampler's fallback
    if (threadIdx.x == 0) out[r] = vocab - 1;
    return;
  }
  if (threadIdx.x == pick) {
    float target = scratch[0];
    int id = hi - 1;
    for (int i = lo; i < hi; ++i) {
      target -= expf((row[i] - mx) * inv_t);
      if (target < 0.0f) { id = i; break; }
    }
    out[r] = id;
  }
}

extern "C" int llm_sample_rows(const float* logits, const float* temperature, const float* uniform,
                               int32_t* out, int rows, int vocab, cudaStream_t stream) {
  if (rows <= 0) return 0;
  launch_kernel(argmax_rows_kernel, rows, 1024, 0, stream, logits, out, vocab);
  launch_kernel(sample_rows_kernel, rows, 256, 0, stream, logits, temperature, uniform, out, vocab);
  return launch_status();
}
