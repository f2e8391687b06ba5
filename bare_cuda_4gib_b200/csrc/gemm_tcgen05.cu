// bfloat16 matrix product out[t, f] = sum_k act[t, k] * w[f, k] on the Blackwell tensor cores:
// TMA loads into 128-byte-swizzled shared memory, tcgen05.mma with the accumulator in tensor
// memory, tcgen05.ld for the epilogue.  This replaces the SIMT matmuls of cuongvng/bare-cuda-4gib
// (engine/kernels/gemm_tiled.cuh:36-96 for m > 16, engine/kernels/gemv_fp16.cu:21-101 for
// m <= 16) with one kernel for prefill and decode.
//
// Two orientations of the same kernel.
// ORIENT 0 (few tokens): the weight matrix is the 128-row MMA operand (A) and the activations are
// the N operand (B): one thread block computes 128 output features for BN tokens, BN in
// {16, 32, 64, 128, 256}.  A decode step therefore still fills the 128 MMA rows with weights,
// which is what has to be streamed from memory.  In tensor memory lane = feature and column =
// token, so an epilogue warp stores 32 consecutive features of one token with one store.
// ORIENT 1 (many tokens): 128 tokens are the MMA rows and BN (128 or 256) output features the
// N operand; lane = token, column = feature, so an epilogue thread stores 16 consecutive
// features of its token with vector stores.
//
// Split K.  gridDim.z thread blocks share the K range of a tile; each writes its float32 partial
// result to out + z * partial_stride.  The consumer kernels (residual add + norm, rotation,
// SwiGLU) add the partials in index order, so no atomics and no reduction pass are needed and
// the result does not depend on timing.
//
// MODE 1 (SwiGLU): w is [gate rows; up rows] and the block stores silu(gate) * up.  ORIENT 0
// makes its 128 MMA rows of 64 gate rows and the matching 64 up rows, so the accumulator holds
// gate in lanes 0..63 and up in lanes 64..127; the two epilogue warps that own the up lanes hand
// their values over through shared memory.  ORIENT 1 loads BN/2 gate rows and the matching BN/2
// up rows as one N operand, so a thread finds gate in column c and up in column BN/2 + c.
//
// Warps: 0 = TMA producer, 1 = tensor memory allocation + MMA issue, 2..5 = epilogue.
// Every wait on an mbarrier is bounded: after about a second without progress the thread sets
// the error word, every role leaves its loop, tensor memory is released and the block returns.

#include "common.cuh"

#include <cuda.h>
#include <string.h>

namespace {

constexpr int BM = 128;      // features per block (MMA M)
constexpr int BK = 64;       // k elements per stage (one 128-byte swizzle row)
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;

constexpr int ERR_TIMEOUT_PRODUCER = 1;
constexpr int ERR_TIMEOUT_MMA = 2;
constexpr int ERR_TIMEOUT_EPILOGUE = 3;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Waits for the phase with the given parity; gives up after limit_ns or when another role
// has already given up.  Returns false on giving up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer();
  for (unsigned spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 63u) {
      if (*abort_flag) return false;
      if (global_timer() - start > limit_ns) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes, swizzled in
// 1024-byte groups of 8 rows (start address and offsets in 16-byte units, Blackwell version 1,
// layout type 2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);  // start address
  d |= (uint64_t)1 << 16;                  // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset: 8 rows of 128 bytes
  d |= (uint64_t)1 << 46;                  // descriptor version
  d |= (uint64_t)2 << 61;                  // 128-byte swizzle
  return d;
}

// Instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// What the epilogue of the tokens-on-rows orientation may do beyond storing the product.
struct RowsExtra {
  // The input was prepared for a norm whose factor is one number per row (see AddTo / Prenormed in
  // the launcher): it is bfloat16(residual * norm weight), and the factor rsqrt(mean of squares +
  // eps) is applied here to the float32 sums.  `sq_in` [sq_items][sq_stride]: parts of every
  // input row's sum of squares, added in index order.  Null: the input is what it is.
  const float* sq_in;
  int sq_items;
  long long sq_stride;
  float norm_width, eps;
  // With `out` the float32 residual stream (accumulate): besides residual += product the epilogue
  // leaves what the next norm's product needs: pre_x = bfloat16(new residual * pre_w) and this
  // tile's part of every row's sum of squares in pre_sq[feature tile][row].  Null: neither.
  __nv_bfloat16* pre_x;
  long long pre_x_stride;
  const void* pre_w;
  int pre_w_dtype;
  float* pre_sq;
  long long pre_sq_stride;
};

constexpr int STAGING_BYTES = 4 * 32 * 32 * 4;   // per epilogue warp 32 rows of 32 float32, for the adding epilogue

// The factor of the norm that the input rows were prepared for (1 without one).
__device__ __forceinline__ float row_scale(const RowsExtra& ex, int t, int n_tokens) {
  if (!ex.sq_in || t >= n_tokens) return 1.0f;
  float sq = 0.0f;
  for (int i = 0; i < ex.sq_items; ++i) sq += ex.sq_in[(long long)i * ex.sq_stride + t];
  return 1.0f / sqrtf(sq / ex.norm_width + ex.eps);
}

// Epilogue of one warp for a tile with tokens on the tensor-memory lanes (lane = token, column =
// feature): the warp's 32 tokens start at `t_first`, the tile's features at f0.  `lane_base` is
// the tensor-memory address of the warp's lanes at the accumulator's first column; `have_acc`
// false means an empty K range (zeros).  MODE 1: gate in column c, up in column BN/2 + c.
// `wait_acc()` waits until the accumulator is complete (false: the block has given up, nothing is
// stored); what does not depend on the accumulator is requested from memory before it is called.
template <int MODE, int DEPTH, typename Wait>
__device__ __forceinline__ void epilogue_tokens_on_rows(uint32_t lane_base, int BN, int F_TILE, int f0, int f_tile_index,
                                                        int t_first, int lane, bool have_acc, void* out, int out_is_f32,
                                                        long long ld_out, int n_tokens, int n_features,
                                                        const RowsExtra& ex, float* staging, Wait&& wait_acc) {
  float* out_f32 = reinterpret_cast<float*>(out);
  __nv_bfloat16* out_bf16 = reinterpret_cast<__nv_bfloat16*>(out);
  if (MODE == 0 && out_is_f32 == 2 && ex.pre_x) {
    // ---- residual += product, with the next norm prepared.  A thread owns a token's row of the
    // accumulator, but rows of the residual stream lie far apart in memory, so the warp passes 32
    // columns at a time through shared memory (16-byte chunks swizzled by row, free of bank
    // conflicts both ways) and then walks over them four rows per instruction, each row's 128
    // bytes read and written by eight neighbouring lanes.  The old residual values and the norm's
    // weights of DEPTH such chunks are in registers at any time: the first ones are requested
    // while the tensor core still works on the tile, and a chunk's registers are refilled for
    // the chunk DEPTH further on as soon as it is done, so the memory's latency is not waited for.
    const int sub = lane >> 3, ch = lane & 7;
    float sq_acc[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) sq_acc[it] = 0.0f;
    float4 old[DEPTH][8], w[DEPTH];
    bool f_ok[DEPTH];
    auto fetch = [&](int d, int cc) {     // (d is a constant wherever this is called)
      const int f = f0 + cc + ch * 4;
      f_ok[d] = cc < F_TILE && f + 4 <= n_features && cc + ch * 4 < F_TILE;   // (a tile's width is a multiple of 16)
      w[d] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (f_ok[d]) {
        if (ex.pre_w_dtype == DT_BF16) {
          const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(ex.pre_w) + f);
          const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
          const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
          w[d] = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
        } else {
          w[d] = *reinterpret_cast<const float4*>(static_cast<const float*>(ex.pre_w) + f);
        }
      }
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int t = t_first + it * 4 + sub;
        old[d][it] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (f_ok[d] && t < n_tokens) old[d][it] = *reinterpret_cast<const float4*>(out_f32 + (long long)t * ld_out + f);
      }
    };
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) fetch(d, 32 * d);
    if (!wait_acc()) return;
#pragma unroll 1
    for (int c0 = 0; c0 < F_TILE; c0 += 32 * DEPTH) {
      if (f0 + c0 >= n_features) break;   // uniform across the block
#pragma unroll
      for (int d = 0; d < DEPTH; ++d) {
        const int cc = c0 + 32 * d, f = f0 + cc + ch * 4;
        if (cc < F_TILE && f0 + cc < n_features) {   // uniform across the warp
          uint32_t v[32];
          if (have_acc) {
            tmem_load16(lane_base + cc, *reinterpret_cast<uint32_t(*)[16]>(&v[0]));
            tmem_load16(lane_base + cc + 16, *reinterpret_cast<uint32_t(*)[16]>(&v[16]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(staging + lane * 32 + ((c ^ (lane & 7)) << 2)) =
                make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = it * 4 + sub, t = t_first + row;
            if (!f_ok[d] || t >= n_tokens) continue;
            const float4 a = *reinterpret_cast<const float4*>(staging + row * 32 + ((ch ^ (row & 7)) << 2));
            const float4 o4 = old[d][it];
            const float4 now = make_float4(o4.x + a.x, o4.y + a.y, o4.z + a.z, o4.w + a.w);
            *reinterpret_cast<float4*>(out_f32 + (long long)t * ld_out + f) = now;
            const __nv_bfloat162 p01 = __floats2bfloat162_rn(now.x * w[d].x, now.y * w[d].y);
            const __nv_bfloat162 p23 = __floats2bfloat162_rn(now.z * w[d].z, now.w * w[d].w);
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t*>(&p01);
            packed.y = *reinterpret_cast<const uint32_t*>(&p23);
            *reinterpret_cast<uint2*>(ex.pre_x + (long long)t * ex.pre_x_stride + f) = packed;
            sq_acc[it] += now.x * now.x;
            sq_acc[it] += now.y * now.y;
            sq_acc[it] += now.z * now.z;
            sq_acc[it] += now.w * now.w;
          }
          __syncwarp();   // the staging rows are about to be overwritten
          fetch(d, cc + 32 * DEPTH);
        }
      }
    }
    // a row's eight lanes add up (in a fixed order), the first of them writes this tile's part
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      float part = sq_acc[it];
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      part += __shfl_xor_sync(0xffffffffu, part, 4);
      const int t = t_first + it * 4 + sub;
      if (ch == 0 && t < n_tokens) ex.pre_sq[(long long)f_tile_index * ex.pre_sq_stride + t] = part;
    }
    return;
  }
  const int t = t_first + lane;
  const float rs = row_scale(ex, t, n_tokens);
  if (!wait_acc()) return;
  const bool vec_ok = out_is_f32 ? (ld_out % 4 == 0 && (reinterpret_cast<uintptr_t>(out_f32) & 15) == 0)
                                 : (ld_out % 8 == 0 && (reinterpret_cast<uintptr_t>(out_bf16) & 15) == 0);
#pragma unroll 1
  for (int c0 = 0; c0 < F_TILE; c0 += 16) {
    if (f0 + c0 >= n_features) break;  // uniform across the block
    uint32_t g[16], u[16];
    if (have_acc) {
      tmem_load16(lane_base + c0, g);
      if (MODE == 1) tmem_load16(lane_base + BN / 2 + c0, u);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) g[j] = u[j] = 0u;
    }
    // (rows past the step's last token hold whatever the activation buffer held before: nothing is
    // computed from them, least of all a division, whose slow path such values would take)
    if (t >= n_tokens) continue;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = __uint_as_float(g[j]) * rs;
      if (MODE == 1) v[j] = v[j] / (1.0f + expf(-v[j])) * (__uint_as_float(u[j]) * rs);
    }
    const int f = f0 + c0;
    const long long at = (long long)t * ld_out + f;
    if (vec_ok && f + 16 <= n_features) {
      if (out_is_f32) {
        float4* dst = reinterpret_cast<float4*>(out_f32 + at);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          float4 w4 = make_float4(v[4 * q4], v[4 * q4 + 1], v[4 * q4 + 2], v[4 * q4 + 3]);
          if (out_is_f32 == 2) {   // accumulate: the output is the float32 residual stream
            const float4 old = dst[q4];
            w4.x += old.x, w4.y += old.y, w4.z += old.z, w4.w += old.w;
          }
          dst[q4] = w4;
        }
      } else {
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          pk[j] = *reinterpret_cast<uint32_t*>(&b);
        }
        uint4* dst = reinterpret_cast<uint4*>(out_bf16 + at);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (f + j < n_features) {
          if (out_is_f32) out_f32[at + j] = out_is_f32 == 2 ? out_f32[at + j] + v[j] : v[j];
          else out_bf16[at + j] = __float2bfloat16_rn(v[j]);
        }
      }
    }
  }
}

// Sizes of a launch that depend on the N tile `bn` (a run-time value: any multiple of 16 up to
// 256, so that the number of tiles can be matched to the number of SMs).
struct Geometry {
  int bn;           // MMA N: tokens (ORIENT 0) or weight rows (ORIENT 1) per tile
  int a_tiles;      // 128-row operand tiles per stage
  int b_bytes;      // bytes of the N operand tile
  int stage_bytes;
  int stages;
  int tmem_cols;    // power of two >= bn * a_tiles, at least 32
  uint32_t idesc;
  unsigned long long wait_ns;   // how long a role waits on an mbarrier before it gives up
  int drop_k_block;             // tests only (llm_gemm_test_hooks): this k block's barrier is armed, its copies are left out
};

constexpr int A_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 8;

// Set by llm_gemm_test_hooks: the wait limit of the launches that follow, and a k block whose copies
// the producer of the non-persistent kernel leaves out, so that a test can watch a bounded wait run out.
static unsigned long long g_wait_ns = WAIT_LIMIT_NS;
static int g_drop_k_block = -1;

static Geometry make_geometry(int bn, int mode, int orient, int blocks_per_sm) {
  Geometry g;
  g.wait_ns = g_wait_ns;
  g.drop_k_block = g_drop_k_block;
  g.bn = bn;
  g.a_tiles = 1;
  g.b_bytes = bn * BK * 2;
  g.stage_bytes = g.a_tiles * A_BYTES + g.b_bytes;
  const int budget = (blocks_per_sm == 2 ? 110 : 200) * 1024;
  g.stages = budget / g.stage_bytes;
  if (g.stages > MAX_STAGES) g.stages = MAX_STAGES;
  int cols = 32;
  while (cols < bn * g.a_tiles) cols *= 2;
  g.tmem_cols = cols;
  g.idesc = instr_desc_bf16(BM, bn);
  return g;
}

// Streaming multiprocessors of the current device, asked once.
static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1)
      n = 148;   // a B200
  }
  return n;
}

static size_t smem_bytes(const Geometry& g) { return (size_t)g.stages * g.stage_bytes + 1024 + 256; }

template <int MODE, int ORIENT, int BLOCKS_PER_SM>
__global__ void __launch_bounds__(NUM_THREADS, BLOCKS_PER_SM)
gemm_tcgen05_kernel(const Geometry geo, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                    void* __restrict__ out, int out_is_f32, int n_tokens, int n_features, int k_blocks,
                    int k_blocks_per_split, long long ld_out, long long partial_stride, int up_row_offset,
                    const RowsExtra ex, int* __restrict__ error_word) {
  const int BN = geo.bn;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + geo.stages * geo.stage_bytes);
  uint64_t* empty_bar = full_bar + geo.stages;
  uint64_t* tmem_full_bar = empty_bar + geo.stages;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // ORIENT 0: 128 features (MODE 1: 64 outputs) x BN tokens.  ORIENT 1: 128 tokens x BN features
  // (MODE 1: BN/2 outputs).
  const int F_TILE = ORIENT == 0 ? (MODE == 1 ? BM / 2 : BM) : (MODE == 1 ? BN / 2 : BN);
  const int f0 = blockIdx.x * F_TILE;
  const int t0 = blockIdx.y * (ORIENT == 0 ? BN : BM);
  const int kb_begin = blockIdx.z * k_blocks_per_split;
  const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);
  const int n_kb = max(0, kb_end - kb_begin);

  // One stage's loads, in two halves: the weight tiles depend on no other kernel and may be
  // fetched before pdl_wait(); the activation tile is another kernel's output and may not.
  // The first half arms the stage's barrier with the bytes of both.
  auto issue_weights = [&](int i, int s, int which) {   // which: 0 = arm + first tile, 1 = second tile, 2 = both
    uint8_t* stage = smem + s * geo.stage_bytes;
    if (which != 1) mbar_expect_tx(&full_bar[s], geo.stage_bytes);
    if (i == geo.drop_k_block) return;   // a test's way to leave a barrier waiting (never set otherwise)
    const int k0 = (kb_begin + i) * BK;
    if (ORIENT == 0) {
      if (which != 1) tma_load_2d(stage, &map_w, &full_bar[s], k0, f0);   // MODE 1: map_w's box has 64 rows
      if (MODE == 1 && which != 0) tma_load_2d(stage + A_BYTES / 2, &map_w, &full_bar[s], k0, up_row_offset + f0);
    } else {
      uint8_t* b_tile = stage + A_BYTES;
      if (which != 1) tma_load_2d(b_tile, &map_w, &full_bar[s], k0, f0);
      // MODE 1: map_w's box has BN/2 rows: gate rows above, the matching up rows below
      if (MODE == 1 && which != 0) tma_load_2d(b_tile + geo.b_bytes / 2, &map_w, &full_bar[s], k0, up_row_offset + f0);
    }
  };
  auto issue_activations = [&](int i, int s) {
    if (i == geo.drop_k_block) return;
    uint8_t* stage = smem + s * geo.stage_bytes;
    const int k0 = (kb_begin + i) * BK;
    if (ORIENT == 0) tma_load_2d(stage + geo.a_tiles * A_BYTES, &map_a, &full_bar[s], k0, t0);
    else tma_load_2d(stage, &map_a, &full_bar[s], k0, t0);
  };
  const int n_early = min(n_kb, geo.stages);  // stages that are free from the start

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    for (int s = 0; s < geo.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int i = 0; i < n_early; ++i) issue_weights(i, i, 2);   // overlaps the tail of the kernel before
    pdl_wait();
    for (int i = 0; i < n_early; ++i) issue_activations(i, i);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)),
                 "r"(geo.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();  // every thread: nothing below may run ahead of the kernels before this one
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Issuing a TMA copy costs the issuing thread a few hundred cycles, so a stage's copies are
    // shared: lane 0 arms the barrier and fetches the weight tile(s), lane 1 the activations.
    // (A third lane for the second weight tile of a SwiGLU product measured slower.)
    if (lane < 2) {
      int armed = n_early;
      // stage and phase advance by counting: a division per k block would slow the issue down
      int s = n_early == geo.stages ? 0 : n_early;
      uint32_t phase = n_early == geo.stages ? 1 : 0;
      for (int i = n_early; i < n_kb; ++i) {
        if (!mbar_wait(&empty_bar[s], phase ^ 1, abort_flag, geo.wait_ns)) {
          *abort_flag = 1;
          atomicCAS(error_word, 0, ERR_TIMEOUT_PRODUCER);
          break;
        }
        if (lane == 1) issue_activations(i, s);
        else issue_weights(i, s, 2);
        armed = i + 1;
        if (++s == geo.stages) { s = 0; phase ^= 1; }
      }
      if (lane == 0 && *abort_flag) {
        // copies already issued still land in shared memory: wait for them (bounded) before leaving
        for (int i = max(0, armed - geo.stages); i < armed; ++i) {
          const unsigned long long start = global_timer();
          while (!mbar_try_wait(&full_bar[i % geo.stages], (i / geo.stages) & 1) &&  // rare path
                 global_timer() - start < geo.wait_ns / 10) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = geo.idesc;
      bool ok = true;
      int s = 0;
      uint32_t phase = 0;
      const uint32_t smem_base = smem_u32(smem);
      for (int i = 0; i < n_kb && ok; ++i) {
        if (!mbar_wait(&full_bar[s], phase, abort_flag, geo.wait_ns)) {
          *abort_flag = 1;
          atomicCAS(error_word, 0, ERR_TIMEOUT_MMA);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_base + s * geo.stage_bytes;
        const uint32_t b_addr = a_addr + geo.a_tiles * A_BYTES;
        const uint64_t desc_a = smem_desc_sw128(a_addr);
        const uint64_t desc_b = smem_desc_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
          umma_bf16(tmem_base, desc_a + koff, desc_b + koff, idesc, acc);
        }
        umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        if (++s == geo.stages) { s = 0; phase ^= 1; }
      }
      umma_commit(tmem_full_bar);    // accumulator complete (or, after giving up, releases the epilogue)
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quad = warp & 3;  // tensor-memory lanes 32 * quad .. + 31 belong to this warp
    auto wait_acc = [&]() -> bool {
      bool ok = mbar_wait(tmem_full_bar, 0, abort_flag, geo.wait_ns);
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(error_word, 0, ERR_TIMEOUT_EPILOGUE);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps agree on whether to go on
      ok = !*abort_flag;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      return ok;
    };
    const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
    float* out_f32 = reinterpret_cast<float*>(out) + (long long)blockIdx.z * partial_stride;
    __nv_bfloat16* out_bf16 = reinterpret_cast<__nv_bfloat16*>(out) + (long long)blockIdx.z * partial_stride;
    if (ORIENT == 1) {
      // (the pipeline's stages are idle once the accumulator is complete: the adding epilogue passes its tiles through them)
      epilogue_tokens_on_rows<MODE, BLOCKS_PER_SM == 1 ? 4 : 1>(
          lane_base, BN, F_TILE, f0, blockIdx.x, t0 + quad * 32, lane, n_kb > 0,
          out_is_f32 ? static_cast<void*>(out_f32) : static_cast<void*>(out_bf16), out_is_f32, ld_out, n_tokens, n_features,
          ex, reinterpret_cast<float*>(smem) + quad * (32 * 32), wait_acc);
    } else if (wait_acc()) {
      if (ORIENT == 0 && MODE == 1) {
        // lanes 0..63 hold gate, lanes 64..127 up, for the block's 64 output features: the up warps
        // park their values in shared memory (the pipeline stages are idle by now), [token][feature]
        float* handover = reinterpret_cast<float*>(smem);
        const int l64 = (quad & 1) * 32 + lane;
        if (quad >= 2) {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            if (t0 + c0 >= n_tokens) break;
            uint32_t u[16];
            if (n_kb > 0) {
              tmem_load16(lane_base + c0, u);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) u[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) handover[(c0 + j) * 64 + l64] = __uint_as_float(u[j]);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
        if (quad < 2) {
          const int f = f0 + l64;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            if (t0 + c0 >= n_tokens) break;
            uint32_t g[16];
            if (n_kb > 0) {
              tmem_load16(lane_base + c0, g);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) g[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c0 + j;
              if (t < n_tokens && f < n_features) {
                const float gate = __uint_as_float(g[j]);
                const float v = gate / (1.0f + expf(-gate)) * handover[(c0 + j) * 64 + l64];
                if (out_is_f32) out_f32[(long long)t * ld_out + f] = v;
                else out_bf16[(long long)t * ld_out + f] = __float2bfloat16_rn(v);
              }
            }
          }
        }
      } else if (ORIENT == 0) {
        const int f = f0 + quad * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          if (t0 + c0 >= n_tokens) break;  // uniform across the warp
          uint32_t g[16];
          if (n_kb > 0) {
            tmem_load16(lane_base + c0, g);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] = 0u;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t < n_tokens && f < n_features) {
              const float v = __uint_as_float(g[j]);
              if (out_is_f32) out_f32[(long long)t * ld_out + f] = v;
              else out_bf16[(long long)t * ld_out + f] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(geo.tmem_cols)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// The same product for many tokens (ORIENT 1, no K split) as a persistent kernel: one block per SM
// walks over output tiles, the stage ring runs on across tile boundaries (no pipeline drain and
// refill per tile, all of shared memory for one ring), and the accumulator alternates between two
// halves of tensor memory, so that the epilogue warps drain tile j while the MMA warp already
// works on tile j + 1.  Consecutive tiles of a block's neighbours share activation rows and weight
// rows (tile index -> token tile fastest), which keeps both operands in L2.
constexpr int ACC_COLS = 256;   // tensor-memory columns per accumulator half

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_persistent_kernel(const Geometry geo, const __grid_constant__ CUtensorMap map_w,
                               const __grid_constant__ CUtensorMap map_a, void* __restrict__ out, int out_is_f32,
                               int n_tokens, int n_features, int n_kb, long long ld_out, int up_row_offset,
                               int f_tiles, int t_tiles, const RowsExtra ex, int* __restrict__ error_word) {
  const int BN = geo.bn;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + geo.stages * geo.stage_bytes);
  uint64_t* empty_bar = full_bar + geo.stages;
  uint64_t* acc_full = empty_bar + geo.stages;      // [2]: the accumulator half holds a finished tile
  uint64_t* acc_empty = acc_full + 2;               // [2]: the epilogue has read it out
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int F_TILE = MODE == 1 ? BN / 2 : BN;
  const int n_tiles = f_tiles * t_tiles;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    for (int s = 0; s < geo.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);   // the four epilogue warps
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)),
                 "r"(2 * ACC_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Issuing a copy costs its thread a few hundred cycles, about what the tensor core needs for
    // a stage of a narrow tile.  So four lanes issue: lanes 0 and 1 take the even k blocks of the
    // block's sequence (weights and barrier / activations), lanes 2 and 3 the odd ones.
    if (lane < 4) {
      const int role = lane & 1, turn = lane >> 1;
      int s = turn % geo.stages, armed = 0;
      uint32_t phase = 0;
      int q = 0;   // k blocks of this thread block so far, over all its tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int f0 = (tile / t_tiles) * F_TILE, t0 = (tile % t_tiles) * BM;
        for (int i = 0; i < n_kb; ++i, ++q) {
          if ((q & 1) != turn) continue;
          if (!mbar_wait(&empty_bar[s], phase ^ 1, abort_flag, geo.wait_ns)) {
            *abort_flag = 1;
            atomicCAS(error_word, 0, ERR_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t* stage = smem + s * geo.stage_bytes;
          const int k0 = i * BK;
          if (role == 0) {
            mbar_expect_tx(&full_bar[s], geo.stage_bytes);
            uint8_t* b_tile = stage + A_BYTES;
            tma_load_2d(b_tile, &map_w, &full_bar[s], k0, f0);
            if (MODE == 1) tma_load_2d(b_tile + geo.b_bytes / 2, &map_w, &full_bar[s], k0, up_row_offset + f0);
          } else {
            tma_load_2d(stage, &map_a, &full_bar[s], k0, t0);
          }
          armed = q + 1;
          s += 2;
          if (s >= geo.stages) { s -= geo.stages; phase ^= 1; }
        }
      }
      armed = max(armed, __shfl_sync(0xfu, armed, 2));
      if (lane == 0 && *abort_flag) {
        // copies already issued still land in shared memory: wait for them (bounded) before leaving
        for (int i = max(0, armed - geo.stages); i < armed; ++i) {
          const unsigned long long start = global_timer();
          while (!mbar_try_wait(&full_bar[i % geo.stages], (i / geo.stages) & 1) &&
                 global_timer() - start < geo.wait_ns / 10) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = geo.idesc, smem_base = smem_u32(smem);
      int s = 0, j = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++j) {
        const int buf = j & 1;
        if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, abort_flag, geo.wait_ns)) {
          *abort_flag = 1;
          atomicCAS(error_word, 0, ERR_TIMEOUT_MMA);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc_addr = tmem_base + buf * ACC_COLS;
        for (int i = 0; i < n_kb; ++i) {
          if (!mbar_wait(&full_bar[s], phase, abort_flag, geo.wait_ns)) {
            *abort_flag = 1;
            atomicCAS(error_word, 0, ERR_TIMEOUT_MMA);
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_base + s * geo.stage_bytes;
          const uint64_t desc_a = smem_desc_sw128(a_addr), desc_b = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
            umma_bf16(acc_addr, desc_a + koff, desc_b + koff, idesc, (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == geo.stages) { s = 0; phase ^= 1; }
        }
        umma_commit(&acc_full[buf]);   // (after giving up this still releases the epilogue)
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quad = warp & 3;
    int j = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++j) {
      const int buf = j & 1;
      const int f0 = (tile / t_tiles) * F_TILE, t0 = (tile % t_tiles) * BM;
      bool ok = true;
      auto wait_acc = [&]() -> bool {
        if (!mbar_wait(&acc_full[buf], (j >> 1) & 1, abort_flag, geo.wait_ns) || *abort_flag) {
          *abort_flag = 1;
          atomicCAS(error_word, 0, ERR_TIMEOUT_EPILOGUE);
          ok = false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        return ok;
      };
      const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16) + buf * ACC_COLS;
      epilogue_tokens_on_rows<MODE, 2>(lane_base, BN, F_TILE, f0, tile / t_tiles, t0 + quad * 32, lane, n_kb > 0, out, out_is_f32,
                                       ld_out, n_tokens, n_features, ex,
                                       reinterpret_cast<float*>(smem + geo.stages * geo.stage_bytes + 256) + quad * (32 * 32),
                                       wait_acc);
      if (!ok) break;
      // this warp has read its lanes of the half out: the MMA warp may overwrite it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * ACC_COLS) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

template <int MODE, int ORIENT, int BLOCKS_PER_SM>
int launch(int bn, const CUtensorMap* map_w, const CUtensorMap* map_a, void* out, int out_is_f32, int n_tokens,
           int n_features, int K, long long ld_out, long long partial_stride, int splits, int up_row_offset,
           const RowsExtra& ex, int* error_word, cudaStream_t stream) {
  const Geometry g = make_geometry(bn, MODE, ORIENT, BLOCKS_PER_SM);
  if (g.stages < 1 || g.tmem_cols * BLOCKS_PER_SM > 512) return ERR_BAD_SIZE;
  auto kern = gemm_tcgen05_kernel<MODE, ORIENT, BLOCKS_PER_SM>;
  static size_t configured = 0;
  const size_t smem = smem_bytes(g);
  if (smem > configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return launch_status();
    configured = smem;
  }
  const int k_blocks = (K + BK - 1) / BK;
  const int per_split = (k_blocks + splits - 1) / splits;
  const int f_tile = ORIENT == 0 ? (MODE == 1 ? BM / 2 : BM) : (MODE == 1 ? bn / 2 : bn);
  const int t_tile = ORIENT == 0 ? bn : BM;
  dim3 grid((n_features + f_tile - 1) / f_tile, (n_tokens + t_tile - 1) / t_tile, splits);
  if (grid.y > 65535 || grid.z > 65535) return ERR_BAD_SIZE;
  launch_kernel(kern, grid, NUM_THREADS, smem, stream, g, *map_w, *map_a, out, out_is_f32, n_tokens, n_features,
                k_blocks, per_split, ld_out, partial_stride, up_row_offset, ex, error_word);
  return launch_status();
}

template <int MODE>
int launch_persistent(int bn, const CUtensorMap* map_w, const CUtensorMap* map_a, void* out, int out_is_f32, int n_tokens,
                      int n_features, int K, long long ld_out, int up_row_offset, const RowsExtra& ex, int* error_word,
                      cudaStream_t stream) {
  const Geometry g = make_geometry(bn, MODE, 1, 1);
  if (g.stages < 2 || g.tmem_cols > ACC_COLS) return ERR_BAD_SIZE;
  auto kern = gemm_tcgen05_persistent_kernel<MODE>;
  static size_t configured = 0;
  const size_t smem = smem_bytes(g) + STAGING_BYTES;   // the adding epilogue's staging rows lie behind the barriers
  if (smem > configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return launch_status();
    configured = smem;
  }
  const int f_tile = MODE == 1 ? bn / 2 : bn;
  const int f_tiles = (n_features + f_tile - 1) / f_tile, t_tiles = (n_tokens + BM - 1) / BM;
  const long long tiles = (long long)f_tiles * t_tiles;
  const int grid = tiles < sm_count() ? (int)tiles : sm_count();
  launch_kernel(kern, grid, NUM_THREADS, smem, stream, g, *map_w, *map_a, out, out_is_f32, n_tokens, n_features,
                (K + BK - 1) / BK, ld_out, up_row_offset, f_tiles, t_tiles, ex, error_word);
  return launch_status();
}

}  // namespace

// Writes a 128-byte CUtensorMap for a row-major bfloat16 matrix [rows, cols] (row stride in
// elements) with a box of box_rows x 64 columns and the 128-byte swizzle.  Out-of-range parts of
// a box read as zero.  The base must be 16-byte aligned and the row stride a multiple of 8.
extern "C" int llm_gemm_tensor_map(void* map_out, const void* base, long long rows, long long cols,
                                   long long row_stride, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return 1000 + (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride % 8) || rows <= 0 || cols <= 0) return ERR_BAD_ALIGN;
  if (box_rows <= 0 || box_rows > 256) return ERR_BAD_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

// For tests of the bounded waits: the launches that follow give up on an mbarrier after `wait_ns`
// nanoseconds (0: the default of one second), and the producer of the non-persistent kernel arms
// the barrier of k block `drop_k_block` of every tile without issuing its copies (-1: none), so the
// MMA issuer's wait for it runs out: the kernel reports "MMA issuer" in the error word, releases its
// tensor memory and returns.  Call with (0, -1) to put things back.
extern "C" void llm_gemm_test_hooks(long long wait_ns, int drop_k_block) {
  g_wait_ns = wait_ns > 0 ? (unsigned long long)wait_ns : WAIT_LIMIT_NS;
  g_drop_k_block = drop_k_block;
}

// out[z][t, f] (z < splits) = partial sums of act[t, :] . w[f, :]; mode 1: silu(gate) * up with
// w = [gate; up], the up rows starting at `up_row_offset` (splits must be 1 then).
// `bn` is the N tile, a multiple of 16 up to 256 (of 32 for orient 1 with mode 1).
// `accumulate` (orient 1, mode 0, float32 out, no split): out[t, f] += the product, which is how a
// projection adds itself into the residual stream.
// orient 0: bn tokens per tile; map_a's box must have bn rows, map_w's 128 (64 in mode 1).
// orient 1: bn weight rows per tile; map_a's box must have 128 rows, map_w's bn rows (bn / 2 in mode 1).
// Orient 1 only, both optional (see RowsExtra):
// `sq_in` [sq_items][sq_stride]: the activations are bfloat16(residual * norm weight) and the norm's
// factor per row, 1 / sqrt(sum of the parts / norm_width + eps), is applied to the sums;
// `pre_x` (with accumulate): the kernel also writes pre_x[t, f] = bfloat16(out[t, f] * pre_w[f]) and
// pre_sq[feature tile][t] = that tile's part of the row's sum of squares (ceil(n_features / bn) tiles).
extern "C" int llm_gemm_bf16(const void* map_w, const void* map_a, void* out, int out_dtype, int n_tokens,
                             int n_features, int K, long long ld_out, long long partial_stride, int splits,
                             int bn, int mode, int orient, int up_row_offset, int accumulate, const float* sq_in,
                             int sq_items, long long sq_stride, float norm_width, float eps, void* pre_x,
                             long long pre_x_stride, const void* pre_w, int pre_w_dtype, float* pre_sq,
                             long long pre_sq_stride, int* error_word, cudaStream_t stream) {
  if (n_tokens <= 0 || n_features <= 0) return 0;
  if (K <= 0 || splits <= 0 || (mode == 1 && splits != 1)) return ERR_BAD_SIZE;
  if (splits > 1 && out_dtype != DT_F32) return ERR_BAD_DTYPE;
  if (out_dtype != DT_F32 && out_dtype != DT_BF16) return ERR_BAD_DTYPE;
  CUtensorMap mw_copy, ma_copy;  // the caller's buffers need not be 64-byte aligned
  memcpy(&mw_copy, map_w, sizeof(CUtensorMap));
  memcpy(&ma_copy, map_a, sizeof(CUtensorMap));
  const CUtensorMap* mw = &mw_copy;
  const CUtensorMap* ma = &ma_copy;
  if (accumulate && (orient != 1 || mode != 0 || splits != 1 || out_dtype != DT_F32)) return ERR_BAD_SIZE;
  const int f32 = out_dtype == DT_F32 ? (accumulate ? 2 : 1) : 0;   // 2: out[t, f] += result
  if (bn < 16 || bn > 256 || bn % 16 || (mode == 1 && orient == 1 && bn % 32)) return ERR_BAD_SIZE;
  RowsExtra ex = {};
  if (sq_in) {
    if (orient != 1 || sq_items < 1 || sq_stride < n_tokens || !(norm_width > 0.0f)) return ERR_BAD_SIZE;
    ex.sq_in = sq_in, ex.sq_items = sq_items, ex.sq_stride = sq_stride, ex.norm_width = norm_width, ex.eps = eps;
  }
  if (pre_x) {
    if (!accumulate || !pre_w || !pre_sq || pre_sq_stride < n_tokens || n_features % 4 || ld_out % 4 || pre_x_stride % 4)
      return ERR_BAD_SIZE;
    if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(pre_w)) & 15 || reinterpret_cast<uintptr_t>(pre_x) & 7)
      return ERR_BAD_ALIGN;
    if (pre_w_dtype != DT_F32 && pre_w_dtype != DT_BF16) return ERR_BAD_DTYPE;
    ex.pre_x = static_cast<__nv_bfloat16*>(pre_x), ex.pre_x_stride = pre_x_stride, ex.pre_w = pre_w;
    ex.pre_w_dtype = pre_w_dtype, ex.pre_sq = pre_sq, ex.pre_sq_stride = pre_sq_stride;
  }
  // Two thread blocks per SM let one block's epilogue overlap the other's main loop, at the price
  // of half the pipeline depth each: worth it only when there are more tiles than SMs and at
  // least three stages still fit (two for the SwiGLU tiles, whose long epilogue gains most).
  const Geometry two = make_geometry(bn, mode, orient, 2);
  const long long f_tile = orient == 0 ? (mode == 1 ? BM / 2 : BM) : (mode == 1 ? bn / 2 : bn), t_tile = orient == 0 ? bn : BM;
  const long long tiles = ((n_features + f_tile - 1) / f_tile) * ((n_tokens + t_tile - 1) / t_tile) * splits;
  const bool pair = tiles > sm_count() && two.tmem_cols <= 256 && two.stages >= ((orient == 1 && mode == 1) ? 2 : 3);
  if (orient == 1 && splits == 1 && tiles > sm_count() && bn >= 192) {
    // More tiles than SMs: one block per SM walks over them (see the persistent kernel).  Only for
    // wide tiles: a stage of a narrow tile is shorter on the tensor core than the one issuing
    // thread's round of waiting for it, issuing its instructions and committing, and then two
    // blocks per SM with an issuing thread each are faster.
    if (mode == 0) return launch_persistent<0>(bn, mw, ma, out, f32, n_tokens, n_features, K, ld_out, up_row_offset, ex, error_word, stream);
    return launch_persistent<1>(bn, mw, ma, out, f32, n_tokens, n_features, K, ld_out, up_row_offset, ex, error_word, stream);
  }
#define GEMM_CASE(MODE_, ORIENT_)                                                                            \
  if (mode == MODE_ && orient == ORIENT_)                                                                    \
    return pair ? launch<MODE_, ORIENT_, 2>(bn, mw, ma, out, f32, n_tokens, n_features, K, ld_out,           \
                                            partial_stride, splits, up_row_offset, ex, error_word, stream)  \
                : launch<MODE_, ORIENT_, 1>(bn, mw, ma, out, f32, n_tokens, n_features, K, ld_out,           \
                                            partial_stride, splits, up_row_offset, ex, error_word, stream)
  GEMM_CASE(0, 0);
  GEMM_CASE(1, 0);
  GEMM_CASE(0, 1);
  GEMM_CASE(1, 1);
  return ERR_BAD_SIZE;
#undef GEMM_CASE
}
