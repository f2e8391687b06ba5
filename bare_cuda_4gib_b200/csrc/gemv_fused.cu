// Few-token matrix products with the work around them fused in: out[t, n] = sum_k x[t, k] W[n, k]
// for up to 32 tokens (the decode step and short prompt portions), bfloat16 weights, float32 sums.
//
// With so few tokens the product is bound by reading W once, and a step's time by the number of
// kernels and the memory round trips between them.  So this kernel takes its input in one of
// three forms and finishes its output in one of four:
//   input   PRO_BF16   x is a bfloat16 matrix in global memory
//           PRO_NORM   x = rms_norm(residual row) * weight, computed here from the float32
//                      residual stream (cuongvng/bare-cuda-4gib engine/kernels/rmsnorm.cu:26-40)
//           PRO_PRENORMED  the same norm, prepared by the product that last added into the
//                      residual stream: x arrives as bfloat16(residual * weight) with the rows'
//                      sums of squares in parts, and since the norm's factor rsqrt(mean + eps) is
//                      one number per token it is applied to the float32 sums on the way out
//   output  EPI_STORE  plain store (float32 or bfloat16)
//           EPI_ADD    residual[t, n] += result                (residual_add.cu:20); on request
//                      it also leaves what PRO_PRENORMED of the next product needs: bfloat16(new
//                      residual * next norm's weight) and this item's part of the sums of squares
//           EPI_SWIGLU W = [gate; up]: out[t, i] = silu(gate_i) * up_i        (swiglu.cu:22-23)
//           EPI_ROPE   W = [Wq; Wk; Wv]: rotates q and k by position, writes q to `out` and k, v
//                      into the paged cache                    (rope.cu:25-47, model.cpp:548-556)
//
// Layout of the work.  The tensor-core instruction mma.sync m16n8k16 takes 16 rows of W as A and
// 8 tokens as B.  Thread (g, t) of a warp (g = lane / 4, t = lane % 4) owns rows g and g + 8 of
// the 16, so an "item" is two groups of 8 rows of W that belong together: neighbouring rows for
// a plain product, 8 gate rows with their 8 up rows for SwiGLU, 8 features of a head with their
// rotation partners (half a head further) for the rotation.  The epilogue then finds both
// members of a pair in one thread.  The inner dimension is a sum and may be taken in any order
// as long as A and B agree: a thread reads 16 contiguous bytes (8 values of k) of each of its two
// rows and of its token's x and feeds them to two instructions.
//
// One block per SM (two, with one item each, when there are a few more items than SMs).  A
// producer warp streams the block's items through a ring of shared-memory stages (16 row pieces
// of up to `kc` values each, one bulk copy per piece, landing on an mbarrier); it starts before
// the kernel has waited for its predecessor in the stream, since weights are never written.
// Eight consumer warps split each stage's k range, multiply out of shared memory, and at the end
// of an item add their partial sums in warp order, so a result depends neither on the batch nor
// on the grid.  x for all tokens sits in shared memory for the whole kernel.  Every
// wait on an mbarrier is bounded: after about a second without progress the thread records an
// error code, and from then on every wait of the block returns at once, so the block still
// reaches its barriers and returns (its results are then invalid, which the error word tells).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;                       // consumer warps
constexpr int CONSUMERS = WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;        // plus the producer warp
constexpr int MAX_STAGES = 12;
constexpr int ROW_PAD = 64;                    // bytes between row pieces of a stage beyond their data:
                                               // keeps the 16-byte reads of a quarter warp on distinct banks
constexpr int SMEM_BUDGET = 220 * 1024;        // dynamic shared memory of one block per SM
constexpr int SMEM_HALF = 110 * 1024;          // ... of two blocks per SM
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;
constexpr int ERR_GEMV_PRODUCER = 21, ERR_GEMV_CONSUMER = 22;

enum { PRO_BF16 = 0, PRO_NORM = 1, PRO_PRENORMED = 2 };
constexpr int SQ_SLOTS = 32;                  // token slots per item in the sums-of-squares parts
enum { EPI_STORE = 0, EPI_ADD = 1, EPI_SWIGLU = 2, EPI_ROPE = 3 };


struct GemvArgs {
  const __nv_bfloat16* w;   // [w_rows, k] row-major
  int w_rows, k, n_items, tokens;
  int x_ld;                 // shared-memory row stride of x in elements
  int kc, stages;           // k values per stage of the ring, number of stages
  int norm_rows;            // PRO_NORM: residual rows staged in shared memory at a time
  int first_aliased;        // PRO_NORM: stages from this one on double as that staging area (else = stages)
  int* error_word;
  // input
  const void* x;            // PRO_BF16: bfloat16 [tokens, k]; PRO_NORM: float32 residual rows
  long long x_stride;       // elements between rows of x
  const void* norm_w;       // PRO_NORM: [k]
  int norm_w_dtype;
  float eps;
  const int32_t* row_index; // PRO_NORM, PRO_PRENORMED: token i reads row row_index[i] (null: i)
  const float* sq_in;       // PRO_PRENORMED: [sq_items][sq_stride] parts of the rows' sums of squares
  int sq_items;
  long long sq_stride;
  // EPI_ADD, optional: what the next product's PRO_PRENORMED needs
  __nv_bfloat16* pre_x;     // [tokens, n_out] = bfloat16(new residual * pre_w)
  long long pre_x_stride;
  const void* pre_w;        // the next norm's weight [n_out]
  int pre_w_dtype;
  float* pre_sq;            // [n_items][SQ_SLOTS]
  // output
  void* out;                // EPI_STORE/EPI_SWIGLU: [tokens, n]; EPI_ADD: float32 residual; EPI_ROPE: q [tokens, q_heads * d]
  int out_dtype;
  long long out_stride;
  int n_out;                // valid output features (rows of W for a plain product, the gate rows for SwiGLU)
  int up_offset;            // EPI_SWIGLU: first up row of W
  // rotation and cache
  PagedCache cache;
  const int32_t* positions;
  const int32_t* row_seq;
  const float* inv_freq;    // [d / 2], null: no rotation
  int q_heads, write_cache;
};

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
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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

// Waits for the phase with the given parity.  Gives up after WAIT_LIMIT_NS, or at once when some
// thread of the block has given up before: records `code`, raises the block's flag, returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up, int* error_word, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*gave_up) return false;
  const unsigned long long start = global_timer();
  for (unsigned spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 63u) {
      if (*gave_up) return false;
      if (global_timer() - start > WAIT_LIMIT_NS) {
        *gave_up = 1;
        if (error_word) atomicCAS(error_word, 0, code);
        return false;
      }
    }
  }
}

// One contiguous piece of global memory into shared memory; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The two rows of W that thread group g reads for `item` (clamped into W; `valid` tells whether
// the item's feature for this g exists at all).
template <int EPI>
__device__ __forceinline__ void item_rows(const GemvArgs& a, int item, int g, int& lo, int& hi) {
  if (EPI == EPI_SWIGLU) {
    lo = min(item * 8 + g, a.n_out - 1);
    hi = a.up_offset + lo;
  } else if (EPI == EPI_ROPE) {
    const int d = a.cache.head_dim, groups = d / 16;
    const int h = item / groups, p = item % groups;
    lo = h * d + p * 8 + g;
    hi = lo + d / 2;
  } else {
    lo = min(item * 16 + g, a.w_rows - 1);
    hi = min(item * 16 + g + 8, a.w_rows - 1);
  }
}

template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(THREADS, PRO == PRO_NORM ? 1 : 2) gemv_fused_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int row_stride = a.kc * 2 + ROW_PAD, stage_bytes = 16 * row_stride;
  uint8_t* ring = smem;                                                              // [stages][16][row_stride]
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ring + (size_t)a.stages * stage_bytes);   // [8 * NT][x_ld]
  float* red = reinterpret_cast<float*>(xs + (size_t)8 * NT * a.x_ld);               // [2][WARPS][NT * 4][32]
  float* scale_s = red + 2 * WARPS * NT * 4 * 32;                                    // PRO_PRENORMED: [SQ_SLOTS]
  float* norm_ws = scale_s + SQ_SLOTS;                                               // PRO_NORM: [k]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(norm_ws + (PRO == PRO_NORM ? a.k : 0));
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* x_bar = empty_bar + MAX_STAGES;
  uint64_t* norm_done = x_bar + 1;
  volatile int* gave_up = reinterpret_cast<volatile int*>(norm_done + 1);
  // PRO_NORM: residual rows are staged as float32 [norm_rows][k] in the ring's last stages, which
  // the producer leaves alone until the norm is done
  float* staging = reinterpret_cast<float*>(ring + (size_t)a.first_aliased * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], WARPS);
    }
    mbar_init(x_bar, 1);
    mbar_init(norm_done, 1);
    *gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == WARPS) {
    // ---- producer: lanes 0..7 fetch the items' "lo" rows, lanes 8..15 the "hi" rows
    int stage = 0;
    uint32_t phase = 0;
    uint32_t in_flight = 0, in_flight_parity = 0;   // per stage: a load was issued / with which parity
    bool staging_free = false;
    for (int item = blockIdx.x; item < a.n_items; item += gridDim.x) {
      int lo, hi;
      item_rows<EPI>(a, item, lane & 7, lo, hi);
      const __nv_bfloat16* src_row = a.w + (long long)(lane < 8 ? lo : hi) * a.k;
      for (int k0 = 0; k0 < a.k; k0 += a.kc) {
        const int len = min(a.kc, a.k - k0);
        bool ok = true;
        if (PRO == PRO_NORM && stage >= a.first_aliased && !staging_free) {
          if (lane == 0) ok = mbar_wait(norm_done, 0, gave_up, a.error_word, ERR_GEMV_PRODUCER);
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) goto producer_done;
          staging_free = true;
        }
        if (lane == 0) ok = mbar_wait(&empty_bar[stage], phase ^ 1u, gave_up, a.error_word, ERR_GEMV_PRODUCER);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) goto producer_done;
        if (lane == 0) mbar_expect_tx(&full_bar[stage], 16u * len * 2u);
        __syncwarp();
        if (lane < 16)
          bulk_load(ring + (size_t)stage * stage_bytes + lane * row_stride, src_row + k0, len * 2, &full_bar[stage]);
        in_flight |= 1u << stage;
        in_flight_parity = (in_flight_parity & ~(1u << stage)) | (phase << stage);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  producer_done:
    // If the block gave up, copies may still be on their way into its shared memory: wait for
    // them (bounded) before the block may return.
    if (*gave_up && lane == 0)
      for (int s = 0; s < a.stages; ++s)
        if (in_flight & (1u << s)) {
          const unsigned long long start = global_timer();
          while (!mbar_try_wait(&full_bar[s], (in_flight_parity >> s) & 1u) && global_timer() - start < WAIT_LIMIT_NS) {}
        }
    return;
  }

  // ---- consumers
  if (PRO == PRO_NORM) {     // the norm's weight is no kernel's output: fetch it before waiting
    for (int i = threadIdx.x; i < a.k; i += CONSUMERS)
      norm_ws[i] = a.norm_w_dtype == DT_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.norm_w)[i])
                                             : static_cast<const float*>(a.norm_w)[i];
  }
  pdl_wait();
  // x for every token into shared memory (rows past the last token are zero).  Rows come in as
  // bulk copies, which unlike loads into registers are not limited by the SM's load queue.
  if (PRO == PRO_NORM) {
    const float* res = static_cast<const float*>(a.x);
    const int n4 = a.k / 4;
    uint32_t x_phase = 0;
    consumer_barrier();       // norm_ws is complete
    for (int r0 = 0; r0 < 8 * NT; r0 += a.norm_rows) {
      const int batch = min(a.norm_rows, a.tokens - r0);     // rows of this batch that exist
      if (batch > 0) {
        if (warp == 0) {
          if (lane == 0) mbar_expect_tx(x_bar, (uint32_t)batch * a.k * 4u);
          __syncwarp();
          for (int j = lane; j < batch; j += 32) {
            const int r = r0 + j;
            bulk_load(staging + (size_t)j * a.k, res + (long long)(a.row_index ? a.row_index[r] : r) * a.x_stride,
                      (uint32_t)a.k * 4u, x_bar);
          }
        }
        mbar_wait(x_bar, x_phase, gave_up, a.error_word, ERR_GEMV_CONSUMER);
        x_phase ^= 1u;
      }
      for (int j = warp; j < a.norm_rows && r0 + j < 8 * NT; j += WARPS) {
        uint2* dst = reinterpret_cast<uint2*>(xs + (size_t)(r0 + j) * a.x_ld);
        if (j >= batch) {
          for (int i = lane; i < n4; i += 32) dst[i] = make_uint2(0u, 0u);
          continue;
        }
        const float4* src = reinterpret_cast<const float4*>(staging + (size_t)j * a.k);
        float sq = 0.0f;
        for (int i = lane; i < n4; i += 32) {
          const float4 u = src[i];
          sq += u.x * u.x;
          sq += u.y * u.y;
          sq += u.z * u.z;
          sq += u.w * u.w;
        }
        sq = warp_sum(sq);
        const float scale = 1.0f / sqrtf(sq / (float)a.k + a.eps);
        for (int i = lane; i < n4; i += 32) {
          const float4 u = src[i];
          const float4 w = reinterpret_cast<const float4*>(norm_ws)[i];
          const __nv_bfloat162 o01 = __floats2bfloat162_rn(u.x * scale * w.x, u.y * scale * w.y);
          const __nv_bfloat162 o23 = __floats2bfloat162_rn(u.z * scale * w.z, u.w * scale * w.w);
          uint2 o;
          o.x = *reinterpret_cast<const uint32_t*>(&o01);
          o.y = *reinterpret_cast<const uint32_t*>(&o23);
          dst[i] = o;
        }
      }
      if (r0 + a.norm_rows < 8 * NT) consumer_barrier();   // the staging rows are about to be overwritten
    }
  } else {
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(a.x);
    if (warp == 0) {
      if (lane == 0) mbar_expect_tx(x_bar, (uint32_t)a.tokens * a.k * 2u);
      __syncwarp();
      for (int r = lane; r < a.tokens; r += 32)
        bulk_load(xs + (size_t)r * a.x_ld, x + (long long)(a.row_index ? a.row_index[r] : r) * a.x_stride,
                  (uint32_t)a.k * 2u, x_bar);
    }
    const int per_row = a.k / 8;
    for (int r = a.tokens; r < 8 * NT; ++r)
      for (int c = threadIdx.x; c < per_row; c += CONSUMERS)
        *reinterpret_cast<uint4*>(xs + (size_t)r * a.x_ld + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    if (PRO == PRO_PRENORMED) {
      // the norm's factor per token from the parts of its row's sum of squares: lanes take items
      // lane, lane + 32, ..., then the warp adds up (the same order whatever the batch)
      for (int tok = warp; tok < a.tokens; tok += WARPS) {
        const int src = a.row_index ? a.row_index[tok] : tok;
        float sq = 0.0f;
        for (int i = lane; i < a.sq_items; i += 32) sq += a.sq_in[(long long)i * a.sq_stride + src];
        sq = warp_sum(sq);
        if (lane == 0) scale_s[tok] = 1.0f / sqrtf(sq / (float)a.k + a.eps);
      }
    }
    mbar_wait(x_bar, 0, gave_up, a.error_word, ERR_GEMV_CONSUMER);
  }
  consumer_barrier();
  if (PRO == PRO_NORM && threadIdx.x == 0) mbar_arrive(norm_done);

  int buf = 0, stage = 0;
  uint32_t phase = 0;
  for (int item = blockIdx.x; item < a.n_items; item += gridDim.x) {
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;

    // What the epilogue needs from memory does not depend on the sums: fetch it before the
    // barrier (old residual values; positions, angles and cache addresses).
    float old_lo[2] = {0.0f, 0.0f}, old_hi[2] = {0.0f, 0.0f}, rot_sin[2] = {0.0f, 0.0f}, rot_cos[2] = {1.0f, 1.0f};
    long long cache_at[2] = {-1, -1};
    if (warp < NT) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int tok = warp * 8 + 2 * t + j;
        if (tok >= a.tokens) continue;
        if (EPI == EPI_ADD) {
          const float* res = static_cast<const float*>(a.out) + (long long)tok * a.out_stride;
          if (item * 16 + g < a.n_out) old_lo[j] = res[item * 16 + g];
          if (item * 16 + g + 8 < a.n_out) old_hi[j] = res[item * 16 + g + 8];
        } else if (EPI == EPI_ROPE) {
          const int d = a.cache.head_dim, groups = d / 16;
          const int h = item / groups, i = (item % groups) * 8 + g;
          const int pos = a.positions[tok];
          if (h < a.q_heads + a.cache.kv_heads && a.inv_freq) sincosf((float)pos * a.inv_freq[i], &rot_sin[j], &rot_cos[j]);
          if (h >= a.q_heads && a.write_cache) {
            const bool is_v = h >= a.q_heads + a.cache.kv_heads;
            cache_at[j] = cache_offset(a.cache, a.row_seq[tok], pos, h - a.q_heads - (is_v ? a.cache.kv_heads : 0));
          }
        }
      }
    }

    for (int k0 = 0; k0 < a.k; k0 += a.kc) {
      const int n_steps = min(a.kc, a.k - k0) / 32;
      const int s_begin = warp * n_steps / WARPS, s_end = (warp + 1) * n_steps / WARPS;
      mbar_wait(&full_bar[stage], phase, gave_up, a.error_word, ERR_GEMV_CONSUMER);
      const uint8_t* lo_row = ring + (size_t)stage * stage_bytes + g * row_stride + 16 * t;
      const uint8_t* hi_row = lo_row + 8 * row_stride;
#pragma unroll 4
      for (int s = s_begin; s < s_end; ++s) {
        const uint4 lo = *reinterpret_cast<const uint4*>(lo_row + s * 64);
        const uint4 hi = *reinterpret_cast<const uint4*>(hi_row + s * 64);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const uint4 b = *reinterpret_cast<const uint4*>(xs + (size_t)(n * 8 + g) * a.x_ld + k0 + s * 32 + 8 * t);
          mma_bf16(acc[n], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
          mma_bf16(acc[n], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == a.stages) {
        stage = 0;
        phase ^= 1u;
      }
    }

    float* mine = red + ((size_t)(buf * WARPS + warp) * NT * 4) * 32;
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) mine[(n * 4 + i) * 32 + lane] = acc[n][i];
    consumer_barrier();
    // Warp n of the first NT warps finishes token group n: sums over the warps in index order,
    // then the epilogue.  v[0], v[1]: row "lo" for tokens 2t and 2t + 1; v[2], v[3]: row "hi".
    if (warp < NT) {
      const int n = warp;
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += red[((size_t)(buf * WARPS + w) * NT * 4 + n * 4 + i) * 32 + lane];
        v[i] = s;
      }
      float sq_mine[2] = {0.0f, 0.0f};   // EPI_ADD with pre outputs: this thread's share of its two tokens' sums of squares
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int tok = n * 8 + 2 * t + j;
        if (tok >= a.tokens) continue;
        float lo_v = v[j], hi_v = v[2 + j];
        if (PRO == PRO_PRENORMED) {
          lo_v *= scale_s[tok];
          hi_v *= scale_s[tok];
        }
        if (EPI == EPI_STORE || EPI == EPI_ADD) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int row = item * 16 + g + 8 * half;
            if (row >= a.n_out) continue;
            const float val = half ? hi_v : lo_v;
            const long long at = (long long)tok * a.out_stride + row;
            if (EPI == EPI_ADD) {
              const float now = (half ? old_hi[j] : old_lo[j]) + val;
              static_cast<float*>(a.out)[at] = now;
              if (a.pre_x) {
                const float w = a.pre_w_dtype == DT_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.pre_w)[row])
                                                         : static_cast<const float*>(a.pre_w)[row];
                a.pre_x[(long long)tok * a.pre_x_stride + row] = __float2bfloat16_rn(now * w);
                sq_mine[j] += now * now;
              }
            }
            else if (a.out_dtype == DT_F32) static_cast<float*>(a.out)[at] = val;
            else static_cast<__nv_bfloat16*>(a.out)[at] = __float2bfloat16_rn(val);
          }
        } else if (EPI == EPI_SWIGLU) {
          const int col = item * 8 + g;
          if (col >= a.n_out) continue;
          const float val = lo_v / (1.0f + expf(-lo_v)) * hi_v;
          const long long at = (long long)tok * a.out_stride + col;
          if (a.out_dtype == DT_F32) static_cast<float*>(a.out)[at] = val;
          else static_cast<__nv_bfloat16*>(a.out)[at] = __float2bfloat16_rn(val);
        } else {  // EPI_ROPE
          const int d = a.cache.head_dim, groups = d / 16, half = d / 2;
          const int h = item / groups, i = (item % groups) * 8 + g;   // head of [q; k; v], feature in the lower half
          const float first = lo_v * rot_cos[j] - hi_v * rot_sin[j];  // v heads keep cos 1, sin 0
          const float second = hi_v * rot_cos[j] + lo_v * rot_sin[j];
          if (h < a.q_heads) {
            const long long at = (long long)tok * a.out_stride + (long long)h * d + i;
            if (a.out_dtype == DT_F32) {
              static_cast<float*>(a.out)[at] = first;
              static_cast<float*>(a.out)[at + half] = second;
            } else {
              static_cast<__nv_bfloat16*>(a.out)[at] = __float2bfloat16_rn(first);
              static_cast<__nv_bfloat16*>(a.out)[at + half] = __float2bfloat16_rn(second);
            }
          } else if (cache_at[j] >= 0) {
            const bool is_v = h >= a.q_heads + a.cache.kv_heads;
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_v ? a.cache.v : a.cache.k) + cache_at[j] + i;
            dst[0] = __float2bfloat16_rn(first);
            dst[half] = __float2bfloat16_rn(second);
          }
        }
      }
      if (EPI == EPI_ADD && a.pre_x) {
        // the item's 16 rows are spread over the 8 lanes that share t: add them up, lane g = 0 writes
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          float part = sq_mine[j];
          part += __shfl_xor_sync(0xffffffffu, part, 4);
          part += __shfl_xor_sync(0xffffffffu, part, 8);
          part += __shfl_xor_sync(0xffffffffu, part, 16);
          const int tok = n * 8 + 2 * t + j;
          if (g == 0 && tok < a.tokens) a.pre_sq[(size_t)item * SQ_SLOTS + tok] = part;
        }
      }
    }
    buf ^= 1;
  }
}

template <int NT, int PRO, int EPI>
int launch(const GemvArgs& a, size_t smem, int grid, cudaStream_t stream) {
  auto kern = gemv_fused_kernel<NT, PRO, EPI>;
  static bool raised = false;   // one instantiation, one attribute (per process; one device per process)
  if (!raised) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET) != cudaSuccess)
      return launch_status();
    raised = true;
  }
  launch_kernel(kern, grid, THREADS, smem, stream, a);
  return launch_status();
}

template <int NT, int PRO>
int launch_epi(int epi, const GemvArgs& a, size_t smem, int grid, cudaStream_t stream) {
  switch (epi) {
    case EPI_STORE: return launch<NT, PRO, EPI_STORE>(a, smem, grid, stream);
    case EPI_ADD: return launch<NT, PRO, EPI_ADD>(a, smem, grid, stream);
    case EPI_SWIGLU: return launch<NT, PRO, EPI_SWIGLU>(a, smem, grid, stream);
    case EPI_ROPE: return launch<NT, PRO, EPI_ROPE>(a, smem, grid, stream);
  }
  return ERR_BAD_SIZE;
}

template <int NT>
int launch_pro(int pro, int epi, const GemvArgs& a, size_t smem, int grid, cudaStream_t stream) {
  if (pro == PRO_BF16) return launch_epi<NT, PRO_BF16>(epi, a, smem, grid, stream);
  if (pro == PRO_NORM) return launch_epi<NT, PRO_NORM>(epi, a, smem, grid, stream);
  if (pro == PRO_PRENORMED) return launch_epi<NT, PRO_PRENORMED>(epi, a, smem, grid, stream);
  return ERR_BAD_SIZE;
}

// How a launch lays out shared memory: the stage size kc (k values), the number of stages, the
// residual rows staged at a time, and the total.  Returns false if x and two stages do not fit.
struct SmemPlan {
  int x_ld, kc, stages, norm_rows, first_aliased;
  size_t bytes;
};

static bool plan_smem(int tokens, int k, int pro, size_t budget, int min_stages, SmemPlan& p) {
  if (tokens < 1 || tokens > 32 || k < 32 || k % 32) return false;
  const int nt = (tokens + 7) / 8;
  p.x_ld = k + ((k * 2) % 128 == 64 ? 0 : 32);
  constexpr int kc_wish = 2048;   // the longest row piece of a stage: 4 KB per bulk copy (the copy unit's cost is per copy)
  const size_t fixed = (size_t)8 * nt * p.x_ld * 2 + (size_t)2 * WARPS * nt * 4 * 32 * 4 + SQ_SLOTS * 4 +
                       (pro == PRO_NORM ? (size_t)k * 4 : 0) + (2 * MAX_STAGES + 2) * 8 + 16;
  // the stage size: the longest piece of a row (k / n values, a multiple of 32, at most kc_wish)
  // of which two stages fit; longer pieces mean fewer copies per byte
  for (int n = 1; n <= k / 32; ++n) {
    if (k % (32 * n) || k / n > kc_wish) continue;
    const int use = k / n;
    if (use < 128 && n > 1) break;
    const size_t stage = (size_t)16 * (use * 2 + ROW_PAD);
    if (fixed + min_stages * stage > budget) continue;
    size_t stages = (budget - fixed) / stage;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    p.kc = use, p.stages = (int)stages, p.bytes = fixed + stages * stage;
    p.norm_rows = 0, p.first_aliased = (int)stages;
    if (pro == PRO_NORM) {
      // the staging area takes the ring's last stages; all eight rows of a token group at once if
      // that leaves a stage for the weights meanwhile, else fewer rows at a time
      for (int rows = 8; rows >= 1; rows /= 2) {
        const size_t aliased = ((size_t)rows * k * 4 + stage - 1) / stage;
        if (aliased < stages || (rows == 1 && aliased <= stages)) {
          p.norm_rows = rows, p.first_aliased = (int)(stages - aliased);
          break;
        }
      }
      if (p.norm_rows == 0) continue;
    }
    return true;
  }
  return false;
}

}  // namespace


// Shared memory the kernel needs for `tokens` tokens and inner dimension k (0: not supported).
extern "C" long long llm_gemv_fused_smem(int tokens, int k) {
  SmemPlan p;
  return plan_smem(tokens, k, PRO_NORM, SMEM_BUDGET, 2, p) ? (long long)p.bytes : 0;
}

extern "C" int llm_gemv_fused(const void* w, int w_rows, int k, int tokens, int pro, int epi,
                              const void* x, long long x_stride, const void* norm_w, int norm_w_dtype, float eps,
                              const int32_t* row_index, void* out, int out_dtype, long long out_stride, int n_out,
                              int up_offset, void* k_base, void* v_base, const int32_t* block_table,
                              long long page_stride, int table_stride, int page_tokens, int kv_heads, int head_dim,
                              const int32_t* positions, const int32_t* row_seq, const float* inv_freq, int q_heads,
                              int write_cache, const float* sq_in, int sq_items, long long sq_stride, void* pre_x, long long pre_x_stride,
                              const void* pre_w, int pre_w_dtype, float* pre_sq, int max_blocks, int* error_word, cudaStream_t stream) {
  SmemPlan plan;
  if (!plan_smem(tokens, k, pro, SMEM_BUDGET, 2, plan)) return ERR_BAD_SIZE;
  if (out_dtype != DT_F32 && out_dtype != DT_BF16) return ERR_BAD_DTYPE;
  if (epi == EPI_ADD && out_dtype != DT_F32) return ERR_BAD_DTYPE;
  if (tokens > SQ_SLOTS || (pro == PRO_PRENORMED && (!sq_in || sq_items < 1 || sq_stride < 1)) || (pre_x && (epi != EPI_ADD || !pre_w || !pre_sq)))
    return ERR_BAD_SIZE;
  const auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!aligned16(w) || !aligned16(x) || (pro != PRO_NORM && x_stride % 8) || (pro == PRO_NORM && x_stride % 4) ||
      (pro == PRO_NORM && !aligned16(norm_w)))
    return ERR_BAD_ALIGN;
  GemvArgs a = {};
  a.w = static_cast<const __nv_bfloat16*>(w);
  a.w_rows = w_rows, a.k = k, a.tokens = tokens;
  a.x_ld = plan.x_ld, a.kc = plan.kc, a.stages = plan.stages, a.norm_rows = plan.norm_rows, a.first_aliased = plan.first_aliased, a.error_word = error_word;
  a.x = x, a.x_stride = x_stride, a.norm_w = norm_w, a.norm_w_dtype = norm_w_dtype, a.eps = eps, a.row_index = row_index;
  a.out = out, a.out_dtype = out_dtype, a.out_stride = out_stride, a.n_out = n_out, a.up_offset = up_offset;
  a.cache = PagedCache{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  a.positions = positions, a.row_seq = row_seq, a.inv_freq = inv_freq, a.q_heads = q_heads, a.write_cache = write_cache;
  a.sq_in = sq_in, a.sq_items = sq_items, a.sq_stride = sq_stride;
  a.pre_x = static_cast<__nv_bfloat16*>(pre_x), a.pre_x_stride = pre_x_stride, a.pre_w = pre_w, a.pre_w_dtype = pre_w_dtype;
  a.pre_sq = pre_sq;
  if (epi == EPI_SWIGLU) {
    if (n_out < 1 || up_offset < n_out || up_offset + n_out > w_rows) return ERR_BAD_SIZE;
    a.n_items = (n_out + 7) / 8;
  } else if (epi == EPI_ROPE) {
    if (head_dim < 16 || head_dim % 16 || (q_heads + 2 * kv_heads) * head_dim != w_rows) return ERR_BAD_SIZE;
    a.n_items = (q_heads + 2 * kv_heads) * (head_dim / 16);
  } else {
    if (n_out < 1 || n_out > w_rows) return ERR_BAD_SIZE;
    a.n_items = (n_out + 15) / 16;
  }
  const int nt = (tokens + 7) / 8;
  int grid = a.n_items < max_blocks ? a.n_items : max_blocks;
  if (grid < 1) return ERR_BAD_SIZE;
  // A product with a few more items than SMs (one and a bit per block) would keep most SMs waiting
  // for the blocks that run two.  If a block with one whole-row stage fits twice on an SM, every
  // item gets a block of its own instead and all of them stream at once.
  SmemPlan one;
  if (pro != PRO_NORM && a.n_items > max_blocks && a.n_items <= 2 * max_blocks &&
      plan_smem(tokens, k, pro, SMEM_HALF, 1, one) && one.kc == k) {
    plan = one;
    plan.stages = 1, plan.bytes = plan.bytes - (size_t)(one.stages - 1) * 16 * (one.kc * 2 + ROW_PAD);
    a.kc = plan.kc, a.stages = 1, a.first_aliased = 1;
    grid = a.n_items;
  }
  const size_t smem = plan.bytes;
  switch (nt) {
    case 1: return launch_pro<1>(pro, epi, a, smem, grid, stream);
    case 2: return launch_pro<2>(pro, epi, a, smem, grid, stream);
    case 3: return launch_pro<3>(pro, epi, a, smem, grid, stream);
    case 4: return launch_pro<4>(pro, epi, a, smem, grid, stream);
  }
  return ERR_BAD_SIZE;
}
