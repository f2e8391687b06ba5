// Paged attention for steps whose requests bring very few tokens (the decode step): at most 16
// packed rows (tokens x query heads of one key/value group) per request and key/value head,
// bfloat16, float32 softmax and sums.  Same arithmetic as attention_mma.cu (which follows
// cuongvng/bare-cuda-4gib engine/kernels/attention_qk.cu:49-68, softmax.cu:28-42,
// attention_av.cu:24-44); what differs is how the memory latency is taken: once.
//
// A decode step at batch 8 reads 17 MB of keys and values per layer, about 2.5 us of memory
// time, so the kernel's time is the length of its chain of dependent memory trips.  Here:
//   * A tile's key blocks (64 positions each, 32 at head size 128) are dealt round-robin to the warps of a thread
//     block cluster: `gridDim.z` blocks (up to 8) of four warps.  Every warp requests all of its
//     key and value blocks at once, as TMA copies over the cache pool's tensor map straight into
//     128-byte-swizzled shared memory (one trip for the whole tile), runs its own flash-attention
//     state over them, and no warp waits for another while it does.
//   * Whatever no kernel of the step writes is read before the kernel waits for its predecessor
//     in the stream: the step's metadata (written by the host before the step's first kernel) and
//     every key block that lies wholly below the step's first new position.
//   * A block merges its warps' states in its own shared memory and sends row r's merged state to
//     block r % gridDim.z of the cluster (stores into distributed shared memory).  After one
//     cluster barrier each block merges the rows it owns over the blocks in index order (so the
//     result does not depend on timing) and writes them.  No scratch in global memory, no
//     atomics, no second kernel, and nobody reads another block's memory after the barrier.
// Waits on mbarriers are bounded (about a second; then the error word is set and the block goes
// on to its barriers with whatever it has, so that it still returns).
//
// HEAD_DIM (-DHEAD_DIM=64 or 128) is a compile-time constant: the tensor map copies boxes of 64
// columns.

#include "common.cuh"

#include <cuda.h>
#include <string.h>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int D = HEAD_DIM;
static_assert(D == 64 || D == 128, "HEAD_DIM must be 64 or 128");
// A warp's request for one key block is 16 KB of keys and 16 KB of values whatever the head size: 64
// positions at head size 64, 32 at 128 (measured at head size 128, batch 8 to 64 and contexts of 2,048
// to 8,192: 0.79 to 0.93 of the copy bandwidth with 32 positions, 0.55 to 0.74 with 64, whose 146 KB of
// shared memory leave room for one block per SM only).
#ifndef DECODE_KEY_BLOCK
#define DECODE_KEY_BLOCK (HEAD_DIM == 128 ? 32 : 64)
#endif
constexpr int BN = DECODE_KEY_BLOCK;        // keys per block
static_assert(BN == 32 || BN == 64, "key blocks of 32 or 64 positions");
constexpr int BM = 16;                      // packed rows per tile
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int SUBS = D / 64;                // 64-column sub-tiles per key row
constexpr int SUB_BYTES = BN * 128;         // one sub-tile: [BN keys][128 bytes], swizzled
constexpr int KV_BYTES = 2 * SUBS * SUB_BYTES;   // keys then values of one block
constexpr int MAX_SLOTS = 3;                // key blocks a warp may have in flight
constexpr int QLD = D + 8;
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;
constexpr int ERR_DECODE_ATTENTION = 31;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

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
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up, int* error_word) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*gave_up) return false;
  const unsigned long long start = global_timer();
  for (unsigned spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 63u) {
      if (*gave_up) return false;
      if (global_timer() - start > WAIT_LIMIT_NS) {
        *gave_up = 1;
        if (error_word) atomicCAS(error_word, 0, ERR_DECODE_ATTENTION);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `local` (a shared-memory address of this block) in block `rank` of the cluster.
__device__ __forceinline__ uint32_t peer_smem(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` in a sub-tile written by TMA with
// the 128-byte swizzle (the tile starts on a 1024-byte boundary).
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }


struct DecodeArgs {
  const __nv_bfloat16* q;      // [tokens, q_heads, D]
  __nv_bfloat16* out;          // [tokens, q_heads * D]
  const int32_t* block_table;  // [batch sequences][table_stride]
  int table_stride, page_tokens, kv_heads, q_heads;
  long long page_rows, k_row0, v_row0, pool_rows;   // the pool seen as rows of D elements
  int box_rows;                // rows per TMA box: divides 64 and the page size
  int slots;                   // key blocks per warp in flight
  const int32_t* seq_q_start;
  const int32_t* seq_q_len;
  const int32_t* seq_kv_len;
  const int32_t* tile_seq;
  const int32_t* tile_index;
  float scale_log2;
  int window;
  int* error_word;
};

__global__ void __launch_bounds__(THREADS)
attention_decode_kernel(const __grid_constant__ CUtensorMap pool_map, const DecodeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv = smem;                                                       // [WARPS][slots][KV_BYTES]
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(kv + (size_t)WARPS * a.slots * KV_BYTES);   // [BM][QLD]
  float* recv = reinterpret_cast<float*>(Qs + BM * QLD);                   // [n_splits][rows owned][D + 4], written by the cluster
  const int owned_rows = (BM + (int)gridDim.z - 1) / (int)gridDim.z;
  uint64_t* full = reinterpret_cast<uint64_t*>(recv + (size_t)gridDim.z * owned_rows * (D + 4));   // [WARPS][MAX_SLOTS]
  volatile int* gave_up = reinterpret_cast<volatile int*>(full + WARPS * MAX_SLOTS);
  // the warps' final states, read by the whole cluster (over the key/value area, which is free by then)
  float* st_o = reinterpret_cast<float*>(kv);       // [WARPS][BM][D]
  float* st_m = st_o + WARPS * BM * D;              // [WARPS][BM]
  float* st_l = st_m + WARPS * BM;                  // [WARPS][BM]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_splits = gridDim.z, split = blockIdx.z;
  if (threadIdx.x == 0) {
    for (int i = 0; i < WARPS * MAX_SLOTS; ++i) mbar_init(&full[i], 1);
    *gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&pool_map)) : "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  // The step's metadata is written by the host before the step's first kernel and by no kernel:
  // it is read without waiting for the kernel before this one.
  const int tile = blockIdx.x, kvh = blockIdx.y;
  const int seq = a.tile_seq[tile];
  if (seq < 0) {         // the same for every block of the cluster
    pdl_wait();
    return;
  }
  // Every block of the cluster reports that it runs; the wait for this phase stands before the
  // first store into another block's shared memory, by when it has long completed.
  if (n_splits > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  const int group = a.q_heads / a.kv_heads;
  const int q_start = a.seq_q_start[seq], q_len = a.seq_q_len[seq], kv_len = a.seq_kv_len[seq];
  const int row0 = a.tile_index[tile] * BM;
  const int n_rows = q_len * group;
  const int pos0 = kv_len - q_len;
  const int last_token = min(q_len - 1, (row0 + BM - 1) / group), first_token = row0 / group;
  const int hi_key = pos0 + last_token;
  const int tile_min_pos = pos0 + first_token, tile_max_pos = pos0 + last_token;
  const int lo_key = a.window > 0 ? max(0, pos0 + first_token - a.window + 1) : 0;
  const int kb_lo = lo_key / BN, kb_hi = hi_key / BN;   // inclusive
  // this warp's key blocks: kb_lo + gw, kb_lo + gw + stride, ...
  const int stride = WARPS * n_splits, gw = split * WARPS + warp;
  const int my_blocks = kb_lo + gw > kb_hi ? 0 : (kb_hi - kb_lo - gw) / stride + 1;

  const int32_t* table_row = a.block_table + (long long)seq * a.table_stride;
  const int pieces = BN / a.box_rows;
  uint8_t* my_kv = kv + (size_t)warp * a.slots * KV_BYTES;
  uint64_t* my_full = full + warp * MAX_SLOTS;

  // requests block j of this warp into slot j % slots: lane p looks piece p up, lanes 0 and 1 issue
  auto request = [&](int j) {
    const int slot = j % a.slots;
    const uint32_t k_base = smem_u32(my_kv) + slot * KV_BYTES, v_base = k_base + SUBS * SUB_BYTES;
    const int key0 = (kb_lo + gw + j * stride) * BN;
    long long my_row = -1;
    if (lane < pieces) {
      const int key = key0 + lane * a.box_rows;
      if (key < kv_len) {
        const int page = __ldg(table_row + key / a.page_tokens);
        if (page >= 0) my_row = (long long)page * a.page_rows + (long long)kvh * a.page_tokens + key % a.page_tokens;
      }
    }
    const uint32_t all = pieces < 32 ? (1u << pieces) - 1u : 0xffffffffu;
    const uint32_t held = __ballot_sync(0xffffffffu, my_row >= 0) & all;
    const uint32_t missing = ~held & all;
    if (missing) {   // pieces past the request's end or without a page: zeros, visible to nobody but this warp
      for (int piece = 0; piece < pieces; ++piece) {
        if (!((missing >> piece) & 1u)) continue;
        for (int sub = 0; sub < SUBS; ++sub)
          for (int i = lane; i < a.box_rows * 8; i += 32) {
            const uint32_t off = sub * SUB_BYTES + piece * a.box_rows * 128 + i * 16;
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(k_base + off), "r"(0) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_base + off), "r"(0) : "memory");
          }
      }
      __syncwarp();
    }
    if (lane == 0) mbar_expect_tx(&my_full[slot], (uint32_t)__popc(held) * 2u * SUBS * a.box_rows * 128u);
    __syncwarp();
    for (int piece = 0; piece < pieces; ++piece) {
      const long long row = __shfl_sync(0xffffffffu, my_row, piece);
      if (lane > 1 || row < 0) continue;
      const uint32_t base = lane == 0 ? k_base : v_base;
      const long long cache_row0 = lane == 0 ? a.k_row0 : a.v_row0;
      for (int sub = 0; sub < SUBS; ++sub)
        tma_load_2d(base + sub * SUB_BYTES + piece * a.box_rows * 128, &pool_map, &my_full[slot], sub * 64, (int)(row + cache_row0));
    }
  };
  // key blocks wholly below the step's first new position hold what earlier steps wrote: they
  // are requested at once; the others after the kernel before this one has finished
  const int first_wave = min(my_blocks, a.slots);
  uint32_t deferred = 0;
  for (int j = 0; j < first_wave; ++j) {
    if ((kb_lo + gw + j * stride) * BN + BN <= pos0) request(j);
    else deferred |= 1u << j;
  }
  pdl_wait();
  for (int j = 0; j < first_wave; ++j)
    if ((deferred >> j) & 1u) request(j);

  // ---- Q (rows beyond the request's packed rows are zero), then its fragments into registers
  constexpr int CHUNKS = D / 8;
  for (int i = threadIdx.x; i < BM * CHUNKS; i += THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS, R = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < n_rows) {
      const int token = R / group, head = kvh * group + R % group;
      v = *reinterpret_cast<const uint4*>(a.q + ((long long)(q_start + token) * a.q_heads + head) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(Qs + r * QLD + c * 8) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks)
    ldmatrix_x4(qf[ks], smem_u32(Qs + (lane & 15) * QLD + ks * 16 + (lane >> 4) * 8));

  int row_pos[2];
  float m[2], l[2], o[D / 8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = row0 + (lane >> 2) + h * 8;
    row_pos[h] = R < n_rows ? pos0 + R / group : -1;
    m[h] = -INFINITY;
    l[h] = 0.0f;
  }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  constexpr int NT = BN / 8;
  for (int j = 0; j < my_blocks; ++j) {
    const int slot = j % a.slots;
    mbar_wait(&my_full[slot], (uint32_t)(j / a.slots) & 1u, gave_up, a.error_word);
    const uint32_t k_base = smem_u32(my_kv) + slot * KV_BYTES, v_base = k_base + SUBS * SUB_BYTES;
    const int kb = kb_lo + gw + j * stride;
    const int key0 = kb * BN;

    float s[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    const int mid = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int col = ks * 16 + (mid & 1) * 8;           // first of the 8 feature columns this lane addresses
#pragma unroll
      for (int nt = 0; nt < NT; nt += 2) {
        uint32_t kf[4];
        const int key = (nt + (mid >> 1)) * 8 + (lane & 7);
        ldmatrix_x4(kf, k_base + (col / 64) * SUB_BYTES + swizzled(key, (col % 64) / 8));
        mma_bf16(s[nt], qf[ks], kf[0], kf[1]);
        mma_bf16(s[nt + 1], qf[ks], kf[2], kf[3]);
      }
    }

    const bool all_visible = key0 + BN - 1 <= tile_min_pos && (a.window <= 0 || key0 > tile_max_pos - a.window);
    float mx[2] = {-INFINITY, -INFINITY};
    if (all_visible) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float v = s[nt][e] * a.scale_log2;
          s[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const bool visible = key <= row_pos[h] && (a.window <= 0 || key > row_pos[h] - a.window);
          const float v = visible ? s[nt][e] * a.scale_log2 : -INFINITY;
          s[nt][e] = v;
          mx[h] = fmaxf(mx[h], v);
        }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
      corr[h] = fast_exp2(m[h] - m_use[h]);
      m[h] = m_new;
      l[h] *= corr[h];
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
    }
    uint32_t pf[NT / 2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float p0 = fast_exp2(s[nt][0] - m_use[0]), p1 = fast_exp2(s[nt][1] - m_use[0]);
      const float p2 = fast_exp2(s[nt][2] - m_use[1]), p3 = fast_exp2(s[nt][3] - m_use[1]);
      l[0] += p0 + p1;
      l[1] += p2 + p3;
      pf[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      const int key = kk * 16 + (mid & 1) * 8 + (lane & 7);
#pragma unroll
      for (int dt = 0; dt < D / 8; dt += 2) {
        uint32_t vf[4];
        const int col = (dt + (mid >> 1)) * 8;
        ldmatrix_x4_trans(vf, v_base + (col / 64) * SUB_BYTES + swizzled(key, (col % 64) / 8));
        mma_bf16(o[dt], pf[kk], vf[0], vf[1]);
        mma_bf16(o[dt + 1], pf[kk], vf[2], vf[3]);
      }
    }
    // the slot is free again: this warp's next block that uses it may be requested
    if (j + a.slots < my_blocks) {
      __syncwarp();
      request(j + a.slots);
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }

  // ---- the warps' states into shared memory (every warp of the block is done with its slots)
  __syncthreads();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + h * 8;
    if ((lane & 3) == 0) {
      st_m[warp * BM + r] = m[h];
      st_l[warp * BM + r] = l[h];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      float* dst = st_o + ((size_t)(warp * BM + r)) * D + i * 8 + (lane & 3) * 2;
      dst[0] = o[i][h * 2 + 0];
      dst[1] = o[i][h * 2 + 1];
    }
  }
  __syncthreads();
  if (n_splits > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");   // all blocks of the cluster have started
  // ---- this block's warps merged, per row and eight columns a thread; row r goes to block r % n_splits
  constexpr int STATE = D + 4;   // floats per row state: D sums (relative to m), then m and l (16-byte rows)
  for (int i = threadIdx.x; i < BM * (D / 8); i += THREADS) {
    const int r = i / (D / 8), c8 = i % (D / 8);
    if (row0 + r >= n_rows) continue;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, st_m[w * BM + r]);
    float L = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float f = exp2f(st_m[w * BM + r] - M);
        L += st_l[w * BM + r] * f;
        const float* src = st_o + ((size_t)(w * BM + r)) * D + c8 * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += src[e] * f;
      }
    }
    const int owner = r % n_splits;
    const uint32_t local = smem_u32(recv + ((size_t)split * owned_rows + r / n_splits) * STATE);
    const uint32_t dst = n_splits > 1 ? peer_smem(local, owner) : local;
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + c8 * 32), "f"(acc[0]), "f"(acc[1]), "f"(acc[2]), "f"(acc[3]) : "memory");
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + c8 * 32 + 16), "f"(acc[4]), "f"(acc[5]), "f"(acc[6]), "f"(acc[7]) : "memory");
    if (c8 == 0) asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(dst + D * 4), "f"(M), "f"(L) : "memory");
  }
  if (n_splits > 1) cluster_sync();
  else __syncthreads();

  // ---- the rows this block owns, merged over the blocks in index order
  for (int i = threadIdx.x; i < owned_rows * (D / 4); i += THREADS) {
    const int slot = i / (D / 4), c4 = i % (D / 4);
    const int r = slot * n_splits + split, R = row0 + r;
    if (r >= BM || R >= n_rows) continue;
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, recv[((size_t)z * owned_rows + slot) * STATE + D]);
    float L = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (M != -INFINITY) {
      for (int z = 0; z < n_splits; ++z) {
        const float* st = recv + ((size_t)z * owned_rows + slot) * STATE;
        const float f = exp2f(st[D] - M);
        L += st[D + 1] * f;
        const float4 v = *reinterpret_cast<const float4*>(st + c4 * 4);
        acc.x += v.x * f;
        acc.y += v.y * f;
        acc.z += v.z * f;
        acc.w += v.w * f;
      }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    const int token = R / group, head = kvh * group + R % group;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(a.out + ((long long)(q_start + token) * a.q_heads + head) * D + c4 * 4) = packed;
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

size_t smem_bytes(int slots) {
  const size_t kv = (size_t)WARPS * slots * KV_BYTES;
  const size_t states = (size_t)WARPS * BM * (D + 2) * 4;
  return 1024 + (kv > states ? kv : states) + (size_t)BM * QLD * 2 + (size_t)(BM + 8) * (D + 4) * 4 +
         WARPS * MAX_SLOTS * 8 + 16;
}

}  // namespace

extern "C" int llm_attention_decode_head_dim() { return D; }
extern "C" int llm_attention_decode_key_block() { return BN; }


// Writes the 128-byte tensor map of a cache group's pool: `rows` rows of D bfloat16 starting at
// `base` (16-byte aligned), boxes of 64 columns x `box_rows` rows, 128-byte swizzle.
extern "C" int llm_attention_decode_pool_map(void* map_out, const void* base, long long rows, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return 1000 + (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || rows <= 0 || box_rows <= 0 || box_rows > 64) return ERR_BAD_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

// Tiles of 16 packed rows (the tile list of llm_attention_mma's decode shape).  `n_splits` blocks
// (1..8) share a tile's key blocks as one cluster; `slots` (1..3) key blocks per warp are in
// flight.  `pool_map`: llm_attention_decode_pool_map over `pool_base`, in which k_base and v_base
// lie, with boxes of `box_rows` rows (a multiple of 8 that divides 64 and the page size).
extern "C" int llm_attention_decode(const void* pool_map, const void* pool_base, long long pool_rows, int box_rows,
                                    const void* q, void* out, void* k_base, void* v_base, const int32_t* block_table,
                                    long long page_stride, int table_stride, int page_tokens, int kv_heads,
                                    int head_dim, const int32_t* seq_q_start, const int32_t* seq_q_len,
                                    const int32_t* seq_kv_len, const int32_t* tile_seq, const int32_t* tile_index,
                                    int n_tiles, int n_splits, int slots, int q_heads, float scale, int window,
                                    int* error_word, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (head_dim != D || q_heads % kv_heads || kv_heads > 65535 || n_splits < 1 || n_splits > 8 || slots < 1 ||
      slots > MAX_SLOTS)
    return ERR_BAD_SIZE;
  if (box_rows < 8 || box_rows % 8 || BN % box_rows || page_tokens % box_rows) return ERR_BAD_SIZE;
  const long long k_off = reinterpret_cast<const char*>(k_base) - reinterpret_cast<const char*>(pool_base);
  const long long v_off = reinterpret_cast<const char*>(v_base) - reinterpret_cast<const char*>(pool_base);
  if (k_off < 0 || v_off < 0 || k_off % (D * 2) || v_off % (D * 2) || page_stride % D) return ERR_BAD_ALIGN;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) return ERR_BAD_ALIGN;
  const size_t smem = smem_bytes(slots);
  if (smem > 227 * 1024) return ERR_BAD_SIZE;
  static size_t raised = 0;
  if (smem > raised) {
    if (cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return launch_status();
    raised = smem;
  }
  CUtensorMap map;   // the caller's buffer need not be 64-byte aligned
  memcpy(&map, pool_map, sizeof(CUtensorMap));
  DecodeArgs a;
  a.q = reinterpret_cast<const __nv_bfloat16*>(q);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.block_table = block_table;
  a.table_stride = table_stride, a.page_tokens = page_tokens, a.kv_heads = kv_heads, a.q_heads = q_heads;
  a.page_rows = page_stride / D, a.k_row0 = k_off / (D * 2), a.v_row0 = v_off / (D * 2), a.pool_rows = pool_rows;
  a.box_rows = box_rows, a.slots = slots;
  a.seq_q_start = seq_q_start, a.seq_q_len = seq_q_len, a.seq_kv_len = seq_kv_len;
  a.tile_seq = tile_seq, a.tile_index = tile_index;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.error_word = error_word;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, kv_heads, n_splits);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (n_splits > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 1;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = n_splits;
    ++n_attr;
  }
  if (pdl_enabled()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  cudaLaunchKernelEx(&cfg, attention_decode_kernel, map, a);
  return launch_status();
}
