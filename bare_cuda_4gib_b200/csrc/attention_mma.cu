// Paged flash attention for bfloat16 on the tensor cores (mma.sync m16n8k16, float32 softmax and
// accumulators), one kernel for prefill portions, decode rows and mixed batches.  It replaces
// the three-kernel attention of cuongvng/bare-cuda-4gib (engine/kernels/attention_qk.cu:49-68,
// softmax.cu:28-42, attention_av.cu:24-44), which materialises [heads, T, keys] scores.
//
// Rows.  The query heads that share one key/value head are packed into the rows of a tile:
// packed row R of a request = (token R / group, head R % group).  A thread block owns one tile
// of BM packed rows of one request and one key/value head, so a key block loaded once serves
// every head of the group.  Keys are visited in blocks of 64 positions, copied from the
// request's pages into padded shared memory with cp.async (two stages for the prefill shape, four
// for the decode shape, whose few rows leave the loads' latency exposed).
//
// Two shapes of the same kernel:
//   WARPS_M = 4, WARPS_N = 1: each warp 16 * MT rows and all 64 keys of a block (prefill); MT = 2
//   (128 rows per block) for head sizes up to 64, where the registers allow it: a key fragment
//   read from shared memory then feeds two row tiles, which halves the shared-memory traffic;
//   WARPS_M = 1, WARPS_N = 4: 16 rows, each warp 16 of the 64 keys of a block (decode); the
//   warps' partial softmax states are merged through shared memory.
// gridDim.z > 1 splits a tile's key blocks over several thread blocks; each writes a
// normalised partial output and its log-sum-exp to scratch memory and counts itself done; the
// block that counts last merges the tile's partial results in split order (so the sum does not
// depend on which block that is) and sets the counter back to zero.  No block waits for another.
// Softmax runs in base 2: scores are multiplied by scale * log2(e).
//
// HEAD_DIM is a compile-time constant (-DHEAD_DIM=64): a multiple of 16 up to 128.

#include "common.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int D = HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 128, "HEAD_DIM must be a multiple of 16 up to 128");
constexpr int BN = 64;        // keys per block
constexpr int LDS = D + 8;    // padded row length in shared memory (conflict-free ldmatrix)
constexpr int CHUNKS = D / 8; // 16-byte chunks per row

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x for softmax weights: the hardware approximation (relative error about 2^-22, far below the
// bfloat16 rounding of the probabilities that follows); -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct AttnArgs {
  const __nv_bfloat16* q;      // [tokens, q_heads, D]
  __nv_bfloat16* out;          // [tokens, q_heads * D]
  PagedCache cache;
  const int32_t* seq_q_start;  // per batch sequence: first row of its tokens in this step
  const int32_t* seq_q_len;    // tokens it brings
  const int32_t* seq_kv_len;   // its length after this step
  const int32_t* tile_seq;     // per tile: batch sequence (-1: nothing to do)
  const int32_t* tile_index;   // per tile: which BM-row tile of the sequence's packed rows
  float* part_o;               // scratch for split keys: [tile][kv head][split][BM][D], normalised
  float* part_lse;             // [tile][kv head][split][BM], base-2 log-sum-exp (-inf: no keys)
  int* counters;               // [tile][kv head]: splits done; zero before and after every launch
  int q_heads;
  float scale_log2;
  int window;                  // <= 0: every key
};

template <int WARPS_M, int WARPS_N, int MT>
__global__ void __launch_bounds__(WARPS_M* WARPS_N * 32)
attention_mma_kernel(AttnArgs a) {
  constexpr int NW = WARPS_M * WARPS_N;
  constexpr int NT_THREADS = NW * 32;
  constexpr int WR = 16 * MT;            // rows per warp
  constexpr int BM = WR * WARPS_M;
  constexpr int KEYS_W = BN / WARPS_N;  // keys of a block that one warp handles
  constexpr int NT = KEYS_W / 8;        // score n-tiles per warp
  static_assert(NT % 2 == 0, "a warp handles keys in pairs of n-tiles");
  constexpr int STAGES = WARPS_N > 1 ? 4 : 2;  // key/value blocks in flight

  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [BM][LDS]
  __nv_bfloat16* Ks = Qs + BM * LDS;                                   // [STAGES][BN][LDS]
  __nv_bfloat16* Vs = Ks + STAGES * BN * LDS;                          // [STAGES][BN][LDS]

  pdl_launch_dependents();
  pdl_wait();
  // later tiles of a request see more keys: start them first
  const int tile = gridDim.x - 1 - blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, n_splits = gridDim.z;
  const int seq = a.tile_seq[tile];
  if (seq < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp / WARPS_N, wn = warp % WARPS_N;
  const int group = a.q_heads / a.cache.kv_heads;
  const int q_start = a.seq_q_start[seq], q_len = a.seq_q_len[seq], kv_len = a.seq_kv_len[seq];
  const int row0 = a.tile_index[tile] * BM;  // first packed row of the tile
  const int n_rows = q_len * group;
  const int pos0 = kv_len - q_len;           // position of the request's first token in this step

  // ---- key blocks this thread block visits
  const int last_token = min(q_len - 1, (row0 + BM - 1) / group);
  const int first_token = row0 / group;
  const int hi_key = pos0 + last_token;  // newest visible key of any row
  // positions of the tile's valid rows: [tile_min_pos, tile_max_pos].  Rows past the request's
  // last packed row are never stored, so it does not matter what they "see" in unmasked blocks
  // (their queries are zero, their scores finite).
  const int tile_min_pos = pos0 + first_token;
  const int tile_max_pos = pos0 + last_token;
  int lo_key = 0;
  if (a.window > 0) lo_key = max(0, pos0 + first_token - a.window + 1);
  const int kb_lo = lo_key / BN, kb_hi = hi_key / BN;  // inclusive
  const int n_kb_total = kb_hi - kb_lo + 1;
  const int per_split = (n_kb_total + n_splits - 1) / n_splits;
  const int kb_begin = kb_lo + split * per_split;
  const int kb_end = min(kb_hi + 1, kb_begin + per_split);  // exclusive

  // ---- stage Q (rows beyond the request's packed rows are zero)
  for (int i = threadIdx.x; i < BM * CHUNKS; i += NT_THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const int R = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < n_rows) {
      const int token = R / group, head = kvh * group + R % group;
      v = *reinterpret_cast<const uint4*>(a.q + ((long long)(q_start + token) * a.q_heads + head) * D + c * 8);
    }
    *reinterpret_cast<uint4*>(Qs + r * LDS + c * 8) = v;
  }

  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.cache.k);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.cache.v);
  // Page lookups.  When a page holds a multiple of 64 positions, a key block lies inside one page:
  // one table entry per block, and each thread's offsets inside the block never change.  Smaller
  // pages are looked up per row.
  const int page_tokens = a.cache.page_tokens;
  const bool block_in_page = (page_tokens % BN) == 0;
  const int32_t* table_row = a.cache.block_table + (long long)seq * a.cache.table_stride;
  const long long head_offset = (long long)kvh * page_tokens * D;
  constexpr int LOADS = (BN * CHUNKS + NT_THREADS - 1) / NT_THREADS;   // 16-byte chunks per thread and block
  // copies block kb into its stage (nothing if kb is past the end) and closes one cp.async group
  auto load_block = [&](int kb, int stage) {
    if (kb < kb_end) {
      __nv_bfloat16* ks = Ks + stage * BN * LDS;
      __nv_bfloat16* vs = Vs + stage * BN * LDS;
      const int key0 = kb * BN;
      long long block_base = -1;
      if (block_in_page) {
        const int page = __ldg(table_row + key0 / page_tokens);
        if (page >= 0) block_base = (long long)page * a.cache.page_stride + head_offset + (long long)(key0 % page_tokens) * D;
      }
#pragma unroll
      for (int j = 0; j < LOADS; ++j) {
        const int i = threadIdx.x + j * NT_THREADS;
        if (BN * CHUNKS % NT_THREADS != 0 && i >= BN * CHUNKS) break;
        const int r = i / CHUNKS, c = i % CHUNKS;
        long long src = 0;
        bool valid = key0 + r < kv_len;
        if (block_in_page) {
          valid = valid && block_base >= 0;
          if (valid) src = block_base + r * D + c * 8;
        } else if (valid) {
          const int key = key0 + r;
          const int page = __ldg(table_row + key / page_tokens);
          valid = page >= 0;
          if (valid) src = (long long)page * a.cache.page_stride + head_offset + (long long)(key % page_tokens) * D + c * 8;
        }
        cp_async16(ks + r * LDS + c * 8, kc + src, valid);
        cp_async16(vs + r * LDS + c * 8, vc + src, valid);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) load_block(kb_begin + st, st);
  __syncthreads();  // Q staged

  // ---- Q fragments stay in registers
  uint32_t qf[MT][D / 16][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
      ldmatrix_x4(qf[mt][ks], Qs + (wm * WR + mt * 16 + (lane & 15)) * LDS + ks * 16 + (lane >> 4) * 8);

  // this thread's rows: two per row tile
  int row_pos[MT][2];
  float m[MT][2], l[MT][2];
  float o[MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int R = row0 + wm * WR + mt * 16 + (lane >> 2) + h * 8;
      row_pos[mt][h] = R < n_rows ? pos0 + R / group : -1;  // -1: no key is visible
      m[mt][h] = -INFINITY;
      l[mt][h] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.0f;
  }

  for (int kb = kb_begin; kb < kb_end; ++kb) {
    const int stage = (kb - kb_begin) % STAGES;
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();  // block kb has landed; everyone is done with the stage used one block ago
    load_block(kb + STAGES - 1, (kb - kb_begin + STAGES - 1) % STAGES);
    const __nv_bfloat16* ks_ = Ks + stage * BN * LDS;
    const __nv_bfloat16* vs_ = Vs + stage * BN * LDS;
    const int key0 = kb * BN + wn * KEYS_W;  // first key this warp scores

    float s[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < NT; ++i) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int nt = 0; nt < NT; nt += 2) {
        uint32_t kf[4];
        const int mid = lane >> 3;
        ldmatrix_x4(kf, ks_ + (wn * KEYS_W + (nt + (mid >> 1)) * 8 + (lane & 7)) * LDS + ks * 16 + (mid & 1) * 8);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(s[mt][nt], qf[mt][ks], kf[0], kf[1]);
          mma_bf16(s[mt][nt + 1], qf[mt][ks], kf[2], kf[3]);
        }
      }
    }

    // a block wholly below every row's position and inside every row's window needs no mask
    const bool all_visible = kb * BN + BN - 1 <= tile_min_pos && (a.window <= 0 || kb * BN > tile_max_pos - a.window);
    uint32_t pf[MT][NT / 2][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      // scale, mask, running maximum
      float mx[2] = {-INFINITY, -INFINITY};
      if (all_visible) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float v = s[mt][nt][e] * a.scale_log2;
            s[mt][nt][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
          }
        }
      } else {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            const bool visible = key <= row_pos[mt][h] && (a.window <= 0 || key > row_pos[mt][h] - a.window);
            const float v = visible ? s[mt][nt][e] * a.scale_log2 : -INFINITY;
            s[mt][nt][e] = v;
            mx[h] = fmaxf(mx[h], v);
          }
        }
      }
      float corr[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[mt][h], mx[h]);
        m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
        corr[h] = fast_exp2(m[mt][h] - m_use[h]);  // m = -inf gives 0; an unchanged maximum gives exactly 1
        m[mt][h] = m_new;
        l[mt][h] *= corr[h];
      }
      // most blocks leave every row's maximum where it was: nothing to rescale then
      if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          o[mt][i][0] *= corr[0];
          o[mt][i][1] *= corr[0];
          o[mt][i][2] *= corr[1];
          o[mt][i][3] *= corr[1];
        }
      }
      // probabilities, as A fragments for P V
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float p0 = fast_exp2(s[mt][nt][0] - m_use[0]), p1 = fast_exp2(s[mt][nt][1] - m_use[0]);
        const float p2 = fast_exp2(s[mt][nt][2] - m_use[1]), p3 = fast_exp2(s[mt][nt][3] - m_use[1]);
        l[mt][0] += p0 + p1;
        l[mt][1] += p2 + p3;
        pf[mt][nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
        pf[mt][nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
    }
#pragma unroll
    for (int kk = 0; kk < KEYS_W / 16; ++kk) {
#pragma unroll
      for (int dt = 0; dt < D / 8; dt += 2) {
        uint32_t vf[4];
        const int mid = lane >> 3;
        ldmatrix_x4_trans(vf, vs_ + (wn * KEYS_W + kk * 16 + (mid & 1) * 8 + (lane & 7)) * LDS + (dt + (mid >> 1)) * 8);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_bf16(o[mt][dt], pf[mt][kk], vf[0], vf[1]);
          mma_bf16(o[mt][dt + 1], pf[mt][kk], vf[2], vf[3]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[mt][h] += __shfl_xor_sync(0xffffffffu, l[mt][h], 1);
      l[mt][h] += __shfl_xor_sync(0xffffffffu, l[mt][h], 2);
    }

  // ---- merge the warps that shared rows, through shared memory (reuses the K/V stages)
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(Ks);      // [WARPS_N][BM][D]
  float* red_m = red_o + WARPS_N * BM * D;          // [WARPS_N][BM]
  float* red_l = red_m + WARPS_N * BM;              // [WARPS_N][BM]
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = wm * WR + mt * 16 + (lane >> 2) + h * 8;
      if ((lane & 3) == 0) {
        red_m[wn * BM + r] = m[mt][h];
        red_l[wn * BM + r] = l[mt][h];
      }
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        float* dst = red_o + ((long long)(wn * BM + r)) * D + i * 8 + (lane & 3) * 2;
        dst[0] = o[mt][i][h * 2 + 0];
        dst[1] = o[mt][i][h * 2 + 1];
      }
    }
  __syncthreads();
  const long long item = ((long long)tile * gridDim.y + kvh) * n_splits + split;
  for (int i = threadIdx.x; i < BM * CHUNKS; i += NT_THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const int R = row0 + r;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS_N; ++w) M = fmaxf(M, red_m[w * BM + r]);
    float L = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS_N; ++w) {
        const float f = exp2f(red_m[w * BM + r] - M);
        L += red_l[w * BM + r] * f;
        const float* src = red_o + ((long long)(w * BM + r)) * D + c * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += src[e] * f;
      }
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    if (n_splits == 1) {
      if (R < n_rows) {
        const int token = R / group, head = kvh * group + R % group;
        uint4 packed;
        packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
        packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
        packed.z = pack_bf16(acc[4] * inv, acc[5] * inv);
        packed.w = pack_bf16(acc[6] * inv, acc[7] * inv);
        *reinterpret_cast<uint4*>(a.out + ((long long)(q_start + token) * a.q_heads + head) * D + c * 8) = packed;
      }
    } else {
      float* dst = a.part_o + (item * BM + r) * D + c * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = acc[e] * inv;
      if (c == 0) a.part_lse[item * BM + r] = L > 0.0f ? M + log2f(L) : -INFINITY;
    }
  }
  if (n_splits == 1) return;

  // ---- the last block of this tile to get here merges the splits
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  int* counter = a.counters + (long long)tile * gridDim.y + kvh;
  if (threadIdx.x == 0) is_last = atomicAdd(counter, 1) == n_splits - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const long long item0 = ((long long)tile * gridDim.y + kvh) * n_splits;
  // all log-sum-exps first, in one parallel pass, into shared memory (the K/V stages are free)
  float* lse = reinterpret_cast<float*>(Ks);   // [n_splits][BM]
  constexpr int LSE_CAPACITY = STAGES * BN * LDS * 2 * 2 / 4;
  const bool lse_fits = n_splits * BM <= LSE_CAPACITY;
  if (lse_fits) {
    __syncthreads();  // everyone is done with red_o / red_m
    for (int i = threadIdx.x; i < n_splits * BM; i += NT_THREADS) lse[i] = __ldcg(a.part_lse + item0 * BM + i);
    __syncthreads();
  }
  for (int i = threadIdx.x; i < BM * CHUNKS; i += NT_THREADS) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const int R = row0 + r;
    if (R >= n_rows) continue;
    auto lse_at = [&](int z) { return lse_fits ? lse[z * BM + r] : __ldcg(a.part_lse + (item0 + z) * BM + r); };
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, lse_at(z));
    float W = 0.0f, acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (M != -INFINITY) {
#pragma unroll 4
      for (int z = 0; z < n_splits; ++z) {   // independent loads: several are in flight at once
        const float w = exp2f(lse_at(z) - M);
        const float4* src = reinterpret_cast<const float4*>(a.part_o + ((item0 + z) * BM + r) * D + c * 8);
        const float4 lo = __ldcg(src), hi = __ldcg(src + 1);
        W += w;
        acc[0] += w * lo.x; acc[1] += w * lo.y; acc[2] += w * lo.z; acc[3] += w * lo.w;
        acc[4] += w * hi.x; acc[5] += w * hi.y; acc[6] += w * hi.z; acc[7] += w * hi.w;
      }
    }
    const float inv = W > 0.0f ? 1.0f / W : 0.0f;
    const int token = R / group, head = kvh * group + R % group;
    uint4 packed;
    packed.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    packed.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    packed.z = pack_bf16(acc[4] * inv, acc[5] * inv);
    packed.w = pack_bf16(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(a.out + ((long long)(q_start + token) * a.q_heads + head) * D + c * 8) = packed;
  }
  if (threadIdx.x == 0) *counter = 0;
}

template <int WARPS_M, int WARPS_N, int MT>
constexpr size_t smem_bytes() {
  constexpr int BM = 16 * MT * WARPS_M;
  constexpr int STAGES = WARPS_N > 1 ? 4 : 2;
  constexpr size_t tiles = (size_t)(BM + 2 * STAGES * BN) * LDS * 2;
  constexpr size_t merge = (size_t)BM * LDS * 2 + (size_t)WARPS_N * BM * (D + 2) * 4;
  return tiles > merge ? tiles : merge;
}

template <int WARPS_M, int WARPS_N, int MT>
int launch(const AttnArgs& a, int n_tiles, int kv_heads, int n_splits, cudaStream_t stream) {
  auto kern = attention_mma_kernel<WARPS_M, WARPS_N, MT>;
  constexpr size_t smem = smem_bytes<WARPS_M, WARPS_N, MT>();
  static bool configured = false;
  if (!configured) {
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return launch_status();
    configured = true;
  }
  dim3 grid(n_tiles, kv_heads, n_splits);
  launch_kernel(kern, grid, WARPS_M * WARPS_N * 32, smem, stream, a);
  return launch_status();
}

}  // namespace

constexpr int PREFILL_MT = D <= 64 ? 2 : 1;   // row tiles per warp in the prefill shape

extern "C" int llm_attention_head_dim() { return D; }

// Rows of a tile in the prefill shape (the decode shape has 16).
extern "C" int llm_attention_prefill_rows() { return 64 * PREFILL_MT; }

// 32-bit words of scratch that `n_tiles` tiles of `rows_per_tile` rows need when split `n_splits`
// ways: LLM_ATTENTION_COUNTER_WORDS counters (one per tile and kv head; they must be zero before
// the first launch and every launch leaves them zero), then partial outputs, then their
// log-sum-exps.
#define LLM_ATTENTION_COUNTER_WORDS 4096
extern "C" long long llm_attention_scratch_floats(int n_tiles, int kv_heads, int n_splits, int rows_per_tile) {
  return LLM_ATTENTION_COUNTER_WORDS + (long long)n_tiles * kv_heads * n_splits * rows_per_tile * (D + 1);
}

// rows_per_tile: llm_attention_prefill_rows() (prefill shape) or 16 (decode shape).  `scratch` (llm_attention_scratch_floats
// words, its first LLM_ATTENTION_COUNTER_WORDS zero) is needed when n_splits > 1.
extern "C" int llm_attention_mma(const void* q, void* out, void* k_base, void* v_base, const int32_t* block_table,
                                 long long page_stride, int table_stride, int page_tokens, int kv_heads,
                                 int head_dim, const int32_t* seq_q_start, const int32_t* seq_q_len,
                                 const int32_t* seq_kv_len, const int32_t* tile_seq, const int32_t* tile_index,
                                 int n_tiles, int rows_per_tile, int n_splits, float* scratch, int q_heads,
                                 float scale, int window, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (head_dim != D || q_heads % kv_heads || n_splits < 1 || n_splits > 65535 || kv_heads > 65535) return ERR_BAD_SIZE;
  if (n_splits > 1 && !scratch) return ERR_BAD_SIZE;
  if (n_splits > 1 && (long long)n_tiles * kv_heads > LLM_ATTENTION_COUNTER_WORDS) return ERR_BAD_SIZE;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k_base) |
       reinterpret_cast<uintptr_t>(v_base)) & 15)
    return ERR_BAD_ALIGN;
  AttnArgs a;
  a.q = reinterpret_cast<const __nv_bfloat16*>(q);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.cache = PagedCache{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  a.seq_q_start = seq_q_start;
  a.seq_q_len = seq_q_len;
  a.seq_kv_len = seq_kv_len;
  a.tile_seq = tile_seq;
  a.tile_index = tile_index;
  a.counters = reinterpret_cast<int*>(scratch);
  a.part_o = scratch ? scratch + LLM_ATTENTION_COUNTER_WORDS : nullptr;
  a.part_lse = scratch ? a.part_o + (long long)n_tiles * kv_heads * n_splits * rows_per_tile * D : nullptr;
  a.q_heads = q_heads;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  if (rows_per_tile == 64 * PREFILL_MT) return launch<4, 1, PREFILL_MT>(a, n_tiles, kv_heads, n_splits, stream);
  if (rows_per_tile == 16) return launch<1, 4, 1>(a, n_tiles, kv_heads, n_splits, stream);
  return ERR_BAD_SIZE;
}

// ---------------------------------------------------------------------------------------------
// Entry point that allocates nothing (declared in attention_no_alloc.h; it has no counterpart in
// cuongvng/bare-cuda-4gib).  Same computation as llm_attention_mma, but the scratch memory for
// split keys is a fixed array inside this library instead of a buffer the caller allocates.

#include "attention_no_alloc.h"

static __device__ __align__(256) float g_static_scratch[LLM_ATTENTION_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
// Device address of g_static_scratch, looked up once per device.  In host code the array's name
// is only a handle for the runtime, never an address a kernel may be given.
float* g_static_scratch_address[MAX_DEVICES] = {};
}  // namespace

extern "C" int llm_attention_mma_static_scratch(const void* q, void* out, void* k_base, void* v_base,
                                                const int32_t* block_table, long long page_stride,
                                                int table_stride, int page_tokens, int kv_heads, int head_dim,
                                                const int32_t* seq_q_start, const int32_t* seq_q_len,
                                                const int32_t* seq_kv_len, const int32_t* tile_seq,
                                                const int32_t* tile_index, int n_tiles, int rows_per_tile,
                                                int n_splits, int q_heads, float scale, int window,
                                                cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (n_splits < 1 || kv_heads < 1 || (rows_per_tile != 16 && rows_per_tile != 64 * PREFILL_MT)) return ERR_BAD_SIZE;
  const long long need = llm_attention_scratch_floats(n_tiles, kv_heads, n_splits, rows_per_tile);
  if (n_splits > 1 && need > (long long)LLM_ATTENTION_STATIC_SCRATCH_FLOATS) return LLM_ERR_STATIC_SCRATCH_TOO_SMALL;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return 1000 + (int)e;
  if (device < 0 || device >= MAX_DEVICES) return ERR_BAD_SIZE;
  // the array's address belongs to the current device: a stream of another device must not get it
  int stream_device = device;
  if (cudaStreamGetDevice(stream, &stream_device) == cudaSuccess) {
    if (stream_device != device) return LLM_ERR_STATIC_SCRATCH_WRONG_DEVICE;
  } else {
    (void)cudaGetLastError();     // the runtime cannot tell (a capturing stream, say): the caller's word stands
  }
  if (!g_static_scratch_address[device]) {
    float* address = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch);
    if (e != cudaSuccess) return 1000 + (int)e;
    g_static_scratch_address[device] = address;
  }
  return llm_attention_mma(q, out, k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads,
                           head_dim, seq_q_start, seq_q_len, seq_kv_len, tile_seq, tile_index, n_tiles,
                           rows_per_tile, n_splits, g_static_scratch_address[device], q_heads, scale, window, stream);
}

extern "C" float* llm_attention_static_scratch_address(void) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return nullptr;
  return g_static_scratch_address[device];
}
