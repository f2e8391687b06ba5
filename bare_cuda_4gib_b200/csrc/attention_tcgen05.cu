// Paged flash attention for prefill portions on the Blackwell tensor cores: both matrix products
// of attention are tcgen05.mma with their accumulators in tensor memory.  It covers the prefill
// shape of csrc/attention_mma.cu (same arguments, same packing of the query heads that share a
// key/value head into the rows of a tile) for head sizes 64 and 128; the decode shape stays with
// the cluster decode kernel.  As there, nothing of cuongvng/bare-cuda-4gib's [heads, T, keys] score
// buffer exists (engine/kernels/attention_qk.cu:49-68, softmax.cu:28-42, attention_av.cu:24-44).
//
// One thread block = one or two tiles of 128 packed rows of one request and one key/value head (two
// at head size 128: they see (almost) the same keys, so every key and value block is brought into
// shared memory once for both; one at head size 64, where two blocks share an SM instead).  Keys are
// visited in blocks of 128 positions:
//   loader warp    copies the blocks' keys and values from the request's pages into 128-byte-
//                  swizzled shared memory with TMA (one tensor map over the cache group's whole
//                  pool, a box per page piece).  Key tiles and value tiles go through ONE ring of
//                  slots in the order K(0) V(0) K(1) V(1) ..., each slot given back by the commit of
//                  the last product that reads it (4 slots at head size 64, 3 at 128);
//   MMA thread     S_g = Q_g K^T (M 128, N 128, K head size) into tile g's S columns of tensor memory;
//   softmax warps  a group of four warps per tile; group g owns tile g and sees every key block of it.
//                  First it stages Q_g with cp.async.  Then, one thread per row: read the row of S
//                  from tensor memory once, 64 columns at a time, scale, mask, running maximum and
//                  sum in float32 (base 2, kept in several independent partial maxima and sums so
//                  that no long dependent chain forms), write P as bfloat16 into swizzled shared
//                  memory (the A operand of the second product);
//   MMA thread     O_g (+)= P_g V (M 128, N 64 per 64 value columns, K 128): O accumulates in
//                  tensor memory over all key blocks; V stays as it lies in the cache
//                  ([key][channel]) and is described to the MMA as an MN-major operand;
//   softmax warps  the maximum that the exponentials are taken against follows the row's true
//                  maximum only when that has grown by more than 2^8, so O (and the row's sum, and
//                  the half row of P that may already be written) is rescaled rarely; at the end
//                  every thread divides its row of O by its sum and stores it: no merge between threads.
// While one group exponentiates, the other (of the same block or of the SM's other block) reads its S,
// and a block's MMA thread serves whichever of its groups is ready next.
// A request's last page may hold, behind its last key, what an earlier request left there: masked
// scores never see it, but 0 x NaN would reach O through P V, so the loader clears those value rows
// in shared memory before the last block's P V may run.
// Every mbarrier wait is bounded: on a timeout the thread sets the error word, all roles leave
// their loops, tensor memory is released and the block returns.

#include "common.cuh"

#include <cuda.h>
#include <string.h>

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace {

constexpr int D = HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention kernel is built for head sizes 64 and 128");
constexpr int KA = D / 64;       // 64-wide sub-tiles ("atoms") along the head dimension
constexpr int BM = 128;          // packed rows per tile (one softmax group)
// Head size 64: one tile per block and two blocks per SM (112 KB of shared memory and 256 columns of
// tensor memory each), so one block's start and end hide behind the other's key blocks (2,048-token
// prompt 44.1 -> 42.8 us, 8,192 tokens 511 -> 473 us).  Head size 128 has room for one block per SM
// only: two tiles per block, which then share every key and value tile.
#ifndef ATTN_TILES
#define ATTN_TILES (HEAD_DIM == 64 ? 1 : 2)
#endif
constexpr int TILES = ATTN_TILES;   // tiles per block (1: two blocks share an SM)
static_assert(TILES == 1 || TILES == 2, "one or two tiles per block");
constexpr int BLOCK_ROWS = TILES * BM;
constexpr int BN = 128;          // keys per block
constexpr int SUB = 128 * 128;   // bytes of a [128 rows x 64 bf16] swizzled sub-tile
constexpr int Q_BYTES = KA * SUB;        // one tile's queries
constexpr int TILE_BYTES = KA * SUB;     // one key tile or one value tile
constexpr int P_BYTES = 2 * SUB;         // [128 rows x 128 keys] as two sub-tiles
#ifndef ATTN_SLOTS
#define ATTN_SLOTS (HEAD_DIM == 64 ? 4 : 3)
#endif
constexpr int SLOTS = ATTN_SLOTS;   // key and value tiles in flight (what shared memory allows)
constexpr int SOFTMAX_THREADS = 128 * TILES, LOADER_THREADS = 32;
constexpr int MMA_WARP = SOFTMAX_THREADS / 32;
constexpr int NUM_THREADS = SOFTMAX_THREADS + 32 + LOADER_THREADS;   // warps 0-7 softmax, 8 MMA, 9 loader
constexpr int TMEM_COLS = 256 * TILES;
constexpr int O_COL = TILES * BN;  // first tensor-memory column of the P V results (the S buffers lie before it)
constexpr int GROUP_THREADS = 128;
constexpr int S_PIECE = 64;      // columns of S a softmax thread holds in registers at a time (one sub-tile of P)
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;
constexpr size_t SMEM_BYTES = TILES * Q_BYTES + SLOTS * TILE_BYTES + TILES * P_BYTES + 256;   // 2 * SLOTS + 11 barriers, 2 words

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
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
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer();
  for (unsigned spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 63u) == 63u) {
      if (*abort_flag) return false;
      if (global_timer() - start > WAIT_LIMIT_NS) return false;
    }
  }
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a [rows x 64 bf16] sub-tile
// with the 128-byte swizzle: rows are 128 bytes, groups of 8 rows are 1024 bytes, and the chunk
// index is XORed with the row's index inside its group.
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

// Shared-memory matrix descriptor, 128-byte swizzle, 1024 bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// float32 accumulator, bfloat16 operands, A K-major; B K-major or (b_mn = 1) MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_load32_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_stores() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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
  // the cache group's pool seen as rows of D elements: row = page * page_rows + k_row0 (or v_row0)
  // + kv head * page_tokens + position in page; the tensor map's box is 64 columns x box_rows rows
  long long page_rows, k_row0, v_row0;
  int box_rows;
  const __nv_bfloat16* q;      // [tokens, q_heads, D]
  __nv_bfloat16* out;          // [tokens, q_heads * D]
  PagedCache cache;
  const int32_t* seq_q_start;
  const int32_t* seq_q_len;
  const int32_t* seq_kv_len;
  const int32_t* tile_seq;     // per tile: batch sequence (-1: nothing to do)
  const int32_t* tile_index;   // per tile: which 128-row tile of the sequence's packed rows
  int q_heads;
  float scale_log2;
  int window;
  int* error_word;
};

constexpr int ERR_LOADER = 11, ERR_MMA = 12, ERR_SOFTMAX = 13, ERR_LAYOUT = 14;

__global__ void __launch_bounds__(NUM_THREADS, TILES == 1 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap pool_map, AttnArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];   // swizzled tiles need 1024-byte alignment (checked below)
  uint8_t* q_smem = smem;                              // [TILES][KA sub-tiles]
  uint8_t* ring = q_smem + TILES * Q_BYTES;            // [SLOTS][KA sub-tiles]: key and value tiles in turn
  uint8_t* p_smem = ring + SLOTS * TILE_BYTES;         // [TILES][two sub-tiles of 64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + TILES * P_BYTES);
  uint64_t* tile_full = bars;               // [SLOTS] loader -> MMA: the slot's tile has landed
  uint64_t* tile_empty = tile_full + SLOTS; // [SLOTS] MMA (commit) -> loader
  uint64_t* q_full = tile_empty + SLOTS;    // [2] softmax group -> MMA: Q_g staged
  uint64_t* s_full = q_full + 2;            // [2] MMA (commit) -> softmax, per group
  uint64_t* p_full = s_full + 2;            // [2] softmax -> MMA: P written, per group
  uint64_t* o_full = p_full + 2;            // [2] MMA (commit) -> softmax, per group: P(i) V is complete
  uint64_t* s_free = o_full + 2;            // [2] softmax -> MMA: the group holds its S values in registers
  uint64_t* v_clean = s_free + 2;           // loader -> MMA: the last value tile holds no stale rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(v_clean + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023) {   // never seen; refuse rather than compute with a broken layout
    if (threadIdx.x == 0) atomicCAS(a.error_word, 0, ERR_LAYOUT);
    return;
  }
  // ---- what this block works on (uniform across the block).  The tile list and the requests'
  // lengths are written by the host before the step's first kernel, so they may be read ahead of
  // pdl_wait(); their latency then hides behind the barrier set-up and the tensor-memory allocation.
  // blocks are handed out with x fastest: all key/value heads of the latest tile first (it sees
  // the most keys), then of the tile before it, ... so the longest blocks of the whole grid start first
  const int tile = gridDim.y - 1 - blockIdx.y, kvh = blockIdx.x;
  const int seq = a.tile_seq[tile];
  int q_start = 0, q_len = 0, kv_len = 0, row0 = 0, n_rows = 0, pos0 = 0, group = 1;
  // per group (tile of 128 rows): its key blocks [g_lo, g_hi) and the positions of its first and last row
  int g_lo[TILES] = {}, g_hi[TILES] = {}, g_min_pos[TILES] = {}, g_max_pos[TILES] = {};
  int kb_lo = 0, n_kb = 0;   // the union of the two ranges: what the loader brings
  if (seq >= 0) {
    group = a.q_heads / a.cache.kv_heads;
    q_start = a.seq_q_start[seq];
    q_len = a.seq_q_len[seq];
    kv_len = a.seq_kv_len[seq];
    row0 = a.tile_index[tile] * BLOCK_ROWS;
    n_rows = q_len * group;
    pos0 = kv_len - q_len;
    int lo_all = 1 << 30, hi_all = 0;
#pragma unroll
    for (int g = 0; g < TILES; ++g) {
      const int first_row = row0 + g * BM;
      if (first_row >= n_rows) continue;
      const int first_token = first_row / group, last_token = min(q_len - 1, (first_row + BM - 1) / group);
      g_min_pos[g] = pos0 + first_token;
      g_max_pos[g] = pos0 + last_token;
      const int lo_key = a.window > 0 ? max(0, g_min_pos[g] - a.window + 1) : 0;
      g_lo[g] = lo_key / BN;
      g_hi[g] = g_max_pos[g] / BN + 1;
      lo_all = min(lo_all, g_lo[g]);
      hi_all = max(hi_all, g_hi[g]);
    }
    if (hi_all > 0) kb_lo = lo_all, n_kb = hi_all - lo_all;
  }
  // the key block that holds the request's last key, if positions behind that key share it
  const int stale_block = (seq >= 0 && kv_len % BN != 0) ? (kv_len - 1) / BN : -1;
  const bool clean_needed = stale_block >= kb_lo && stale_block < kb_lo + n_kb;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&pool_map)) : "memory");
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(&tile_full[s], 1);
      mbar_init(&tile_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&q_full[b], GROUP_THREADS);
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], GROUP_THREADS);
      mbar_init(&o_full[b], 1);
      mbar_init(&s_free[b], GROUP_THREADS);
    }
    mbar_init(v_clean, LOADER_THREADS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  if (warp > MMA_WARP) {
    // ------------------------------------------------------------------ loader warp
    // Tile n of the ring is the keys (n even) or the values (n odd) of key block n / 2: one TMA box
    // per piece of a page (a page holds box_rows or more positions of a key block).  A piece whose
    // page is not held (given back by a window), or that lies wholly behind the request's last key,
    // is filled with zeros by the warp instead; its keys are masked, but stale shared memory must not
    // reach P V.
    const int page_tokens = a.cache.page_tokens;
    const int32_t* table_row = a.cache.block_table + (long long)max(seq, 0) * a.cache.table_stride;
    const int pieces = BN / a.box_rows;   // at most 16: lane p looks piece p up, lanes 0 and 1 issue the copies
    const uint32_t piece_mask = (pieces < 32) ? ((1u << pieces) - 1u) : 0xffffffffu;
    const int page_shift = (page_tokens & (page_tokens - 1)) == 0 ? __ffs(page_tokens) - 1 : -1;
    long long my_row = -1;     // lane p: the pool row (without the cache's K or V offset) of piece p, or -1
    auto look_up = [&](int jj) {
      const int key = (kb_lo + jj) * BN + lane * a.box_rows;
      my_row = -1;
      if (lane < pieces && key < kv_len) {
        const int block = page_shift >= 0 ? key >> page_shift : key / page_tokens;
        const int in_page = page_shift >= 0 ? key & (page_tokens - 1) : key % page_tokens;
        const int page = __ldg(table_row + block);
        if (page >= 0) my_row = (long long)page * a.page_rows + (long long)kvh * page_tokens + in_page;
      }
    };
    auto issue_tile = [&](int n) {
      const int slot = n % SLOTS;
      const uint32_t base = smem_u32(ring) + slot * TILE_BYTES;
      const bool values = n & 1;
      if (!values) look_up(n >> 1);    // the value tile that follows uses the same rows
      const uint32_t held = __ballot_sync(0xffffffffu, my_row >= 0) & piece_mask;
      const uint32_t missing = ~held & piece_mask;
      if (missing) {   // rare: zero the pieces without a page, and make the stores visible to the MMA
        for (int piece = 0; piece < pieces; ++piece) {
          if (!((missing >> piece) & 1u)) continue;
          for (int at = 0; at < KA; ++at)
            for (int i = lane; i < a.box_rows * 8; i += 32)
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + at * SUB + piece * a.box_rows * 128 + i * 16), "r"(0) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
      }
      if (lane == 0) mbar_expect_tx(&tile_full[slot], (uint32_t)__popc(held) * KA * a.box_rows * 128u);   // also the one arrival
      __syncwarp();
      const long long row0_of_cache = values ? a.v_row0 : a.k_row0;
      for (int piece = 0; piece < pieces; ++piece) {     // lanes 0 and 1 take the pieces in turn: issuing is what takes the time
        const long long row = __shfl_sync(0xffffffffu, my_row, piece);
        if (lane != (piece & 1) || row < 0) continue;
        for (int at = 0; at < KA; ++at)
          tma_load_2d(base + at * SUB + piece * a.box_rows * 128, &pool_map, &tile_full[slot], at * 64, (int)(row + row0_of_cache));
      }
    };
    bool ok = true;
    const int n_tiles = 2 * n_kb;
    for (int n = 0; n < n_tiles && ok; ++n) {
      const uint32_t use = (uint32_t)(n / SLOTS);   // how often the slot was filled before
      if (use > 0 && !mbar_wait(&tile_empty[n % SLOTS], (use - 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      issue_tile(n);
    }
    if (ok && clean_needed) {
      // the value tile of the block with the request's last key: once it has landed, clear the rows
      // behind that key (whole pieces behind it were never copied and are zero already)
      const int n = 2 * (stale_block - kb_lo) + 1, slot = n % SLOTS;
      ok = mbar_wait(&tile_full[slot], (n / SLOTS) & 1, abort_flag);
      if (ok) {
        const int first_stale = kv_len - stale_block * BN;           // 1 .. BN - 1
        const int piece_end = min(BN, (first_stale + a.box_rows - 1) / a.box_rows * a.box_rows);
        const uint32_t base = smem_u32(ring) + slot * TILE_BYTES;
        for (int at = 0; at < KA; ++at)
          for (int i = lane; i < (piece_end - first_stale) * 8; i += 32)
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(base + at * SUB + first_stale * 128 + i * 16), "r"(0) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(a.error_word, 0, ERR_LOADER);
    }
    mbar_arrive(v_clean);      // in every case: the MMA thread must not wait in vain
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_kb > 0) {
      constexpr uint32_t idesc_s = instr_desc(BM, BN, 0);
      constexpr uint32_t idesc_o = instr_desc(BM, 64, 1);
      auto active = [&](int g, int jj) { return kb_lo + jj >= g_lo[g] && kb_lo + jj < g_hi[g]; };
      // S_g = Q_g K(jj)^T into group g's S buffer; `last`: no product after this one reads the key tile
      auto issue_s = [&](int g, int jj, bool last) {
        const int slot = (2 * jj) % SLOTS;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = smem_u32(ring) + slot * TILE_BYTES, q_addr = smem_u32(q_smem) + g * Q_BYTES;
#pragma unroll
        for (int at = 0; at < KA; ++at)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + g * BN, smem_desc_sw128(q_addr + at * SUB) + 2 * k,
                      smem_desc_sw128(k_addr + at * SUB) + 2 * k, idesc_s, (at > 0 || k > 0) ? 1u : 0u);
        umma_commit(&s_full[g]);
        if (last) umma_commit(&tile_empty[slot]);
      };
      // O_g (+)= P_g V(jj): the group's O accumulates in tensor memory over its key blocks (`first`: overwrite)
      auto issue_pv = [&](int g, int jj, bool last, int i) {     // i: the group's i-th key block
        const int slot = (2 * jj + 1) % SLOTS;
        const bool first = i == 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = smem_u32(ring) + slot * TILE_BYTES;
        const uint32_t p_addr = smem_u32(p_smem) + g * P_BYTES;
#pragma unroll
        for (int vt = 0; vt < KA; ++vt)
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)
            umma_bf16(tmem_base + O_COL + g * D + vt * 64, smem_desc_sw128(p_addr + (kk >> 2) * SUB) + 2 * (kk & 3),
                      smem_desc_sw128(v_addr + vt * SUB) + (uint64_t)(kk * 2048 >> 4), idesc_o, (kk > 0 || !first) ? 1u : 0u);
        umma_commit(&o_full[g]);
        if (last) umma_commit(&tile_empty[slot]);
      };
      // The two groups are served as they come: a group's next S as soon as it reports that it holds the
      // S before it in registers (and the key tile has landed), its P V as soon as it reports P (and has
      // read the O_block before).  Nothing is waited for while the other group could be served.
      bool ok = true;
      int s_next[TILES] = {}, pv_next[TILES] = {};      // per group: its next block to issue S / P V for
      int n_g[TILES];
#pragma unroll
      for (int g = 0; g < TILES; ++g) n_g[g] = g_hi[g] - g_lo[g];
      auto unfinished = [&]() {
        bool any = false;
#pragma unroll
        for (int g = 0; g < TILES; ++g) any = any || pv_next[g] < n_g[g];
        return any;
      };
      auto landed = [&](int n) { return mbar_try_wait(&tile_full[n % SLOTS], (n / SLOTS) & 1); };
      unsigned long long idle_since = 0;
      unsigned idle_spins = 0;
      while (ok && unfinished()) {
        bool progress = false;
#pragma unroll
        for (int g = 0; g < TILES; ++g) {
          const int o = TILES > 1 ? 1 - g : 0;   // the other group, if there is one
          if (s_next[g] < n_g[g]) {
            const int i = s_next[g], jj = g_lo[g] + i - kb_lo;
            if ((i == 0 ? mbar_try_wait(&q_full[g], 0) : mbar_try_wait(&s_free[g], (i - 1) & 1)) && landed(2 * jj)) {
              // the other group is done with K(jj) if it never reads it or has issued its S for it already
              const bool last = TILES == 1 || !active(o, jj) || s_next[o] > kb_lo + jj - g_lo[o];
              issue_s(g, jj, last);
              s_next[g] = i + 1;
              progress = true;
            }
          }
          if (pv_next[g] < s_next[g]) {
            const int i = pv_next[g], jj = g_lo[g] + i - kb_lo;
            if (mbar_try_wait(&p_full[g], (uint32_t)i & 1u) && landed(2 * jj + 1) &&
                (kb_lo + jj != stale_block || mbar_try_wait(v_clean, 0))) {
              const bool last = TILES == 1 || !active(o, jj) || pv_next[o] > kb_lo + jj - g_lo[o];
              issue_pv(g, jj, last, i);
              pv_next[g] = i + 1;
              progress = true;
            }
          }
        }
        if (progress) {
          idle_spins = 0;
        } else if ((++idle_spins & 63u) == 0u) {
          if (idle_spins == 64u) idle_since = global_timer();
          if (*abort_flag || global_timer() - idle_since > WAIT_LIMIT_NS) ok = false;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicCAS(a.error_word, 0, ERR_MMA);
        for (int b = 0; b < TILES; ++b) umma_commit(&s_full[b]);   // release whoever waits
        for (int b = 0; b < TILES; ++b) umma_commit(&o_full[b]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: group g owns tile g, one thread per row
    const int quad = warp & 3, g = warp >> 2;        // tensor-memory lanes 32 * quad ..
    const int gt = threadIdx.x & (GROUP_THREADS - 1);
    const int tile_row0 = row0 + g * BM;
    // Q_g: 128 rows x D in 16-byte chunks, staged by the group's threads (a few chunks each, so one
    // round of global latency); rows past the request's packed rows are zero
    for (int i = gt; i < BM * (D / 8); i += GROUP_THREADS) {
      const int qr = i / (D / 8), c = i % (D / 8);
      const int QR = tile_row0 + qr;
      const bool valid = seq >= 0 && QR < n_rows;
      const int token = valid ? QR / group : 0, head = valid ? kvh * group + QR % group : 0;
      const __nv_bfloat16* src = a.q + ((long long)(q_start + token) * a.q_heads + head) * D + c * 8;
      cp_async16(smem_u32(q_smem) + g * Q_BYTES + (c >> 3) * SUB + swizzled(qr, c & 7), src, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive(&q_full[g]);
    const int r = quad * 32 + lane;                  // row of the tile = tensor-memory lane
    const int R = tile_row0 + r;
    const bool row_valid = seq >= 0 && R < n_rows;
    const int row_pos = row_valid ? pos0 + R / group : -1;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + g * BN, o_addr = lane_addr + O_COL + g * D;
    const int my_lo = g_lo[g], my_n = g_hi[g] - g_lo[g];
    const int tile_min_pos = g_min_pos[g], tile_max_pos = g_max_pos[g];
    // Running softmax of the row.  `m` is the maximum the exponentials are taken against; it follows the
    // true maximum only when that has grown by more than RESCALE_STEP (in base-2 units), so that O, which
    // accumulates in tensor memory over all key blocks, has to be rescaled rarely: with a stale maximum
    // the probabilities reach at most 2^RESCALE_STEP, and since sum and O are taken against the same `m`
    // their quotient is exact either way.
    constexpr float RESCALE_STEP = 8.0f;
    float m = -INFINITY, l = 0.0f;
    // this row of the group's P tiles (swizzled: chunk c of row r lies at c ^ (r % 8) inside the row's 128 bytes)
    const uint32_t p_row = smem_u32(p_smem) + g * P_BYTES + (r >> 3) * 1024 + (r & 7) * 128, p_xor = (uint32_t)(r & 7) << 4;
    // P(k) V of this group is complete
    auto wait_pv = [&](int k) { return mbar_wait(&o_full[g], (uint32_t)k & 1u, abort_flag); };
    bool ok = true;
    for (int i = 0; i < my_n && ok; ++i) {
      const int key0 = (my_lo + i) * BN;
      ok = mbar_wait(&s_full[g], i & 1, abort_flag) && !*abort_flag;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool all_visible = key0 + BN - 1 <= tile_min_pos && (a.window <= 0 || key0 > tile_max_pos - a.window);
      // The row of S is read once, in two pieces of 64 columns (one sub-tile of P each).  Each piece
      // settles the maximum for itself: should the second piece move it, the probabilities of the
      // first, which this thread has just written, are rescaled where they lie (rare, as is every move).
      float l0 = 0.0f, l1 = 0.0f, l2 = 0.0f, l3 = 0.0f;
#pragma unroll
      for (int h = 0; h < BN / S_PIECE; ++h) {
        uint32_t v[S_PIECE];
#pragma unroll
        for (int c = 0; c < S_PIECE; c += 32) tmem_load32_nowait(s_addr + h * S_PIECE + c, v + c);
        tmem_wait_loads();
        if (h == BN / S_PIECE - 1) {   // the last read of S(i): the MMA thread may overwrite the buffer with S(i + 1)
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(&s_free[g]);
        }
        if (!all_visible) {
#pragma unroll
          for (int k = 0; k < S_PIECE; ++k) {
            const int key = key0 + h * S_PIECE + k;
            const bool visible = key <= row_pos && (a.window <= 0 || key > row_pos - a.window);
            if (!visible) v[k] = 0xff800000u;   // -inf: probability 0
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int k = 0; k < S_PIECE; k += 8) {   // four independent partial maxima
          mx0 = fmaxf(mx0, fmaxf(__uint_as_float(v[k]), __uint_as_float(v[k + 1])));
          mx1 = fmaxf(mx1, fmaxf(__uint_as_float(v[k + 2]), __uint_as_float(v[k + 3])));
          mx2 = fmaxf(mx2, fmaxf(__uint_as_float(v[k + 4]), __uint_as_float(v[k + 5])));
          mx3 = fmaxf(mx3, fmaxf(__uint_as_float(v[k + 6]), __uint_as_float(v[k + 7])));
        }
        const float m_new = fmaxf(m, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * a.scale_log2);   // scale > 0: the maximum commutes with it
        // tensor-memory loads and stores are warp-wide: the warp moves its maxima together, as soon as one of
        // its rows has outgrown its own by the step (a row that has not may follow the true maximum just as well)
        const bool move = __any_sync(0xffffffffu, m_new > m + RESCALE_STEP);
        // P(i) goes where P(i - 1) lay: the product that read it must be complete
        if (h == 0 && i > 0 && !wait_pv(i - 1)) {
          ok = false;
          break;
        }
        if (move) {
          const float corr = fast_exp2(m - (m_new == -INFINITY ? 0.0f : m_new));   // m = -inf gives 0
          m = m_new;
          l *= corr;
          if (h > 0) {   // this block's first piece: its partial sums, and its probabilities where this thread wrote them
            l0 *= corr, l1 *= corr, l2 *= corr, l3 *= corr;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t at = p_row + ((uint32_t)(c << 4) ^ p_xor);
              uint32_t w[4];
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(at) : "memory");
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
                w[e] = pack_bf16(__low2float(pair) * corr, __high2float(pair) * corr);
              }
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            }
          }
          if (i > 0) {     // O = O * corr in tensor memory, between two products (the one before is complete: see above)
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t t[32];
              tmem_load32_nowait(o_addr + c0, t);
              tmem_wait_loads();
#pragma unroll
              for (int k = 0; k < 32; ++k) t[k] = __float_as_uint(__uint_as_float(t[k]) * corr);
              tmem_store32(o_addr + c0, t);
            }
            tmem_wait_stores();
          }
        }
        const float m_use = m == -INFINITY ? 0.0f : m;
        // probabilities into shared memory as the A operand of P V (sub-tile h of 64 keys); the row's sum
        // in four independent partial sums
#pragma unroll
        for (int c = 0; c < S_PIECE / 8; ++c) {
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(v[c * 8 + 2 * e]), a.scale_log2, -m_use));
            const float p1 = fast_exp2(fmaf(__uint_as_float(v[c * 8 + 2 * e + 1]), a.scale_log2, -m_use));
            if (e == 0) l0 += p0 + p1;
            else if (e == 1) l1 += p0 + p1;
            else if (e == 2) l2 += p0 + p1;
            else l3 += p0 + p1;
            packed[e] = pack_bf16(p0, p1);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + h * SUB + ((uint32_t)(c << 4) ^ p_xor)),
                       "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]) : "memory");
        }
      }
      if (!ok) break;
      l += (l0 + l1) + (l2 + l3);
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&p_full[g]);
    }
    if (ok && my_n > 0) ok = wait_pv(my_n - 1) && !*abort_flag;
    if (!ok) {
      *abort_flag = 1;
      atomicCAS(a.error_word, 0, ERR_SOFTMAX);
    }
    // ---- every thread finishes its own row: O / l out of tensor memory, rounded to bfloat16, 64 bytes
    // at a time.  Heads that share a key/value head lie side by side in a token's output row, as their
    // rows do in the tile.  (The loads are warp-wide, so rows without an output still take part.)
    if (ok && my_n > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const int token = row_valid ? R / group : 0, head = row_valid ? kvh * group + R % group : 0;
      uint4* dst = reinterpret_cast<uint4*>(a.out + ((long long)(q_start + token) * a.q_heads + head) * D);
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t t[32];
        tmem_load32_nowait(o_addr + c0, t);
        tmem_wait_loads();
        if (row_valid) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            dst[c0 / 8 + c] = make_uint4(pack_bf16(__uint_as_float(t[8 * c]) * inv, __uint_as_float(t[8 * c + 1]) * inv),
                                         pack_bf16(__uint_as_float(t[8 * c + 2]) * inv, __uint_as_float(t[8 * c + 3]) * inv),
                                         pack_bf16(__uint_as_float(t[8 * c + 4]) * inv, __uint_as_float(t[8 * c + 5]) * inv),
                                         pack_bf16(__uint_as_float(t[8 * c + 6]) * inv, __uint_as_float(t[8 * c + 7]) * inv));
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
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

// Writes the 128-byte tensor map of a cache group's pool: `rows` rows of D bfloat16 starting at
// `base` (16-byte aligned), boxes of 64 columns x `box_rows` rows, 128-byte swizzle.
extern "C" int llm_attention_tc_pool_map(void* map_out, const void* base, long long rows, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return 1000 + (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || rows <= 0 || box_rows <= 0 || box_rows > 128) return ERR_BAD_SIZE;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2000 + (int)r;
}

extern "C" int llm_attention_tc_head_dim() { return D; }
extern "C" int llm_attention_tc_rows() { return BLOCK_ROWS; }

// Same arguments as llm_attention_mma without splits and scratch, plus the pool's tensor map
// (llm_attention_tc_pool_map over `pool_base`, which k_base and v_base lie in, with boxes of
// `box_rows` rows: a multiple of 8 that divides both 128 and the page size).  Every tile has 256
// packed rows (llm_attention_tc_rows).
extern "C" int llm_attention_tcgen05(const void* pool_map, const void* pool_base, int box_rows, const void* q, void* out,
                                     void* k_base, void* v_base, const int32_t* block_table,
                                     long long page_stride, int table_stride, int page_tokens, int kv_heads,
                                     int head_dim, const int32_t* seq_q_start, const int32_t* seq_q_len,
                                     const int32_t* seq_kv_len, const int32_t* tile_seq, const int32_t* tile_index,
                                     int n_tiles, int q_heads, float scale, int window, int* error_word,
                                     cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (head_dim != D || q_heads % kv_heads || kv_heads > 65535) return ERR_BAD_SIZE;
  if (box_rows < 8 || box_rows % 8 || BN % box_rows || page_tokens % box_rows) return ERR_BAD_SIZE;
  const long long k_off = reinterpret_cast<const char*>(k_base) - reinterpret_cast<const char*>(pool_base);
  const long long v_off = reinterpret_cast<const char*>(v_base) - reinterpret_cast<const char*>(pool_base);
  if (k_off < 0 || v_off < 0 || k_off % (D * 2) || v_off % (D * 2) || page_stride % D) return ERR_BAD_ALIGN;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(k_base) |
       reinterpret_cast<uintptr_t>(v_base)) & 15)
    return ERR_BAD_ALIGN;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES) !=
        cudaSuccess)
      return launch_status();
    configured = true;
  }
  CUtensorMap map;   // the caller's buffer need not be 64-byte aligned
  memcpy(&map, pool_map, sizeof(CUtensorMap));
  AttnArgs a;
  a.page_rows = page_stride / D;
  a.k_row0 = k_off / (D * 2);
  a.v_row0 = v_off / (D * 2);
  a.box_rows = box_rows;
  a.q = reinterpret_cast<const __nv_bfloat16*>(q);
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.cache = PagedCache{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  a.seq_q_start = seq_q_start;
  a.seq_q_len = seq_q_len;
  a.seq_kv_len = seq_kv_len;
  a.tile_seq = tile_seq;
  a.tile_index = tile_index;
  a.q_heads = q_heads;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.window = window;
  a.error_word = error_word;
  if (n_tiles > 65535) return ERR_BAD_SIZE;
  dim3 grid(kv_heads, n_tiles);
  launch_kernel(attention_tcgen05_kernel, grid, NUM_THREADS, SMEM_BYTES, stream, map, a);
  return launch_status();
}
