// Paged causal attention on the tensor cores for bfloat16, for prefill portions and decoded
// tokens in one launch: a flash-attention loop (scores, online softmax in float32, weighted
// sum) over key/value tiles gathered from cache pages through the block table.
//
// Built for one head size per library: -DPYLON_HEAD_DIM=<multiple of 16, 16..256>.
//
// Work split.  Grid = (query tiles x splits, KV heads, rows).  The query rows of one
// request and one KV head are packed token-major, the heads of the group inside: packed row
// m is token m / G, query head kv_head * G + m % G, for any group size G.  A block takes 64
// packed rows (4 warps x 16) and walks 64-key tiles aligned at absolute position multiples
// of 64; tiles are double-buffered with cp.async.  With more than one split, each split
// walks its share of the tiles and leaves a normalised partial result and its
// log-sum-exp in scratch memory; a second kernel combines them.  Decode steps use splits to
// fill the machine; prefill uses one.
//
// Semantics as raun6k/Pylon's attention call (src/pylon/kv/cache.py:462-476, restated
// 483-491): key j of the same request is visible to the token at position p iff j <= p
// (and j > p - window when a window is set); softmax scale 1/sqrt(d) unless given.
#include "common.cuh"

#include <cuda.h>

#include <mutex>

#ifndef PYLON_HEAD_DIM
#define PYLON_HEAD_DIM 128
#endif

namespace pylon {

constexpr int D = PYLON_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 in 16..256");
constexpr int BLOCK_N = 64, ATT_THREADS = 128;
constexpr int LD = D + 8;              // padded row: ldmatrix rows fall on distinct banks
constexpr int CHUNKS = D / 8;          // 16-byte chunks per row
constexpr int TILE_ELEMS = BLOCK_N * LD;

struct AttentionParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const __nv_bfloat16* k_pages;
  const __nv_bfloat16* v_pages;
  __nv_bfloat16* out;
  float* partial_out;   // [splits, tokens, nq, D]: the tiled kernel's splits
  float* partial_lse;   // [splits, tokens, nq]   (log2 domain)
  float* decode_out;    // [rows * nkv + decode blocks, SMALL_ROWS, D]: the decode kernel's segments
  float* decode_lse;    // [rows * nkv + decode blocks, SMALL_ROWS]
  const int* q_start;
  const int* kv_len;
  const int* block_table;
  int table_width, page_size, num_pages, nq, nkv, group, window, num_splits, total_tokens, num_rows;
  int small_rows_elsewhere;   // rows of at most SMALL_ROWS packed query rows are left to the decode kernel
  int incoming_rows;          // the cluster form's buffers for partial results hold this many packed query rows
  unsigned* counters;         // [rows * nkv], zero between launches: the last block of a decoded (row, KV head) combines its segments
  int* error;                 // set non-zero when a bounded wait for a TMA copy ran out (the output is then void)
  float scale_log2;     // softmax scale * log2(e)
};

constexpr int SMALL_ROWS = 16;   // packed query rows (tokens x group) one MMA tile holds

__device__ __forceinline__ unsigned smem_address(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_address(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_address(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x by the hardware approximation (relative error about 2^-22, exact 0 for -infinity); the
// library's exp2f wraps the same instruction in range handling the softmax does not need.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Gathers keys [tile * 64, tile * 64 + 64) of one KV head into a padded shared tile.  Keys
// at or beyond kv_len, or without a page, are zero-filled.
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* dst, const __nv_bfloat16* pages, const int* table,
                                             int tile, int kv_len, int kv_head, const AttentionParams& p) {
  for (int c = threadIdx.x; c < BLOCK_N * CHUNKS; c += ATT_THREADS) {
    const int r = c / CHUNKS, col = c % CHUNKS;
    const int key = tile * BLOCK_N + r;
    const __nv_bfloat16* src = pages;
    bool valid = key < kv_len;
    if (valid) {
      const int page = table[key / p.page_size];
      valid = page >= 0 && page < p.num_pages;
      if ((page < -1 || page >= p.num_pages) && p.error) atomicExch(p.error, PYLON_ERROR_BAD_PAGE);   // -1: no page (behind a window); anything else outside the pool: a broken table
      if (valid) src = pages + (((size_t)page * p.nkv + kv_head) * p.page_size + key % p.page_size) * D + col * 8;
    }
    cp_async_16(dst + r * LD + col * 8, src, valid);
  }
}

// One contiguous run of a page holds the whole tile when the page size is a multiple of 64:
// one table look-up, then plain 16-byte copies.
__device__ __forceinline__ void load_kv_tile_contiguous(__nv_bfloat16* dst, const __nv_bfloat16* pages, const int* table,
                                                        int tile, int kv_len, int kv_head, const AttentionParams& p) {
  const int key0 = tile * BLOCK_N;
  const int page = key0 < kv_len ? table[key0 / p.page_size] : -1;
  const bool page_ok = page >= 0 && page < p.num_pages;
  if ((page < -1 || page >= p.num_pages) && threadIdx.x == 0 && p.error) atomicExch(p.error, PYLON_ERROR_BAD_PAGE);   // a broken table; -1 is "no page"
  const __nv_bfloat16* base = page_ok ? pages + (((size_t)page * p.nkv + kv_head) * p.page_size + key0 % p.page_size) * D : pages;
#pragma unroll
  for (int i = 0; i < BLOCK_N * CHUNKS / ATT_THREADS; ++i) {
    const int c = threadIdx.x + i * ATT_THREADS;
    const int r = c / CHUNKS, col = c % CHUNKS;
    const bool valid = page_ok && key0 + r < kv_len;
    cp_async_16(dst + r * LD + col * 8, valid ? base + (size_t)c * 8 : pages, valid);
  }
}

// Tiled form for prompt portions.  MT = 16-row MMA tiles per warp: a block takes 64 * MT
// packed query rows, so each key/value fragment read from shared memory serves MT tiles.
template <int MT>
__global__ void __launch_bounds__(ATT_THREADS) paged_attention_mma_kernel(const AttentionParams p) {
  constexpr int BM = 64 * MT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [BM][LD]
  __nv_bfloat16* k_tiles = q_tile + BM * LD;                              // [2][64][LD]
  __nv_bfloat16* v_tiles = k_tiles + 2 * TILE_ELEMS;                      // [2][64][LD]

  const int row = blockIdx.z, kv_head = blockIdx.y;
  const int q0 = p.q_start[row];
  const int q_len = p.q_start[row + 1] - q0;
  const int G = p.group;
  const int packed_rows = q_len * G;
  if (p.small_rows_elsewhere && packed_rows <= SMALL_ROWS) return;   // the decode kernel takes this row
  // Later query tiles see more keys: hand them out first so the longest blocks start first.
  const int q_tiles_here = (packed_rows + BM - 1) / BM;
  const int q_tile_slot = blockIdx.x / p.num_splits, split = blockIdx.x % p.num_splits;
  if (q_tile_slot >= q_tiles_here) return;
  const int m0 = (q_tiles_here - 1 - q_tile_slot) * BM;
  const int kv_len = p.kv_len[row];
  const int pos0 = kv_len - q_len;   // position of the row's first new token
  const int* table = p.block_table + (size_t)row * p.table_width;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int token_first = m0 / G;
  const int last_packed = min(packed_rows, m0 + BM) - 1;
  const int token_last = last_packed / G;
  const int hi = pos0 + token_last;                                                   // last visible key (inclusive)
  const int lo = p.window > 0 ? max(0, pos0 + token_first - p.window + 1) : 0;        // first visible key
  const int first_tile = lo / BLOCK_N, tiles = hi / BLOCK_N - first_tile + 1;
  const int per_split = (tiles + p.num_splits - 1) / p.num_splits;
  const int tile_begin = first_tile + split * per_split;
  const int tile_end = min(first_tile + tiles, tile_begin + per_split);
  const bool contiguous = p.page_size % BLOCK_N == 0;

  // This thread's rows: two per MMA tile.  Packed index, token position, validity.
  int row_pos[MT][2], row_token[MT][2], row_head[MT][2];
  bool row_valid[MT][2];
  int warp_min_pos = 0x7fffffff;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = m0 + (warp * MT + mt) * 16 + g + 8 * h;
      row_valid[mt][h] = m < packed_rows;
      row_token[mt][h] = row_valid[mt][h] ? m / G : 0;
      row_head[mt][h] = kv_head * G + (row_valid[mt][h] ? m % G : 0);
      row_pos[mt][h] = pos0 + row_token[mt][h];
    }
  }
  // Smallest position among the warp's rows (rows past the end count as the first row): tiles
  // wholly at or below it need no mask.
  {
    const int m_first = m0 + warp * MT * 16;
    warp_min_pos = pos0 + (m_first < packed_rows ? m_first / G : 0);
  }
  const bool warp_full = m0 + (warp * MT + MT) * 16 <= packed_rows;   // all rows of the warp exist
  const bool warp_active = m0 + warp * MT * 16 < packed_rows;

  float o[MT][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f; }
  float row_max[MT][2], row_sum[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) { row_max[mt][0] = row_max[mt][1] = -INFINITY; row_sum[mt][0] = row_sum[mt][1] = 0.f; }

  auto load_tile = [&](int stage, int tile) {
    if (contiguous) {
      load_kv_tile_contiguous(k_tiles + stage * TILE_ELEMS, p.k_pages, table, tile, kv_len, kv_head, p);
      load_kv_tile_contiguous(v_tiles + stage * TILE_ELEMS, p.v_pages, table, tile, kv_len, kv_head, p);
    } else {
      load_kv_tile(k_tiles + stage * TILE_ELEMS, p.k_pages, table, tile, kv_len, kv_head, p);
      load_kv_tile(v_tiles + stage * TILE_ELEMS, p.v_pages, table, tile, kv_len, kv_head, p);
    }
  };

  if (tile_begin < tile_end) {
    // Query tile: packed rows m0 .. m0+BM-1, zero-filled past the end.
    for (int c = threadIdx.x; c < BM * CHUNKS; c += ATT_THREADS) {
      const int r = c / CHUNKS, col = c % CHUNKS;
      const int m = m0 + r;
      const bool valid = m < packed_rows;
      const __nv_bfloat16* src = p.q;
      if (valid) src = p.q + (size_t)(q0 + m / G) * p.q_stride + (size_t)(kv_head * G + m % G) * D + col * 8;
      cp_async_16(q_tile + r * LD + col * 8, src, valid);
    }
    load_tile(0, tile_begin);
    cp_async_commit();

    for (int tile = tile_begin; tile < tile_end; ++tile) {
      const int stage = (tile - tile_begin) & 1;
      if (tile + 1 < tile_end) {
        load_tile(stage ^ 1, tile + 1);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const __nv_bfloat16* ks = k_tiles + stage * TILE_ELEMS;
      const __nv_bfloat16* vs = v_tiles + stage * TILE_ELEMS;
      if (warp_active) {
        // S = Q K^T for this warp's 16 * MT rows and the tile's 64 keys.
        float s[MT][BLOCK_N / 8][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < BLOCK_N / 8; ++i) { s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          unsigned a[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            ldmatrix_x4(a[mt], q_tile + ((warp * MT + mt) * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
#pragma unroll
          for (int n2 = 0; n2 < BLOCK_N / 16; ++n2) {
            unsigned b[4];
            ldmatrix_x4(b, ks + (n2 * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16(s[mt][2 * n2], a[mt], b[0], b[1]);
              mma_bf16(s[mt][2 * n2 + 1], a[mt], b[2], b[3]);
            }
          }
        }

        // Mask: key visible iff key <= position (and > position - window) and the row exists.
        // A tile wholly at or below every row's position (and inside every window) needs none.
        const int tile_last_key = tile * BLOCK_N + BLOCK_N - 1;
        const bool no_mask = warp_full && tile_last_key <= warp_min_pos && p.window == 0;
        if (!no_mask) {
          const int key_base = tile * BLOCK_N + 2 * tq;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int n = 0; n < BLOCK_N / 8; ++n) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int h = i >> 1;
                const int key = key_base + n * 8 + (i & 1);
                bool visible = row_valid[mt][h] && key <= row_pos[mt][h];
                if (p.window > 0) visible = visible && key > row_pos[mt][h] - p.window;
                if (!visible) s[mt][n][i] = -INFINITY;
              }
            }
          }
        }

        // Online softmax in float32 (base 2).
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int n = 0; n < BLOCK_N / 8; ++n) mx = fmaxf(mx, fmaxf(s[mt][n][2 * h], s[mt][n][2 * h + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float new_max = fmaxf(row_max[mt][h], mx);
            const float use_max = new_max == -INFINITY ? 0.f : new_max;
            const float alpha = fast_exp2((row_max[mt][h] - use_max) * p.scale_log2);   // 2^-inf = 0 on the first tile
            const float shift = use_max * p.scale_log2;
            float sum = 0.f;
#pragma unroll
            for (int n = 0; n < BLOCK_N / 8; ++n) {
              const float p0 = fast_exp2(s[mt][n][2 * h] * p.scale_log2 - shift);
              const float p1 = fast_exp2(s[mt][n][2 * h + 1] * p.scale_log2 - shift);
              s[mt][n][2 * h] = p0;
              s[mt][n][2 * h + 1] = p1;
              sum += p0 + p1;
            }
            row_sum[mt][h] = row_sum[mt][h] * alpha + sum;
            row_max[mt][h] = new_max;
            // Once a row's maximum has settled alpha is exactly 1: the accumulators are left alone
            // unless some row of the warp moved.
            if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
              for (int i = 0; i < D / 8; ++i) { o[mt][i][2 * h] *= alpha; o[mt][i][2 * h + 1] *= alpha; }
            }
          }
        }

        // O += P V
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          unsigned a[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
            a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
            a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
            a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
          }
#pragma unroll
          for (int d2 = 0; d2 < D / 16; ++d2) {
            unsigned b[4];
            ldmatrix_x4_trans(b, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + d2 * 16 + 8 * (lane >> 4));
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16(o[mt][2 * d2], a[mt], b[0], b[1]);
              mma_bf16(o[mt][2 * d2 + 1], a[mt], b[2], b[3]);
            }
          }
        }
      }  // warp_active
      __syncthreads();   // the stage is overwritten by the load after next
    }
  }

  // Epilogue: normalise and store (or leave a partial result for the combine kernel).
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float sum = row_sum[mt][h];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (!row_valid[mt][h]) continue;
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      const size_t token = (size_t)q0 + row_token[mt][h];
      if (p.num_splits == 1) {
        __nv_bfloat16* dst = p.out + (token * p.nq + row_head[mt][h]) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + 2 * tq) = __floats2bfloat162_rn(o[mt][i][2 * h] * inv, o[mt][i][2 * h + 1] * inv);
      } else {
        const size_t slot = ((size_t)split * p.total_tokens + token) * p.nq + row_head[mt][h];
        float* dst = p.partial_out + slot * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
          *reinterpret_cast<float2*>(dst + i * 8 + 2 * tq) = make_float2(o[mt][i][2 * h] * inv, o[mt][i][2 * h + 1] * inv);
        if (tq == 0) p.partial_lse[slot] = sum > 0.f ? row_max[mt][h] * p.scale_log2 + log2f(sum) : -INFINITY;
      }
    }
  }
}

// -----------------------------------------------------------------------------------------
// Decode form: rows with at most 16 packed query rows (one decoded token times the group, or
// a few tokens).  All four warps share the one 16-row query tile and split every 64-key tile
// between them (16 keys each), each with its own running softmax; the four partial results
// are merged through shared memory at the end.  Key/value tiles run through a three-stage
// cp.async pipeline.  When the page size is a multiple of 64 a tile is one contiguous run of
// a page and is addressed with one table look-up; otherwise keys are gathered one by one.
// -----------------------------------------------------------------------------------------
constexpr int DEC_STAGES = 2;   // two stages leave room for three blocks per SM: warps in flight matter more than depth
// The cluster form runs with two blocks per SM at most and would have room for a third stage, but then only two blocks fit
// an SM at all, and clusters that have to be placed whole on one GPC no longer find room at once: 3.88 ms a step instead of
// 3.25 at batch 12, 2.75 instead of 2.49 at batch 4 (2.11 instead of 2.14 at batch 1).
constexpr int DEC_CLUSTER_STAGES = 2;
// With so few pairs that every block of their 16-block clusters has an SM to itself (one request of eight KV heads), the
// ring holds three tiles, so that more of a block's old tiles are asked for before the kernel waits for the one ahead of
// it: 1,975 against 1,990 us a step at one request.  (Four stages, all of a block's tiles at a context of 4,096, take so
// much shared memory that the output projection's blocks cannot move in beside them and ask for their weights early: 2,215 us.)
constexpr int DEC_LONE_STAGES = 3;

// Two ways to bring a 64-key tile into shared memory.  With a head size that is a multiple of
// 64 and pages that are multiples of 64 keys, TMA copies the tile (one elected thread, boxes of
// 64 keys x 64 values in the 128-byte swizzle, completion on an mbarrier): streaming the cache
// this way reaches 5.9 TB/s where per-thread 16-byte cp.async copies reached 3.4.  Otherwise
// every thread gathers 16-byte pieces with cp.async into rows padded by 8 values.
constexpr bool TMA_HEAD = D % 64 == 0;
template <bool TMA, int STAGES = DEC_STAGES>
struct DecodeTiles {
  static constexpr int ROW = TMA ? D : LD;                        // values between two keys of a box / a padded row
  static constexpr int TILE = BLOCK_N * ROW;                      // one 64-key tile of keys or of values
  static constexpr int STAGE = 2 * TILE;                          // keys then values
  static constexpr size_t STAGE_BYTES = (size_t)STAGES * STAGE * sizeof(__nv_bfloat16);
  // stages (1024-byte aligned for the swizzle), query tile, two mbarriers
  static constexpr size_t SMEM = (TMA ? 1024 : 0) + STAGE_BYTES + (size_t)SMALL_ROWS * LD * sizeof(__nv_bfloat16) + (TMA ? 64 : 0);
  static_assert(STAGE * sizeof(__nv_bfloat16) >= 4 * SMALL_ROWS * D * sizeof(float), "the warps' outputs are merged in one idle stage");
  // Element offset of the 16-byte piece `chunk` (8 values) of key `row` within a tile.
  static __device__ __forceinline__ int offset(int row, int chunk) {
    if (TMA) return (chunk >> 3) * (BLOCK_N * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
    return row * LD + chunk * 8;
  }
};

constexpr unsigned ATT_WAIT_LIMIT = 1u << 22;   // try_wait calls before a wait for a TMA copy gives up
__device__ __forceinline__ void att_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_address(bar)), "r"(count));
}
__device__ __forceinline__ void att_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_address(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool att_mbar_wait(uint64_t* bar, unsigned parity) {
  for (unsigned tries = 0; tries < ATT_WAIT_LIMIT; ++tries) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(smem_address(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// One box of 64 keys x 64 values; no cluster multicast.
__device__ __forceinline__ void att_tma_load(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(smem_address(dst)), "l"((unsigned long long)map), "r"(smem_address(bar)), "r"(x), "r"(y) : "memory");
}

// Thread-block clusters: the address of one's own shared-memory location in another block of the cluster, a load from
// there, and the cluster's barrier (release/acquire: what a block wrote to its shared memory before is visible after).
__device__ __forceinline__ unsigned cluster_address(const void* own, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_address(own)), "r"(rank));
  return remote;
}
__device__ __forceinline__ float cluster_load(unsigned address) {
  float value;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(value) : "r"(address) : "memory");
  return value;
}
__device__ __forceinline__ void cluster_store(unsigned address, float value) {
  asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(address), "f"(value) : "memory");
}
// The two halves of a cluster barrier: a block arrives when it starts and waits before it first writes into another
// block's shared memory, by which time every block of the cluster has started too.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// The decode kernel's warps merge their results through a buffer whose rows lie 4 D bytes apart, a multiple of all 32
// banks: column c of row r sits at c ^ merge_swizzle(r), so that the four rows a half-warp stores at once fall into
// different banks (head sizes that are multiples of 32; others keep their columns).
__device__ __forceinline__ int merge_swizzle(int r) { return D % 32 == 0 ? (r & 3) << 3 : 0; }

// Tiles of 64 keys that a row of decoded tokens (at most SMALL_ROWS packed query rows) walks
// per KV head, and the first of them; 0 for every other row.
__device__ __forceinline__ int decode_row_tiles(const AttentionParams& p, int row, int* first_tile) {
  const int q0 = p.q_start[row];
  const int q_len = p.q_start[row + 1] - q0;
  const int packed_rows = q_len * p.group;
  *first_tile = 0;
  if (packed_rows <= 0 || packed_rows > SMALL_ROWS) return 0;
  const int pos0 = p.kv_len[row] - q_len;
  const int hi = pos0 + q_len - 1;
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  if (hi < lo) return 0;
  *first_tile = lo / BLOCK_N;
  return hi / BLOCK_N - lo / BLOCK_N + 1;
}

constexpr int DEC_PENDING = 16;    // segments a block collects before it publishes them
constexpr int DEC_MIN_TILES = 4;   // a block takes about this many tiles at least: below it, starting and merging cost more than the walk

// The runs: `used` blocks share `total` tiles, block b takes [run_begin(b), run_begin(b + 1)), so the
// runs differ by one tile at most; run_of(x) is the block whose run holds tile x.
// `pairs`: (row, KV head) pairs with tiles.  When the rows are equally long, a number of blocks that is a
// multiple of the pairs makes every run end where a pair ends, and no block has to merge and publish
// twice (30 instead of 35 us at batch 8, context 4096); it is taken if it costs under a fifth of the blocks.
__device__ __forceinline__ int decode_blocks_used(int total, int grid, int pairs) {
  const int used = max(1, min(grid, total / DEC_MIN_TILES));
  const int aligned = pairs > 0 ? used / pairs * pairs : 0;
  return aligned * 5 >= used * 4 ? aligned : used;
}
__device__ __forceinline__ int run_begin(int block, int total, int used) { return (int)((long long)block * total / used); }
__device__ __forceinline__ int run_of(int tile, int total, int used) { return (int)((((long long)tile + 1) * used - 1) / total); }   // a block takes at least this many tiles: below it the merging costs more than the walk

// Decoded rows.  All (row, KV head, tile) triples of the launch form one sequence, row-major,
// and the blocks cut it into equal runs, so every block reads the same number of bytes however
// the requests' lengths differ.  A run may end inside a (row, KV head) pair and go on into
// the next: each piece ("segment") is walked by the block's four warps, 16 keys of every tile
// each, and merged.  A pair that lies in one block is written out at once; the segments of a
// pair that spans blocks leave normalised partial results in scratch slot (pair + block), and
// the block that finishes last (a counter per pair) combines them.
//
// map_k, map_v (TMA form only): the page pools as matrices [pages x KV heads x page size, D]
// with boxes of 64 rows x 64 values.
//
// CLUSTER > 0 (TMA form, launches with so few (row, KV head) pairs that CLUSTER blocks for each are all resident): the
// blocks of a thread-block cluster share one pair, each walks an equal share of its tiles, and the partial results are
// combined through distributed shared memory: every block sends each other block the slice of its result that the
// other one adds up (stores into that block's shared memory, which nobody waits for), and after one cluster barrier each
// block adds up what it was sent and leaves.  No scratch, fence, counter or second trip to L2; with one request the
// combination of 16 partial results per head was most of the kernel's time.  (Fetching the slices from the other
// blocks instead took a second barrier, so that nobody left while it was being read: 3,000 to 4,000 cycles for the
// loads and that barrier, measured at one request.)
template <bool TMA, int CLUSTER = 0, int CLUSTER_STAGES = DEC_CLUSTER_STAGES>
__global__ void __launch_bounds__(ATT_THREADS, D <= 128 && CLUSTER_STAGES <= 2 ? 3 : 1) paged_attention_decode_kernel(const AttentionParams p, const __grid_constant__ CUtensorMap map_k,
                                                                              const __grid_constant__ CUtensorMap map_v) {
  constexpr int STAGES = CLUSTER ? CLUSTER_STAGES : DEC_STAGES;
  using Tiles = DecodeTiles<TMA, STAGES>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* smem_base = TMA ? reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023) : smem_raw;
  __nv_bfloat16* stages = reinterpret_cast<__nv_bfloat16*>(smem_base);                 // [STAGES][2][64 keys]
  __nv_bfloat16* q_tile = stages + STAGES * Tiles::STAGE;                          // [16][LD]
  uint64_t* tile_full = reinterpret_cast<uint64_t*>(q_tile + SMALL_ROWS * LD);         // [STAGES], TMA form
  // cluster form: what the other blocks send - [CLUSTER][slice] partial results, then [CLUSTER][SMALL_ROWS] log-sum-exps
  float* incoming = reinterpret_cast<float*>(tile_full + 8);
  __shared__ int plan[4];   // tiles of the launch; the row this block starts in; tiles before that row; blocks with a run
  __shared__ int pending[DEC_PENDING][6];   // segments to publish: pair, first block, segments, q0, packed rows, KV head
  __shared__ bool pending_last[DEC_PENDING];
  __shared__ float row_lse[SMALL_ROWS];
  __shared__ float merge_max[4 * SMALL_ROWS], merge_sum[4 * SMALL_ROWS];   // the four warps' softmax statistics

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int G = p.group;
  if (TMA && threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) att_mbar_init(&tile_full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // The rows' lengths were written long before the kernel ahead of this one started, so the plan
  // can be made while that kernel finishes; the queries and the newest keys are its work.
  const int cluster_pair = CLUSTER ? (int)blockIdx.x / (CLUSTER ? CLUSTER : 1) : 0, cluster_rank = CLUSTER ? (int)blockIdx.x % (CLUSTER ? CLUSTER : 1) : 0;
  int cluster_first = 0, cluster_tiles = 0;
  if (CLUSTER) {
    cluster_tiles = decode_row_tiles(p, cluster_pair / p.nkv, &cluster_first);
    if (cluster_tiles == 0) {   // not a row of decoded tokens: the whole cluster leaves
      grid_dependency_wait();   // a grid must not end before the grid ahead of it has: the next kernel's wait sees only this one
      return;
    }
    cluster_arrive();   // "this block has started"; waited for before the first store into another block's shared memory
  }
  if (!CLUSTER && warp == 0) {
    int unused;
    const int first_chunk = lane < p.num_rows ? decode_row_tiles(p, lane, &unused) : 0;   // kept: most launches have at most 32 rows
    int total = first_chunk, with_tiles = first_chunk > 0;
    for (int base = 32; base < p.num_rows; base += 32) {
      const int tiles = base + lane < p.num_rows ? decode_row_tiles(p, base + lane, &unused) : 0;
      total += tiles;
      with_tiles += tiles > 0;
    }
#pragma unroll
    for (int offset = 16; offset; offset >>= 1) {
      total += __shfl_xor_sync(0xffffffffu, total, offset);
      with_tiles += __shfl_xor_sync(0xffffffffu, with_tiles, offset);
    }
    total *= p.nkv;
    const int used = decode_blocks_used(total, gridDim.x, with_tiles * p.nkv);
    const int begin = (int)blockIdx.x < used ? run_begin(blockIdx.x, total, used) : total;
    int found_row = -1, found_before = 0;
    if (begin < total) {
      int before = 0;
      for (int base = 0; base < p.num_rows && found_row < 0; base += 32) {
        const int tiles = (base == 0 ? first_chunk : (base + lane < p.num_rows ? decode_row_tiles(p, base + lane, &unused) : 0)) * p.nkv;
        int inclusive = tiles;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
          const int below = __shfl_up_sync(0xffffffffu, inclusive, offset);
          if (lane >= offset) inclusive += below;
        }
        const int exclusive = before + inclusive - tiles;
        const unsigned hit = __ballot_sync(0xffffffffu, tiles > 0 && exclusive <= begin && begin < exclusive + tiles);
        if (hit) {
          found_row = base + __ffs(hit) - 1;
          found_before = __shfl_sync(0xffffffffu, exclusive, __ffs(hit) - 1);
        }
        before += __shfl_sync(0xffffffffu, inclusive, 31);
      }
    }
    if (lane == 0) { plan[0] = total; plan[1] = found_row; plan[2] = found_before; plan[3] = used; }
  }
  __syncthreads();
  const int total_tiles = CLUSTER ? 0 : plan[0];
  if (!CLUSTER && plan[1] < 0) {   // no run for this block
    grid_dependency_wait();   // a grid must not end before the grid ahead of it has: the next kernel's wait sees only this one
    return;
  }
  const int blocks_used = CLUSTER ? 1 : plan[3];
  const int run_end = CLUSTER ? 0 : run_begin(blockIdx.x + 1, total_tiles, blocks_used);
  const bool contiguous = p.page_size % BLOCK_N == 0;
  int position = CLUSTER ? 0 : run_begin(blockIdx.x, total_tiles, blocks_used), row = CLUSTER ? 0 : plan[1], before = CLUSTER ? 0 : plan[2];
  bool cluster_share_taken = false;
  unsigned issued = 0, consumed = 0;   // tiles of this block so far: stage = count % STAGES

  // The next piece of this block's run: tiles [tile_begin, tile_end) of one (row, KV head).
  struct Segment {
    int kv_head, tile_begin, tile_end, pair, first_block, segments, q0, packed_rows, kv_len, pos0;
    const int* table;
  };
  auto next_segment = [&](Segment& s) -> bool {
    if (CLUSTER) {   // one segment: this block's share of the cluster's pair
      if (cluster_share_taken) return false;
      cluster_share_taken = true;
      const int cluster_row = cluster_pair / p.nkv;
      s.kv_head = cluster_pair % p.nkv;
      s.tile_begin = cluster_first + (int)((long long)cluster_rank * cluster_tiles / (CLUSTER ? CLUSTER : 1));
      s.tile_end = cluster_first + (int)((long long)(cluster_rank + 1) * cluster_tiles / (CLUSTER ? CLUSTER : 1));
      s.pair = cluster_pair; s.first_block = 0; s.segments = CLUSTER;
      s.q0 = p.q_start[cluster_row];
      const int q_len = p.q_start[cluster_row + 1] - s.q0;
      s.packed_rows = q_len * G;
      s.kv_len = p.kv_len[cluster_row];
      s.pos0 = s.kv_len - q_len;
      s.table = p.block_table + (size_t)cluster_row * p.table_width;
      return s.tile_end > s.tile_begin;
    }
    while (position < run_end && row < p.num_rows) {
      int first_tile;
      const int row_tiles = decode_row_tiles(p, row, &first_tile);
      if (row_tiles == 0) { ++row; continue; }
      const int within = position - before;
      s.kv_head = within / row_tiles;
      s.tile_begin = first_tile + within % row_tiles;
      s.tile_end = s.tile_begin + min(run_end - position, row_tiles - within % row_tiles);
      const int pair_start = before + s.kv_head * row_tiles;
      s.first_block = run_of(pair_start, total_tiles, blocks_used);
      s.segments = run_of(pair_start + row_tiles - 1, total_tiles, blocks_used) - s.first_block + 1;   // blocks this pair lies in
      s.pair = row * p.nkv + s.kv_head;
      s.q0 = p.q_start[row];
      const int q_len = p.q_start[row + 1] - s.q0;
      s.packed_rows = q_len * G;
      s.kv_len = p.kv_len[row];
      s.pos0 = s.kv_len - q_len;
      s.table = p.block_table + (size_t)row * p.table_width;
      position += s.tile_end - s.tile_begin;
      if (position - before == row_tiles * p.nkv) { before += row_tiles * p.nkv; ++row; }   // the next segment starts the next row
      return true;
    }
    return false;
  };
  // Starts the copy of one tile into the next stage of the ring.
  auto issue_tile = [&](const Segment& s, int tile) {
    __nv_bfloat16* dst = stages + (issued % STAGES) * Tiles::STAGE;
    if (TMA) {
      if (threadIdx.x == 0) {
        // A tile lies in one page.  Without a page for it the row coordinate points past the
        // pool and TMA fills the boxes with zeros.
        const int key0 = tile * BLOCK_N;
        const int page = s.table[key0 / p.page_size];
        const bool page_ok = page >= 0 && page < p.num_pages;
        if ((page < -1 || page >= p.num_pages) && p.error) atomicExch(p.error, PYLON_ERROR_BAD_PAGE);   // a broken table; -1 is "no page"
        const int y = page_ok ? (page * p.nkv + s.kv_head) * p.page_size + key0 % p.page_size : p.num_pages * p.nkv * p.page_size;
        uint64_t* bar = &tile_full[issued % STAGES];
        // The stage was read with ordinary loads (ldmatrix) until the barrier before this; TMA is another proxy, which
        // that barrier alone does not order behind them.
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        att_mbar_expect_tx(bar, (unsigned)(Tiles::STAGE * sizeof(__nv_bfloat16)));
#pragma unroll
        for (int box = 0; box < D / 64; ++box) {
          att_tma_load(dst + box * (BLOCK_N * 64), &map_k, bar, box * 64, y);
          att_tma_load(dst + Tiles::TILE + box * (BLOCK_N * 64), &map_v, bar, box * 64, y);
        }
      }
    } else if (contiguous) {
      load_kv_tile_contiguous(dst, p.k_pages, s.table, tile, s.kv_len, s.kv_head, p);
      load_kv_tile_contiguous(dst + Tiles::TILE, p.v_pages, s.table, tile, s.kv_len, s.kv_head, p);
    } else {
      load_kv_tile(dst, p.k_pages, s.table, tile, s.kv_len, s.kv_head, p);
      load_kv_tile(dst + Tiles::TILE, p.v_pages, s.table, tile, s.kv_len, s.kv_head, p);
    }
    ++issued;
  };
  // Starts the copy of a segment's packed query rows (cp.async; the caller commits the group).
  auto load_query = [&](const Segment& s) {
    for (int c = threadIdx.x; c < SMALL_ROWS * CHUNKS; c += ATT_THREADS) {
      const int r = c / CHUNKS, col = c % CHUNKS;
      const bool valid = r < s.packed_rows;
      const __nv_bfloat16* src = p.q;
      if (valid) src = p.q + (size_t)(s.q0 + r / G) * p.q_stride + (size_t)(s.kv_head * G + r % G) * D + col * 8;
      cp_async_16(q_tile + r * LD + col * 8, src, valid);
    }
  };

  // Segments of pairs that other blocks share leave partial results; the block publishes them
  // together (one fence and one round of counter updates for all of them, at the end of its run
  // or when the list is full), and combines those pairs for which it turns out to be last.
  int pending_count = 0;
  auto publish_and_combine = [&]() {
    if (pending_count == 0) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x < pending_count)
      pending_last[threadIdx.x] = atomicAdd(p.counters + pending[threadIdx.x][0], 1u) == (unsigned)pending[threadIdx.x][2] - 1u;
    __syncthreads();
    for (int entry = 0; entry < pending_count; ++entry) {
      if (!pending_last[entry]) continue;
      const int pair = pending[entry][0], first_block = pending[entry][1], segments = pending[entry][2];
      const int q0 = pending[entry][3], packed_rows = pending[entry][4], kv_head = pending[entry][5];
      __threadfence();
      // One trip to L2: every thread asks for its four values of up to eight segments and for
      // those segments' log-sum-exps at once, then weighs and adds them.  More segments go round
      // again, the sum so far rescaled as in the attention loop itself.
      constexpr int SLOT_VECTORS = SMALL_ROWS * D / 4;
      const size_t slot0 = (size_t)pair + first_block;
      const float4* partials = reinterpret_cast<const float4*>(p.decode_out + slot0 * SMALL_ROWS * D);
      const float* lses = p.decode_lse + slot0 * SMALL_ROWS;
      for (int v = threadIdx.x; v < packed_rows * (D / 4); v += ATT_THREADS) {
        const int r = v / (D / 4), col = (v % (D / 4)) * 4;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        float run_max = -INFINITY, run_total = 0.f;
        for (int s2 = 0; s2 < segments; s2 += 8) {
          float4 part[8];
          float lse[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int segment = min(s2 + j, segments - 1);
            part[j] = __ldcg(partials + (size_t)segment * SLOT_VECTORS + v);
            lse[j] = s2 + j < segments ? __ldcg(lses + (size_t)segment * SMALL_ROWS + r) : -INFINITY;
          }
          float new_max = run_max;
#pragma unroll
          for (int j = 0; j < 8; ++j) new_max = fmaxf(new_max, lse[j]);
          if (new_max == -INFINITY) continue;   // nothing visible in these segments
          const float alpha = fast_exp2(run_max - new_max);   // 0 for the first round
          sum.x *= alpha; sum.y *= alpha; sum.z *= alpha; sum.w *= alpha;
          run_total *= alpha;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float weight = fast_exp2(lse[j] - new_max);   // 0 for -infinity
            sum.x += weight * part[j].x; sum.y += weight * part[j].y; sum.z += weight * part[j].z; sum.w += weight * part[j].w;
            run_total += weight;
          }
          run_max = new_max;
        }
        const float inv = run_total > 0.f ? 1.f / run_total : 0.f;
        const size_t token = (size_t)q0 + r / G;
        const int head = kv_head * G + r % G;
        __nv_bfloat16* dst = p.out + (token * p.nq + head) * D + col;
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(sum.x * inv, sum.y * inv), pack_bf16(sum.z * inv, sum.w * inv));
      }
      if (threadIdx.x == 0) p.counters[pair] = 0u;   // ready for the next launch
    }
    pending_count = 0;
  };

  Segment current, following;
  bool have = next_segment(current);
  const bool had_tiles = have;   // cluster form: this block has a share of the pair's tiles
  bool waited = false;       // for the kernel before this one (programmatic dependent launch)
  bool prefetched = false;   // the segment's query and first tile were asked for while the one before it was merged
  while (have) {
    const bool have_following = next_segment(following);
    const int kv_head = current.kv_head, tile_begin = current.tile_begin, tile_end = current.tile_end, pair = current.pair;
    const int first_block = current.first_block, segments = current.segments, q0 = current.q0, packed_rows = current.packed_rows;
    const int kv_len = current.kv_len, pos0 = current.pos0;
    int issued_ahead = 0;   // tiles of this segment asked for before the wait for the kernel ahead (first segment only)

    int row_pos[2];
    bool row_valid[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = g + 8 * h;
      row_valid[h] = m < packed_rows;
      row_pos[h] = pos0 + (row_valid[h] ? m / G : 0);
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};

    auto issue = [&](int tile) {
      if (tile < tile_end) issue_tile(current, tile);
      if (!TMA) cp_async_commit();   // an empty group keeps the count of groups in step with the tiles
    };
    if (!prefetched) {
      if (!waited) {
        // Tiles that end before the row's first new token hold nothing the kernel before this one writes: as many
        // of them as the ring has stages are asked for before this kernel waits for that one.  The queries and the
        // newest keys are its work.
        if (TMA) {
          while (issued_ahead < STAGES && tile_begin + issued_ahead < tile_end && (tile_begin + issued_ahead + 1) * BLOCK_N <= pos0) {
            issue_tile(current, tile_begin + issued_ahead);
            ++issued_ahead;
          }
        }
        grid_dependency_wait();
        allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
        waited = true;
      }
      load_query(current);
      if (TMA) cp_async_commit();   // otherwise the first tile's group carries the query
      for (int s = issued_ahead; s < STAGES - 1; ++s) issue(tile_begin + s);   // the ring runs STAGES - 1 tiles ahead
    }

    const bool upper_rows_unused = packed_rows <= 8;
    // The query fragments stay in registers when the head is small enough to leave room.
    constexpr bool Q_IN_REGISTERS = D <= 128;
    unsigned q_frag[Q_IN_REGISTERS ? D / 16 : 1][4];
    bool q_loaded = false;

    bool tile_prefetched = false;   // the following segment's first tile is on its way
    for (int tile = tile_begin; tile < tile_end; ++tile) {
      if (tile + STAGES - 1 < tile_begin + issued_ahead) {
        // asked for before the wait
      } else if (TMA && STAGES == 2 && tile + 1 == tile_end && have_following) {
        // The ring has a free stage and this segment no tile for it: the following segment's
        // first tile comes in while this one's last tile is multiplied and the warps are merged.
        issue_tile(following, following.tile_begin);
        tile_prefetched = true;
      } else {
        issue(tile + STAGES - 1);
      }
      const __nv_bfloat16* ks = stages + (consumed % STAGES) * Tiles::STAGE;
      const __nv_bfloat16* vs = ks + Tiles::TILE;
      if (TMA) {
        if (tile == tile_begin) {
          cp_async_wait<0>();
          __syncthreads();   // the query tile is in
        }
        if (!att_mbar_wait(&tile_full[consumed % STAGES], (consumed / STAGES) & 1)) {
          if (p.error) atomicExch(p.error, 1);
          if (!CLUSTER) return;   // every thread of the block gives up on the same copy
          break;                  // in a cluster the others wait for this block at the barrier: it goes there, its result void
        }
        if (tile * BLOCK_N + BLOCK_N > kv_len) {
          // Keys past the row's length are masked, but their values (whatever the page held) still
          // meet a weight of zero in the product: make them zero, as the gathering form does.
          const int first_unused = kv_len - tile * BLOCK_N;
          for (int c = threadIdx.x; c < BLOCK_N * CHUNKS; c += ATT_THREADS) {
            const int r = c / CHUNKS;
            if (r >= first_unused) *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(vs) + Tiles::offset(r, c % CHUNKS)) = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // before TMA writes this stage again
          __syncthreads();
        }
      } else {
        cp_async_wait<STAGES - 1>();
        __syncthreads();
      }
      ++consumed;
      const int key_row = warp * 16 + (lane & 7);   // the key this lane addresses in ldmatrix, before the 8-row offsets
      if (Q_IN_REGISTERS && !q_loaded) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          ldmatrix_x4(q_frag[Q_IN_REGISTERS ? kk : 0], q_tile + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
        q_loaded = true;
      }

      // Even and odd k-steps accumulate separately: four independent MMA chains instead of two.
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      float s_odd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        unsigned a_loaded[4], b[4];
        if (!Q_IN_REGISTERS) ldmatrix_x4(a_loaded, q_tile + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
        const unsigned (&a)[4] = Q_IN_REGISTERS ? q_frag[Q_IN_REGISTERS ? kk : 0] : a_loaded;
        ldmatrix_x4(b, ks + Tiles::offset(key_row + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
        if (kk & 1) {
          mma_bf16(s_odd[0], a, b[0], b[1]);
          mma_bf16(s_odd[1], a, b[2], b[3]);
        } else {
          mma_bf16(s[0], a, b[0], b[1]);
          mma_bf16(s[1], a, b[2], b[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] += s_odd[n][i];
      // Tiles that end at or before the row's first new token, with no window, are visible whole.
      if (p.window > 0 || tile * BLOCK_N + BLOCK_N - 1 > pos0) {
        const int key_base = tile * BLOCK_N + warp * 16 + 2 * tq;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int h = i >> 1;
            const int key = key_base + n * 8 + (i & 1);
            bool visible = row_valid[h] && key <= row_pos[h];
            if (p.window > 0) visible = visible && key > row_pos[h] - p.window;
            if (!visible) s[n][i] = -INFINITY;
          }
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // One decoded token times a group of up to 8 fills rows 0..7 only: rows 8..15 hold zero
        // queries, their scores stay zero and nothing of them is stored.
        if (h == 1 && upper_rows_unused) continue;
        float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float new_max = fmaxf(row_max[h], mx);
        const float use_max = new_max == -INFINITY ? 0.f : new_max;
        const float alpha = fast_exp2((row_max[h] - use_max) * p.scale_log2);
        const float shift = use_max * p.scale_log2;
        float sum = 0.f;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const float p0 = fast_exp2(s[n][2 * h] * p.scale_log2 - shift);
          const float p1 = fast_exp2(s[n][2 * h + 1] * p.scale_log2 - shift);
          s[n][2 * h] = p0;
          s[n][2 * h + 1] = p1;
          sum += p0 + p1;
        }
        row_sum[h] = row_sum[h] * alpha + sum;
        row_max[h] = new_max;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][2 * h] *= alpha; o[i][2 * h + 1] *= alpha; }
      }
      unsigned a[4];
      a[0] = pack_bf16(s[0][0], s[0][1]);
      a[1] = pack_bf16(s[0][2], s[0][3]);
      a[2] = pack_bf16(s[1][0], s[1][1]);
      a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int d2 = 0; d2 < D / 16; ++d2) {
        unsigned b[4];
        ldmatrix_x4_trans(b, vs + Tiles::offset(key_row + 8 * ((lane >> 3) & 1), d2 * 2 + (lane >> 4)));
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      }
      __syncthreads();   // everyone is done with this stage before it is loaded again
    }
    if (!TMA) cp_async_wait<0>();

    // While this segment is merged and written out, the next one's query is on its way into the
    // query tile, which every warp has read; its first tile went into the stage that is not the
    // one read last (where the merge happens).
    prefetched = false;
    if (TMA && STAGES == 2 && have_following) {
      load_query(following);
      cp_async_commit();
      if (!tile_prefetched) issue_tile(following, following.tile_begin);
      prefetched = true;
    }

    // Merge the four warps: each leaves its (max, sum, unnormalised output) in shared memory.
    __nv_bfloat16* idle_stage = stages + ((consumed + STAGES - 1) % STAGES) * Tiles::STAGE;   // the stage read last
    // [4][16][D]: exactly one stage of the TMA form; columns swizzled by row (merge_swizzle)
    float* merge_o = reinterpret_cast<float*>(idle_stage);
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (h == 1 && upper_rows_unused) continue;   // nothing reads rows 8..15 of the merge buffers then
      float sum = row_sum[h];
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      const int r = g + 8 * h;
      if (tq == 0) {
        merge_max[warp * SMALL_ROWS + r] = row_max[h];
        merge_sum[warp * SMALL_ROWS + r] = sum;
      }
      float* dst = merge_o + ((size_t)warp * SMALL_ROWS + r) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(dst + ((i * 8 + 2 * tq) ^ merge_swizzle(r))) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
    }
    __syncthreads();
    // Per row, once: the warps' weights 2^(max_w - max) over the total, and the log-sum-exp.
    if (threadIdx.x < packed_rows) {
      const int r = threadIdx.x;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mx = fmaxf(mx, merge_max[w * SMALL_ROWS + r]);
      float weight[4], total = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float m = merge_max[w * SMALL_ROWS + r];
        weight[w] = m == -INFINITY ? 0.f : fast_exp2((m - mx) * p.scale_log2);
        total += weight[w] * merge_sum[w * SMALL_ROWS + r];
      }
      const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) merge_max[w * SMALL_ROWS + r] = weight[w] * inv;   // from here on: the warp's share
      row_lse[r] = total > 0.f ? mx * p.scale_log2 + log2f(total) : -INFINITY;     // the segment's log-sum-exp (log2)
    }
    __syncthreads();
    const size_t slot = (size_t)pair + blockIdx.x;
    if (CLUSTER) {
      // The block's normalised result goes to the start of the stages, where the other blocks of the cluster find it:
      // first into registers, since the merge buffers may lie in the same place.
      float mine[SMALL_ROWS * D / ATT_THREADS];
#pragma unroll
      for (int i = 0; i < SMALL_ROWS * D / ATT_THREADS; ++i) {
        const int e = threadIdx.x + i * ATT_THREADS, r = e / D, col = e % D;
        mine[i] = 0.f;
        if (e < packed_rows * D) {
#pragma unroll
          for (int w = 0; w < 4; ++w) mine[i] += merge_max[w * SMALL_ROWS + r] * merge_o[((size_t)w * SMALL_ROWS + r) * D + (col ^ merge_swizzle(r))];
        }
      }
      cluster_wait();   // every block of the cluster has started
      // Element e of the pair's result belongs to the block that adds up slice e / slice_length.
      const int slice_length = (packed_rows * D + CLUSTER - 1) / (CLUSTER ? CLUSTER : 1), slice_stride = (p.incoming_rows * D + CLUSTER - 1) / (CLUSTER ? CLUSTER : 1);
#pragma unroll
      for (int i = 0; i < SMALL_ROWS * D / ATT_THREADS; ++i) {
        const int e = threadIdx.x + i * ATT_THREADS;
        if (e < packed_rows * D) cluster_store(cluster_address(incoming + cluster_rank * slice_stride + e % slice_length, e / slice_length), mine[i]);
      }
      for (int x = threadIdx.x; x < CLUSTER * SMALL_ROWS; x += ATT_THREADS) {
        const int r = x % SMALL_ROWS;
        if (r < packed_rows)
          cluster_store(cluster_address(incoming + (CLUSTER ? CLUSTER : 1) * slice_stride + cluster_rank * SMALL_ROWS + r, x / SMALL_ROWS), row_lse[r]);
      }
    }
    for (int e = threadIdx.x; !CLUSTER && e < packed_rows * D; e += ATT_THREADS) {
      const int r = e / D, col = e % D;
      float value = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) value += merge_max[w * SMALL_ROWS + r] * merge_o[((size_t)w * SMALL_ROWS + r) * D + (col ^ merge_swizzle(r))];
      if (segments == 1) {
        const size_t token = (size_t)q0 + r / G;
        const int head = kv_head * G + r % G;
        p.out[(token * p.nq + head) * D + col] = __float2bfloat16_rn(value);
      } else {
        p.decode_out[(slot * SMALL_ROWS + r) * D + col] = value;
        if (col == 0) p.decode_lse[slot * SMALL_ROWS + r] = row_lse[r];
      }
    }

    if (!CLUSTER && segments > 1) {
      if (threadIdx.x == 0) {
        int* entry = pending[pending_count];
        entry[0] = pair; entry[1] = first_block; entry[2] = segments; entry[3] = q0; entry[4] = packed_rows; entry[5] = kv_head;
      }
      if (++pending_count == DEC_PENDING) publish_and_combine();
    }
    if (TMA) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the merge buffers were written where TMA writes next
    __syncthreads();   // the query tile and the stages are free for the next segment
    current = following;
    have = have_following;
  }
  if (!CLUSTER) {
    if (!waited) grid_dependency_wait();   // a block without a segment: no grid ends before the grid ahead of it has
    publish_and_combine();
    return;
  }

  // The cluster's blocks combine their results: each block the slice of the (packed row, value) elements that the others
  // sent it.
  constexpr int SIZE = CLUSTER ? CLUSTER : 1;
  {
    const int cluster_row = cluster_pair / p.nkv;
    const int q0 = p.q_start[cluster_row];
    const int packed_rows = (p.q_start[cluster_row + 1] - q0) * G;
    const int kv_head = cluster_pair % p.nkv;
    const int slice_length = (packed_rows * D + SIZE - 1) / SIZE, slice_stride = (p.incoming_rows * D + SIZE - 1) / SIZE;
    float* incoming_lse = incoming + SIZE * slice_stride;
    if (!had_tiles) {
      // no tiles for this block: nothing visible in its share, and nothing sent but that
      cluster_wait();   // every block of the cluster has started
      for (int x = threadIdx.x; x < SIZE * SMALL_ROWS; x += ATT_THREADS)
        if (x % SMALL_ROWS < packed_rows) cluster_store(cluster_address(incoming_lse + cluster_rank * SMALL_ROWS + x % SMALL_ROWS, x / SMALL_ROWS), -INFINITY);
    }
    if (!waited) {   // only a block without tiles comes here without having waited
      grid_dependency_wait();
      allow_dependents();
    }
    cluster_barrier();   // what every block sent is there
    for (int x = threadIdx.x; x < slice_length && cluster_rank * slice_length + x < packed_rows * D; x += ATT_THREADS) {
      const int e = cluster_rank * slice_length + x, r = e / D, col = e % D;
      float lse[SIZE], part[SIZE];
#pragma unroll
      for (int c = 0; c < SIZE; ++c) {
        lse[c] = incoming_lse[c * SMALL_ROWS + r];
        part[c] = incoming[c * slice_stride + x];
      }
      float top = -INFINITY;
#pragma unroll
      for (int c = 0; c < SIZE; ++c) top = fmaxf(top, lse[c]);
      float sum = 0.f, total = 0.f;
#pragma unroll
      for (int c = 0; c < SIZE; ++c) {
        if (lse[c] == -INFINITY) continue;   // a block without visible keys: whatever lies in its place does not count
        const float weight = fast_exp2(lse[c] - top);
        sum += weight * part[c];
        total += weight;
      }
      const size_t token = (size_t)q0 + r / G;
      const int head = kv_head * G + r % G;
      p.out[(token * p.nq + head) * D + col] = __float2bfloat16_rn(total > 0.f ? sum / total : 0.f);
    }
  }
}

// out[token, head] = sum_s w_s partial[s] / sum_s w_s with w_s = 2^(lse_s - max lse).  One
// warp per (token, head).
// skip_small: tokens of rows with at most SMALL_ROWS packed query rows are left alone (the decode
// kernel wrote them).
__global__ void combine_splits_kernel(const float* __restrict__ partial_out, const float* __restrict__ partial_lse,
                                      __nv_bfloat16* __restrict__ out, int num_splits, long long items, const int* __restrict__ q_start,
                                      int num_rows, int nq, int group, int skip_small) {
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  if (skip_small) {
    const int token = (int)(item / nq);
    int lo = 0, hi = num_rows - 1;   // the last row that starts at or before the token
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (q_start[mid] <= token) lo = mid; else hi = mid - 1;
    }
    if ((q_start[lo + 1] - q_start[lo]) * group <= SMALL_ROWS) return;
  }
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, partial_lse[(size_t)s * items + item]);
  float acc[(D + 31) / 32];
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) acc[i] = 0.f;
  float total = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float lse = partial_lse[(size_t)s * items + item];
    if (lse == -INFINITY) continue;
    const float w = exp2f(lse - mx);
    total += w;
    const float* src = partial_out + ((size_t)s * items + item) * D;
#pragma unroll
    for (int i = 0; i < (D + 31) / 32; ++i) {
      const int e = lane + 32 * i;
      if (e < D) acc[i] += w * src[e];
    }
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
  for (int i = 0; i < (D + 31) / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < D) out[(size_t)item * D + e] = __float2bfloat16_rn(acc[i] * inv);
  }
}

constexpr size_t ATT_SMEM_1 = (size_t)(64 * LD + 4 * TILE_ELEMS) * sizeof(__nv_bfloat16);
constexpr size_t ATT_SMEM_2 = (size_t)(128 * LD + 4 * TILE_ELEMS) * sizeof(__nv_bfloat16);
constexpr bool WIDE_TILES = D <= 128;   // two MMA tiles per warp keep their accumulators in registers up to this head size

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_attention_head_dim() { return D; }

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &result) != cudaSuccess || result != cudaDriverEntryPointSuccess)
      symbol = nullptr;
    return (EncodeTiled)symbol;
  }();
  return fn;
}

// Tensor map of a page pool [pages, KV heads, page size, D] seen as a matrix of rows of D values, boxes of 64 rows x 64
// values in the 128-byte swizzle.  The last few maps are kept: a model asks for the same pools at every step.
static bool page_pool_map(CUtensorMap* map, const void* pages, long long rows) {
  struct Known { const void* pages; long long rows; CUtensorMap map; };
  static Known known[64];
  static int count = 0, next = 0;
  static std::mutex mutex;
  std::lock_guard<std::mutex> guard(mutex);
  for (int i = 0; i < count; ++i)
    if (known[i].pages == pages && known[i].rows == rows) { *map = known[i].map; return true; }
  EncodeTiled encode = encode_tiled();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)D * sizeof(__nv_bfloat16)};
  cuuint32_t box[2] = {64, (cuuint32_t)BLOCK_N};
  cuuint32_t element_strides[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  known[next].pages = pages; known[next].rows = rows; known[next].map = *map;
  next = (next + 1) % 64;
  if (count < 64) ++count;
  return true;
}

constexpr size_t DEC_SMEM_TMA = DecodeTiles<TMA_HEAD>::SMEM, DEC_SMEM_GATHER = DecodeTiles<false>::SMEM;
// The cluster form: its stages and query tile, then what the other blocks of the cluster send (partial results of
// `rows` packed query rows in all, and every block's log-sum-exps).
constexpr size_t DEC_SMEM_CLUSTER_BASE = DecodeTiles<TMA_HEAD, DEC_CLUSTER_STAGES>::SMEM;
constexpr size_t DEC_SMEM_LONE_BASE = DecodeTiles<TMA_HEAD, DEC_LONE_STAGES>::SMEM;
constexpr size_t dec_smem_cluster(int rows, int cluster, bool lone = false) {
  return (lone ? DEC_SMEM_LONE_BASE : DEC_SMEM_CLUSTER_BASE) + ((size_t)rows * D + cluster + (size_t)cluster * SMALL_ROWS) * sizeof(float);
}
constexpr size_t DEC_SMEM_CLUSTER = dec_smem_cluster(SMALL_ROWS, 16);   // the most
static bool clusters_of_16() {
  static const bool allowed = [] {
    if (!TMA_HEAD) return false;
    auto kernel = paged_attention_decode_kernel<TMA_HEAD, TMA_HEAD ? 16 : 0>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) { cudaGetLastError(); return false; }
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_CLUSTER) != cudaSuccess) { cudaGetLastError(); return false; }
    // does the device place such a cluster at all?
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(16); config.blockDim = dim3(ATT_THREADS); config.dynamicSmemBytes = DEC_SMEM_CLUSTER;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 16; attribute[0].val.clusterDim.y = 1; attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute; config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) { cudaGetLastError(); return false; }
    return clusters >= 1;
  }();
  return allowed;
}
constexpr size_t DEC_SMEM_MOST = DEC_SMEM_TMA > DEC_SMEM_GATHER ? DEC_SMEM_TMA : DEC_SMEM_GATHER;

// Clusters of 16 blocks are beyond the portable size: the kernel has to opt in, and the device may refuse.
static bool clusters_of_16();

static int decode_sm_count() {
  static int counts[pylon::MAX_DEVICES] = {};
  int& count = counts[pylon::current_device_slot()];
  if (count == 0) {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) value = 0;
    count = value;
  }
  return count;
}

// Blocks of the decode kernel: as many as are resident at once, of the form that needs more
// shared memory.
extern "C" int pylon_attention_decode_blocks() {
  static int resident_on[pylon::MAX_DEVICES] = {};
  int& resident = resident_on[pylon::current_device_slot()];
  if (resident == 0) {
    int device = 0, sm_count = 0, per_sm = 0, per_sm_tma = 0;
    if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return -1;
    if (cudaFuncSetAttribute(paged_attention_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_GATHER) != cudaSuccess) return -1;
    if (cudaFuncSetAttribute(paged_attention_decode_kernel<TMA_HEAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_TMA) != cudaSuccess) return -1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, paged_attention_decode_kernel<false>, ATT_THREADS, DEC_SMEM_GATHER) != cudaSuccess || per_sm < 1) return -1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_tma, paged_attention_decode_kernel<TMA_HEAD>, ATT_THREADS, DEC_SMEM_TMA) != cudaSuccess || per_sm_tma < 1) return -1;
    resident = (per_sm_tma < per_sm ? per_sm_tma : per_sm) * sm_count;
  }
  return resident;
}

// Scratch floats a call needs: `num_splits` splits of the tiled kernel over `total_tokens`
// tokens (none for one split) and the decode kernel's segment slots (none for decode_blocks = 0).
extern "C" long long pylon_attention_scratch_floats(int num_splits, int total_tokens, int nq, int num_rows, int nkv, int decode_blocks) {
  long long floats = 0;
  if (num_splits > 1) floats += (long long)num_splits * total_tokens * nq * (D + 1);
  if (decode_blocks > 0) floats += ((long long)num_rows * nkv + decode_blocks) * SMALL_ROWS * (D + 1);
  return floats;
}

// q: bfloat16 [tokens, >= nq*D] with q_stride elements between tokens; pages: bfloat16
// [num_pages, nkv, page_size, D]; out: bfloat16 [tokens, nq, D]; q_start: int32 [rows + 1];
// kv_len: int32 [rows]; block_table: int32 [rows, table_width]; max_q: the longest row (or an
// upper bound); num_splits: key/value splits of rows with more than 16 packed query rows;
// decode_blocks: blocks of the kernel for the other rows (1 .. pylon_attention_decode_blocks()); 0 with several rows: the caller knows that
// none of them is that short, and the tiled kernel takes them all;
// scratch: float32, pylon_attention_scratch_floats() long, contents arbitrary; counters:
// num_rows * nkv unsigned integers that are zero before the call (and zero again after it).
// scratch and counters may be null when num_splits = 1 and no row can have 16 packed rows or fewer
// (one row and max_q * group > 16).  error: null, or one int in device memory that a kernel sets
// non-zero when its bounded wait for a TMA copy ran out (the output is then void).  skip_large != 0: rows with
// more than 16 packed query rows are left alone (another kernel writes them).  rows_alike != 0: the caller knows that
// the rows of decoded tokens hold about equally many keys; with few of them, each (row, KV head) pair then gets a
// thread-block cluster of its own (with rows of very different lengths that would leave most blocks idle: the result is
// right either way).
extern "C" int pylon_paged_attention_mma(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                         void* out, float* scratch, unsigned* counters, const int* q_start, const int* kv_len,
                                         const int* block_table, int table_width, int page_size, int num_pages,
                                         int nq, int nkv, int window, float scale, int num_rows, int total_tokens,
                                         int max_q, int num_splits, int decode_blocks, int skip_large, int rows_alike, int* error,
                                         cudaStream_t stream) {
  if (num_rows <= 0 || total_tokens <= 0) return 0;
  if (nkv < 1 || nq < 1 || nq % nkv) PYLON_REFUSE("paged_attention_mma: %d query heads over %d KV heads", nq, nkv);
  if (page_size < 1 || table_width < 1 || window < 0 || max_q < 1 || num_splits < 1)
    PYLON_REFUSE("paged_attention_mma: page size %d, table width %d, window %d, longest row %d, splits %d", page_size,
                 table_width, window, max_q, num_splits);
  if (((uintptr_t)q % 16) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || ((uintptr_t)out % 8) || (q_stride % 8))
    PYLON_REFUSE("paged_attention_mma: q and pages must be 16-byte aligned and the token stride a multiple of 8");
  if (!(scale > 0.f)) PYLON_REFUSE("paged_attention_mma: the softmax scale must be positive");
  if (nkv > 65535 || num_rows > 65535) PYLON_REFUSE("paged_attention_mma: %d KV heads, %d rows", nkv, num_rows);
  const int group = nq / nkv;
  const long long packed_max = (long long)max_q * group;
  const bool any_large = packed_max > SMALL_ROWS;
  // A lone large row leaves nothing for the decode kernel; nor does a caller who knows that every row is large and
  // says so by asking for no decode blocks (the tiled kernel then takes every row, whatever its size).
  const bool maybe_small = !any_large || (num_rows > 1 && decode_blocks > 0);
  const bool run_tiled = any_large && !skip_large;
  if (!run_tiled) num_splits = 1;                        // no row for the tiled kernel
  if (num_splits > 1 && scratch == nullptr) PYLON_REFUSE("paged_attention_mma: splits need scratch memory");
  if (maybe_small) {
    const int most = pylon_attention_decode_blocks();
    if (most < 1) PYLON_REFUSE("paged_attention_mma: the decode kernel does not fit on this device");
    if (decode_blocks < 1 || decode_blocks > most) PYLON_REFUSE("paged_attention_mma: %d decode blocks, 1 to %d are possible", decode_blocks, most);
    if (scratch == nullptr || counters == nullptr) PYLON_REFUSE("paged_attention_mma: rows of decoded tokens need scratch memory and counters");
  }
  static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(paged_attention_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_SMEM_1);
    if (err == cudaSuccess && WIDE_TILES)
      err = cudaFuncSetAttribute(paged_attention_mma_kernel<WIDE_TILES ? 2 : 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_SMEM_2);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(paged_attention_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_GATHER);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(paged_attention_decode_kernel<TMA_HEAD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_TMA);
#define PYLON_CLUSTER_CASE(N)                                                                                                   \
    if (err == cudaSuccess && TMA_HEAD)                                                                                         \
      err = cudaFuncSetAttribute(paged_attention_decode_kernel<TMA_HEAD, TMA_HEAD ? N : 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM_CLUSTER);
    PYLON_CLUSTER_CASE(16) PYLON_CLUSTER_CASE(8) PYLON_CLUSTER_CASE(6) PYLON_CLUSTER_CASE(4) PYLON_CLUSTER_CASE(3) PYLON_CLUSTER_CASE(2)
#undef PYLON_CLUSTER_CASE
    if (err == cudaSuccess && TMA_HEAD && dec_smem_cluster(SMALL_ROWS, 16, true) <= 227 * 1024 && clusters_of_16()) {
      auto lone = paged_attention_decode_kernel<TMA_HEAD, TMA_HEAD ? 16 : 0, DEC_LONE_STAGES>;
      err = cudaFuncSetAttribute(lone, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (err == cudaSuccess) err = cudaFuncSetAttribute(lone, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dec_smem_cluster(SMALL_ROWS, 16, true));
    }
    if (err != cudaSuccess) PYLON_REFUSE("paged_attention_mma: %s", cudaGetErrorString(err));
    configured = true;
  }
  AttentionParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
  p.out = (__nv_bfloat16*)out;
  const long long items = (long long)total_tokens * nq;
  float* decode_scratch = scratch;
  p.partial_out = p.partial_lse = nullptr;
  if (num_splits > 1) {
    p.partial_out = scratch;
    p.partial_lse = scratch + (size_t)num_splits * items * D;
    decode_scratch = scratch + (size_t)num_splits * items * (D + 1);
  }
  const size_t slots = (size_t)num_rows * nkv + (maybe_small ? decode_blocks : 0);
  p.decode_out = decode_scratch;
  p.decode_lse = decode_scratch ? decode_scratch + slots * SMALL_ROWS * D : nullptr;
  p.counters = counters;
  p.error = error;
  p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.nq = nq; p.nkv = nkv; p.group = group; p.window = window; p.num_splits = num_splits; p.total_tokens = total_tokens;
  p.num_rows = num_rows;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.small_rows_elsewhere = maybe_small ? 1 : 0;
  p.incoming_rows = (int)(packed_max < SMALL_ROWS ? packed_max : SMALL_ROWS);
  if (run_tiled) {
    // 128-row blocks when the rows are long enough to fill them and the accumulators fit.
    const bool wide = WIDE_TILES && packed_max >= 256;
    const int block_rows = wide ? 128 : 64;
    const long long q_tiles = (packed_max + block_rows - 1) / block_rows;
    if (q_tiles * num_splits > 2147483647LL) PYLON_REFUSE("paged_attention_mma: too many query tiles");
    dim3 grid((unsigned)(q_tiles * num_splits), nkv, num_rows);
    if (wide)
      paged_attention_mma_kernel<WIDE_TILES ? 2 : 1><<<grid, ATT_THREADS, ATT_SMEM_2, stream>>>(p);
    else
      paged_attention_mma_kernel<1><<<grid, ATT_THREADS, ATT_SMEM_1, stream>>>(p);
  }
  if (maybe_small) {
    CUtensorMap map_k = {}, map_v = {};
    const long long pool_rows = (long long)num_pages * nkv * page_size;
    const bool tma = TMA_HEAD && page_size % BLOCK_N == 0 && pool_rows < 2147483647LL - BLOCK_N;
    if (tma) {
      if (!page_pool_map(&map_k, k_pages, pool_rows) || !page_pool_map(&map_v, v_pages, pool_rows))
        PYLON_REFUSE("paged_attention_mma: the tensor maps of the page pools could not be made");
      // Few pairs of about equal length: a cluster of blocks for each (16 where the device places such clusters), as large as leaves two blocks to an SM (with three,
      // clusters measured slower than the runs: 3.23 against 2.97 ms a step at batch 8) and within the caller's blocks.
      const long long pairs = (long long)num_rows * nkv;
      int size = 0;
      if (TMA_HEAD && rows_alike) {
        const long long room = 2LL * decode_sm_count() / pairs;
        size = (room >= 16 && clusters_of_16()) ? 16 : room >= 8 ? 8 : room >= 6 ? 6 : room >= 4 ? 4 : room >= 3 ? 3 : room >= 2 ? 2 : 0;
        if (pairs * size > decode_blocks) size = 0;
      }
#define PYLON_CLUSTER_CASE(N)                                                                                                   \
      if (size == N) launch_dependent_cluster(paged_attention_decode_kernel<TMA_HEAD, TMA_HEAD ? N : 0>, dim3((unsigned)(pairs * N)), dim3(ATT_THREADS), dec_smem_cluster(p.incoming_rows, N), \
                                              stream, N, p, map_k, map_v);
      if (size == 16 && pairs * 16 <= decode_sm_count() && dec_smem_cluster(SMALL_ROWS, 16, true) <= 227 * 1024) {   // every block an SM to itself
        launch_dependent_cluster(paged_attention_decode_kernel<TMA_HEAD, TMA_HEAD ? 16 : 0, DEC_LONE_STAGES>, dim3((unsigned)(pairs * 16)), dim3(ATT_THREADS),
                                 dec_smem_cluster(p.incoming_rows, 16, true), stream, 16, p, map_k, map_v);
        size = -1;
      }
      PYLON_CLUSTER_CASE(16) PYLON_CLUSTER_CASE(8) PYLON_CLUSTER_CASE(6) PYLON_CLUSTER_CASE(4) PYLON_CLUSTER_CASE(3) PYLON_CLUSTER_CASE(2)
#undef PYLON_CLUSTER_CASE
      if (size == 0)
        launch_dependent(paged_attention_decode_kernel<TMA_HEAD>, dim3(decode_blocks), dim3(ATT_THREADS), DEC_SMEM_TMA, stream, p, map_k, map_v);
    } else {
      launch_dependent(paged_attention_decode_kernel<false>, dim3(decode_blocks), dim3(ATT_THREADS), DEC_SMEM_GATHER, stream, p, map_k, map_v);
    }
  }
  if (num_splits > 1) {
    const int warps = 4;
    launch_dependent(combine_splits_kernel, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream,
                     (const float*)p.partial_out, (const float*)p.partial_lse, p.out, num_splits, items, q_start, num_rows, nq, group,
                     maybe_small ? 1 : 0);
  }
  PYLON_CHECK_LAUNCH("paged_attention_mma");
}
