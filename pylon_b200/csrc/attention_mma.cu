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
  float* partial_out;   // [splits, tokens, nq, D]
  float* partial_lse;   // [splits, tokens, nq]   (log2 domain)
  const int* q_start;
  const int* kv_len;
  const int* block_table;
  int table_width, page_size, num_pages, nq, nkv, group, window, num_splits, total_tokens;
  int small_rows_elsewhere;   // rows of at most SMALL_ROWS packed query rows are left to the decode kernel
  unsigned* counters;         // [rows * nkv], zero between launches: lets the last split of a decode row combine the splits itself
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
constexpr int DEC_STAGE_ELEMS = 2 * TILE_ELEMS;   // keys then values
constexpr size_t DEC_SMEM = (size_t)(SMALL_ROWS * LD + DEC_STAGES * DEC_STAGE_ELEMS) * sizeof(__nv_bfloat16);
static_assert(DEC_STAGES * DEC_STAGE_ELEMS * sizeof(__nv_bfloat16) >= 4 * SMALL_ROWS * (D + 2) * sizeof(float), "merge buffers reuse the tile stages");

__global__ void __launch_bounds__(ATT_THREADS) paged_attention_decode_kernel(const AttentionParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][LD]
  __nv_bfloat16* stages = q_tile + SMALL_ROWS * LD;                      // [DEC_STAGES][2][64][LD]

  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int row = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
  const int q0 = p.q_start[row];
  const int q_len = p.q_start[row + 1] - q0;
  const int G = p.group;
  const int packed_rows = q_len * G;
  if (packed_rows <= 0 || packed_rows > SMALL_ROWS) return;   // larger rows belong to the tiled kernel
  const int kv_len = p.kv_len[row];
  const int pos0 = kv_len - q_len;
  const int* table = p.block_table + (size_t)row * p.table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;

  const int hi = pos0 + q_len - 1;
  const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int first_tile = lo / BLOCK_N, tiles = hi / BLOCK_N - first_tile + 1;
  const int per_split = (tiles + p.num_splits - 1) / p.num_splits;
  const int tile_begin = first_tile + split * per_split;
  const int tile_end = min(first_tile + tiles, tile_begin + per_split);
  const bool contiguous = p.page_size % BLOCK_N == 0;

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
    if (tile < tile_end) {
      __nv_bfloat16* dst = stages + ((tile - tile_begin) % DEC_STAGES) * DEC_STAGE_ELEMS;
      if (contiguous) {
        load_kv_tile_contiguous(dst, p.k_pages, table, tile, kv_len, kv_head, p);
        load_kv_tile_contiguous(dst + TILE_ELEMS, p.v_pages, table, tile, kv_len, kv_head, p);
      } else {
        load_kv_tile(dst, p.k_pages, table, tile, kv_len, kv_head, p);
        load_kv_tile(dst + TILE_ELEMS, p.v_pages, table, tile, kv_len, kv_head, p);
      }
    }
    cp_async_commit();   // an empty group keeps the count of groups in step with the tiles
  };

  if (tile_begin < tile_end) {
    for (int c = threadIdx.x; c < SMALL_ROWS * CHUNKS; c += ATT_THREADS) {
      const int r = c / CHUNKS, col = c % CHUNKS;
      const bool valid = r < packed_rows;
      const __nv_bfloat16* src = p.q;
      if (valid) src = p.q + (size_t)(q0 + r / G) * p.q_stride + (size_t)(kv_head * G + r % G) * D + col * 8;
      cp_async_16(q_tile + r * LD + col * 8, src, valid);
    }
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; ++s) issue(tile_begin + s);

    const bool upper_rows_unused = packed_rows <= 8;
    // The query fragments stay in registers when the head is small enough to leave room.
    constexpr bool Q_IN_REGISTERS = D <= 128;
    unsigned q_frag[Q_IN_REGISTERS ? D / 16 : 1][4];
    bool q_loaded = false;

    for (int tile = tile_begin; tile < tile_end; ++tile) {
      issue(tile + DEC_STAGES - 1);
      cp_async_wait<DEC_STAGES - 1>();
      __syncthreads();
      const __nv_bfloat16* ks = stages + ((tile - tile_begin) % DEC_STAGES) * DEC_STAGE_ELEMS + warp * 16 * LD;
      const __nv_bfloat16* vs = ks + TILE_ELEMS;
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
        ldmatrix_x4(b, ks + ((lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
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
        ldmatrix_x4_trans(b, vs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + d2 * 16 + 8 * (lane >> 4));
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      }
      __syncthreads();   // everyone is done with this stage before it is loaded again
    }
    cp_async_wait<0>();
  }

  // Merge the four warps: each leaves its (max, sum, unnormalised output) in shared memory.
  float* merge_o = reinterpret_cast<float*>(stages);                 // [4][16][D]
  float* merge_max = merge_o + 4 * SMALL_ROWS * D;                   // [4][16]
  float* merge_sum = merge_max + 4 * SMALL_ROWS;                     // [4][16]
  __syncthreads();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
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
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8 + 2 * tq) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < packed_rows * D; e += ATT_THREADS) {
    const int r = e / D, col = e % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, merge_max[w * SMALL_ROWS + r]);
    float total = 0.f, value = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float m = merge_max[w * SMALL_ROWS + r];
      const float weight = m == -INFINITY ? 0.f : exp2f((m - mx) * p.scale_log2);
      total += weight * merge_sum[w * SMALL_ROWS + r];
      value += weight * merge_o[((size_t)w * SMALL_ROWS + r) * D + col];
    }
    const float inv = total > 0.f ? 1.f / total : 0.f;
    const size_t token = (size_t)q0 + r / G;
    const int head = kv_head * G + r % G;
    if (p.num_splits == 1) {
      p.out[(token * p.nq + head) * D + col] = __float2bfloat16_rn(value * inv);
    } else {
      const size_t slot = ((size_t)split * p.total_tokens + token) * p.nq + head;
      p.partial_out[slot * D + col] = value * inv;
      if (col == 0) p.partial_lse[slot] = total > 0.f ? mx * p.scale_log2 + log2f(total) : -INFINITY;
    }
  }

  if (p.num_splits > 1 && p.counters != nullptr) {
    // The split that finishes last for this (row, KV head) combines all of them; the others
    // have published their partial results (fence, then the counter).
    __shared__ bool last_split;
    __threadfence();
    __syncthreads();
    unsigned* counter = p.counters + (size_t)row * p.nkv + kv_head;
    if (threadIdx.x == 0) last_split = atomicAdd(counter, 1u) == (unsigned)p.num_splits - 1u;
    __syncthreads();
    if (!last_split) return;
    __threadfence();
    const size_t items = (size_t)p.total_tokens * p.nq;
    // The splits' weights first (one trip to L2 for all of them), then the weighted sum with
    // several partial results in flight per thread.
    float* weights = reinterpret_cast<float*>(stages);   // [SMALL_ROWS][splits]; the stages are idle now
    __shared__ float row_total[SMALL_ROWS];
    const int splits = p.num_splits;
    __syncthreads();
    for (int e = threadIdx.x; e < packed_rows * splits; e += ATT_THREADS) {
      const int r = e / splits, s2 = e % splits;
      const size_t item = ((size_t)q0 + r / G) * p.nq + kv_head * G + r % G;
      weights[r * splits + s2] = __ldcg(p.partial_lse + (size_t)s2 * items + item);
    }
    __syncthreads();
    if (threadIdx.x < packed_rows) {
      const int r = threadIdx.x;
      float mx = -INFINITY;
      for (int s2 = 0; s2 < splits; ++s2) mx = fmaxf(mx, weights[r * splits + s2]);
      float total = 0.f;
      for (int s2 = 0; s2 < splits; ++s2) {
        const float lse = weights[r * splits + s2];
        const float weight = lse == -INFINITY ? 0.f : exp2f(lse - mx);
        weights[r * splits + s2] = weight;
        total += weight;
      }
      row_total[r] = total;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < packed_rows * D; e += ATT_THREADS) {
      const int r = e / D, col = e % D;
      const size_t item = ((size_t)q0 + r / G) * p.nq + kv_head * G + r % G;
      const float* src = p.partial_out + item * D + col;
      float value = 0.f;
      int s2 = 0;
      for (; s2 + 4 <= splits; s2 += 4) {
        const float v0 = __ldcg(src + (size_t)(s2 + 0) * items * D), v1 = __ldcg(src + (size_t)(s2 + 1) * items * D);
        const float v2 = __ldcg(src + (size_t)(s2 + 2) * items * D), v3 = __ldcg(src + (size_t)(s2 + 3) * items * D);
        value += weights[r * splits + s2] * v0 + weights[r * splits + s2 + 1] * v1 + weights[r * splits + s2 + 2] * v2 + weights[r * splits + s2 + 3] * v3;
      }
      for (; s2 < splits; ++s2) value += weights[r * splits + s2] * __ldcg(src + (size_t)s2 * items * D);
      const float total = row_total[r];
      p.out[item * D + col] = __float2bfloat16_rn(total > 0.f ? value / total : 0.f);
    }
    if (threadIdx.x == 0) *counter = 0u;   // ready for the next launch
  }
}

// out[token, head] = sum_s w_s partial[s] / sum_s w_s with w_s = 2^(lse_s - max lse).  One
// warp per (token, head).
__global__ void combine_splits_kernel(const float* __restrict__ partial_out, const float* __restrict__ partial_lse,
                                      __nv_bfloat16* __restrict__ out, int num_splits, long long items) {
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
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

// Scratch floats needed for `num_splits` splits over `total_tokens` tokens (0 for one split).
extern "C" long long pylon_attention_scratch_floats(int num_splits, int total_tokens, int nq) {
  if (num_splits <= 1) return 0;
  return (long long)num_splits * total_tokens * nq * (D + 1);
}

// q: bfloat16 [tokens, >= nq*D] with q_stride elements between tokens; pages: bfloat16
// [num_pages, nkv, page_size, D]; out: bfloat16 [tokens, nq, D]; q_start: int32 [rows + 1];
// kv_len: int32 [rows]; block_table: int32 [rows, table_width]; max_q: the longest row (or an
// upper bound); scratch: float32, pylon_attention_scratch_floats() long when num_splits > 1;
// counters: null, or num_rows * nkv unsigned integers that are zero before the call (and zero
// again after it): with them the splits of decoded rows are combined inside the attention
// kernel instead of by a second launch.
extern "C" int pylon_paged_attention_mma(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                         void* out, float* scratch, unsigned* counters, const int* q_start, const int* kv_len,
                                         const int* block_table, int table_width, int page_size, int num_pages,
                                         int nq, int nkv, int window, float scale, int num_rows, int total_tokens,
                                         int max_q, int num_splits, cudaStream_t stream) {
  if (num_rows <= 0 || total_tokens <= 0) return 0;
  if (nkv < 1 || nq < 1 || nq % nkv) PYLON_REFUSE("paged_attention_mma: %d query heads over %d KV heads", nq, nkv);
  if (page_size < 1 || table_width < 1 || window < 0 || max_q < 1 || num_splits < 1)
    PYLON_REFUSE("paged_attention_mma: page size %d, table width %d, window %d, longest row %d, splits %d", page_size,
                 table_width, window, max_q, num_splits);
  if (((uintptr_t)q % 16) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || ((uintptr_t)out % 4) || (q_stride % 8))
    PYLON_REFUSE("paged_attention_mma: q and pages must be 16-byte aligned and the token stride a multiple of 8");
  if (!(scale > 0.f)) PYLON_REFUSE("paged_attention_mma: the softmax scale must be positive");
  if (num_splits > 1 && scratch == nullptr) PYLON_REFUSE("paged_attention_mma: splits need scratch memory");
  if (nkv > 65535 || num_rows > 65535) PYLON_REFUSE("paged_attention_mma: %d KV heads, %d rows", nkv, num_rows);
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(paged_attention_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_SMEM_1);
    if (err == cudaSuccess && WIDE_TILES)
      err = cudaFuncSetAttribute(paged_attention_mma_kernel<WIDE_TILES ? 2 : 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_SMEM_2);
    if (err == cudaSuccess) err = cudaFuncSetAttribute(paged_attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DEC_SMEM);
    if (err != cudaSuccess) PYLON_REFUSE("paged_attention_mma: %s", cudaGetErrorString(err));
    configured = true;
  }
  AttentionParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.k_pages = (const __nv_bfloat16*)k_pages; p.v_pages = (const __nv_bfloat16*)v_pages;
  p.out = (__nv_bfloat16*)out;
  const long long items = (long long)total_tokens * nq;
  p.partial_out = scratch; p.partial_lse = scratch ? scratch + (size_t)num_splits * items * D : nullptr;
  p.counters = counters;
  p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.nq = nq; p.nkv = nkv; p.group = nq / nkv; p.window = window; p.num_splits = num_splits; p.total_tokens = total_tokens;
  p.scale_log2 = scale * 1.4426950408889634f;
  const long long packed_max = (long long)max_q * p.group;
  const bool any_large = packed_max > SMALL_ROWS;
  const bool maybe_small = !any_large || num_rows > 1;   // a lone large row leaves nothing for the decode kernel
  p.small_rows_elsewhere = maybe_small ? 1 : 0;
  if (any_large) {
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
    dim3 grid(num_splits, nkv, num_rows);
    launch_dependent(paged_attention_decode_kernel, grid, dim3(ATT_THREADS), DEC_SMEM, stream, p);
  }
  if (num_splits > 1 && (any_large || counters == nullptr)) {
    const int warps = 4;
    launch_dependent(combine_splits_kernel, dim3((unsigned)((items + warps - 1) / warps)), dim3(warps * 32), 0, stream,
                     (const float*)p.partial_out, (const float*)p.partial_lse, p.out, num_splits, items);
  }
  PYLON_CHECK_LAUNCH("paged_attention_mma");
}
