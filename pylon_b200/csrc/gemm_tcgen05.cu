// C[M, N] = A[M, K] * B[N, K]^T for bfloat16 on the fifth-generation tensor cores: operands
// staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), multiplied by
// tcgen05.mma issued from one thread, accumulated in float32 in tensor memory, read back with
// tcgen05.ld for the epilogue.  For the products of prompt portions (many rows).
//
// One persistent block per SM walks 128 x BN output tiles.  Six warps with fixed roles:
//   warp 0      TMA producer: fills a ring of STAGES shared-memory stages (A 128 x 64, B BN x 64)
//   warp 1      MMA issuer: four tcgen05.mma (K = 16 each) per stage into one of two
//               accumulator buffers in tensor memory; tcgen05.commit frees the stage and, after
//               the last stage of a tile, hands the accumulator to the epilogue
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its quarter of the 128 lanes),
//               convert, lay 32 rows x 32 or 64 columns out in shared memory in the swizzle a
//               TMA store expects and let TMA write them (whole sectors, clipped at the
//               matrix's edge; a lane storing its own row left half-written sectors and cost a
//               fifth of the time); with SWIGLU the columns hold gate and up values in
//               alternating groups of 8 and silu(gate) * up is stored, half as wide
// so the epilogue of one tile overlaps the products of the next.  Tiles wider than 256 columns (288: nine of them
// cover the 2,560 columns of an output or down projection, so that 2,048 rows are 144 tiles, one round over 148 SMs,
// where 160 tiles of 256 columns are a full round and a nearly empty one) take two products per step of k (the tensor
// core's N ends at 256) and have one accumulator buffer, since two would not fit in tensor memory: their epilogue
// does not overlap the next tile.  All waits on mbarriers are
// bounded: a wait that runs out sets an error word for the host and the block winds down
// (frees its tensor memory and returns) instead of hanging.
//
// No TMA load here uses cluster multicast.
//
// Stands in for the library product behind raun6k/Pylon's nn.Linear at prefill
// (src/pylon/model/layers.py:26-27,126,138).
#include "common.cuh"

#include <cuda.h>

namespace pylon {

constexpr int TC_BM = 128, TC_BK = 64, TC_THREADS = 192;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;   // try_wait calls before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// Waits for the phase with the given parity to complete; false if the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t tries = 0; tries < TC_WAIT_LIMIT; ++tries) {
    uint32_t done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// Shared memory -> global through a tensor map; the rows and columns outside the matrix are not written.  The store
// joins the thread's open bulk group: tma_store_commit() closes it.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
               ::"l"((uint64_t)map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// Until all but the newest `Pending` stores of this thread have read their shared memory.
template <int Pending>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(Pending) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive float32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tc_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16)
// in the 128-byte swizzle TMA wrote: start address, 1024 bytes between groups of 8 rows,
// descriptor version 1, swizzle mode 128B.
__device__ __forceinline__ uint64_t tc_smem_desc(const void* tile) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);   // start address, 16-byte units
  desc |= (uint64_t)(1024 >> 4) << 32;                   // stride between 8-row groups
  desc |= (uint64_t)1 << 46;                             // descriptor version (sm_100)
  desc |= (uint64_t)2 << 61;                             // 128-byte swizzle
  return desc;
}

// Instruction descriptor for kind::f16: bfloat16 A and B, float32 D, both K-major, M x N.
__host__ __device__ constexpr uint32_t tc_instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// silu for a bfloat16 result.  The approximate division has no slow path: the exact one takes a subroutine for a zero
// numerator, and the rows of a last, partly filled tile are all zeros (a 1,984-row product took 167 us instead of 146).
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int TC_STAGING_BYTES = 4 * 2 * 32 * 128;   // four epilogue warps x two buffers x 32 rows x up to 128 bytes

template <int BN>
struct TcShared {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
  static constexpr int PIECES = BN > 256 ? 2 : 1;            // products (and boxes of B) per step of k: the tensor core's N and a TMA box end at 256
  static constexpr int PIECE_ROWS = BN / PIECES;
  static constexpr int ACCUMULATORS = 2 * BN <= 512 ? 2 : 1;  // buffers in tensor memory (512 columns)
  static_assert(PIECE_ROWS % 16 == 0 && PIECE_ROWS <= 256 && (PIECE_ROWS * 128) % 1024 == 0, "a piece of B must be a valid N and start on a swizzle group");
  static constexpr int FIT = (227 * 1024 - 1024 /* alignment slack */ - 256 /* barriers */ - TC_STAGING_BYTES) / (A_BYTES + B_BYTES);
  static constexpr int STAGES = FIT > 6 ? 6 : FIT;
  static constexpr size_t BYTES = (size_t)STAGES * (A_BYTES + B_BYTES) + TC_STAGING_BYTES + 1024 + 256;
};

// Columns of the output that one TMA store writes: 64 (128-byte rows, 128-byte swizzle) where the tile's width divides
// into such groups, else 32 (64-byte rows, 64-byte swizzle).  With SWIGLU an output column takes two of the accumulator.
template <int BN, bool SWIGLU>
struct TcStore {
  static constexpr int COLUMNS = BN % (SWIGLU ? 128 : 64) == 0 ? 64 : 32;
  static constexpr int ACCUMULATOR_COLUMNS = COLUMNS * (SWIGLU ? 2 : 1);
  static constexpr int ROW_BYTES = COLUMNS * 2;
  static constexpr uint32_t SWIZZLE_MASK = ROW_BYTES == 128 ? 7 : 3;   // the 16-byte unit index is XORed with these bits of (offset / 128)
  static_assert(BN % ACCUMULATOR_COLUMNS == 0, "the tile's width must divide into whole stores");
};

// What the epilogue of a fused QKV product needs to finish the heads it holds (TC_ROTATE): q and k heads are normalised
// (RMSNorm over the head, when weights are given) and rotated by the tables, q goes to a tensor of its own, k and v into
// their pages at the token's slot.
struct RotateArgs {
  __nv_bfloat16* q_out;            // [M, nq * D], row stride ldq
  long long ldq;
  const float* q_weight;           // [D] or null
  const float* k_weight;
  float eps;
  const float* cos_table;          // [table_positions, D / 2]
  const float* sin_table;
  int table_positions;
  const int* positions;            // [M]
  const int* token_row;            // [M]; negative: a padding token, which belongs to no request
  const int* block_table;          // [rows, table_width]
  int table_width, page_size;
  __nv_bfloat16* k_pages;          // [num_pages, nkv, page_size, D]
  __nv_bfloat16* v_pages;
  int num_pages, nq, nkv;
  int* page_error;                 // set to PYLON_ERROR_BAD_PAGE when a block table names a page that is not there
};
enum TcMode { TC_PLAIN = 0, TC_SWIGLU = 1, TC_ROTATE = 2 };

// The epilogue of a fused QKV product for one warp's 32 token rows (lane = row = lane of tensor memory) and the BN / D
// heads of its tile, head by head, in two turns.  Row-wise: a thread reads its row of the head from tensor memory, sums
// its squares in float32 and lays the row down in the warp's staging rows as bfloat16 (16-byte units XORed with the row,
// so that neither these writes nor the reads along a row meet in a bank).  Then column-wise, row by row: lane l holds the
// columns l * PER.. of the lower half and their rotation partners in the upper half, so the angles of a row are one
// coalesced 128- or 256-byte read, the norm weights sit in registers, and a row leaves as whole sectors, into q or the
// token's slot of its page.  (With the rotation row-wise as well, every thread read its own row of the tables: 32 lines a
// load, which the little L1 that the ring leaves could not hold; a tile's epilogue then took longer than its products.)
template <int BN, int D>
__device__ __forceinline__ void rotate_epilogue(const RotateArgs& rot, uint32_t taddr, unsigned char* staging, int row0, int n0, int M, int lane) {
  constexpr int HALF = D / 2, UNITS = D / 8, ROW_BYTES = D * 2, PER = HALF / 32;   // PER columns of each half to a lane: 2 or 1
  static_assert((D == 64 || D == 128) && BN % D == 0 && 32 * ROW_BYTES <= 2 * 32 * 128, "head size 64 or 128, whole heads in a tile");
  const int t = row0 + lane;
  const bool live = t < M;
  const int pos = live ? rot.positions[t] : 0;
  const int row = live ? rot.token_row[t] : -1;
  long long page_offset = -1;   // elements from the pages' start to this token's slot of KV head 0; negative: nothing is written
  if (row >= 0) {
    const int page = rot.block_table[(size_t)row * rot.table_width + pos / rot.page_size];
    if (page >= 0 && page < rot.num_pages) page_offset = ((long long)page * rot.nkv * rot.page_size + pos % rot.page_size) * D;
    else if (rot.page_error) atomicExch(rot.page_error, PYLON_ERROR_BAD_PAGE);   // always there for a prepared step: else the host is told
  }
  const int table_row = pos < rot.table_positions ? pos : rot.table_positions - 1;   // the host checks the range
  const int heads = rot.nq + 2 * rot.nkv;
  const int column = lane * PER;   // this lane's columns of the lower half in the column-wise turn
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += D) {
    const int head = (n0 + c0) / D;
    if (head >= heads) break;
    const bool is_q = head < rot.nq, is_v = head >= rot.nq + rot.nkv;
    const float* weight = is_v ? nullptr : (is_q ? rot.q_weight : rot.k_weight);
    float sumsq = 0.f;
#pragma unroll 1
    for (int part = 0; part < D / 32; ++part) {
      uint32_t raw[32];
      tc_load_32(taddr + c0 + part * 32, raw);
      if (weight) {
#pragma unroll
        for (int j = 0; j < 32; ++j) sumsq += __uint_as_float(raw[j]) * __uint_as_float(raw[j]);
      }
#pragma unroll
      for (int unit = 0; unit < 4; ++unit) {
        const uint32_t physical = (uint32_t)(part * 4 + unit) ^ (uint32_t)(lane & (UNITS - 1));
        *reinterpret_cast<uint4*>(staging + lane * ROW_BYTES + (physical << 4)) =
            make_uint4(pack2(__uint_as_float(raw[unit * 8]), __uint_as_float(raw[unit * 8 + 1])), pack2(__uint_as_float(raw[unit * 8 + 2]), __uint_as_float(raw[unit * 8 + 3])),
                       pack2(__uint_as_float(raw[unit * 8 + 4]), __uint_as_float(raw[unit * 8 + 5])), pack2(__uint_as_float(raw[unit * 8 + 6]), __uint_as_float(raw[unit * 8 + 7])));
      }
    }
    const float inv = weight ? rsqrtf(sumsq / (float)D + rot.eps) : 1.f;
    float w_lower[PER], w_upper[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      w_lower[i] = weight ? weight[column + i] : 1.f;
      w_upper[i] = weight ? weight[HALF + column + i] : 1.f;
    }
    __syncwarp();
    const int kv_head = is_q ? 0 : (head - rot.nq) % rot.nkv;
    __nv_bfloat16* pages = is_v ? rot.v_pages : rot.k_pages;
    const uint32_t lower_byte = (uint32_t)column * 2, upper_byte = (uint32_t)(HALF + column) * 2;
    // Eight rows at a time: first everything they read (angles, staged values), then the arithmetic and the stores, so
    // that the loads of a batch are in flight together (a load cannot pass a store that might write what it reads).
    constexpr int BATCH = 8;
#pragma unroll 1
    for (int r0 = 0; r0 < 32 && row0 + r0 < M; r0 += BATCH) {
      long long offsets[BATCH];
      float inv_of[BATCH], c[BATCH][PER], sn[BATCH][PER], a[BATCH][PER], b[BATCH][PER];
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int r = r0 + i;
        offsets[i] = __shfl_sync(0xffffffffu, page_offset, r);
        inv_of[i] = __shfl_sync(0xffffffffu, inv, r);
        const int table_r = __shfl_sync(0xffffffffu, table_row, r);   // rows past the end have position 0: any row of the tables will do
        if (!is_v) {
          const float* cos_at = rot.cos_table + (size_t)table_r * HALF + column;
          const float* sin_at = rot.sin_table + (size_t)table_r * HALF + column;
          if (PER == 2) {
            const float2 cv = *reinterpret_cast<const float2*>(cos_at), sv = *reinterpret_cast<const float2*>(sin_at);
            c[i][0] = cv.x; c[i][PER - 1] = cv.y; sn[i][0] = sv.x; sn[i][PER - 1] = sv.y;
          } else {
            c[i][0] = cos_at[0]; sn[i][0] = sin_at[0];
          }
        }
        const unsigned char* source = staging + r * ROW_BYTES;
        const uint32_t swizzle = (uint32_t)(r & (UNITS - 1));
        const unsigned char* lower_src = source + ((((lower_byte >> 4) ^ swizzle) << 4) | (lower_byte & 15));
        const unsigned char* upper_src = source + ((((upper_byte >> 4) ^ swizzle) << 4) | (upper_byte & 15));
        if (PER == 2) {
          const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(lower_src)), fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(upper_src));
          a[i][0] = fa.x; a[i][PER - 1] = fa.y; b[i][0] = fb.x; b[i][PER - 1] = fb.y;
        } else {
          a[i][0] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(lower_src));
          b[i][0] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(upper_src));
        }
      }
#pragma unroll
      for (int i = 0; i < BATCH; ++i) {
        const int r = r0 + i;
        if (row0 + r >= M || (!is_q && offsets[i] < 0)) continue;
        if (!is_v) {
#pragma unroll
          for (int e = 0; e < PER; ++e) {
            const float first = a[i][e] * inv_of[i] * w_lower[e], second = b[i][e] * inv_of[i] * w_upper[e];
            a[i][e] = first * c[i][e] - second * sn[i][e];
            b[i][e] = second * c[i][e] + first * sn[i][e];
          }
        }
        __nv_bfloat16* dst = is_q ? rot.q_out + (size_t)(row0 + r) * rot.ldq + (size_t)head * D : pages + offsets[i] + (size_t)kv_head * rot.page_size * D;
        if (PER == 2) {
          *reinterpret_cast<uint32_t*>(dst + column) = pack2(a[i][0], a[i][PER - 1]);
          *reinterpret_cast<uint32_t*>(dst + HALF + column) = pack2(b[i][0], b[i][PER - 1]);
        } else {
          dst[column] = __float2bfloat16_rn(a[i][0]);
          dst[HALF + column] = __float2bfloat16_rn(b[i][0]);
        }
      }
    }
    __syncwarp();   // the next head writes the same staging rows
  }
}

// error: 0 = fine; otherwise 1 producer, 2 MMA issuer, 3 epilogue gave up waiting.
template <int BN, int MODE, int D>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                      const __grid_constant__ CUtensorMap map_b,
                                                                      const __grid_constant__ CUtensorMap map_c, int M, int N, int K,
                                                                      int* __restrict__ error, const RotateArgs rot) {
  constexpr bool SWIGLU = MODE == TC_SWIGLU;
  using S = TcShared<BN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* a_tiles = smem;
  unsigned char* b_tiles = smem + (size_t)STAGES * S::A_BYTES;
  unsigned char* staging = b_tiles + (size_t)STAGES * S::B_BYTES;   // 1024-byte aligned: every stage is a multiple of that
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + TC_STAGING_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;      // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + BN - 1) / BN;
  const int total_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  constexpr int ACCUMULATORS = S::ACCUMULATORS;
  constexpr int TMEM_COLUMNS = ACCUMULATORS * BN <= 256 ? 256 : 512;   // the accumulator buffers; allocations are powers of two
  if (warp == 1) {   // the whole warp allocates
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_base_slot)), "r"(TMEM_COLUMNS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // Barriers and tensor memory are set up while the kernel before this one finishes (dependent launch); its output is
  // read, and anything written, only from here on.
  grid_dependency_wait();
  allow_dependents();

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;   // neighbours in the grid share their B tile
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) { atomicExch(error, 1); alive = false; break; }
          mbar_expect_tx(&full[stage], S::A_BYTES + S::B_BYTES);
          tma_load_2d(a_tiles + (size_t)stage * S::A_BYTES, &map_a, &full[stage], kb * TC_BK, m0);
#pragma unroll
          for (int piece = 0; piece < S::PIECES; ++piece)
            tma_load_2d(b_tiles + (size_t)stage * S::B_BYTES + (size_t)piece * S::PIECE_ROWS * 128, &map_b, &full[stage], kb * TC_BK, n0 + piece * S::PIECE_ROWS);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc_instr_desc(TC_BM, S::PIECE_ROWS);
      uint32_t stage = 0, phase = 0;
      uint32_t round = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++round) {
        const uint32_t buffer = round % ACCUMULATORS, buffer_phase = (round / ACCUMULATORS) & 1;
        if (!mbar_wait(&acc_empty[buffer], buffer_phase ^ 1)) { atomicExch(error, 2); break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buffer * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase)) { atomicExch(error, 2); alive = false; break; }
          tc_fence_after();
          const uint64_t a_desc = tc_smem_desc(a_tiles + (size_t)stage * S::A_BYTES);
          const uint64_t b_desc = tc_smem_desc(b_tiles + (size_t)stage * S::B_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)   // 16 k-values = 32 bytes further along the swizzled row: +2 in 16-byte units
#pragma unroll
            for (int piece = 0; piece < S::PIECES; ++piece)   // a piece of B lies PIECE_ROWS rows of 128 bytes further on, its columns of the accumulator likewise
              tc_mma(tmem_d + piece * S::PIECE_ROWS, a_desc + 2 * k, b_desc + 2 * k + (uint64_t)((piece * S::PIECE_ROWS * 128) >> 4), idesc, (kb | k) != 0 ? 1u : 0u);
          tc_commit(&empty[stage]);   // the stage is free once these products have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (alive) tc_commit(&acc_full[buffer]);   // the accumulator is complete once all products are
      }
    }
  } else {
    // Epilogue: warp w reads the quarter (w % 4) of the 128 lanes; lane = output row.
    using Store = TcStore<BN, SWIGLU>;
    const int quarter = warp & 3;
    unsigned char* my_staging = staging + (size_t)quarter * 2 * 32 * 128;
    const int out_columns = SWIGLU ? N / 2 : N;
    uint32_t round = 0, staged = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++round) {
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * BN;
      const uint32_t buffer = round % ACCUMULATORS, buffer_phase = (round / ACCUMULATORS) & 1;
      if (!mbar_wait(&acc_full[buffer], buffer_phase)) { atomicExch(error, 3); break; }
      tc_fence_after();
      const int row0 = m0 + quarter * 32;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buffer * BN;
      if constexpr (MODE == TC_ROTATE) {
        rotate_epilogue<BN, D>(rot, taddr, my_staging, row0, n0, M, lane);
      } else
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += Store::ACCUMULATOR_COLUMNS, ++staged) {
        unsigned char* stage_rows = my_staging + (staged & 1) * (32 * 128);
        if (lane == 0) tma_store_wait_read<1>();   // the store that last read this buffer is two stores back
        __syncwarp();
#pragma unroll
        for (int part = 0; part < Store::ACCUMULATOR_COLUMNS / 32; ++part) {
          uint32_t raw[32];
          tc_load_32(taddr + c0 + part * 32, raw);
          uint32_t packed[16];
          if (SWIGLU) {   // [g0..g7 u0..u7 g8..g15 u8..u15] -> 16 outputs
#pragma unroll
            for (int group = 0; group < 2; ++group)
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const float g0 = __uint_as_float(raw[group * 16 + j]), g1 = __uint_as_float(raw[group * 16 + j + 1]);
                const float u0 = __uint_as_float(raw[group * 16 + 8 + j]), u1 = __uint_as_float(raw[group * 16 + 8 + j + 1]);
                packed[group * 4 + j / 2] = pack2(silu_fast(g0) * u0, silu_fast(g1) * u1);
              }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) packed[j] = pack2(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1]));
          }
          constexpr int UNITS = SWIGLU ? 2 : 4;   // 16-byte units this part adds to the row
#pragma unroll
          for (int unit = 0; unit < UNITS; ++unit) {
            uint32_t offset = (uint32_t)lane * Store::ROW_BYTES + (uint32_t)(part * UNITS + unit) * 16;
            offset ^= ((offset >> 7) & Store::SWIZZLE_MASK) << 4;
            *reinterpret_cast<uint4*>(stage_rows + offset) = make_uint4(packed[unit * 4], packed[unit * 4 + 1], packed[unit * 4 + 2], packed[unit * 4 + 3]);
          }
        }
        fence_async_shared();   // the writes above, before the TMA engine reads them
        __syncwarp();
        const int out_column = (n0 + c0) / (SWIGLU ? 2 : 1);
        if (lane == 0) {
          if (row0 < M && out_column < out_columns) tma_store_2d(&map_c, stage_rows, out_column, row0);
          // A group for every turn of this loop, empty where the rows lie outside the matrix and nothing is stored: the wait
          // at the loop's head counts groups ("all but the newest have read their buffer"), and a turn without one would let
          // the turn after it write the buffer that the last real store is still reading.  (Seen with a last row tile
          // whose lower quarters lie outside the matrix: the tile a block had stored just before it came out wrong in places.)
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buffer]);   // four warps: the buffer may be overwritten
    }
    if (MODE != TC_ROTATE && lane == 0) tma_store_wait_all();
  }

  // Wind down: every role comes here, also after a wait that ran out.
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLUMNS));
  }
}

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

// Tensor map of a row-major bfloat16 matrix [rows, cols] (row stride ld elements) with boxes of box_rows x box_cols
// (64 columns: 128-byte swizzle; 32: 64-byte swizzle).
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows, int box_cols = TC_BK) {
  EncodeTiled encode = encode_tiled();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool SWIGLU>
static int launch_tcgen05(const CUtensorMap& map_a, const CUtensorMap& map_b, __nv_bfloat16* c, int M, int N, int K, long long ldc,
                          int* error, int sm_count, cudaStream_t stream) {
  auto kernel = gemm_tcgen05_kernel<BN, SWIGLU ? TC_SWIGLU : TC_PLAIN, 128>;
  static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShared<BN>::BYTES);
    if (err != cudaSuccess) PYLON_REFUSE("gemm_tcgen05: %s", cudaGetErrorString(err));
    configured = true;
  }
  CUtensorMap map_c;
  if (!make_map(&map_c, c, M, SWIGLU ? N / 2 : N, ldc, 32, TcStore<BN, SWIGLU>::COLUMNS)) PYLON_REFUSE("gemm_tcgen05: the output's tensor map could not be made");
  const int tiles = ((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
  const int blocks = tiles < sm_count ? tiles : sm_count;
  launch_dependent<LAUNCH_GEMM>(kernel, dim3(blocks), dim3(TC_THREADS), TcShared<BN>::BYTES, stream, map_a, map_b, map_c, M, N, K, error, RotateArgs{});
  PYLON_CHECK_LAUNCH("gemm_tcgen05");
}

template <int BN, int D>
static int launch_rotate(const CUtensorMap& map_a, const CUtensorMap& map_b, int M, int N, int K, const RotateArgs& rot, int* error, int sm_count,
                         cudaStream_t stream) {
  auto kernel = gemm_tcgen05_kernel<BN, TC_ROTATE, D>;
  static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShared<BN>::BYTES);
    if (err != cudaSuccess) PYLON_REFUSE("gemm_tcgen05_qkv: %s", cudaGetErrorString(err));
    configured = true;
  }
  const int tiles = ((M + TC_BM - 1) / TC_BM) * ((N + BN - 1) / BN);
  const int blocks = tiles < sm_count ? tiles : sm_count;
  launch_dependent<LAUNCH_GEMM>(kernel, dim3(blocks), dim3(TC_THREADS), TcShared<BN>::BYTES, stream, map_a, map_b, map_a /* no output map */, M, N, K, error,
                                rot);
  PYLON_CHECK_LAUNCH("gemm_tcgen05_qkv");
}

static int forced_columns = 0;

}  // namespace pylon

// For measurements: every later product uses tiles of 128 x columns (288, 256, 192, 160 or 128); 0 returns to the choice by size.
extern "C" int pylon_gemm_tcgen05_force_tile(int columns) {
  pylon::forced_columns = columns;
  return 0;
}

// x: bfloat16 [M, K] (row stride ldx), w: bfloat16 [N, K] (row stride ldw), y: bfloat16 [M, N], or [M, N / 2] with swiglu
// (row stride ldy).  K and the strides multiples of 8, N a multiple of 8 (16 with swiglu), x, w and y 16-byte aligned.
// swiglu != 0: w's rows alternate in groups of 8 between gate and up rows and y receives silu(gate) * up.
// error: one int in device memory; the kernel sets it non-zero if one of its waits ran out (the result is then void).
extern "C" int pylon_gemm_tcgen05_bf16(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw,
                                       long long ldy, int swiglu, int* error, int sm_count, cudaStream_t stream) {
  using namespace pylon;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldy % 8) PYLON_REFUSE("gemm_tcgen05: K = %d and the row strides must be multiples of 8", K);
  if (N % (swiglu ? 16 : 8)) PYLON_REFUSE("gemm_tcgen05: N = %d must be a multiple of %d", N, swiglu ? 16 : 8);
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)y % 16)) PYLON_REFUSE("gemm_tcgen05: x, w and y must be 16-byte aligned");
  if (ldx < K || ldw < K || ldy < (swiglu ? N / 2 : N)) PYLON_REFUSE("gemm_tcgen05: a row stride is shorter than its row");
  if (!error || sm_count < 1) PYLON_REFUSE("gemm_tcgen05: an error word and the SM count are needed");
  // Tile width: the one whose rounds over the SMs cover the fewest columns (a persistent block
  // takes ceil(tiles / SMs) tiles; the last round is often nearly empty with wide tiles).
  const long long tiles_m = (M + TC_BM - 1) / TC_BM;
  int bn = 128;
  long long best = -1;
  for (int candidate : {288, 256, 192, 160, 128}) {
    if (forced_columns && candidate != forced_columns) continue;
    if (swiglu && (candidate == 160 || candidate == 288)) continue;   // their accumulator columns do not divide into stores of 32 output columns
    const long long tiles = tiles_m * ((N + candidate - 1) / candidate);
    const long long rounds = (tiles + sm_count - 1) / sm_count;
    // A tile's time is what its operands take to arrive from L2, (128 + width) rows of k a step, plus its start and end:
    // one pass of all SMs over their tiles took 11.9, 12.2, 13.9 and 16.3 us at widths 128, 160, 192 and 256 (k = 2,560), which is width + 213.
    long long cost = rounds * (candidate + 213);
    if (candidate > 256) cost += rounds * 100;   // one accumulator buffer: the epilogue of a tile holds up the next (21 us a round)
    if (best < 0 || cost < best) { best = cost; bn = candidate; }
  }
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, x, M, K, ldx, TC_BM) || !make_map(&map_b, w, N, K, ldw, bn > 256 ? bn / 2 : bn))
    PYLON_REFUSE("gemm_tcgen05: the tensor maps could not be made");
  __nv_bfloat16* out = (__nv_bfloat16*)y;
#define PYLON_TC_CASE(BN_)                                                                                          \
  if (bn == BN_) {                                                                                                  \
    if (swiglu) return launch_tcgen05<BN_, true>(map_a, map_b, out, M, N, K, ldy, error, sm_count, stream);         \
    return launch_tcgen05<BN_, false>(map_a, map_b, out, M, N, K, ldy, error, sm_count, stream);                    \
  }
  PYLON_TC_CASE(256) PYLON_TC_CASE(192)
#undef PYLON_TC_CASE
  if (bn == 288) return launch_tcgen05<288, false>(map_a, map_b, out, M, N, K, ldy, error, sm_count, stream);
  if (bn == 160) return launch_tcgen05<160, false>(map_a, map_b, out, M, N, K, ldy, error, sm_count, stream);
  if (swiglu) return launch_tcgen05<128, true>(map_a, map_b, out, M, N, K, ldy, error, sm_count, stream);
  return launch_tcgen05<128, false>(map_a, map_b, out, M, N, K, ldy, error, sm_count, stream);
}

// The fused QKV product with its heads finished in the epilogue: x bfloat16 [M, K], w bfloat16 [(nq + 2 nkv) * d, K] (q rows,
// then k, then v); q and k heads are normalised over the head (weights float32 [d], or null for none) and rotated by the
// float32 cos/sin tables [table_positions, d / 2] at positions[t] (pairs (j, j + d / 2)); q goes to q_out bfloat16
// [M, nq * d] (row stride ldq), k and v into the pages [num_pages, nkv, page_size, d] at the slot that the token's row of
// the block table names (token_row[t] negative: a padding token, nothing written).  d 64 or 128.  page_error: set to
// PYLON_ERROR_BAD_PAGE when a block table names a page that is not there (nothing is written for that token).
extern "C" int pylon_gemm_tcgen05_qkv_rotate(const void* x, const void* w, void* q_out, int M, int K, long long ldx, long long ldw, long long ldq,
                                             const float* q_weight, const float* k_weight, float eps, const float* cos_table, const float* sin_table,
                                             int table_positions, const int* positions, const int* token_row, const int* block_table, int table_width,
                                             int page_size, void* k_pages, void* v_pages, int num_pages, int nq, int nkv, int head_dim, int* page_error,
                                             int* error, int sm_count, cudaStream_t stream) {
  using namespace pylon;
  if (M <= 0) return 0;
  if (head_dim != 64 && head_dim != 128) PYLON_REFUSE("gemm_tcgen05_qkv: head size %d (64 or 128)", head_dim);
  if (nq < 1 || nkv < 1 || page_size < 1 || table_width < 1 || num_pages < 1 || table_positions < 1)
    PYLON_REFUSE("gemm_tcgen05_qkv: %d query heads, %d KV heads, pages of %d, tables of %d, %d pages, %d positions", nq, nkv, page_size, table_width, num_pages, table_positions);
  const int N = (nq + 2 * nkv) * head_dim;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldq % 8) PYLON_REFUSE("gemm_tcgen05_qkv: K = %d and the row strides must be multiples of 8", K);
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)q_out % 16) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) ||
      ((uintptr_t)cos_table % 16) || ((uintptr_t)sin_table % 16) || ((uintptr_t)q_weight % 16) || ((uintptr_t)k_weight % 16))
    PYLON_REFUSE("gemm_tcgen05_qkv: x, w, q, the pages, the tables and the norm weights must be 16-byte aligned");
  if (ldx < K || ldw < K || ldq < (long long)nq * head_dim) PYLON_REFUSE("gemm_tcgen05_qkv: a row stride is shorter than its row");
  if (!x || !w || !q_out || !cos_table || !sin_table || !positions || !token_row || !block_table || !k_pages || !v_pages || !error || sm_count < 1)
    PYLON_REFUSE("gemm_tcgen05_qkv: a tensor, the error word or the SM count is missing");
  RotateArgs rot;
  rot.q_out = (__nv_bfloat16*)q_out; rot.ldq = ldq; rot.q_weight = q_weight; rot.k_weight = k_weight; rot.eps = eps;
  rot.cos_table = cos_table; rot.sin_table = sin_table; rot.table_positions = table_positions; rot.positions = positions;
  rot.token_row = token_row; rot.block_table = block_table; rot.table_width = table_width; rot.page_size = page_size;
  rot.k_pages = (__nv_bfloat16*)k_pages; rot.v_pages = (__nv_bfloat16*)v_pages; rot.num_pages = num_pages; rot.nq = nq; rot.nkv = nkv;
  rot.page_error = page_error;
  // Tile width: a multiple of the head size; the one whose rounds over the SMs cover the fewest columns.
  const long long tiles_m = (M + TC_BM - 1) / TC_BM;
  int bn = 128;
  long long best = -1;
  for (int candidate : {256, 192, 128}) {
    if (candidate % head_dim || (forced_columns && candidate != forced_columns)) continue;
    const long long tiles = tiles_m * ((N + candidate - 1) / candidate);
    const long long rounds = (tiles + sm_count - 1) / sm_count;
    const long long cost = rounds * (candidate + 213);   // as for the plain product
    if (best < 0 || cost < best) { best = cost; bn = candidate; }
  }
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, x, M, K, ldx, TC_BM) || !make_map(&map_b, w, N, K, ldw, bn)) PYLON_REFUSE("gemm_tcgen05_qkv: the tensor maps could not be made");
  if (head_dim == 128) {
    if (bn == 256) return launch_rotate<256, 128>(map_a, map_b, M, N, K, rot, error, sm_count, stream);
    return launch_rotate<128, 128>(map_a, map_b, M, N, K, rot, error, sm_count, stream);
  }
  if (bn == 256) return launch_rotate<256, 64>(map_a, map_b, M, N, K, rot, error, sm_count, stream);
  if (bn == 192) return launch_rotate<192, 64>(map_a, map_b, M, N, K, rot, error, sm_count, stream);
  return launch_rotate<128, 64>(map_a, map_b, M, N, K, rot, error, sm_count, stream);
}
