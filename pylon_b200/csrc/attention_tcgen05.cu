// Paged causal attention for prompt portions on the fifth-generation tensor cores, bfloat16.
//
// Built for one head size per library: -DPYLON_HEAD_DIM=64 or 128.  Pages must hold a multiple
// of 64 keys (a 64-key tile then lies in one page and TMA can fetch it as boxes).
//
// One block takes 128 packed query rows of one request and one KV head (packed row m is token
// m / G, query head kv_head * G + m % G, for any group size G) and walks the 64-key tiles its
// rows can see.  Six warps with fixed roles:
//   warps 0..3  softmax: thread i owns row i, which is lane i of tensor memory.  It reads its
//               64 scores with tcgen05.ld, scales and masks them, keeps the running maximum
//               and sum in float32 (no shuffles: a row is one thread), writes the weights as
//               bfloat16 back into tensor memory over the scores it has read (tcgen05.st, two
//               weights to a column), and at the end divides the output row by its sum and
//               stores it.
//   warp 4      TMA producer: keys and values of a tile as 64 x 64 boxes into a two-stage ring
//   warp 5      MMA issuer: S = Q K^T (tcgen05.mma, M 128, N 64, accumulator in tensor memory,
//               two score buffers so that the scores of tile t + 1 are computed while tile t
//               goes through the softmax), then O += P V (M 128, N = head size; the weights are
//               the A operand, read from tensor memory; V is read straight from its [key][value]
//               tile as the MN-major operand).  The weights never touch shared memory, which the
//               operand reads of the N = 64 products keep busy as it is, and no softmax thread
//               waits for the weights' buffer to come free: 504 against 529 us at 8,192 tokens.
// The output accumulator stays in tensor memory.  When a row's maximum grows, the row is
// rescaled there (tcgen05.ld, multiply, tcgen05.st) - but only when it grew by more than 2^8:
// up to that, the old maximum stays the reference point, which changes nothing in exact
// arithmetic and keeps every weight below 256.
//
// Two blocks fit on an SM (shared memory 96 KB, tensor memory 256 columns each), so one
// block's softmax overlaps the other's products.  All waits on mbarriers are bounded: a wait
// that runs out sets an error word for the host and every role winds down (tensor memory is
// freed) instead of hanging.  No TMA load here uses cluster multicast.
//
// Semantics as raun6k/Pylon's attention call (src/pylon/kv/cache.py:462-476, restated
// 483-491): key j of the same request is visible to the token at position p iff j <= p (and
// j > p - window when a window is set); softmax scale 1/sqrt(d) unless given.
#include "common.cuh"

#include <cuda.h>

#include <mutex>

#ifndef PYLON_HEAD_DIM
#define PYLON_HEAD_DIM 128
#endif

namespace pylon {

constexpr int D = PYLON_HEAD_DIM;
static_assert(D == 64 || D == 128, "the tcgen05 attention is built for head sizes 64 and 128");
constexpr int FA_BM = 128, FA_BN = 64, FA_STAGES = 2, FA_THREADS = 192;
constexpr int FA_SMALL_ROWS = 16;                  // rows with at most this many packed query rows belong to the decode kernel
constexpr int FA_Q_BYTES = FA_BM * D * 2;          // D / 64 panels of [128 rows][64 values]
constexpr int FA_TILE_BYTES = FA_BN * D * 2;       // keys or values of one tile: D / 64 boxes of [64 keys][64 values]
constexpr int FA_STAGE_BYTES = 2 * FA_TILE_BYTES;
constexpr size_t FA_SMEM_USED = (size_t)FA_Q_BYTES + FA_STAGES * FA_STAGE_BYTES + 128 /* barriers: 15 x 8 bytes and the tensor-memory address */;
// At least 80 KB: never more than two blocks on an SM, so that their 2 x 256 columns of tensor memory always fit and no
// block waits in tcgen05.alloc for another to finish.
constexpr size_t FA_SMEM = FA_SMEM_USED > 80 * 1024 ? FA_SMEM_USED : 80 * 1024;
constexpr int FA_S_COLUMNS = FA_BN, FA_O_COLUMN = 2 * FA_BN;       // two score buffers, then the output
constexpr int FA_TMEM_COLUMNS = 256;                                // 128 + D rounded up to a power of two
constexpr unsigned FA_WAIT_LIMIT = 1u << 22;
constexpr float FA_RESCALE_STEP = 8.f;             // log2: a row is rescaled when its maximum grew by more than this

struct FaParams {
  const __nv_bfloat16* q;
  long long q_stride;
  __nv_bfloat16* out;
  const int* q_start;
  const int* kv_len;
  const int* block_table;
  int table_width, page_size, num_pages, nq, nkv, group, window, skip_small, first_row;
  float scale_log2;
  int* error;
};

__device__ __forceinline__ unsigned fa_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(fa_smem(bar)), "r"(count));
}
__device__ __forceinline__ void fa_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(fa_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fa_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ bool fa_mbar_wait(uint64_t* bar, unsigned parity) {
  for (unsigned tries = 0; tries < FA_WAIT_LIMIT; ++tries) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(fa_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
// One look at the barrier, without waiting.
__device__ __forceinline__ bool fa_mbar_test(uint64_t* bar, unsigned parity) {
  unsigned done;
  asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(done) : "r"(fa_smem(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void fa_tma_load(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(fa_smem(dst)), "l"((unsigned long long)map), "r"(fa_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fa_fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void fa_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ void fa_mma(unsigned tmem_d, uint64_t a_desc, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void fa_tmem_load_32(unsigned taddr, unsigned (&r)[32]) {
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
__device__ __forceinline__ void fa_tmem_store_32(unsigned taddr, const unsigned (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
// The product with the A operand in tensor memory (the weights) and B through a shared-memory descriptor.
__device__ __forceinline__ void fa_mma_a_tmem(unsigned tmem_d, unsigned tmem_a, uint64_t b_desc, unsigned idesc, unsigned accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 16 consecutive 32-bit columns of this thread's tensor-memory lane; the caller waits for the stores.
__device__ __forceinline__ void fa_tmem_store_16(unsigned taddr, const unsigned* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void fa_tmem_wait_stores() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned fa_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Shared-memory descriptors (version 1 of sm_100, 128-byte swizzle).  Rows of 128 bytes, eight rows
// to a 1024-byte group.
//   K-major (the reduced dimension runs along a row: Q, K, P): groups follow one another along the
//   rows of the operand; the stride between them is 1024 bytes.
//   MN-major (the operand's own dimension runs along a row: V as [key][value]): a group is 8 keys x 64
//   values; `leading` is the distance to the next 64 values, `stride` to the next 8 keys.
__device__ __forceinline__ uint64_t fa_desc(const void* tile, unsigned leading_bytes, unsigned stride_bytes) {
  uint64_t desc = 0;
  desc |= (uint64_t)((fa_smem(tile) & 0x3FFFF) >> 4);
  desc |= (uint64_t)((leading_bytes >> 4) & 0x3FFF) << 16;
  desc |= (uint64_t)((stride_bytes >> 4) & 0x3FFF) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// Instruction descriptor for kind::f16: bfloat16 A and B, float32 D, M x N; b_mn_major: B is read MN-major.
__host__ __device__ constexpr unsigned fa_instr_desc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}

// Grid (KV heads, rows, query tiles).  error: 1 producer, 2 MMA issuer, 3 softmax gave up waiting; 4 shared memory misaligned.
__global__ void __launch_bounds__(FA_THREADS, 2) attention_tcgen05_kernel(const FaParams p, const __grid_constant__ CUtensorMap map_k,
                                                                           const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* q_tile = smem;
  unsigned char* stages = q_tile + FA_Q_BYTES;
  uint64_t* k_full = reinterpret_cast<uint64_t*>(stages + FA_STAGES * FA_STAGE_BYTES);   // [2] the keys of a tile have landed
  uint64_t* k_empty = k_full + 2;      // [2] ... and are read (their scores are computed)
  uint64_t* v_full = k_empty + 2;      // [2] the same for the values
  uint64_t* v_empty = v_full + 2;      // [2]
  uint64_t* s_full = v_empty + 2;      // [2] scores of a tile are in tensor memory
  // [2] weights of tile t are in tensor memory, over its scores (and the output rescaled): barrier t % 2.  The softmax
  // threads wait for nothing between two tiles but the scores, so they may be done with tile t + 1 while the issuer still
  // waits for the values of tile t: with one barrier its wait by parity for tile t would then look at the phase of tile
  // t + 2 and never end.  (Until the weights went into tensor memory the softmax threads waited for the weighted sum of
  // tile t before they wrote the weights of tile t + 1, and could not get that far ahead.)
  uint64_t* p_full = s_full + 2;
  // [2] the weighted sum of tile t is added to the output: barrier t % 2.  A softmax thread waits for it only when it has
  // to (a row to rescale; the end), and a wait by parity can tell a phase only from its neighbours: with one barrier a
  // thread that skipped two tiles' waits would take the phase before last for the one it asks for.  With two, the phase
  // before (tile t - 2) is always complete when tile t's scores are: the products run in the order they were issued.
  uint64_t* pv_done = p_full + 2;
  uint64_t* q_full = pv_done + 2;      // the query tile is in shared memory
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(q_full + 1);

  const int row = p.first_row + blockIdx.y, kv_head = blockIdx.x;
  const int q0 = p.q_start[row];
  const int q_len = p.q_start[row + 1] - q0;
  const int G = p.group;
  const int packed_rows = q_len * G;
  // A block that has nothing to do still waits for the kernel ahead before it leaves: if every block left at once, this
  // grid would end before that kernel, and the next kernel's wait, which sees only this grid, would let it read too early.
  if (packed_rows <= 0 || (p.skip_small && packed_rows <= FA_SMALL_ROWS)) { grid_dependency_wait(); return; }
  // Later query tiles see more keys: hand them out first (the query tile runs slowest in the grid, so the longest
  // blocks of all heads and rows start first).
  const int q_tiles = (packed_rows + FA_BM - 1) / FA_BM;
  if ((int)blockIdx.z >= q_tiles) { grid_dependency_wait(); return; }
  const int m0 = (q_tiles - 1 - (int)blockIdx.z) * FA_BM;
  const int kv_len = p.kv_len[row];
  const int pos0 = kv_len - q_len;   // position of the row's first new token
  const int* table = p.block_table + (size_t)row * p.table_width;
  const int token_lo = m0 / G, token_hi = min(q_len - 1, (m0 + FA_BM - 1) / G);
  const int key_hi = pos0 + token_hi;
  const int key_lo = p.window > 0 ? max(0, pos0 + token_lo - p.window + 1) : 0;
  const int first_tile = key_lo / FA_BN, num_tiles = key_hi / FA_BN - first_tile + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((fa_smem(smem) & 1023u) != 0) {   // the swizzle arithmetic below assumes it
    if (threadIdx.x == 0) atomicExch(p.error, 4);
    grid_dependency_wait();
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      fa_mbar_init(&k_full[s], 1); fa_mbar_init(&k_empty[s], 1); fa_mbar_init(&v_full[s], 1); fa_mbar_init(&v_empty[s], 1);
      fa_mbar_init(&s_full[s], 1);
    }
    fa_mbar_init(&p_full[0], 128);
    fa_mbar_init(&p_full[1], 128);
    fa_mbar_init(&pv_done[0], 1);
    fa_mbar_init(&pv_done[1], 1);
    fa_mbar_init(q_full, 128);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 5) {   // the whole warp allocates
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(fa_smem(tmem_slot)), "r"(FA_TMEM_COLUMNS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  fa_fence_before();
  __syncthreads();
  fa_fence_after();
  const unsigned tmem_base = *tmem_slot;
  // Barriers and tensor memory are set up while the kernel before this one finishes (dependent launch); the queries and
  // the newest keys are its work: they are read, and anything written, only from here on.
  grid_dependency_wait();
  allow_dependents();

  if (warp == 4) {
    // ---- TMA producer ----
    if (lane == 0) {
      for (int t = 0; t < num_tiles; ++t) {
        const int stage = t & 1;
        const unsigned parity = ((t >> 1) & 1) ^ 1;
        // A tile lies in one page.  Without a page for it the row coordinate points past the pool and TMA fills the boxes
        // with zeros.
        const int key0 = (first_tile + t) * FA_BN;
        const int page = table[key0 / p.page_size];
        const bool page_ok = page >= 0 && page < p.num_pages;
        if (page < -1 || page >= p.num_pages) atomicExch(p.error, PYLON_ERROR_BAD_PAGE);   // a broken table; -1 is "no page" (behind a window)
        const int y = page_ok ? (page * p.nkv + kv_head) * p.page_size + key0 % p.page_size : p.num_pages * p.nkv * p.page_size;
        unsigned char* dst = stages + stage * FA_STAGE_BYTES;
        // The keys' half of a stage is free as soon as its scores are computed, a whole tile before the values' half.
        if (!fa_mbar_wait(&k_empty[stage], parity)) { atomicExch(p.error, 1); break; }
        fa_mbar_expect_tx(&k_full[stage], FA_TILE_BYTES);
#pragma unroll
        for (int box = 0; box < D / 64; ++box) fa_tma_load(dst + box * (FA_BN * 128), &map_k, &k_full[stage], box * 64, y);
        if (!fa_mbar_wait(&v_empty[stage], parity)) { atomicExch(p.error, 1); break; }
        fa_mbar_expect_tx(&v_full[stage], FA_TILE_BYTES);
#pragma unroll
        for (int box = 0; box < D / 64; ++box) fa_tma_load(dst + FA_TILE_BYTES + box * (FA_BN * 128), &map_v, &v_full[stage], box * 64, y);
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr unsigned idesc_s = fa_instr_desc(FA_BM, FA_BN, false);
      constexpr unsigned idesc_o = fa_instr_desc(FA_BM, D, true);
      bool alive = fa_mbar_wait(q_full, 0);
      if (!alive) atomicExch(p.error, 2);
      auto scores = [&](int t) {   // S[t % 2] = Q K(t)^T; the keys have landed
        fa_fence_after();
        const unsigned char* k_tile = stages + (t & 1) * FA_STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {   // 16 values = 32 bytes along the swizzled row: +2 in 16-byte units; 64 values to a panel
          const uint64_t a = fa_desc(q_tile + (kk / 4) * (FA_BM * 128), 16, 1024) + 2 * (kk % 4);
          const uint64_t b = fa_desc(k_tile + (kk / 4) * (FA_BN * 128), 16, 1024) + 2 * (kk % 4);
          fa_mma(tmem_base + (t & 1) * FA_S_COLUMNS, a, b, idesc_s, kk != 0 ? 1u : 0u);
        }
        fa_commit(&k_empty[t & 1]);
        fa_commit(&s_full[t & 1]);
      };
      auto weighted_sum = [&](int t) {   // O += P(t) V(t); the weights are written
        fa_fence_after();
        const unsigned char* v_tile = stages + (t & 1) * FA_STAGE_BYTES + FA_TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < FA_BN / 16; ++kk) {   // 16 keys: 32 bytes along a row of P, two 8-key groups (2048 bytes) down V
          const uint64_t b = fa_desc(v_tile + kk * 2048, FA_BN * 128, 1024);
          fa_mma_a_tmem(tmem_base + FA_O_COLUMN, tmem_base + (t & 1) * FA_S_COLUMNS + kk * 8, b, idesc_o, (t | kk) != 0 ? 1u : 0u);
        }
        fa_commit(&v_empty[t & 1]);
        fa_commit(&pv_done[t & 1]);
      };
      if (alive) {
        alive = fa_mbar_wait(&k_full[0], 0);
        if (alive) scores(0); else atomicExch(p.error, 2);
      }
      // Per tile two things are to be issued, whichever can go first: the scores of the next tile (its keys must have
      // landed) and the weighted sum of this one (its weights must be written and its values landed).
      for (int t = 0; t < num_tiles && alive; ++t) {
        bool scores_due = t + 1 < num_tiles, sum_due = true;
        const unsigned next_parity = ((t + 1) >> 1) & 1, parity = (t >> 1) & 1;
        for (unsigned tries = 0; (scores_due || sum_due) && alive; ++tries) {
          if (scores_due && fa_mbar_test(&k_full[(t + 1) & 1], next_parity)) { scores(t + 1); scores_due = false; }
          if (sum_due && fa_mbar_test(&p_full[t & 1], parity) && fa_mbar_test(&v_full[t & 1], parity)) { weighted_sum(t); sum_due = false; }
          if (tries == FA_WAIT_LIMIT) { atomicExch(p.error, 2); alive = false; }
        }
      }
    }
  } else {
    // ---- softmax and output: thread = packed row = lane of tensor memory ----
    const int r = threadIdx.x;
    const int m = m0 + r;
    const bool valid = m < packed_rows;
    const int token = valid ? m / G : 0;
    const int head = kv_head * G + (valid ? m % G : 0);
    const int pos = pos0 + token;
    // The query row, in the layout the tensor core reads: 128-byte rows, 16-byte unit u of row r at u ^ (r % 8).
    {
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)(q0 + token) * p.q_stride + (size_t)head * D);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        const uint4 v = valid ? src[c] : make_uint4(0u, 0u, 0u, 0u);   // an ordinary load: the kernel that wrote the queries overlaps this one's start
        *reinterpret_cast<uint4*>(q_tile + (c / 8) * (FA_BM * 128) + r * 128 + (((c % 8) ^ (r & 7)) << 4)) = v;
      }
      fa_fence_async_shared();
      fa_mbar_arrive(q_full);
    }
    const unsigned lane_base = tmem_base + ((unsigned)(warp * 32) << 16);
    float reference = -INFINITY;   // the maximum the weights refer to (log2 units, scaled)
    float sum = 0.f;
    bool alive = true;
    for (int t = 0; t < num_tiles; ++t) {
      if (!fa_mbar_wait(&s_full[t & 1], (t >> 1) & 1)) { atomicExch(p.error, 3); alive = false; break; }
      fa_fence_after();
      float s[FA_BN];
      {
        unsigned raw[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          fa_tmem_load_32(lane_base + (t & 1) * FA_S_COLUMNS + half * 32, raw);
#pragma unroll
          for (int j = 0; j < 32; ++j) s[half * 32 + j] = __uint_as_float(raw[j]);
        }
      }
      const int key0 = (first_tile + t) * FA_BN;
      // Tiles that end at or before the block's first token, with no window and only valid rows, are visible whole.
      if (p.window > 0 || key0 + FA_BN - 1 > pos0 + token_lo || !valid) {
#pragma unroll
        for (int j = 0; j < FA_BN; ++j) {
          const int key = key0 + j;
          bool visible = valid && key <= pos;
          if (p.window > 0) visible = visible && key > pos - p.window;
          if (!visible) s[j] = -INFINITY;
        }
      }
      // Eight chains side by side: one chain of 63 dependent comparisons would cost more than the exponentials.
      float lane_max[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) lane_max[j] = s[j];
#pragma unroll
      for (int j = 8; j < FA_BN; ++j) lane_max[j & 7] = fmaxf(lane_max[j & 7], s[j]);
      float tile_max = fmaxf(fmaxf(fmaxf(lane_max[0], lane_max[1]), fmaxf(lane_max[2], lane_max[3])),
                             fmaxf(fmaxf(lane_max[4], lane_max[5]), fmaxf(lane_max[6], lane_max[7])));
      tile_max *= p.scale_log2;   // the scale is positive: the largest score stays the largest
      // The reference moves only when the maximum has grown by more than the step (or was not set yet).
      const bool move = tile_max > reference + FA_RESCALE_STEP || (reference == -INFINITY && tile_max > -INFINITY);
      const float alpha = move ? (reference == -INFINITY ? 0.f : fa_exp2(reference - tile_max)) : 1.f;
      if (move) reference = tile_max;
      const float use = reference == -INFINITY ? 0.f : reference;
      // The weights first, in registers: the product of the tile before this one may still be running.
      sum *= alpha;
      float part_sum[4] = {0.f, 0.f, 0.f, 0.f};   // four chains, for the same reason
      unsigned packed[FA_BN / 2];
#pragma unroll
      for (int j = 0; j < FA_BN; j += 2) {
        const float w0 = fa_exp2(fmaf(s[j], p.scale_log2, -use)), w1 = fa_exp2(fmaf(s[j + 1], p.scale_log2, -use));   // 0 for masked keys
        part_sum[(j >> 1) & 3] += w0 + w1;
        packed[j / 2] = fa_pack(w0, w1);
      }
      sum += (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
      // The weights go into tensor memory over this tile's scores, two to a column (this lane's scores are in registers
      // and nothing else reads these columns before the weighted sum).  The output may be rescaled once the tile before
      // this one is added up: only then is that product waited for.
      if (t > 0 && __any_sync(0xffffffffu, move)) {   // tcgen05.ld/st are warp-wide: rows that stay multiply by one
        if (!fa_mbar_wait(&pv_done[(t - 1) & 1], ((t - 1) >> 1) & 1)) { atomicExch(p.error, 3); alive = false; break; }
        fa_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          unsigned raw[32];
          fa_tmem_load_32(lane_base + FA_O_COLUMN + c * 32, raw);
#pragma unroll
          for (int j = 0; j < 32; ++j) raw[j] = __float_as_uint(__uint_as_float(raw[j]) * alpha);
          fa_tmem_store_32(lane_base + FA_O_COLUMN + c * 32, raw);
        }
      }
      fa_tmem_store_16(lane_base + (t & 1) * FA_S_COLUMNS, packed);
      fa_tmem_store_16(lane_base + (t & 1) * FA_S_COLUMNS + 16, packed + 16);
      if (key0 + FA_BN > kv_len) {
        // Keys past the row's length are masked, but their values (whatever the page held) still meet a weight of zero in
        // the product: make them zero, once they have landed.
        if (!fa_mbar_wait(&v_full[t & 1], (t >> 1) & 1)) { atomicExch(p.error, 3); alive = false; break; }
        unsigned char* v_tile = stages + (t & 1) * FA_STAGE_BYTES + FA_TILE_BYTES;
        const int first_unused = kv_len - key0;
        for (int c = r; c < FA_BN * (D / 8); c += 128) {
          const int key = c / (D / 8), unit = c % (D / 8);
          if (key >= first_unused)
            *reinterpret_cast<uint4*>(v_tile + (unit / 8) * (FA_BN * 128) + key * 128 + (((unit % 8) ^ (key & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
        fa_fence_async_shared();   // the zeroed values, before the tensor core reads them
      }
      fa_tmem_wait_stores();
      fa_fence_before();
      fa_mbar_arrive(&p_full[t & 1]);
    }
    if (alive && !fa_mbar_wait(&pv_done[(num_tiles - 1) & 1], ((num_tiles - 1) >> 1) & 1)) { atomicExch(p.error, 3); alive = false; }
    if (alive) {
      fa_fence_after();
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(q0 + token) * p.nq + head) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        unsigned raw[32];
        fa_tmem_load_32(lane_base + FA_O_COLUMN + c * 32, raw);   // warp-wide: rows that are not stored load all the same
        if (valid) {
#pragma unroll
          for (int j = 0; j < 32; j += 8)
            *reinterpret_cast<uint4*>(dst + c * 32 + j) = make_uint4(
                fa_pack(__uint_as_float(raw[j]) * inv, __uint_as_float(raw[j + 1]) * inv), fa_pack(__uint_as_float(raw[j + 2]) * inv, __uint_as_float(raw[j + 3]) * inv),
                fa_pack(__uint_as_float(raw[j + 4]) * inv, __uint_as_float(raw[j + 5]) * inv), fa_pack(__uint_as_float(raw[j + 6]) * inv, __uint_as_float(raw[j + 7]) * inv));
        }
      }
    }
  }

  // Wind down: every role comes here, also after a wait that ran out.
  fa_fence_before();
  __syncthreads();
  if (warp == 5) {
    fa_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(FA_TMEM_COLUMNS));
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
  cuuint32_t box[2] = {64, (cuuint32_t)FA_BN};
  cuuint32_t element_strides[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  known[next].pages = pages; known[next].rows = rows; known[next].map = *map;
  next = (next + 1) % 64;
  if (count < 64) ++count;
  return true;
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_attention_tcgen05_head_dim() { return D; }

// q: bfloat16 [tokens, >= nq*D] with q_stride elements between tokens; pages: bfloat16 [num_pages, nkv, page_size, D] with
// page_size a multiple of 64; out: bfloat16 [tokens, nq, D]; q_start: int32 [rows + 1]; kv_len: int32 [rows]; block_table:
// int32 [rows, table_width]; rows [first_row, first_row + num_rows) of those arrays are attended to (a caller that knows
// which rows bring prompt portions names just those); max_q: the longest row (or an upper bound).  skip_small != 0: rows
// with at most 16 packed query rows (tokens x group) are left alone (another kernel writes them).  error: one int in device memory that the kernel sets
// non-zero when one of its bounded waits ran out (the output is then void).
extern "C" int pylon_paged_attention_tcgen05(const void* q, long long q_stride, const void* k_pages, const void* v_pages, void* out,
                                             const int* q_start, const int* kv_len, const int* block_table, int table_width,
                                             int page_size, int num_pages, int nq, int nkv, int window, float scale, int first_row,
                                             int num_rows, int max_q, int skip_small, int* error, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (nkv < 1 || nq < 1 || nq % nkv) PYLON_REFUSE("paged_attention_tcgen05: %d query heads over %d KV heads", nq, nkv);
  if (page_size < 64 || page_size % 64) PYLON_REFUSE("paged_attention_tcgen05: pages of %d keys; a multiple of 64 is needed", page_size);
  if (table_width < 1 || window < 0 || max_q < 1) PYLON_REFUSE("paged_attention_tcgen05: table width %d, window %d, longest row %d", table_width, window, max_q);
  if (((uintptr_t)q % 16) || ((uintptr_t)k_pages % 16) || ((uintptr_t)v_pages % 16) || ((uintptr_t)out % 16) || (q_stride % 8))
    PYLON_REFUSE("paged_attention_tcgen05: q, pages and out must be 16-byte aligned and the token stride a multiple of 8");
  if (!(scale > 0.f)) PYLON_REFUSE("paged_attention_tcgen05: the softmax scale must be positive");
  if (nkv > 65535 || num_rows > 65535 || first_row < 0) PYLON_REFUSE("paged_attention_tcgen05: %d KV heads, %d rows from row %d", nkv, num_rows, first_row);
  if (!error) PYLON_REFUSE("paged_attention_tcgen05: an error word is needed");
  const long long pool_rows = (long long)num_pages * nkv * page_size;
  if (pool_rows >= 2147483647LL - FA_BN) PYLON_REFUSE("paged_attention_tcgen05: the page pool has too many rows for a tensor map coordinate");
  static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FA_SMEM);
    if (err != cudaSuccess) PYLON_REFUSE("paged_attention_tcgen05: %s", cudaGetErrorString(err));
    configured = true;
  }
  CUtensorMap map_k, map_v;
  if (!page_pool_map(&map_k, k_pages, pool_rows) || !page_pool_map(&map_v, v_pages, pool_rows))
    PYLON_REFUSE("paged_attention_tcgen05: the tensor maps of the page pools could not be made");
  FaParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out;
  p.q_start = q_start; p.kv_len = kv_len; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.nq = nq; p.nkv = nkv; p.group = nq / nkv; p.window = window; p.skip_small = skip_small; p.first_row = first_row;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.error = error;
  const long long q_tiles = ((long long)max_q * p.group + FA_BM - 1) / FA_BM;
  if (q_tiles > 65535) PYLON_REFUSE("paged_attention_tcgen05: too many query tiles");
  launch_dependent(attention_tcgen05_kernel, dim3(nkv, num_rows, (unsigned)q_tiles), dim3(FA_THREADS), FA_SMEM, stream, p, map_k, map_v);
  PYLON_CHECK_LAUNCH("paged_attention_tcgen05");
}
