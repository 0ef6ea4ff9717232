// x * w^T for at most 64 activation rows - the products of a decode step - in three forms:
//   partial sums   y[part] = x[:, k-slice(part)] * w[:, k-slice(part)]^T as float32, for results that go into
//                  the residual stream (attention output and down projections); whoever reads y adds the parts up
//   product        y = x * w^T in bfloat16 (one slice of k)
//   SwiGLU         w's rows alternate in groups of 8 between gate and up rows; y = silu(gate) * up in bfloat16
//
// These products are small (20 to 50 MB of weights) and bound by how soon their bytes are in
// flight, not by arithmetic.  One block takes a 64-row slab of w and one slice of k.  A producer
// thread asks TMA for the slab box by box (64 rows x 64 k, 128-byte swizzle; the 8 x 64 box of x
// rides on the same mbarrier) into a ring that holds a block's whole share, so all of it is on
// its way after one round trip; four consumer warps (16 weight rows each) multiply with
// mma.sync, w as the 16-row A operand, x as 8-column B operands (MT of them for up to 8 * MT rows).  Streaming a matrix this
// way took 6.4 us for the 2560 x 4096 output projection where per-thread 16-byte loads took 10.
//
// All waits on mbarriers are bounded: a wait that runs out sets an error word for the host and
// the block returns.  No TMA load here uses cluster multicast.
//
// Stands in for the library product behind raun6k/Pylon's nn.Linear at decode
// (src/pylon/model/layers.py:26-27,138).
#include "common.cuh"

#include <cuda.h>

#include <mutex>
#include <unordered_map>

namespace pylon {

constexpr int ST_ROWS = 64, ST_BK = 64, ST_CONSUMERS = 4, ST_THREADS = 32 * (1 + ST_CONSUMERS);
constexpr int ST_W_BYTES = ST_ROWS * ST_BK * 2;
enum StreamForm { ST_PARTIAL = 0, ST_PRODUCT = 1, ST_SWIGLU = 2 };
// MT: 8-row tiles of x.  A stage holds the box of w and the box of x; as many stages as fit in 64 KB (three blocks to an SM).
template <int MT>
struct StreamRing {
  static constexpr int X_BYTES = 8 * MT * ST_BK * 2, STAGE_BYTES = ST_W_BYTES + X_BYTES;
  static constexpr int STAGES = (64 * 1024) / STAGE_BYTES;
  static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 128 /* barriers */;
};
constexpr unsigned ST_WAIT_LIMIT = 1u << 22;   // try_wait calls before a wait gives up

__device__ __forceinline__ unsigned st_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void st_mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(st_smem(bar)), "r"(count));
}
__device__ __forceinline__ void st_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(st_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void st_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(st_smem(bar)) : "memory");
}
__device__ __forceinline__ bool st_mbar_wait(uint64_t* bar, unsigned parity) {
  for (unsigned tries = 0; tries < ST_WAIT_LIMIT; ++tries) {
    unsigned done;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(done) : "r"(st_smem(bar)), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void st_tma_load(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(st_smem(dst)), "l"((unsigned long long)map), "r"(st_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void st_ldmatrix_x4(unsigned (&r)[4], unsigned address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void st_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Grid (parts, slabs of 64 weight rows).  y: float32 [parts, M, N] (ST_PARTIAL), bfloat16 [M, N] (ST_PRODUCT) or
// bfloat16 [M, N / 2] (ST_SWIGLU), row stride ldy for the last two.  error: 1 the producer, 2 a consumer gave up waiting.
template <int MT, int FORM>
__global__ void __launch_bounds__(ST_THREADS, 3) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                                     void* __restrict__ y, int M, int N, int K, long long ldy, int* __restrict__ error) {
  using Ring = StreamRing<MT>;
  constexpr int STAGES = Ring::STAGES, STAGE_BYTES = Ring::STAGE_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + (size_t)STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = blockIdx.x, parts = gridDim.x, n0 = blockIdx.y * ST_ROWS;
  const int k_boxes = (K + ST_BK - 1) / ST_BK;
  const int box_begin = (int)((long long)part * k_boxes / parts), box_end = (int)((long long)(part + 1) * k_boxes / parts);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) { st_mbar_init(&full[s], 1); st_mbar_init(&empty[s], ST_CONSUMERS); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: the boxes that fit in the ring are asked for before
      // this kernel waits for it (a dependent launch may start while that kernel is still running); the activations'
      // boxes follow after the wait, on the same barriers.
      const int ahead = min(STAGES, box_end - box_begin);
      for (int i = 0; i < ahead; ++i) {
        st_mbar_expect_tx(&full[i], STAGE_BYTES);   // rows past N, M or K arrive as zeros and count all the same
        st_tma_load(stages + (size_t)i * STAGE_BYTES, &map_w, &full[i], (box_begin + i) * ST_BK, n0);
      }
      grid_dependency_wait();
      allow_dependents();
      for (int i = 0; i < ahead; ++i)
        st_tma_load(stages + (size_t)i * STAGE_BYTES + ST_W_BYTES, &map_x, &full[i], (box_begin + i) * ST_BK, 0);
      unsigned stage = 0, phase = 1;   // the ring has gone round once
      for (int box = box_begin + ahead; box < box_end; ++box) {
        if (!st_mbar_wait(&empty[stage], phase ^ 1)) { atomicExch(error, 1); break; }
        // The consumers read the stage with ordinary loads (ldmatrix); TMA, which writes it next, is another proxy, and
        // the barrier alone does not order the two.  Without this fence the next box's first rows now and then landed
        // under a warp's last reads: one weight row in some 1,500 calls off by a box's worth of its sum, for every token.
        // (The same fence in every consumer warp, before it gives the stage back, cost 6 % of a decode step; here 1.7 %.)
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        unsigned char* dst = stages + (size_t)stage * STAGE_BYTES;
        st_mbar_expect_tx(&full[stage], STAGE_BYTES);
        st_tma_load(dst, &map_w, &full[stage], box * ST_BK, n0);
        st_tma_load(dst + ST_W_BYTES, &map_x, &full[stage], box * ST_BK, 0);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    return;
  }
  grid_dependency_wait();   // before the result is written: its memory may be what that kernel still reads

  // Consumers.  In the 128-byte swizzle the 16-byte unit u of row r sits at unit u ^ (r % 8).
  const int slab_row = (warp - 1) * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);   // this lane's row of w for ldmatrix
  const unsigned w_row_offset = (unsigned)slab_row * 128, w_xor = (unsigned)(slab_row & 7);
  const unsigned x_row_offset = (unsigned)(lane & 7) * 128, x_xor = (unsigned)(lane & 7);
  float acc[MT][2][4];   // per tile of x: even and odd k-steps, two MMA chains
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][0][i] = acc[j][1][i] = 0.f;
  unsigned stage = 0, phase = 0;
  bool alive = true;
  for (int box = box_begin; box < box_end; ++box) {
    if (!st_mbar_wait(&full[stage], phase)) { atomicExch(error, 2); alive = false; break; }
    const unsigned w_box = st_smem(stages + (size_t)stage * STAGE_BYTES), x_box = w_box + ST_W_BYTES;
#pragma unroll
    for (int half = 0; half < 2; ++half) {   // 32 k each
      unsigned a[2][4];
#pragma unroll
      for (int step = 0; step < 2; ++step)    // 16 k each
        st_ldmatrix_x4(a[step], w_box + w_row_offset + ((((unsigned)(4 * half + 2 * step) + (lane >> 4)) ^ w_xor) << 4));
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        unsigned b[4];                         // x: units 4 * half .. + 3 of rows 8j .. 8j + 7
        st_ldmatrix_x4(b, x_box + (unsigned)(j * 8 * 128) + x_row_offset + ((((unsigned)(4 * half) + (lane >> 3)) ^ x_xor) << 4));
        st_mma(acc[j][0], a[0], b[0], b[1]);
        st_mma(acc[j][1], a[1], b[2], b[3]);
      }
    }
    __syncwarp();
    if (lane == 0) st_mbar_arrive(&empty[stage]);
    if (++stage == STAGES) { stage = 0; phase ^= 1; }
  }
  if (!alive) return;

  // Accumulator element i of lane (g, t): weight row g + 8 * (i / 2), activation row 2 * t + (i % 2) of its tile.
  const int g = lane >> 2, t = lane & 3;
  const int row0 = n0 + (warp - 1) * 16 + g;   // the weight row of elements 0 and 1; elements 2 and 3: row0 + 8
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = acc[j][0][i] + acc[j][1][i];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int m = j * 8 + 2 * t + e;
      if (m >= M) continue;
      if (FORM == ST_PARTIAL) {
        float* out = reinterpret_cast<float*>(y) + ((size_t)part * M + m) * N;
        if (row0 < N) out[row0] = v[e];
        if (row0 + 8 < N) out[row0 + 8] = v[2 + e];
      } else if (FORM == ST_PRODUCT) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(y) + (size_t)m * ldy;
        if (row0 < N) out[row0] = __float2bfloat16_rn(v[e]);
        if (row0 + 8 < N) out[row0 + 8] = __float2bfloat16_rn(v[2 + e]);
      } else {   // rows row0 (gate) and row0 + 8 (its up row) are both this lane's
        if (row0 + 8 < N) {
          const float gate = v[e], up = v[2 + e];
          reinterpret_cast<__nv_bfloat16*>(y)[(size_t)m * ldy + (n0 + (warp - 1) * 16) / 2 + g] = __float2bfloat16_rn(__fdividef(gate, 1.f + __expf(-gate)) * up);   // approximate division: ample for bfloat16, no slow path
        }
      }
    }
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

// Tensor map of a row-major bfloat16 matrix [rows, cols] (row stride ld elements) with boxes of box_rows x 64 columns
// in the 128-byte swizzle.  Maps are kept by their arguments: a model multiplies by the same matrices at every step.
static bool matrix_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  struct Key {
    const void* base; long long rows, cols, ld; int box_rows;
    bool operator==(const Key& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
  };
  struct Hash {
    size_t operator()(const Key& k) const { return std::hash<const void*>()(k.base) ^ (size_t)(k.rows * 1315423911LL) ^ (size_t)(k.cols * 2654435761LL) ^ (size_t)k.box_rows; }
  };
  static std::unordered_map<Key, CUtensorMap, Hash> known;
  static std::mutex mutex;
  std::lock_guard<std::mutex> guard(mutex);
  const Key key{base, rows, cols, ld, box_rows};
  auto found = known.find(key);
  if (found != known.end()) { *map = found->second; return true; }
  EncodeTiled encode = encode_tiled();
  if (!encode) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)ST_BK, (cuuint32_t)box_rows};
  cuuint32_t element_strides[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (known.size() >= 4096) known.clear();   // activations come and go; the weights' maps are made again on demand
  known.emplace(key, *map);
  return true;
}

template <int MT, int FORM>
static int launch_stream(const CUtensorMap& map_w, const CUtensorMap& map_x, void* y, int M, int N, int K, long long ldy, int parts, int slabs,
                         int* error, cudaStream_t stream) {
  auto kernel = gemm_stream_kernel<MT, FORM>;
  static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)StreamRing<MT>::SMEM);
    if (err != cudaSuccess) PYLON_REFUSE("gemm_stream: %s", cudaGetErrorString(err));
    configured = true;
  }
  launch_dependent<LAUNCH_GEMM>(kernel, dim3(parts, slabs), dim3(ST_THREADS), StreamRing<MT>::SMEM, stream, map_w, map_x, y, M, N, K, ldy, error);
  PYLON_CHECK_LAUNCH("gemm_stream");
}

template <int FORM>
static int dispatch_stream(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw, long long ldy, int parts,
                           int* error, cudaStream_t stream, const char* name) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) PYLON_REFUSE("%s: M = %d is more than 64 rows", name, M);
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8) PYLON_REFUSE("%s: K = %d and the row strides must be multiples of 8", name, K);
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)y % 4)) PYLON_REFUSE("%s: x and w must be 16-byte aligned", name);
  if (ldx < K || ldw < K) PYLON_REFUSE("%s: a row stride is shorter than its row", name);
  const int k_boxes = (K + ST_BK - 1) / ST_BK, slabs = (N + ST_ROWS - 1) / ST_ROWS;
  if (parts < 1 || parts > k_boxes || parts > 65535 || slabs > 65535) PYLON_REFUSE("%s: %d parts over %d slices of k, %d slabs", name, parts, k_boxes, slabs);
  if (!error) PYLON_REFUSE("%s: an error word is needed", name);
  const int tiles = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  CUtensorMap map_w, map_x;
  if (!matrix_map(&map_w, w, N, K, ldw, ST_ROWS) || !matrix_map(&map_x, x, M, K, ldx, 8 * tiles)) PYLON_REFUSE("%s: the tensor maps could not be made", name);
  if (tiles == 1) return launch_stream<1, FORM>(map_w, map_x, y, M, N, K, ldy, parts, slabs, error, stream);
  if (tiles == 2) return launch_stream<2, FORM>(map_w, map_x, y, M, N, K, ldy, parts, slabs, error, stream);
  if (tiles == 4) return launch_stream<4, FORM>(map_w, map_x, y, M, N, K, ldy, parts, slabs, error, stream);
  return launch_stream<8, FORM>(map_w, map_x, y, M, N, K, ldy, parts, slabs, error, stream);
}

}  // namespace pylon

// x: bfloat16 [M, K] (row stride ldx), M <= 64; w: bfloat16 [N, K] (row stride ldw); y: float32 [parts, M, N] contiguous,
// whose sum over the first dimension is x @ w.T.  K and the row strides multiples of 8, x and w 16-byte aligned,
// 1 <= parts <= number of 64-wide slices of k.  error: one int in device memory that the kernel sets non-zero if one of its
// waits ran out (the result is then void).
extern "C" int pylon_gemm_stream_partial(const void* x, const void* w, float* y, int M, int N, int K, long long ldx, long long ldw,
                                         int parts, int* error, cudaStream_t stream) {
  return pylon::dispatch_stream<pylon::ST_PARTIAL>(x, w, y, M, N, K, ldx, ldw, N, parts, error, stream, "gemm_stream_partial");
}

// The product itself: y bfloat16 [M, N], row stride ldy.
extern "C" int pylon_gemm_stream_bf16(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw,
                                      long long ldy, int* error, cudaStream_t stream) {
  if (ldy < N) PYLON_REFUSE("gemm_stream_bf16: a row stride is shorter than its row");
  return pylon::dispatch_stream<pylon::ST_PRODUCT>(x, w, y, M, N, K, ldx, ldw, ldy, 1, error, stream, "gemm_stream_bf16");
}

// silu(x gate^T) * (x up^T): w's rows are interleaved in groups of 8 (rows 16b..16b+7 gate rows 8b..8b+7, rows 16b+8..16b+15
// the matching up rows; N a multiple of 16); y bfloat16 [M, N / 2], row stride ldy.
extern "C" int pylon_gemm_stream_swiglu(const void* x, const void* w, void* y, int M, int N, int K, long long ldx, long long ldw,
                                        long long ldy, int* error, cudaStream_t stream) {
  if (N % 16 || ldy < N / 2) PYLON_REFUSE("gemm_stream_swiglu: N = %d must be a multiple of 16 and the result N / 2 columns wide", N);
  return pylon::dispatch_stream<pylon::ST_SWIGLU>(x, w, y, M, N, K, ldx, ldw, ldy, 1, error, stream, "gemm_stream_swiglu");
}
