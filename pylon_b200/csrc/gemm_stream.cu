// y[part] = x[:, k-slice(part)] * w[:, k-slice(part)]^T for at most 8 activation rows, as float32
// partial sums over `parts` slices of k: the product of a decode step whose result goes into
// the residual stream (attention output and feed-forward down projections).  Whoever reads y
// adds the parts up.
//
// These products are small (20 to 50 MB of weights) and bound by how soon their bytes are in
// flight, not by arithmetic.  One block takes a 64-row slab of w and one slice of k.  A producer
// thread asks TMA for the slab box by box (64 rows x 64 k, 128-byte swizzle; the 8 x 64 box of x
// rides on the same mbarrier) into a ring that holds a block's whole share, so all of it is on
// its way after one round trip; four consumer warps (16 weight rows each) multiply with
// mma.sync, w as the 16-row A operand, x as the 8-column B operand.  Streaming a matrix this
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

constexpr int ST_ROWS = 64, ST_BK = 64, ST_STAGES = 7, ST_CONSUMERS = 4, ST_THREADS = 32 * (1 + ST_CONSUMERS);
constexpr int ST_W_BYTES = ST_ROWS * ST_BK * 2, ST_X_BYTES = 8 * ST_BK * 2, ST_STAGE_BYTES = ST_W_BYTES + ST_X_BYTES;
constexpr size_t ST_SMEM = (size_t)ST_STAGES * ST_STAGE_BYTES + 1024 /* alignment slack */ + 128 /* barriers */;
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

// Grid (parts, slabs of 64 weight rows).  error: 1 the producer, 2 a consumer gave up waiting.
__global__ void __launch_bounds__(ST_THREADS, 3) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                                  float* __restrict__ y, int M, int N, int K, int* __restrict__ error) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(stages + (size_t)ST_STAGES * ST_STAGE_BYTES);
  uint64_t* empty = full + ST_STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = blockIdx.x, parts = gridDim.x, n0 = blockIdx.y * ST_ROWS;
  const int k_boxes = (K + ST_BK - 1) / ST_BK;
  const int box_begin = (int)((long long)part * k_boxes / parts), box_end = (int)((long long)(part + 1) * k_boxes / parts);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < ST_STAGES; ++s) { st_mbar_init(&full[s], 1); st_mbar_init(&empty[s], ST_CONSUMERS); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  if (warp == 0) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: the boxes that fit in the ring are asked for before
      // this kernel waits for it (a dependent launch may start while that kernel is still running); the activations'
      // boxes follow after the wait, on the same barriers.
      const int ahead = min(ST_STAGES, box_end - box_begin);
      for (int i = 0; i < ahead; ++i) {
        st_mbar_expect_tx(&full[i], ST_STAGE_BYTES);   // rows past N, M or K arrive as zeros and count all the same
        st_tma_load(stages + (size_t)i * ST_STAGE_BYTES, &map_w, &full[i], (box_begin + i) * ST_BK, n0);
      }
      grid_dependency_wait();
      allow_dependents();
      for (int i = 0; i < ahead; ++i)
        st_tma_load(stages + (size_t)i * ST_STAGE_BYTES + ST_W_BYTES, &map_x, &full[i], (box_begin + i) * ST_BK, 0);
      unsigned stage = 0, phase = 1;   // the ring has gone round once
      for (int box = box_begin + ahead; box < box_end; ++box) {
        if (!st_mbar_wait(&empty[stage], phase ^ 1)) { atomicExch(error, 1); break; }
        unsigned char* dst = stages + (size_t)stage * ST_STAGE_BYTES;
        st_mbar_expect_tx(&full[stage], ST_STAGE_BYTES);
        st_tma_load(dst, &map_w, &full[stage], box * ST_BK, n0);
        st_tma_load(dst + ST_W_BYTES, &map_x, &full[stage], box * ST_BK, 0);
        if (++stage == ST_STAGES) { stage = 0; phase ^= 1; }
      }
    }
    return;
  }
  grid_dependency_wait();   // before the result is written: its memory may be what that kernel still reads

  // Consumers.  In the 128-byte swizzle the 16-byte unit u of row r sits at unit u ^ (r % 8).
  const int slab_row = (warp - 1) * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);   // this lane's row of w for ldmatrix
  const unsigned w_row_offset = (unsigned)slab_row * 128, w_xor = (unsigned)(slab_row & 7);
  const unsigned x_row_offset = (unsigned)(lane & 7) * 128, x_xor = (unsigned)(lane & 7);
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // even and odd k-steps: two MMA chains
  unsigned stage = 0, phase = 0;
  bool alive = true;
  for (int box = box_begin; box < box_end; ++box) {
    if (!st_mbar_wait(&full[stage], phase)) { atomicExch(error, 2); alive = false; break; }
    const unsigned w_box = st_smem(stages + (size_t)stage * ST_STAGE_BYTES), x_box = w_box + ST_W_BYTES;
#pragma unroll
    for (int half = 0; half < 2; ++half) {   // 32 k each
      unsigned b[4];                          // x: units 4 * half .. + 3 of rows 0..7
      st_ldmatrix_x4(b, x_box + x_row_offset + ((((unsigned)(4 * half) + (lane >> 3)) ^ x_xor) << 4));
#pragma unroll
      for (int step = 0; step < 2; ++step) {  // 16 k each
        unsigned a[4];
        st_ldmatrix_x4(a, w_box + w_row_offset + ((((unsigned)(4 * half + 2 * step) + (lane >> 4)) ^ w_xor) << 4));
        st_mma(acc[step], a, b[2 * step], b[2 * step + 1]);
      }
    }
    __syncwarp();
    if (lane == 0) st_mbar_arrive(&empty[stage]);
    if (++stage == ST_STAGES) { stage = 0; phase ^= 1; }
  }
  if (!alive) return;

  // Accumulator element i of lane (g, t): weight row g + 8 * (i / 2), activation row 2 * t + (i % 2).
  const int g = lane >> 2, t = lane & 3;
  float* out = y + (size_t)part * M * N;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n0 + (warp - 1) * 16 + g + 8 * (i >> 1), m = 2 * t + (i & 1);
    if (n < N && m < M) out[(size_t)m * N + n] = acc[0][i] + acc[1][i];
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

}  // namespace pylon

// x: bfloat16 [M, K] (row stride ldx), M <= 8; w: bfloat16 [N, K] (row stride ldw); y: float32 [parts, M, N] contiguous,
// whose sum over the first dimension is x @ w.T.  K and the row strides multiples of 8, x and w 16-byte aligned,
// 1 <= parts <= number of 64-wide slices of k.  error: one int in device memory that the kernel sets non-zero if one of its
// waits ran out (the result is then void).
extern "C" int pylon_gemm_stream_partial(const void* x, const void* w, float* y, int M, int N, int K, long long ldx, long long ldw,
                                         int parts, int* error, cudaStream_t stream) {
  using namespace pylon;
  if (M <= 0 || N <= 0) return 0;
  if (M > 8) PYLON_REFUSE("gemm_stream: M = %d is more than 8 rows", M);
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8) PYLON_REFUSE("gemm_stream: K = %d and the row strides must be multiples of 8", K);
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)y % 4)) PYLON_REFUSE("gemm_stream: x and w must be 16-byte aligned");
  if (ldx < K || ldw < K) PYLON_REFUSE("gemm_stream: a row stride is shorter than its row");
  const int k_boxes = (K + ST_BK - 1) / ST_BK, slabs = (N + ST_ROWS - 1) / ST_ROWS;
  if (parts < 1 || parts > k_boxes || parts > 65535 || slabs > 65535) PYLON_REFUSE("gemm_stream: %d parts over %d slices of k, %d slabs", parts, k_boxes, slabs);
  if (!error) PYLON_REFUSE("gemm_stream: an error word is needed");
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ST_SMEM);
    if (err != cudaSuccess) PYLON_REFUSE("gemm_stream: %s", cudaGetErrorString(err));
    configured = true;
  }
  CUtensorMap map_w, map_x;
  if (!matrix_map(&map_w, w, N, K, ldw, ST_ROWS) || !matrix_map(&map_x, x, M, K, ldx, 8)) PYLON_REFUSE("gemm_stream: the tensor maps could not be made");
  launch_dependent<LAUNCH_GEMM>(gemm_stream_kernel, dim3(parts, slabs), dim3(ST_THREADS), ST_SMEM, stream, map_w, map_x, y, M, N, K, error);
  PYLON_CHECK_LAUNCH("gemm_stream");
}
