// y[M, N] = x[M, K] * W[N, K]^T for bfloat16 with few rows (M <= 64): the matrix products
// of a decode step, where the time goes to streaming the weights from HBM once.
//
// The weight matrix is the "A" operand of mma.sync.m16n8k16 (16 weight rows x 16 k) and the
// activations are "B" (16 k x 8 rows of x), so 16 output features fill the tensor core's M
// dimension however small the batch is.  Every thread loads its fragments straight from
// global memory as 16-byte vectors: lane (g, t) reads W[n0+g][k0+8t .. k0+8t+7] (and row
// n0+g+8) and x[m][k0+8t ..]; since a dot product does not care in which order k is summed,
// those 8 consecutive elements serve as the lane's k-slots of two MMAs, and no shared-memory
// staging or ldmatrix is needed.  The warps of a block take interleaved 32-wide k-steps of
// the same weight rows (so a block reads contiguous 512-byte runs) and their partial sums
// are added in shared memory in a fixed order.  Loads are double-buffered in registers.
//
// Stands in for the library products raun6k/Pylon's nn.Linear layers call at decode
// (src/pylon/model/layers.py:26-27,126,138; src/pylon/model/model.py:144).
#include "common.cuh"

namespace pylon {

__device__ __forceinline__ uint4 load_stream_16(const void* p) {   // weights: read once, keep out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Activations: shared by every block, so they may stay in L1; an ordinary (coherent) load, because under a dependent
// launch the kernel that writes them may still be running when this one starts.
__device__ __forceinline__ uint4 load_cached_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename OutT>
__device__ __forceinline__ void store_out(OutT* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// MT: 8-row tiles of x (M <= 8 * MT).  NT: 16-row tiles of W per block.  WARPS: k-split
// inside a block.
template <int MT, int NT, int WARPS, int UNROLL, typename OutT>
__global__ void __launch_bounds__(WARPS * 32) gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                 OutT* __restrict__ y, int M, int N, int K, long long ldx, long long ldw, long long ldy) {
  extern __shared__ float reduce[];   // [WARPS][NT * 16][MT * 8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * (NT * 16);
  const int step_begin = 0, k_steps = (K + 31) / 32;

  const __nv_bfloat16* w_rows[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = min(n0 + nt * 16 + g + 8 * h, N - 1);   // rows past N read a valid row and are not stored
      w_rows[nt][h] = w + (size_t)n * ldw + t * 8;
    }
  }
  const __nv_bfloat16* x_rows[MT];
  bool x_valid[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int m = mt * 8 + g;
    x_valid[mt] = m < M;
    x_rows[mt] = x + (size_t)(x_valid[mt] ? m : 0) * ldx + t * 8;
  }

  float acc[NT][MT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[nt][mt][0] = acc[nt][mt][1] = acc[nt][mt][2] = acc[nt][mt][3] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  constexpr int STRIDE = WARPS * UNROLL;   // k-steps between a warp's successive groups of UNROLL steps
  // Two register buffers: the loads of the next group are in flight while this group's MMAs run.
  uint4 wa[UNROLL][NT][2], xa[UNROLL][MT], wb[UNROLL][NT][2], xb[UNROLL][MT];
  auto load_weights = [&](uint4 (&wf)[UNROLL][NT][2], int ks0) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (ks0 + u * WARPS) * 32;
      // K is a multiple of 8: a lane's 8 elements are all in or all out; steps past this block's share load nothing
      const bool in_range = k + t * 8 < K && ks0 + u * WARPS < k_steps;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        wf[u][nt][0] = in_range ? load_stream_16(w_rows[nt][0] + k) : zero;
        wf[u][nt][1] = in_range ? load_stream_16(w_rows[nt][1] + k) : zero;
      }
    }
  };
  auto load_activations = [&](uint4 (&xf)[UNROLL][MT], int ks0) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (ks0 + u * WARPS) * 32;
      const bool in_range = k + t * 8 < K && ks0 + u * WARPS < k_steps;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xf[u][mt] = (in_range && x_valid[mt]) ? load_cached_16(x_rows[mt] + k) : zero;
    }
  };
  auto multiply = [&](const uint4 (&wf)[UNROLL][NT][2], const uint4 (&xf)[UNROLL][MT]) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 lo = wf[u][nt][0], hi = wf[u][nt][1];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 b = xf[u][mt];
          mma_16816(acc[nt][mt], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
          mma_16816(acc[nt][mt], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
      }
    }
  };

  // The weights do not depend on the kernel before this one: the fragments of both register
  // buffers are on their way before this kernel waits for its activations.  (Asking L2 for the block's whole
  // weight slab up front with cp.async.bulk.prefetch.L2 was measured slower: 22 against 18
  // microseconds on the 19456 x 2560 product.)
  int ks0 = step_begin + warp;
  load_weights(wa, ks0);
  bool second_loaded = ks0 + STRIDE < k_steps;   // both register buffers are filled before the wait
  if (second_loaded) load_weights(wb, ks0 + STRIDE);
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  load_activations(xa, ks0);
  for (; ks0 < k_steps; ks0 += 2 * STRIDE) {
    const bool more = ks0 + STRIDE < k_steps;
    if (more) {
      if (!second_loaded) load_weights(wb, ks0 + STRIDE);
      second_loaded = false;
      load_activations(xb, ks0 + STRIDE);
    }
    multiply(wa, xa);
    if (more) {
      if (ks0 + 2 * STRIDE < k_steps) { load_weights(wa, ks0 + 2 * STRIDE); load_activations(xa, ks0 + 2 * STRIDE); }
      multiply(wb, xb);
    }
  }

  // Add the warps' partial sums in a fixed order and store.  Accumulator element i of lane
  // (g, t): weight row g + 8 * (i / 2), x row 2 * t + (i % 2).
  constexpr int ROWS = NT * 16, COLS = MT * 8;
  float* mine = reduce + (size_t)warp * ROWS * COLS;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) mine[(mt * 8 + 2 * t + (i & 1)) * ROWS + nt * 16 + g + 8 * (i >> 1)] = acc[nt][mt][i];
  __syncthreads();
  for (int e = threadIdx.x; e < ROWS * COLS; e += WARPS * 32) {
    const int m = e / ROWS, n = n0 + e % ROWS;
    if (m < M && n < N) {
      float sum = 0.f;
#pragma unroll
      for (int wv = 0; wv < WARPS; ++wv) sum += reduce[(size_t)wv * ROWS * COLS + e];
      store_out<OutT>(y + (size_t)m * ldy + n, sum);
    }
  }
}

template <int MT, int NT, int WARPS, int UNROLL, typename OutT>
static int launch_skinny(const __nv_bfloat16* x, const __nv_bfloat16* w, OutT* y, int M, int N, int K, long long ldx,
                         long long ldw, long long ldy, cudaStream_t stream) {
  constexpr size_t smem = (size_t)WARPS * NT * 16 * MT * 8 * sizeof(float);
  auto kernel = gemm_skinny_kernel<MT, NT, WARPS, UNROLL, OutT>;
  if (smem > 48 * 1024) {
    static bool configured_on[pylon::MAX_DEVICES] = {};   // function attributes belong to a device
  bool& configured = configured_on[pylon::current_device_slot()];
    if (!configured) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) PYLON_REFUSE("gemm_skinny: %s", cudaGetErrorString(err));
      configured = true;
    }
  }
  const int blocks = (N + NT * 16 - 1) / (NT * 16);
  launch_dependent<LAUNCH_GEMM>(kernel, dim3(blocks), dim3(WARPS * 32), smem, stream, x, w, y, M, N, K, ldx, ldw, ldy);
  PYLON_CHECK_LAUNCH("gemm_skinny");
}

template <typename OutT>
static int dispatch_skinny(const __nv_bfloat16* x, const __nv_bfloat16* w, OutT* y, int M, int N, int K, long long ldx,
                           long long ldw, long long ldy, cudaStream_t stream) {
  if (M <= 8) return launch_skinny<1, 1, 8, 2, OutT>(x, w, y, M, N, K, ldx, ldw, ldy, stream);
  if (M <= 16) return launch_skinny<2, 1, 8, 2, OutT>(x, w, y, M, N, K, ldx, ldw, ldy, stream);
  if (M <= 32) return launch_skinny<4, 1, 8, 1, OutT>(x, w, y, M, N, K, ldx, ldw, ldy, stream);
  return launch_skinny<8, 2, 4, 1, OutT>(x, w, y, M, N, K, ldx, ldw, ldy, stream);
}

}  // namespace pylon

// x: bfloat16 [M, K] (row stride ldx), w: bfloat16 [N, K] (row stride ldw), y: [M, N] (row
// stride ldy) in bfloat16 (out_dtype 1) or float32 (out_dtype 0).  M <= 64; K and the row
// strides of x and w multiples of 8; x and w 16-byte aligned.
extern "C" int pylon_gemm_skinny_bf16(const void* x, const void* w, void* y, int M, int N, int K, long long ldx,
                                      long long ldw, long long ldy, int out_dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) PYLON_REFUSE("gemm_skinny: M = %d is more than 64 rows", M);
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8) PYLON_REFUSE("gemm_skinny: K = %d and the row strides must be multiples of 8", K);
  if (((uintptr_t)x % 16) || ((uintptr_t)w % 16)) PYLON_REFUSE("gemm_skinny: x and w must be 16-byte aligned");
  if (ldx < K || ldw < K || ldy < N) PYLON_REFUSE("gemm_skinny: a row stride is shorter than its row");
  if (out_dtype == PYLON_DTYPE_BF16)
    return pylon::dispatch_skinny<__nv_bfloat16>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, M, N, K, ldx, ldw, ldy, stream);
  if (out_dtype == PYLON_DTYPE_F32)
    return pylon::dispatch_skinny<float>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)y, M, N, K, ldx, ldw, ldy, stream);
  PYLON_REFUSE("gemm_skinny: unknown result dtype %d", out_dtype);
}
