// Shared helpers of the sm_100a kernels: element types, 32-bit conversions, reductions,
// and the error convention of the C entry points.
//
// Every entry point is `extern "C" int pylon_<name>(..., cudaStream_t stream)`.  It returns
// 0 when the launch was enqueued, or a negative code: -1 for arguments it refuses (the text
// is kept for pylon_last_error()), -2 when the CUDA runtime refused the launch.  No entry
// point allocates memory or synchronises.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

// Codes a kernel leaves in the error word it is given (0: all is well).  1 to 4: a bounded wait of the kernel ran out
// or its shared memory was not where it must be (each kernel's own meaning).
#define PYLON_ERROR_BAD_PAGE 5   // a block table named a page that the pool does not have: nothing was read or written there
#define PYLON_DTYPE_F32 0
#define PYLON_DTYPE_BF16 1

namespace pylon {

// What a library sets up once per device (function attributes, occupancy figures) is kept in small arrays indexed
// by the current device's number.
constexpr int MAX_DEVICES = 64;
inline int current_device_slot() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0) device = 0;
  return device % MAX_DEVICES;
}
// Multiprocessors of the current device (asked once per device): grid-stride kernels size their grids by it.
inline int multiprocessors() {
  static int counts[MAX_DEVICES] = {};
  int& count = counts[current_device_slot()];
  if (count == 0) {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) == cudaSuccess && cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) == cudaSuccess) count = value;
  }
  return count > 0 ? count : 1;
}

// Text of the last refused call in this thread's library.
inline char* last_error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

#define PYLON_REFUSE(...)                                              \
  do {                                                                 \
    snprintf(pylon::last_error_buffer(), 512, __VA_ARGS__);            \
    return -1;                                                         \
  } while (0)

#define PYLON_CHECK_LAUNCH(name)                                       \
  do {                                                                 \
    cudaError_t err__ = cudaGetLastError();                            \
    if (err__ != cudaSuccess) {                                        \
      snprintf(pylon::last_error_buffer(), 512, "%s: %s", name,        \
               cudaGetErrorString(err__));                             \
      return -2;                                                       \
    }                                                                  \
    return 0;                                                          \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds
// at least 33 floats of shared memory.  Safe to call repeatedly with the same scratch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? scratch[lane] : 0.f;
    w = warp_sum(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < warps ? scratch[lane] : -INFINITY;
    w = warp_max(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

// Programmatic dependent launch: a kernel launched with launch_dependent() may start while
// the kernel before it in the stream is still running.  It must call grid_dependency_wait()
// before it reads anything that kernel writes (and before it writes anything that kernel
// reads); what it does before that - index arithmetic, loads of weights - overlaps the
// predecessor's tail.  allow_dependents() lets the next kernel in the stream start early in
// the same way.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

// On for every launch made through launch_dependent unless PYLON_B200_PDL says otherwise ("0": off; "gemm": only
// the weight-streaming products).  Each of these kernels does what does not depend on its predecessor before it
// waits (the products ask for their first weights, the decode attention makes its plan from the rows' lengths and
// asks for its first old tile, the rotation looks up position, page and angles, the norm loads its weights) and lets
// its own dependents start only after its wait, so at most two kernels share the GPU.  Measured on the decode step of
// the Qwen3-4B shape, batch 8: 3.06 ms with, 3.26 ms without (batch 1: 2.50 against 2.79 ms).
enum LaunchKind { LAUNCH_OTHER = 0, LAUNCH_GEMM = 1 };
inline bool dependent_launch_enabled(LaunchKind kind) {
  static const int mode = [] {
    const char* value = getenv("PYLON_B200_PDL");
    if (!value || value[0] == '1') return 1;
    return value[0] == 'g' ? 2 : 0;
  }();
  return mode == 1 || (mode == 2 && kind == LAUNCH_GEMM);
}

template <LaunchKind KIND = LAUNCH_OTHER, typename... KernelArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled(KIND) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// The same with the grid's blocks grouped into thread-block clusters of `cluster` along x (the grid's x a multiple of it).
template <LaunchKind KIND = LAUNCH_OTHER, typename... KernelArgs, typename... Args>
inline cudaError_t launch_dependent_cluster(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster,
                                            Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = dependent_launch_enabled(KIND) ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

}  // namespace pylon

// One copy per shared library (each library is built from one translation unit; weak in case
// several are linked together).
extern "C" __attribute__((weak)) const char* pylon_last_error() { return pylon::last_error_buffer(); }
