// Paged attention with split keys/values for callers that cannot allocate device memory.
//
// pylon_paged_attention_mma (attention_mma.cu) asks its caller for scratch memory when it
// splits the keys of a request over several blocks.  A caller that has no allocator to turn
// to at that moment — because the GPU's memory is already handed out to the last byte,
// because an allocation could stall a latency-critical loop, or because it links this
// library without PyTorch — uses pylon_paged_attention_mma_static instead: the same
// kernels, with the scratch in a fixed array inside this library.
//
// Rules of use:
//  * The scratch is PYLON_STATIC_SCRATCH_FLOATS floats (16 MiB).  A call needs
//    num_splits * total_tokens * nq * (head size + 1) floats when num_splits > 1 and none
//    otherwise; a call that needs more is refused with an error text and launches nothing.
//  * The first call on each device looks up the array's device address and raises the
//    kernels' shared-memory limit.  Make that first call outside any stream capture; later
//    calls only launch kernels and may be captured like any other launch.
//  * All calls on a device share the one array, and it keeps what the last call left.
//    Nothing in it has to start at zero: every slot a call reads was written earlier in
//    the same call.  But two calls whose kernels overlap on the GPU (different streams, or
//    graphs replayed side by side) race on it; keep calls that use splits in one stream
//    order.
//  * No cudaMalloc, cudaFree or allocating library routine is called, here or in the kernels.
//
// The array's name is a host-side handle in host code, not a device address; the address the
// kernels get comes from cudaGetSymbolAddress, once per device, with that device current.
#include "attention_static.h"

#include <mutex>

#include "attention_mma.cu"

static __device__ __align__(256) float pylon_static_scratch[PYLON_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* scratch_of_device[MAX_DEVICES] = {nullptr};
std::mutex setup_mutex;

// Device address of the built-in scratch on the current device (nullptr and an error text
// if the runtime refuses).
float* static_scratch_address() {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= MAX_DEVICES) {
    snprintf(pylon::last_error_buffer(), 512, "paged_attention_mma_static: no usable current device (%s)",
             err == cudaSuccess ? "index out of range" : cudaGetErrorString(err));
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(setup_mutex);
  if (scratch_of_device[device] == nullptr) {
    float* address = nullptr;
    err = cudaGetSymbolAddress((void**)&address, pylon_static_scratch);
    if (err != cudaSuccess || address == nullptr) {
      snprintf(pylon::last_error_buffer(), 512, "paged_attention_mma_static: cudaGetSymbolAddress failed (%s)", cudaGetErrorString(err));
      return nullptr;
    }
    scratch_of_device[device] = address;
  }
  return scratch_of_device[device];
}
}  // namespace

extern "C" long long pylon_static_scratch_floats() { return (long long)PYLON_STATIC_SCRATCH_FLOATS; }

extern "C" int pylon_paged_attention_mma_static(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                                void* out, const int* q_start, const int* kv_len, const int* block_table,
                                                int table_width, int page_size, int num_pages, int nq, int nkv, int window,
                                                float scale, int num_rows, int total_tokens, int max_q, int num_splits,
                                                cudaStream_t stream) {
  if (num_rows <= 0 || total_tokens <= 0) return 0;
  if (num_splits < 1 || nq < 1) PYLON_REFUSE("paged_attention_mma_static: splits %d, query heads %d", num_splits, nq);
  const long long needed = pylon_attention_scratch_floats(num_splits, total_tokens, nq);
  if (needed > (long long)PYLON_STATIC_SCRATCH_FLOATS)
    PYLON_REFUSE("paged_attention_mma_static: %d splits over %d tokens and %d heads need %lld floats of scratch; the built-in scratch holds %u",
                 num_splits, total_tokens, nq, needed, PYLON_STATIC_SCRATCH_FLOATS);
  float* scratch = static_scratch_address();
  if (scratch == nullptr) return -2;
  return pylon_paged_attention_mma(q, q_stride, k_pages, v_pages, out, scratch, nullptr, q_start, kv_len, block_table, table_width,
                                   page_size, num_pages, nq, nkv, window, scale, num_rows, total_tokens, max_q, num_splits, stream);
}
