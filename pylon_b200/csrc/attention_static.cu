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
//    pylon_attention_scratch_floats() of them: room for the splits of long rows and for the
//    segments of decoded rows.  The number of blocks for decoded rows is chosen here, as
//    many as the device holds at once, fewer if the scratch would not hold their slots; a
//    call that needs more than the array even then is refused with an error text and
//    launches nothing.
//  * The counters by which the blocks of a decoded row find out which of them is last are a
//    second fixed array (PYLON_STATIC_COUNTERS entries; rows x KV heads beyond that are
//    refused).  They start at zero when the library is loaded and every launch that runs to
//    its end leaves them at zero.  A kernel that gives up a bounded wait (pylon_static_error_word()
//    is then non-zero and that call's output void) can leave counters of the rows it shared
//    behind: call pylon_static_reset() before the entry point is used again.
//  * The first call on each device looks up the arrays' device addresses and raises the
//    kernels' shared-memory limit.  Make that first call outside any stream capture; later
//    calls only launch kernels and may be captured like any other launch.
//  * All calls on a device share the arrays, and the scratch keeps what the last call left.
//    Nothing in it has to start at zero: every slot a call reads was written earlier in
//    the same call.  But two calls whose kernels overlap on the GPU (different streams, or
//    graphs replayed side by side) race on them; keep calls in one stream order.
//  * No cudaMalloc, cudaFree or allocating library routine is called, here or in the kernels.
//
// The arrays' names are host-side handles in host code, not device addresses; the addresses
// the kernels get come from cudaGetSymbolAddress, once per device, with that device current.
#include "attention_static.h"

#include <mutex>

#include "attention_mma.cu"

static __device__ __align__(256) float pylon_static_scratch[PYLON_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned pylon_static_counters[PYLON_STATIC_COUNTERS];
static __device__ int pylon_static_error;   // set by a kernel whose bounded wait for a TMA copy ran out

namespace {
using pylon::MAX_DEVICES;
float* scratch_of_device[MAX_DEVICES] = {nullptr};
unsigned* counters_of_device[MAX_DEVICES] = {nullptr};
int* error_of_device[MAX_DEVICES] = {nullptr};
std::mutex setup_mutex;

// Device addresses of the built-in scratch and counters on the current device (nullptr and an
// error text if the runtime refuses).
float* static_scratch_address(unsigned** counters, int** error) {
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
    unsigned* counter_address = nullptr;
    err = cudaGetSymbolAddress((void**)&counter_address, pylon_static_counters);
    if (err != cudaSuccess || counter_address == nullptr) {
      snprintf(pylon::last_error_buffer(), 512, "paged_attention_mma_static: cudaGetSymbolAddress failed (%s)", cudaGetErrorString(err));
      return nullptr;
    }
    int* error_address = nullptr;
    err = cudaGetSymbolAddress((void**)&error_address, pylon_static_error);
    if (err != cudaSuccess || error_address == nullptr) {
      snprintf(pylon::last_error_buffer(), 512, "paged_attention_mma_static: cudaGetSymbolAddress failed (%s)", cudaGetErrorString(err));
      return nullptr;
    }
    counters_of_device[device] = counter_address;
    error_of_device[device] = error_address;
    scratch_of_device[device] = address;
  }
  *counters = counters_of_device[device];
  *error = error_of_device[device];
  return scratch_of_device[device];
}
}  // namespace

extern "C" long long pylon_static_scratch_floats() { return (long long)PYLON_STATIC_SCRATCH_FLOATS; }

// 0, or non-zero after a kernel of an earlier call on the current device gave up waiting for a TMA copy (its output is
// void); -1 if the word cannot be read.  Synchronises the device.
extern "C" int pylon_static_error_word() {
  int value = -1;
  if (cudaMemcpyFromSymbol(&value, pylon_static_error, sizeof(int)) != cudaSuccess) return -1;
  return value;
}

// Puts the built-in counters and the error word of the current device back to zero.  For use after
// pylon_static_error_word() came back non-zero: the kernel that gave up did not take part in the count of the rows it
// shared, so their counters are not where the next call expects them.  Waits for the device first (nothing of an
// earlier call may still be counting).  0, or -2 with an error text.  Allocates nothing.
extern "C" int pylon_static_reset() {
  unsigned* counters = nullptr;
  int* error = nullptr;
  if (static_scratch_address(&counters, &error) == nullptr) return -2;
  cudaError_t err = cudaDeviceSynchronize();
  if (err == cudaSuccess) err = cudaMemset(counters, 0, sizeof(unsigned) * PYLON_STATIC_COUNTERS);
  if (err == cudaSuccess) err = cudaMemset(error, 0, sizeof(int));
  if (err == cudaSuccess) err = cudaDeviceSynchronize();
  if (err != cudaSuccess) {
    snprintf(pylon::last_error_buffer(), 512, "pylon_static_reset: %s", cudaGetErrorString(err));
    return -2;
  }
  return 0;
}

// For tests of the error handling, which make no kernel give up: writes counter `pair` and the error word from the
// host, as a kernel that ran out of patience would have left them.  0, or -2 with an error text.
extern "C" int pylon_static_inject(int pair, unsigned count, int error_code) {
  unsigned* counters = nullptr;
  int* error = nullptr;
  if (static_scratch_address(&counters, &error) == nullptr) return -2;
  if (pair < 0 || pair >= (int)PYLON_STATIC_COUNTERS) PYLON_REFUSE("pylon_static_inject: counter %d of %u", pair, PYLON_STATIC_COUNTERS);
  cudaError_t err = cudaDeviceSynchronize();
  if (err == cudaSuccess) err = cudaMemcpy(counters + pair, &count, sizeof(unsigned), cudaMemcpyHostToDevice);
  if (err == cudaSuccess) err = cudaMemcpy(error, &error_code, sizeof(int), cudaMemcpyHostToDevice);
  if (err != cudaSuccess) {
    snprintf(pylon::last_error_buffer(), 512, "pylon_static_inject: %s", cudaGetErrorString(err));
    return -2;
  }
  return 0;
}

extern "C" int pylon_paged_attention_mma_static(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                                void* out, const int* q_start, const int* kv_len, const int* block_table,
                                                int table_width, int page_size, int num_pages, int nq, int nkv, int window,
                                                float scale, int num_rows, int total_tokens, int max_q, int num_splits,
                                                cudaStream_t stream) {
  if (num_rows <= 0 || total_tokens <= 0) return 0;
  if (num_splits < 1 || nq < 1 || nkv < 1 || max_q < 1) PYLON_REFUSE("paged_attention_mma_static: splits %d, query heads %d, KV heads %d, longest row %d", num_splits, nq, nkv, max_q);
  // Rows of decoded tokens (at most 16 packed query rows) can occur unless the call is one long row.
  const bool maybe_small = (long long)max_q * (nq / nkv) <= pylon::SMALL_ROWS || num_rows > 1;
  int decode_blocks = 0;
  if (maybe_small) {
    if ((long long)num_rows * nkv > (long long)PYLON_STATIC_COUNTERS)
      PYLON_REFUSE("paged_attention_mma_static: %d rows x %d KV heads need more than the %u built-in counters", num_rows, nkv, PYLON_STATIC_COUNTERS);
    decode_blocks = pylon_attention_decode_blocks();
    if (decode_blocks < 1) PYLON_REFUSE("paged_attention_mma_static: the decode kernel does not fit on this device");
    while (decode_blocks > 1 && pylon_attention_scratch_floats(num_splits, total_tokens, nq, num_rows, nkv, decode_blocks) > (long long)PYLON_STATIC_SCRATCH_FLOATS)
      decode_blocks /= 2;
  }
  const long long needed = pylon_attention_scratch_floats(num_splits, total_tokens, nq, num_rows, nkv, decode_blocks);
  if (needed > (long long)PYLON_STATIC_SCRATCH_FLOATS)
    PYLON_REFUSE("paged_attention_mma_static: %d splits over %d tokens and %d heads, %d rows and %d decode blocks need %lld floats of scratch; the built-in scratch holds %u",
                 num_splits, total_tokens, nq, num_rows, decode_blocks, needed, PYLON_STATIC_SCRATCH_FLOATS);
  unsigned* counters = nullptr;
  int* error = nullptr;
  float* scratch = static_scratch_address(&counters, &error);
  if (scratch == nullptr) return -2;
  return pylon_paged_attention_mma(q, q_stride, k_pages, v_pages, out, scratch, counters, q_start, kv_len, block_table, table_width,
                                   page_size, num_pages, nq, nkv, window, scale, num_rows, total_tokens, max_q, num_splits, decode_blocks, 0,
                                   0 /* nothing is known about the rows' lengths */, error, stream);
}
