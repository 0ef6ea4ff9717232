// Paged causal attention, the plain form: one block per (token, query head), any head size
// up to 512, any page size, any group size, optional window.  It is the attention of the
// true 32-bit path and the fall-back of the bfloat16 path for head sizes the tensor-core
// kernel is not built for.  Scores, softmax and the weighted sum are float32.
//
// Semantics (raun6k/Pylon: src/pylon/kv/cache.py:462-476 on the GPU, its exact restatement
// 483-491): a token at position p of its request attends the keys at positions j <= p of
// the same request (and j > p - window when a window is given); scale 1/sqrt(head size)
// unless another is passed; query head h reads KV head h / (nq / nkv).
//
// The keys of a token are walked in chunks of 128 positions aligned at position 0, so a
// token's result depends on its position only, not on how the step was cut or batched.
#include "common.cuh"

namespace pylon {

constexpr int SIMPLE_THREADS = 128;
constexpr int SIMPLE_MAX_DIMS_PER_THREAD = 4;  // head size <= 512

template <typename T>
__global__ void __launch_bounds__(SIMPLE_THREADS) paged_attention_simple_kernel(
    const T* __restrict__ q, long long q_token_stride, const T* __restrict__ k_pages,
    const T* __restrict__ v_pages, T* __restrict__ out, const int* __restrict__ positions,
    const int* __restrict__ token_row, const int* __restrict__ block_table, int table_width, int page_size,
    int num_pages, int nq, int nkv, int d, int window, float scale) {
  extern __shared__ long long shared[];
  long long* offsets = shared;                                      // [128] element offsets of key rows
  float* probs = reinterpret_cast<float*>(offsets + SIMPLE_THREADS);  // [128]
  float* scratch = probs + SIMPLE_THREADS;                          // [33]
  float* qs = scratch + 34;                                         // [d]

  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kv_head = h / (nq / nkv);
  const int pos = positions[t];
  const int row = token_row[t];
  if (row < 0) return;   // a padding token of a step padded to a captured size: it belongs to no request, its output is never read
  const int* table = block_table + (size_t)row * table_width;
  const T* qrow = q + (size_t)t * q_token_stride + (size_t)h * d;
  for (int e = tid; e < d; e += SIMPLE_THREADS) qs[e] = to_float<T>(qrow[e]) * scale;

  const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  float acc[SIMPLE_MAX_DIMS_PER_THREAD];
#pragma unroll
  for (int k = 0; k < SIMPLE_MAX_DIMS_PER_THREAD; ++k) acc[k] = 0.f;
  float running_max = -INFINITY, running_sum = 0.f;
  __syncthreads();

  for (int c0 = (lo / SIMPLE_THREADS) * SIMPLE_THREADS; c0 <= pos; c0 += SIMPLE_THREADS) {
    const int j = c0 + tid;
    float score = -INFINITY;
    long long offset = -1;
    if (j >= lo && j <= pos) {
      const int page = table[j / page_size];
      if (page >= 0 && page < num_pages) {
        offset = (((long long)page * nkv + kv_head) * page_size + j % page_size) * d;
        const T* krow = k_pages + offset;
        float dot = 0.f;
        for (int e = 0; e < d; ++e) dot = fmaf(qs[e], to_float<T>(krow[e]), dot);
        score = dot;
      }
    }
    offsets[tid] = offset;
    const float chunk_max = block_max(score, scratch);
    const float new_max = fmaxf(running_max, chunk_max);
    // new_max is finite: the chunk holds at least key `pos` (or an earlier chunk did).
    const float p = offset >= 0 ? expf(score - new_max) : 0.f;
    probs[tid] = p;
    const float chunk_sum = block_sum(p, scratch);  // also orders probs/offsets writes
    const float rescale = running_max == -INFINITY ? 0.f : expf(running_max - new_max);
    running_sum = running_sum * rescale + chunk_sum;
    running_max = new_max;
    const int valid = pos - c0 + 1 < SIMPLE_THREADS ? pos - c0 + 1 : SIMPLE_THREADS;
#pragma unroll
    for (int k = 0; k < SIMPLE_MAX_DIMS_PER_THREAD; ++k) {
      const int e = tid + k * SIMPLE_THREADS;
      if (e < d) {
        float a = acc[k] * rescale;
        for (int i = 0; i < valid; ++i) {
          const long long off = offsets[i];
          if (off >= 0) a = fmaf(probs[i], to_float<T>(v_pages[off + e]), a);
        }
        acc[k] = a;
      }
    }
    __syncthreads();
  }
  T* orow = out + ((size_t)t * nq + h) * d;
  const float inv = running_sum > 0.f ? 1.f / running_sum : 0.f;
#pragma unroll
  for (int k = 0; k < SIMPLE_MAX_DIMS_PER_THREAD; ++k) {
    const int e = tid + k * SIMPLE_THREADS;
    if (e < d) orow[e] = from_float<T>(acc[k] * inv);
  }
}

}  // namespace pylon

using namespace pylon;

extern "C" int pylon_paged_attention_simple(const void* q, long long q_token_stride, const void* k_pages,
                                            const void* v_pages, void* out, const int* positions,
                                            const int* token_row, const int* block_table, int table_width,
                                            int page_size, int num_pages, int nq, int nkv, int d, int window,
                                            float scale, int num_tokens, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (d < 1 || d > SIMPLE_THREADS * SIMPLE_MAX_DIMS_PER_THREAD)
    PYLON_REFUSE("paged_attention_simple: head size %d is outside 1..%d", d, SIMPLE_THREADS * SIMPLE_MAX_DIMS_PER_THREAD);
  if (nkv < 1 || nq < 1 || nq % nkv) PYLON_REFUSE("paged_attention_simple: %d query heads over %d KV heads", nq, nkv);
  if (nq > 65535) PYLON_REFUSE("paged_attention_simple: %d query heads", nq);
  if (page_size < 1 || table_width < 1 || window < 0)
    PYLON_REFUSE("paged_attention_simple: page size %d, table width %d, window %d", page_size, table_width, window);
  const size_t smem = (size_t)(d + SIMPLE_THREADS + 34) * sizeof(float) + SIMPLE_THREADS * sizeof(long long) + 8;
  dim3 grid(num_tokens, nq);
  if (dtype == PYLON_DTYPE_F32)
    paged_attention_simple_kernel<float><<<grid, SIMPLE_THREADS, smem, stream>>>(
        (const float*)q, q_token_stride, (const float*)k_pages, (const float*)v_pages, (float*)out, positions,
        token_row, block_table, table_width, page_size, num_pages, nq, nkv, d, window, scale);
  else if (dtype == PYLON_DTYPE_BF16)
    paged_attention_simple_kernel<__nv_bfloat16><<<grid, SIMPLE_THREADS, smem, stream>>>(
        (const __nv_bfloat16*)q, q_token_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
        (__nv_bfloat16*)out, positions, token_row, block_table, table_width, page_size, num_pages, nq, nkv, d,
        window, scale);
  else
    PYLON_REFUSE("paged_attention_simple: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("paged_attention_simple");
}
