// Token selection from float32 logits, one block per row: arg-max, and temperature
// sampling with an optional nucleus (top-p) cut.
//
// Definitions follow raun6k/Pylon's Decoder._sample (src/pylon/decode/runner.py:509-525):
// temperature 0 is arg-max; otherwise p = softmax(logits / T); with top_p < 1 the tokens
// are taken in descending order of p and a token is dropped when the mass before it
// exceeds top_p (the first is always kept); the rest is renormalised and one token is
// drawn.  The draw here is an inverse-CDF walk in vocabulary order with a uniform number
// the host supplies per row, so a request's tokens do not depend on what it is batched
// with.  Tokens of exactly equal probability are kept or dropped together.
#include "common.cuh"

namespace pylon {

constexpr int SAMPLE_THREADS = 1024;

struct ArgMax {
  float value;
  int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // larger value wins; equal values: lower index wins; NaN never wins
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax v, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    ArgMax o{__shfl_xor_sync(0xffffffffu, v.value, offset), __shfl_xor_sync(0xffffffffu, v.index, offset)};
    v = better(v, o);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    ArgMax w = lane < warps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      ArgMax o{__shfl_xor_sync(0xffffffffu, w.value, offset), __shfl_xor_sync(0xffffffffu, w.index, offset)};
      w = better(w, o);
    }
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

// Mass of the entries whose weight exceeds the weight with bit pattern `bits`.
__device__ float mass_above(const float* __restrict__ logits, int vocab, float max_logit, float inv_t,
                            unsigned bits, float* scratch) {
  float s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float w = expf((logits[i] - max_logit) * inv_t);
    if (__float_as_uint(w) > bits) s += w;
  }
  return block_sum(s, scratch);
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ ArgMax arg_scratch[33];
  __shared__ float scratch[33];
  __shared__ float prefix[SAMPLE_THREADS];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)row * row_stride;

  ArgMax best{-INFINITY, 0x7fffffff};
  {
    // Sixteen values (four 16-byte loads) in flight per thread: a row of 150,000 logits is read in ten round trips.
    // The order in which a thread meets its values does not matter: `better` breaks ties by index.
    int first_scalar = 0;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
      const float4* x4 = reinterpret_cast<const float4*>(x);
      const int groups = vocab >> 2;
      auto take = [&](const float4& v, int group) {
        best = better(best, ArgMax{v.x, 4 * group});
        best = better(best, ArgMax{v.y, 4 * group + 1});
        best = better(best, ArgMax{v.z, 4 * group + 2});
        best = better(best, ArgMax{v.w, 4 * group + 3});
      };
      int i = tid;
      for (; i + 3 * SAMPLE_THREADS < groups; i += 4 * SAMPLE_THREADS) {
        const float4 v0 = x4[i], v1 = x4[i + SAMPLE_THREADS], v2 = x4[i + 2 * SAMPLE_THREADS], v3 = x4[i + 3 * SAMPLE_THREADS];
        take(v0, i); take(v1, i + SAMPLE_THREADS); take(v2, i + 2 * SAMPLE_THREADS); take(v3, i + 3 * SAMPLE_THREADS);
      }
      for (; i < groups; i += SAMPLE_THREADS) take(x4[i], i);
      first_scalar = groups << 2;
    }
    for (int i = first_scalar + tid; i < vocab; i += SAMPLE_THREADS) best = better(best, ArgMax{x[i], i});
  }
  best = block_argmax(best, arg_scratch);
  const float t = temperature ? temperature[row] : 0.f;
  if (!(t > 0.f) || best.index >= vocab) {  // greedy (or a row of NaN: index stays in range)
    if (tid == 0) out[row] = best.index < vocab ? best.index : 0;
    return;
  }
  const float inv_t = 1.f / t;
  const float max_logit = best.value;

  // Nucleus threshold: the smallest weight bit pattern b with mass_above(b) <= top_p * Z.
  // Weights are in (0, 1], so patterns order like values; a token is kept iff its
  // pattern is >= b.
  unsigned keep_from = 0;
  const float p_keep = top_p ? top_p[row] : 1.f;
  if (p_keep < 1.f) {
    const float total = mass_above(x, vocab, max_logit, inv_t, 0u, scratch);
    const float limit = p_keep * total;
    unsigned lo = 0, hi = __float_as_uint(1.0f);  // mass_above(hi) == 0 <= limit always
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      if (mass_above(x, vocab, max_logit, inv_t, mid, scratch) <= limit) hi = mid; else lo = mid + 1;
    }
    keep_from = lo;
  }

  // Inverse CDF in vocabulary order over the kept tokens; each thread owns one segment.
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = tid * per, end = min(begin + per, vocab);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) {
    const float w = expf((x[i] - max_logit) * inv_t);
    if (__float_as_uint(w) >= keep_from) mine += w;
  }
  prefix[tid] = mine;
  __syncthreads();
  if (tid == 0) {  // serial scan of 1024 partial sums: fixed order, negligible time
    float running = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) { const float v = prefix[i]; prefix[i] = running; running += v; }
    scratch[0] = running;
  }
  __syncthreads();
  const float kept = scratch[0];
  float u = uniform ? uniform[row] : 0.5f;
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  const float target = u * kept;
  __shared__ int chosen;
  if (tid == 0) chosen = -1;
  __syncthreads();
  // The owner of the segment in which the running mass first exceeds the target.
  const float before = prefix[tid];
  if (mine > 0.f && before <= target && target < before + mine) {
    float running = before;
    int pick = -1;
    for (int i = begin; i < end; ++i) {
      const float w = expf((x[i] - max_logit) * inv_t);
      if (__float_as_uint(w) >= keep_from) {
        running += w;
        pick = i;
        if (running > target) break;
      }
    }
    chosen = pick;
  }
  __syncthreads();
  // Rounding at a segment edge can leave no owner: fall back to the most likely token.
  if (tid == 0) out[row] = chosen >= 0 ? chosen : best.index;
}

}  // namespace pylon

// logits: float32 [rows, vocab] with `row_stride` elements between rows.  temperature, top_p
// and uniform are per row (device pointers; null temperature means arg-max for every row).
extern "C" int pylon_sample(const float* logits, long long row_stride, int rows, int vocab,
                            const float* temperature, const float* top_p, const float* uniform, int* out,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) PYLON_REFUSE("sample: vocabulary %d, row stride %lld", vocab, row_stride);
  pylon::sample_kernel<<<rows, pylon::SAMPLE_THREADS, 0, stream>>>(logits, row_stride, vocab, temperature, top_p,
                                                                   uniform, out);
  PYLON_CHECK_LAUNCH("sample");
}
