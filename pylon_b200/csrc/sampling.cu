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

// Where a launch leaves a second copy of its result for the host, in pinned host memory that the device can write
// (null: none): the tokens, and the kernels' error words as they stand when the step's last kernel, this one, runs.  The
// host then needs no copy behind the launch, only to wait for it.
struct SampleMirror {
  int* tokens;          // [rows]
  const int* words;     // [4] on the device
  int* words_copy;      // [4]
};
__device__ __forceinline__ void sample_emit(int* __restrict__ out, const SampleMirror& mirror, int row, int token) {
  out[row] = token;
  if (mirror.tokens) mirror.tokens[row] = token;
  if (row == 0 && mirror.words_copy) {
#pragma unroll
    for (int i = 0; i < 4; ++i) mirror.words_copy[i] = mirror.words[i];
  }
}

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
    const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out, const SampleMirror mirror) {
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
    if (tid == 0) sample_emit(out, mirror, row, best.index < vocab ? best.index : 0);
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
  __shared__ unsigned chosen;   // the lowest index an owner found; all ones: none
  if (tid == 0) chosen = 0xffffffffu;
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
    if (pick >= 0) atomicMin(&chosen, (unsigned)pick);   // rounding can give a target two owners: the lower index, every time
  }
  __syncthreads();
  // Rounding at a segment edge can leave no owner: fall back to the most likely token.
  if (tid == 0) sample_emit(out, mirror, row, chosen != 0xffffffffu ? (int)chosen : best.index);
}


// -----------------------------------------------------------------------------------------
// The same choice with a row spread over a thread-block cluster: every block keeps the weights of
// its slice of the vocabulary in shared memory, so that the passes over the row (the sum, each
// step of the nucleus threshold's bisection, the inverse CDF) read shared memory instead of
// computing 150,000 exponentials from L2 again, and the blocks add their partial sums up through
// distributed shared memory.  With one block per row and top_p < 1 a row of 151,936 logits took
// 990 us (thirty passes); the default sampling options (temperature 0.2, top_p 0.95) take that
// path at every decode step.
//
// Sums are added in a fixed order (threads of a block by block_sum, blocks by rank), and every
// block works out every decision from the same numbers: all of them take the same turns and meet
// at every cluster barrier.
// -----------------------------------------------------------------------------------------
constexpr int SAMPLE_CLUSTER = 8;

__device__ __forceinline__ unsigned sample_cluster_rank() {
  unsigned rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void sample_cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Stores `value` into the same shared-memory location of block `rank` of the cluster.
__device__ __forceinline__ void sample_send(void* own, unsigned rank, unsigned value) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(own)), "r"(rank));
  asm volatile("st.shared::cluster.u32 [%0], %1;\n" ::"r"(remote), "r"(value) : "memory");
}

// One value from every block to every block: `slots` is [SAMPLE_CLUSTER] in each block's shared memory.  The caller uses
// two sets of slots in turn, so that a block that is a step ahead does not write over what another still reads.
__device__ __forceinline__ void sample_exchange(unsigned* slots, unsigned rank, unsigned value) {
  if (threadIdx.x < SAMPLE_CLUSTER) sample_send(&slots[rank], threadIdx.x, value);
  sample_cluster_barrier();
}
__device__ __forceinline__ float sample_total(const unsigned* slots) {
  float total = 0.f;
#pragma unroll
  for (int c = 0; c < SAMPLE_CLUSTER; ++c) total += __uint_as_float(slots[c]);
  return total;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_cluster_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, int slice, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out, const SampleMirror mirror) {
  extern __shared__ float weights[];   // [slice]: this block's share of the row
  __shared__ ArgMax arg_scratch[33];
  __shared__ float scratch[33];
  __shared__ float prefix[SAMPLE_THREADS];
  __shared__ unsigned slots[2][SAMPLE_CLUSTER], index_slots[SAMPLE_CLUSTER];
  __shared__ unsigned chosen;   // the lowest index an owner found; all ones: none
  const unsigned rank = sample_cluster_rank();
  const int row = blockIdx.x / SAMPLE_CLUSTER, tid = threadIdx.x;
  const float* x = logits + (size_t)row * row_stride;
  const int begin = min(vocab, (int)rank * slice), end = min(vocab, begin + slice), count = end - begin;

  // The largest logit: of the slice, then of the row (ties: the lower index).
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = tid; i < count; i += SAMPLE_THREADS) best = better(best, ArgMax{x[begin + i], begin + i});
  best = block_argmax(best, arg_scratch);
  sample_cluster_barrier();   // every block of the cluster has started: its shared memory may be written from here on
  if (tid < SAMPLE_CLUSTER) {
    sample_send(&slots[0][rank], tid, __float_as_uint(best.value));
    sample_send(&index_slots[rank], tid, (unsigned)best.index);
  }
  sample_cluster_barrier();
  best = ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int c = 0; c < SAMPLE_CLUSTER; ++c) best = better(best, ArgMax{__uint_as_float(slots[0][c]), (int)index_slots[c]});
  const float t = temperature ? temperature[row] : 0.f;
  if (!(t > 0.f) || best.index >= vocab) {   // greedy (or a row of NaN: the index stays in range): the same for every block
    if (rank == 0 && tid == 0) sample_emit(out, mirror, row, best.index < vocab ? best.index : 0);
    return;
  }
  const float inv_t = 1.f / t, max_logit = best.value;

  // The weights, once, into shared memory; their sum.
  float mine = 0.f;
  for (int i = tid; i < count; i += SAMPLE_THREADS) {
    const float w = expf((x[begin + i] - max_logit) * inv_t);
    weights[i] = w;
    mine += w;
  }
  int turn = 1;
  sample_exchange(slots[turn], rank, __float_as_uint(block_sum(mine, scratch)));
  const float total = sample_total(slots[turn]);

  // Nucleus threshold: the smallest weight bit pattern b with (mass of the weights above b) <= top_p * Z.  Weights are in
  // (0, 1], so patterns order like values; a token is kept iff its pattern is >= b.
  unsigned keep_from = 0;
  const float p_keep = top_p ? top_p[row] : 1.f;
  if (p_keep < 1.f) {
    const float limit = p_keep * total;
    unsigned lo = 0, hi = __float_as_uint(1.0f);   // nothing lies above 1: that mass is 0 <= limit
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      float above = 0.f;
      for (int i = tid; i < count; i += SAMPLE_THREADS) {
        const float w = weights[i];
        if (__float_as_uint(w) > mid) above += w;
      }
      turn ^= 1;
      sample_exchange(slots[turn], rank, __float_as_uint(block_sum(above, scratch)));
      if (sample_total(slots[turn]) <= limit) hi = mid; else lo = mid + 1;
    }
    keep_from = lo;
  }

  // Inverse CDF in vocabulary order over the kept tokens: each thread owns one segment of the block's slice, each block
  // knows the mass of the blocks before it.
  const int per = (count + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int first = min(count, tid * per), last = min(count, first + per);
  mine = 0.f;
  for (int i = first; i < last; ++i) {
    const float w = weights[i];
    if (__float_as_uint(w) >= keep_from) mine += w;
  }
  prefix[tid] = mine;
  __syncthreads();
  if (tid == 0) {   // serial scan of 1024 partial sums: fixed order, negligible time
    float running = 0.f;
    for (int i = 0; i < SAMPLE_THREADS; ++i) { const float v = prefix[i]; prefix[i] = running; running += v; }
    scratch[0] = running;
  }
  __syncthreads();
  turn ^= 1;
  sample_exchange(slots[turn], rank, __float_as_uint(scratch[0]));
  float before_block = 0.f, kept = 0.f;
#pragma unroll
  for (int c = 0; c < SAMPLE_CLUSTER; ++c) {
    if (c == (int)rank) before_block = kept;
    kept += __uint_as_float(slots[turn][c]);
  }
  float u = uniform ? uniform[row] : 0.5f;
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  const float target = u * kept;
  if (tid == 0) chosen = 0xffffffffu;
  __syncthreads();
  // The owner of the segment in which the running mass first exceeds the target.
  const float before = before_block + prefix[tid];
  if (mine > 0.f && before <= target && target < before + mine) {
    float running = before;
    int pick = -1;
    for (int i = first; i < last; ++i) {
      const float w = weights[i];
      if (__float_as_uint(w) >= keep_from) {
        running += w;
        pick = begin + i;
        if (running > target) break;
      }
    }
    if (pick >= 0) atomicMin(&chosen, (unsigned)pick);   // rounding can give a target two owners: the lower index, every time
  }
  __syncthreads();
  // Block 0 writes the row's token: the first block that found an owner; rounding at a segment's edge can leave none, and
  // then it is the most likely token.
  if (tid == 0) sample_send(&index_slots[rank], 0, chosen);
  sample_cluster_barrier();
  if (rank == 0 && tid == 0) {
    int token = best.index;
    for (int c = SAMPLE_CLUSTER - 1; c >= 0; --c)
      if ((int)index_slots[c] >= 0) token = (int)index_slots[c];
    sample_emit(out, mirror, row, token);
  }
}

}  // namespace pylon

// logits: float32 [rows, vocab] with `row_stride` elements between rows.  temperature, top_p
// and uniform are per row (pointers the device can read: device memory or pinned host memory; null temperature means
// arg-max for every row).  tokens_copy (int [rows]) and words_copy (int [4], with words, the device's four error words):
// pinned host memory, or null; the kernel leaves the tokens, and the words as they stand, there as well.
extern "C" int pylon_sample(const float* logits, long long row_stride, int rows, int vocab,
                            const float* temperature, const float* top_p, const float* uniform, int* out,
                            int* tokens_copy, const int* words, int* words_copy, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (words_copy && !words) PYLON_REFUSE("sample: a copy of the error words without the words");
  const pylon::SampleMirror mirror{tokens_copy, words, words_copy};
  if (vocab <= 0 || row_stride < vocab) PYLON_REFUSE("sample: vocabulary %d, row stride %lld", vocab, row_stride);
  // A row of a large vocabulary goes to a cluster of blocks, where the device places such clusters and a slice of the row
  // fits a block's shared memory: also for arg-max alone, which one block per row reads at a fraction of the bandwidth
  // (16 rows of 151,936 logits: 9.3 us with a block to a row, 6.9 us with a cluster; 5.2 us for one row; from some 32
  // rows on the blocks alone fill the device, and 64 rows take 9.5 us with them, 13.1 us in clusters).
  const int slice = ((vocab + pylon::SAMPLE_CLUSTER - 1) / pylon::SAMPLE_CLUSTER + 3) & ~3;
  const size_t smem = (size_t)slice * sizeof(float);
  if (vocab >= 4096 && smem <= 200 * 1024 && (long long)rows * pylon::SAMPLE_CLUSTER <= 2147483647LL && (temperature || rows <= 32)) {
    static int usable_on[pylon::MAX_DEVICES] = {};   // 0: not asked yet; 1: yes; -1: no
    int& usable = usable_on[pylon::current_device_slot()];
    static size_t configured_smem[pylon::MAX_DEVICES] = {};
    size_t& configured = configured_smem[pylon::current_device_slot()];
    if (usable == 0 || (usable == 1 && smem > configured)) {
      usable = cudaFuncSetAttribute(pylon::sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess ? 1 : -1;
      if (usable == 1) {
        configured = smem;
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(pylon::SAMPLE_CLUSTER); probe.blockDim = dim3(pylon::SAMPLE_THREADS); probe.dynamicSmemBytes = smem;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = pylon::SAMPLE_CLUSTER; attribute[0].val.clusterDim.y = 1; attribute[0].val.clusterDim.z = 1;
        probe.attrs = attribute; probe.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, pylon::sample_cluster_kernel, &probe) != cudaSuccess || clusters < 1) usable = -1;
      }
      if (usable != 1) cudaGetLastError();
    }
    if (usable == 1) {
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3((unsigned)(rows * pylon::SAMPLE_CLUSTER)); config.blockDim = dim3(pylon::SAMPLE_THREADS);
      config.dynamicSmemBytes = smem; config.stream = stream;
      cudaLaunchAttribute attribute[1];
      attribute[0].id = cudaLaunchAttributeClusterDimension;
      attribute[0].val.clusterDim.x = pylon::SAMPLE_CLUSTER; attribute[0].val.clusterDim.y = 1; attribute[0].val.clusterDim.z = 1;
      config.attrs = attribute; config.numAttrs = 1;
      cudaLaunchKernelEx(&config, pylon::sample_cluster_kernel, logits, row_stride, vocab, slice, temperature, top_p, uniform, out, mirror);
      PYLON_CHECK_LAUNCH("sample");
    }
  }
  pylon::sample_kernel<<<rows, pylon::SAMPLE_THREADS, 0, stream>>>(logits, row_stride, vocab, temperature, top_p,
                                                                   uniform, out, mirror);
  PYLON_CHECK_LAUNCH("sample");
}
