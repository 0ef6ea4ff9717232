// Memory-bound kernels around the matrix products: embedding gather, residual add fused
// with RMSNorm, per-head q/k RMSNorm fused with the rotary rotation and the write of keys
// and values into cache pages, SwiGLU.  All arithmetic is float32; `T` is only the type
// activations and cache pages are stored in (float or bfloat16).
//
// Replaces these library call sites of raun6k/Pylon: the embedding lookup
// (src/pylon/model/model.py:133), RMSNorm (src/pylon/model/layers.py:30-40), q/k norm and
// rotation (layers.py:132-134, 73-78), the page write (src/pylon/kv/cache.py:302-313),
// silu(gate)*up (layers.py:27) and the residual adds (layers.py:191,200).
#include "common.cuh"

namespace pylon {

// -----------------------------------------------------------------------------------------
// embedding: residual[t, :] = table[ids[t], :]   (residual stream is float32)
// -----------------------------------------------------------------------------------------
template <typename T>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                    float* __restrict__ out, int width, int vocab, float scale) {
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are validated on the host
  const T* row = table + (size_t)id * width;
  float* dst = out + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_float<T>(row[i]) * scale;   // scale is 1 for models that take the table as it is: exact
}

// -----------------------------------------------------------------------------------------
// tokens that the host does not know yet: ids[t] = sampled[source[t]] where source[t] >= 0
// (the token the sampling kernel chose for that row of the step before, still on the device)
// -----------------------------------------------------------------------------------------
__global__ void take_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source, const int* __restrict__ sampled,
                                   int sampled_rows, int num_tokens) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= num_tokens) return;
  const int from = source[t];
  if (from >= 0 && from < sampled_rows) ids[t] = sampled[from];
}

// -----------------------------------------------------------------------------------------
// residual add + RMSNorm
//   x = residual[row] (+ delta[row]);  if write_residual: residual[row] = x
//   out[r] = x / sqrt(mean(x^2) + eps) * weight          (out row r, compact)
// `rows` (optional) selects which residual rows are normalised; out is [n_rows, width].
// -----------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, const int* __restrict__ rows,
                                   T* __restrict__ out, int width, float eps, int write_residual) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int row = rows ? rows[r] : r;
  float* res = residual + (size_t)row * width;
  const T* del = delta ? delta + (size_t)row * width : nullptr;
  T* dst = out + (size_t)r * width;
  float sumsq = 0.f;
  // Pass 1: form the 32-bit sum, keep it (in the residual or, when it must not be
  // written, recomputed in pass 2) and accumulate the square sum.
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x = res[i];
    if (del) x += to_float<T>(del[i]);
    if (write_residual) res[i] = x;
    sumsq += x * x;
  }
  const float total = block_sum(sumsq, scratch);
  const float inv = rsqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x = res[i];
    if (del && !write_residual) x += to_float<T>(del[i]);
    dst[i] = from_float<T>(x * inv * weight[i]);
  }
}

// Register-resident form for rows of up to 256 * 4 * ITEMS elements whose width is a
// multiple of 4: every thread loads its ITEMS groups of 4 (all loads in flight at once),
// the row is summed once and written once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

constexpr int NORM_THREADS = 256;

// DT: type of the delta (the activation type, or float when the delta comes as `delta_parts`
// float32 partial sums, each [all rows, width], `part_stride` elements apart).
template <typename T, typename DT, int ITEMS>
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_vec_kernel(float* __restrict__ residual, const DT* __restrict__ delta,
                                                                       const float* __restrict__ weight, const int* __restrict__ rows,
                                                                       T* __restrict__ out, int width, float eps, int write_residual,
                                                                       int delta_parts, long long part_stride) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const int groups = width >> 2;
  // The norm's weights do not depend on the kernel before this one: they are on their way while it finishes.
  float4 w[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    w[k] = i < groups ? Vec4<float>::load(weight + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int row = rows ? rows[r] : r;
  float* res = residual + (size_t)row * width;
  const DT* del = delta ? delta + (size_t)row * width : nullptr;
  T* dst = out + (size_t)r * width;
  float4 x[ITEMS];
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    x[k] = i < groups ? Vec4<float>::load(res + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (del) {
#pragma unroll
    for (int k = 0; k < ITEMS; ++k) {
      const int i = threadIdx.x + k * NORM_THREADS;
      if (i < groups) {
        for (int part = 0; part < delta_parts; ++part) {   // in order: the sum does not depend on who wrote which part first
          const float4 d = Vec4<DT>::load(del + (size_t)part * part_stride + 4 * i);
          x[k].x += d.x; x[k].y += d.y; x[k].z += d.z; x[k].w += d.w;
        }
      }
    }
  }
  float sumsq = 0.f;
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) sumsq += x[k].x * x[k].x + x[k].y * x[k].y + x[k].z * x[k].z + x[k].w * x[k].w;
  const float inv = rsqrtf(block_sum(sumsq, scratch) / (float)width + eps);
#pragma unroll
  for (int k = 0; k < ITEMS; ++k) {
    const int i = threadIdx.x + k * NORM_THREADS;
    if (i < groups) {
      if (del && write_residual) Vec4<float>::store(res + 4 * i, x[k]);
      Vec4<T>::store(dst + 4 * i, make_float4(x[k].x * inv * w[k].x, x[k].y * inv * w[k].y, x[k].z * inv * w[k].z, x[k].w * inv * w[k].w));
    }
  }
}

template <typename T, typename DT>
static bool launch_add_rmsnorm_vec(float* residual, const DT* delta, const float* weight, const int* rows, T* out, int n_rows,
                                   int width, float eps, int write_residual, int delta_parts, long long part_stride,
                                   cudaStream_t stream) {
  if (width % 4 || width > NORM_THREADS * 4 * 8) return false;
  if (((uintptr_t)residual % 16) || ((uintptr_t)weight % 16) || ((uintptr_t)out % 8) || (delta && ((uintptr_t)delta % 16))) return false;
  if (part_stride % 4) return false;
  const int items = (width / 4 + NORM_THREADS - 1) / NORM_THREADS;
#define PYLON_NORM_CASE(N)                                                                                     \
  case N:                                                                                                      \
    launch_dependent(add_rmsnorm_vec_kernel<T, DT, N>, dim3(n_rows), dim3(NORM_THREADS), 0, stream, residual, delta, weight, rows, out, width, eps, write_residual, delta_parts, part_stride); \
    return true;
  switch (items) {
    PYLON_NORM_CASE(1) PYLON_NORM_CASE(2) PYLON_NORM_CASE(3) PYLON_NORM_CASE(4)
    PYLON_NORM_CASE(5) PYLON_NORM_CASE(6) PYLON_NORM_CASE(7) PYLON_NORM_CASE(8)
  }
#undef PYLON_NORM_CASE
  return false;
}

template <typename T>
__global__ void residual_add_kernel(float* __restrict__ residual, const T* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) residual[i] += to_float<T>(delta[i]);
}

// -----------------------------------------------------------------------------------------
// q/k RMSNorm + rotary rotation + cache write.  One warp per (token, head).
//   head < nq            : q head, normalised, rotated, written back in place
//   nq <= head < nq+nkv  : k head, normalised, rotated, written to its page slot
//   else                 : v head, copied to its page slot
// Rotation pairs (j, j + rd/2) for j < rd/2 with cos/sin[pos, j]; elements >= rd pass.
// -----------------------------------------------------------------------------------------
template <typename T, int MAX_PER_LANE>
__global__ void qk_norm_rope_kv_write_kernel(
    T* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    float eps, const float* __restrict__ cos_table, const float* __restrict__ sin_table,
    int rotary_dim, int table_positions, const int* __restrict__ positions,
    const int* __restrict__ token_row, const int* __restrict__ block_table, int table_width,
    int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages, int num_pages, int nq, int nkv,
    int d, int num_tokens, int* __restrict__ error) {
  extern __shared__ float exchange[];  // [warps per block][d]
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * heads) return;
  const int t = (int)(item / heads), head = (int)(item % heads);
  T* src = qkv + ((size_t)t * heads + head) * d;
  const int pos = positions[t];

  T* page_dst = nullptr;
  if (head >= nq) {
    const int row = token_row[t];
    if (row < 0) return;   // a padding token of a step padded to a captured size: it belongs to no request
    const int page = block_table[(size_t)row * table_width + pos / page_size];
    if (page < 0 || page >= num_pages) {   // never for a prepared step: nothing is written, and the host is told
      if (lane == 0 && error) atomicExch(error, PYLON_ERROR_BAD_PAGE);
      return;
    }
    const int kv_head = (head - nq) % nkv;
    T* pages = head < nq + nkv ? k_pages : v_pages;
    page_dst = pages + (((size_t)page * nkv + kv_head) * page_size + pos % page_size) * d;
  }
  if (head >= nq + nkv) {  // value: plain copy
    for (int e = lane; e < d; e += 32) page_dst[e] = src[e];
    return;
  }

  float x[MAX_PER_LANE];
  float sumsq = 0.f;
#pragma unroll
  for (int k = 0; k < MAX_PER_LANE; ++k) {
    const int e = lane + 32 * k;
    x[k] = e < d ? to_float<T>(src[e]) : 0.f;
    sumsq += x[k] * x[k];
  }
  const float* weight = head < nq ? q_weight : k_weight;
  if (weight) {
    sumsq = warp_sum(sumsq);
    const float inv = rsqrtf(sumsq / (float)d + eps);
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
      const int e = lane + 32 * k;
      if (e < d) x[k] = x[k] * inv * weight[e];
    }
  }
  T* dst = head < nq ? src : page_dst;
  if (rotary_dim > 0 && cos_table) {
    float* mine = exchange + (size_t)warp * d;
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
      const int e = lane + 32 * k;
      if (e < d) mine[e] = x[k];
    }
    __syncwarp();
    const int half = rotary_dim >> 1;
    const int p = pos < table_positions ? pos : table_positions - 1;  // host checks the range
    const float* c = cos_table + (size_t)p * half;
    const float* s = sin_table + (size_t)p * half;
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
      const int e = lane + 32 * k;
      if (e < d) {
        float y = x[k];
        if (e < half) y = x[k] * c[e] - mine[e + half] * s[e];
        else if (e < rotary_dim) y = x[k] * c[e - half] + mine[e - half] * s[e - half];
        dst[e] = from_float<T>(y);
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < MAX_PER_LANE; ++k) {
      const int e = lane + 32 * k;
      if (e < d) dst[e] = from_float<T>(x[k]);
    }
  }
}

// q/k RMSNorm alone, in place on qkv [T, (nq + 2 nkv) * d]: for position encodings that are not a rotation by a table and
// therefore run between the norms and the cache write.  One warp per (token, q or k head).
template <typename T, int MAX_PER_LANE>
__global__ void qk_norm_kernel(T* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
                               int nq, int nkv, int d, int num_tokens) {
  grid_dependency_wait();
  allow_dependents();
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int normed = nq + nkv;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * normed) return;
  const int t = (int)(item / normed), head = (int)(item % normed);
  const float* weight = head < nq ? q_weight : k_weight;
  if (!weight) return;
  T* src = qkv + ((size_t)t * (nq + 2 * nkv) + head) * d;
  float x[MAX_PER_LANE];
  float sumsq = 0.f;
#pragma unroll
  for (int k = 0; k < MAX_PER_LANE; ++k) {
    const int e = lane + 32 * k;
    x[k] = e < d ? to_float<T>(src[e]) : 0.f;
    sumsq += x[k] * x[k];
  }
  sumsq = warp_sum(sumsq);
  const float inv = rsqrtf(sumsq / (float)d + eps);
#pragma unroll
  for (int k = 0; k < MAX_PER_LANE; ++k) {
    const int e = lane + 32 * k;
    if (e < d) src[e] = from_float<T>(x[k] * inv * weight[e]);
  }
}

// Vector form for head sizes 64, 128 and 256 with the rotation over the whole head: lane l holds
// the CHUNK = d / 32 consecutive elements l * CHUNK .., loaded and stored as one vector; its
// rotation partners (d / 2 further) sit in lane l ^ 16 and come by shuffle.
template <typename T, int CHUNK>
struct HeadChunk;
template <int CHUNK>
struct HeadChunk<__nv_bfloat16, CHUNK> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[CHUNK]) {
    if constexpr (CHUNK == 2) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
      v[0] = f.x; v[1] = f.y;
    } else {
      uint32_t raw[CHUNK / 2];
      if constexpr (CHUNK == 4) { const uint2 r = *reinterpret_cast<const uint2*>(p); raw[0] = r.x; raw[1] = r.y; }
      else { const uint4 r = *reinterpret_cast<const uint4*>(p); raw[0] = r.x; raw[1] = r.y; raw[2] = r.z; raw[3] = r.w; }
#pragma unroll
      for (int i = 0; i < CHUNK / 2; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
      }
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[CHUNK]) {
    uint32_t raw[CHUNK / 2];
#pragma unroll
    for (int i = 0; i < CHUNK / 2; ++i) {
      __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      raw[i] = *reinterpret_cast<uint32_t*>(&b);
    }
    if constexpr (CHUNK == 2) *reinterpret_cast<uint32_t*>(p) = raw[0];
    else if constexpr (CHUNK == 4) *reinterpret_cast<uint2*>(p) = make_uint2(raw[0], raw[1]);
    else *reinterpret_cast<uint4*>(p) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
  }
};
template <int CHUNK>
struct HeadChunk<float, CHUNK> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[CHUNK]) {
#pragma unroll
    for (int i = 0; i < CHUNK; i += 2) { const float2 f = *reinterpret_cast<const float2*>(p + i); v[i] = f.x; v[i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[CHUNK]) {
#pragma unroll
    for (int i = 0; i < CHUNK; i += 2) *reinterpret_cast<float2*>(p + i) = make_float2(v[i], v[i + 1]);
  }
};

// HPW heads of one token per warp: their loads are issued together, so a warp has HPW times the
// bytes in flight per trip to memory (with one head per warp a 2048-token step ran at a third of
// the memory bandwidth); the token's position, page and angles are looked up once.
//
// The projections come either as qkv [T, heads * d] in the activation type (q is then written back in place) or as
// `parts` float32 partial sums [parts, T, heads * d], `part_stride` elements apart, which are added up here (q then goes
// to q_out [T, nq * d]).
template <typename T, int CHUNK, int HPW>
__global__ void qk_norm_rope_kv_write_vec_kernel(
    T* __restrict__ qkv, const float* __restrict__ qkv_parts, int parts, long long part_stride, T* __restrict__ q_out,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions,
    const int* __restrict__ positions, const int* __restrict__ token_row, const int* __restrict__ block_table,
    int table_width, int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages, int num_pages, int nq, int nkv,
    int num_tokens, int* __restrict__ error) {
  constexpr int d = CHUNK * 32, half = d / 2;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const int groups = (heads + HPW - 1) / HPW;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * groups) { grid_dependency_wait(); return; }
  const int t = (int)(item / groups), head_begin = (int)(item % groups) * HPW;
  // Position, page and angles are the step's own data, not the work of the kernel before this one: they are looked up
  // while that kernel finishes.
  const int pos = positions[t];
  size_t page_offset = 0;
  bool page_ok = true;
  if (head_begin + HPW > nq) {   // a key or value head among them
    const int row = token_row[t];   // negative: a padding token of a step padded to a captured size, which belongs to no request
    const int page = row < 0 ? -1 : block_table[(size_t)row * table_width + pos / page_size];
    page_ok = page >= 0 && page < num_pages;   // always for a prepared step: else nothing is written, and the host is told
    if (!page_ok && row >= 0 && lane == 0 && error) atomicExch(error, PYLON_ERROR_BAD_PAGE);
    page_offset = ((size_t)(page_ok ? page : 0) * nkv * page_size + pos % page_size) * d + lane * CHUNK;
  }
  float c[CHUNK], s[CHUNK];
  if (cos_table && head_begin < nq + nkv) {
    const int p = pos < table_positions ? pos : table_positions - 1;   // the host checks the range
    const int column = (lane & 15) * CHUNK;                            // both halves share their angles
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) { c[i] = cos_table[(size_t)p * half + column + i]; s[i] = sin_table[(size_t)p * half + column + i]; }
  }
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  const size_t token_offset = (size_t)t * heads * d + lane * CHUNK;
  float x[HPW][CHUNK];
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    if (head_begin + h >= heads) continue;
    if (qkv_parts) {
      HeadChunk<float, CHUNK>::load(qkv_parts + token_offset + (size_t)(head_begin + h) * d, x[h]);
      for (int part = 1; part < parts; ++part) {   // in order: the sum does not depend on who wrote which part first
        float more[CHUNK];
        HeadChunk<float, CHUNK>::load(qkv_parts + (size_t)part * part_stride + token_offset + (size_t)(head_begin + h) * d, more);
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) x[h][i] += more[i];
      }
    } else {
      HeadChunk<T, CHUNK>::load(qkv + token_offset + (size_t)(head_begin + h) * d, x[h]);
    }
  }
  const bool upper = lane >= 16;
#pragma unroll
  for (int h = 0; h < HPW; ++h) {
    const int head = head_begin + h;
    if (head >= heads) break;
    T* page_dst = nullptr;
    if (head >= nq) {
      if (!page_ok) continue;
      const int kv_head = (head - nq) % nkv;
      page_dst = (head < nq + nkv ? k_pages : v_pages) + page_offset + (size_t)kv_head * page_size * d;
    }
    if (head >= nq + nkv) {   // value: plain copy
      HeadChunk<T, CHUNK>::store(page_dst, x[h]);
      continue;
    }
    const float* weight = head < nq ? q_weight : k_weight;
    if (weight) {
      float sumsq = 0.f;
#pragma unroll
      for (int i = 0; i < CHUNK; ++i) sumsq += x[h][i] * x[h][i];
      sumsq = warp_sum(sumsq);
      const float inv = rsqrtf(sumsq / (float)d + eps);
#pragma unroll
      for (int i = 0; i < CHUNK; ++i) x[h][i] = x[h][i] * inv * weight[lane * CHUNK + i];
    }
    if (cos_table) {
#pragma unroll
      for (int i = 0; i < CHUNK; ++i) {
        const float partner = __shfl_xor_sync(0xffffffffu, x[h][i], 16);
        x[h][i] = upper ? x[h][i] * c[i] + partner * s[i] : x[h][i] * c[i] - partner * s[i];
      }
    }
    T* q_dst = qkv_parts ? q_out + ((size_t)t * nq + head) * d + lane * CHUNK : qkv + token_offset + (size_t)head * d;
    HeadChunk<T, CHUNK>::store(head < nq ? q_dst : page_dst, x[h]);
  }
}

// Many tokens in bfloat16: D / 16 lanes share a head, each with the eight elements 8l.. of the lower half and their
// rotation partners 8l + D/2.. of the upper half as two 16-byte vectors.  The rotation needs no shuffle, the sum of squares
// log2(D / 16) of them, and a warp has 32 / (D / 16) heads per pass with PASSES passes' loads in flight.  (With one head
// across a whole warp, 8 bytes a lane, a 2,048-token step was bound by the instructions issued: 25 us for 50 MB.)
template <int D, int PASSES>
__global__ void __launch_bounds__(128, 5) qk_norm_rope_kv_write_wide_kernel(
    __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions,
    const int* __restrict__ positions, const int* __restrict__ token_row, const int* __restrict__ block_table,
    int table_width, int page_size, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages, int num_pages,
    int nq, int nkv, int num_tokens, int* __restrict__ error) {
  constexpr int LANES = D / 16, HEADS_PER_PASS = 32 / LANES, HALF = D / 2, PER_WARP = HEADS_PER_PASS * PASSES;
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = nq + 2 * nkv;
  const int groups = (heads + PER_WARP - 1) / PER_WARP;
  const long long item = (long long)blockIdx.x * warps_per_block + warp;
  if (item >= (long long)num_tokens * groups) { grid_dependency_wait(); return; }
  const int t = (int)(item / groups), head_begin = (int)(item % groups) * PER_WARP;
  const int sub = lane / LANES, column = (lane % LANES) * 8;   // this lane's head within a pass, its eight columns
  // Position, page and angles are the step's own data: looked up while the kernel before this one finishes.
  const int pos = positions[t];
  size_t page_offset = 0;
  bool page_ok = true;
  if (head_begin + PER_WARP > nq) {   // a key or value head among them
    const int row = token_row[t];   // negative: a padding token of a step padded to a captured size, which belongs to no request
    const int page = row < 0 ? -1 : block_table[(size_t)row * table_width + pos / page_size];
    page_ok = page >= 0 && page < num_pages;   // always for a prepared step: else nothing is written, and the host is told
    if (!page_ok && row >= 0 && lane == 0 && error) atomicExch(error, PYLON_ERROR_BAD_PAGE);
    page_offset = ((size_t)(page_ok ? page : 0) * nkv * page_size + pos % page_size) * D;
  }
  float c[8], s[8];
  if (cos_table && head_begin < nq + nkv) {
    const int p = pos < table_positions ? pos : table_positions - 1;   // the host checks the range
    const float4* cp = reinterpret_cast<const float4*>(cos_table + (size_t)p * HALF + column);
    const float4* sp = reinterpret_cast<const float4*>(sin_table + (size_t)p * HALF + column);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
  }
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  __nv_bfloat16* token = qkv + (size_t)t * heads * D;
  uint4 lower[PASSES], upper[PASSES];
#pragma unroll
  for (int pass = 0; pass < PASSES; ++pass) {
    const int head = head_begin + pass * HEADS_PER_PASS + sub;
    lower[pass] = upper[pass] = make_uint4(0u, 0u, 0u, 0u);
    if (head < heads) {
      lower[pass] = *reinterpret_cast<const uint4*>(token + (size_t)head * D + column);
      upper[pass] = *reinterpret_cast<const uint4*>(token + (size_t)head * D + HALF + column);
    }
  }
#pragma unroll
  for (int pass = 0; pass < PASSES; ++pass) {
    const int head = head_begin + pass * HEADS_PER_PASS + sub;
    float x[16];
    {
      const uint32_t raw[8] = {lower[pass].x, lower[pass].y, lower[pass].z, lower[pass].w, upper[pass].x, upper[pass].y, upper[pass].z, upper[pass].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[i]));
        x[2 * i] = f.x; x[2 * i + 1] = f.y;
      }
    }
    // every lane of the warp takes part in the shuffles, whatever its head is
    float sumsq = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) sumsq += x[i] * x[i];
#pragma unroll
    for (int mask = 1; mask < LANES; mask <<= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, mask);
    if (head >= heads) continue;
    __nv_bfloat16* dst = token + (size_t)head * D;
    if (head >= nq) {
      if (!page_ok) continue;
      const int kv_head = (head - nq) % nkv;
      dst = (head < nq + nkv ? k_pages : v_pages) + page_offset + (size_t)kv_head * page_size * D;
    }
    if (head < nq + nkv) {   // values are copied as they are
      const float* weight = head < nq ? q_weight : k_weight;
      if (weight) {
        const float inv = rsqrtf(sumsq / (float)D + eps);
        const float4* wl = reinterpret_cast<const float4*>(weight + column);
        const float4* wu = reinterpret_cast<const float4*>(weight + HALF + column);
        const float4 w0 = wl[0], w1 = wl[1], w2 = wu[0], w3 = wu[1];
        const float w[16] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w, w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = x[i] * inv * w[i];
      }
      if (cos_table) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float first = x[i], second = x[8 + i];
          x[i] = first * c[i] - second * s[i];
          x[8 + i] = second * c[i] + first * s[i];
        }
      }
    }
    uint32_t packed[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
      packed[i] = *reinterpret_cast<const uint32_t*>(&b);
    }
    if (head >= nq + nkv) {   // bit for bit
      *reinterpret_cast<uint4*>(dst + column) = lower[pass];
      *reinterpret_cast<uint4*>(dst + HALF + column) = upper[pass];
    } else {
      *reinterpret_cast<uint4*>(dst + column) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<uint4*>(dst + HALF + column) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
  }
}

// -----------------------------------------------------------------------------------------
// SwiGLU: out[t, i] = silu(gu[t, i]) * gu[t, inter + i]
// -----------------------------------------------------------------------------------------
// `interleaved`: gate and up columns alternate in groups of 8 ([g0..g7 u0..u7 g8..g15 ...])
// instead of lying in two halves.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total, int interleaved) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / inter;
    const int c = (int)(i - t * inter);
    const int gate_column = interleaved ? (c >> 3) * 16 + (c & 7) : c;
    const int up_column = interleaved ? gate_column + 8 : inter + c;
    const float g = to_float<T>(gate_up[t * 2 * inter + gate_column]);
    const float u = to_float<T>(gate_up[t * 2 * inter + up_column]);
    // float storage is the true 32-bit path: full-precision exponential there
    const float e = sizeof(T) == 4 ? expf(-g) : __expf(-g);
    out[i] = from_float<T>(g / (1.f + e) * u);
  }
}

// Vector form for bfloat16 rows whose width is a multiple of 8 (16-byte accesses).
__global__ void swiglu_bf16x8_kernel(const uint4* __restrict__ gate_up, uint4* __restrict__ out, int inter8,
                                     size_t total8, int interleaved) {
  grid_dependency_wait();
  allow_dependents();   // only now: a kernel that is itself still waiting must not pull the next one onto the SMs
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total8; i += stride) {
    const size_t t = i / inter8;
    const int c = (int)(i - t * inter8);
    uint4 g4 = gate_up[t * 2 * inter8 + (interleaved ? 2 * c : c)];
    uint4 u4 = gate_up[t * 2 * inter8 + (interleaved ? 2 * c + 1 : inter8 + c)];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]);
      const float2 u = __bfloat1622float2(u2[k]);
      // approximate division: no slow path (the exact one takes a subroutine for zero numerators), ample for a bfloat16 result
      o2[k] = __floats2bfloat162_rn(__fdividef(g.x, 1.f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.f + __expf(-g.y)) * u.y);
    }
    out[i] = o4;
  }
}

}  // namespace pylon

using namespace pylon;

// y = x * scale, then (cap > 0) y = cap * tanh(y / cap): what some architectures do to their logits.
__global__ void logit_transform_kernel(float* __restrict__ logits, size_t n, float scale, float cap) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float y = logits[i] * scale;
    if (cap > 0.f) y = cap * tanhf(y / cap);
    logits[i] = y;
  }
}

extern "C" int pylon_logit_transform(float* logits, long long n, float scale, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const long long most = (long long)pylon::multiprocessors() * 16;
  const int blocks = (int)((n + threads - 1) / threads < most ? (n + threads - 1) / threads : most);
  logit_transform_kernel<<<blocks, threads, 0, stream>>>(logits, (size_t)n, scale, cap);
  PYLON_CHECK_LAUNCH("logit_transform");
}

extern "C" int pylon_take_tokens(int* ids, const int* source, const int* sampled, int sampled_rows, int num_tokens, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (sampled_rows <= 0) PYLON_REFUSE("take_tokens: %d sampled rows", sampled_rows);
  take_tokens_kernel<<<(num_tokens + 255) / 256, 256, 0, stream>>>(ids, source, sampled, sampled_rows, num_tokens);
  PYLON_CHECK_LAUNCH("take_tokens");
}

extern "C" int pylon_embed_gather(const int* ids, const void* table, float* out, int num_tokens, int width,
                                  int vocab, int dtype, float scale, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (width <= 0 || vocab <= 0) PYLON_REFUSE("embed_gather: width %d, vocab %d", width, vocab);
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == PYLON_DTYPE_F32)
    embed_gather_kernel<float><<<num_tokens, threads, 0, stream>>>(ids, (const float*)table, out, width, vocab, scale);
  else if (dtype == PYLON_DTYPE_BF16)
    embed_gather_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, out, width, vocab, scale);
  else
    PYLON_REFUSE("embed_gather: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("embed_gather");
}

extern "C" int pylon_add_rmsnorm(float* residual, const void* delta, const float* weight, const int* rows,
                                 void* out, int n_rows, int width, float eps, int write_residual, int dtype,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (width <= 0) PYLON_REFUSE("add_rmsnorm: width %d", width);
  if (rows && write_residual) PYLON_REFUSE("add_rmsnorm: a row selection cannot update the residual");
  const int threads = width >= 4096 ? 512 : (width >= 1024 ? 256 : 128);
  if (dtype == PYLON_DTYPE_F32) {
    if (!launch_add_rmsnorm_vec<float, float>(residual, (const float*)delta, weight, rows, (float*)out, n_rows, width, eps, write_residual, 1, 0, stream))
      add_rmsnorm_kernel<float><<<n_rows, threads, 0, stream>>>(residual, (const float*)delta, weight, rows, (float*)out, width, eps, write_residual);
  } else if (dtype == PYLON_DTYPE_BF16) {
    if (!launch_add_rmsnorm_vec<__nv_bfloat16, __nv_bfloat16>(residual, (const __nv_bfloat16*)delta, weight, rows, (__nv_bfloat16*)out, n_rows, width, eps, write_residual, 1, 0, stream))
      add_rmsnorm_kernel<__nv_bfloat16><<<n_rows, threads, 0, stream>>>(residual, (const __nv_bfloat16*)delta, weight, rows, (__nv_bfloat16*)out, width, eps, write_residual);
  } else {
    PYLON_REFUSE("add_rmsnorm: unknown dtype %d", dtype);
  }
  PYLON_CHECK_LAUNCH("add_rmsnorm");
}

// The same with the delta given as `parts` float32 partial sums [parts, all_rows, width] (contiguous): bfloat16 output,
// width a multiple of 4 and at most 8192.  rows: null (every row: the sum is added to the residual in place, n_rows =
// all_rows) or n_rows int32 row numbers (those rows only, normalised from residual + sum; the residual stays as it is).
extern "C" int pylon_add_parts_rmsnorm(float* residual, const float* delta_parts, int parts, const float* weight, const int* rows,
                                       void* out, int n_rows, int all_rows, int width, float eps, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (parts < 1 || !delta_parts) PYLON_REFUSE("add_parts_rmsnorm: %d parts", parts);
  if (!rows && n_rows != all_rows) PYLON_REFUSE("add_parts_rmsnorm: %d of %d rows without a row selection", n_rows, all_rows);
  if (!launch_add_rmsnorm_vec<__nv_bfloat16, float>(residual, delta_parts, weight, rows, (__nv_bfloat16*)out, n_rows, width, eps, rows ? 0 : 1,
                                                     parts, (long long)all_rows * width, stream))
    PYLON_REFUSE("add_parts_rmsnorm: width %d must be a multiple of 4, at most 8192, with 16-byte aligned buffers", width);
  PYLON_CHECK_LAUNCH("add_parts_rmsnorm");
}

extern "C" int pylon_residual_add(float* residual, const void* delta, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const long long most = (long long)pylon::multiprocessors() * 16;
  const int blocks = (int)((n + threads - 1) / threads < most ? (n + threads - 1) / threads : most);
  if (dtype == PYLON_DTYPE_F32)
    residual_add_kernel<float><<<blocks, threads, 0, stream>>>(residual, (const float*)delta, (size_t)n);
  else if (dtype == PYLON_DTYPE_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(residual, (const __nv_bfloat16*)delta, (size_t)n);
  else
    PYLON_REFUSE("residual_add: unknown dtype %d", dtype);
  PYLON_CHECK_LAUNCH("residual_add");
}

template <typename T>
static int launch_qk_norm_rope(T* qkv, const float* qkv_parts, int parts, long long part_stride, T* q_out, const float* qw, const float* kw, float eps, const float* cos_t,
                               const float* sin_t, int rotary_dim, int table_positions, const int* positions,
                               const int* token_row, const int* block_table, int table_width, int page_size,
                               T* k_pages, T* v_pages, int num_pages, int nq, int nkv, int d, int num_tokens,
                               int* error, cudaStream_t stream) {
  const int warps = 4;
  const long long items = (long long)num_tokens * (nq + 2 * nkv);
  const int blocks = (int)((items + warps - 1) / warps);
  const size_t smem = (size_t)warps * d * sizeof(float);
  // Head sizes 64, 128, 256 rotated over the whole head (or not at all), aligned: the vector form.
  const bool whole = (rotary_dim == d && cos_t) || (rotary_dim == 0 || !cos_t);
  const bool aligned = ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)k_pages % 16 == 0) && ((uintptr_t)v_pages % 16 == 0) &&
                       ((uintptr_t)qkv_parts % 16 == 0) && ((uintptr_t)q_out % 16 == 0) && (part_stride % 4 == 0);
  if (qkv_parts && !(whole && aligned && (d == 64 || d == 128 || d == 256)))
    PYLON_REFUSE("qk_norm_rope_kv_write: partial sums need head size 64, 128 or 256, rotation over the whole head and 16-byte aligned buffers");
  if (whole && aligned && (d == 64 || d == 128 || d == 256)) {
    const float* cos_used = rotary_dim == d ? cos_t : nullptr;
    if constexpr (sizeof(T) == 2) {
      if (num_tokens >= 64 && !qkv_parts && ((uintptr_t)qw % 16 == 0) && ((uintptr_t)kw % 16 == 0) && ((uintptr_t)cos_t % 16 == 0) &&
          ((uintptr_t)sin_t % 16 == 0)) {
        constexpr int PASSES = 3;   // 1, 2 and 4 passes measured the same to slower: 13 to 15 us for 2,048 tokens of 48 heads
        const int per_warp = 32 / (d / 16) * PASSES;
        const long long wide_items = (long long)num_tokens * ((nq + 2 * nkv + per_warp - 1) / per_warp);
        const unsigned wide_blocks = (unsigned)((wide_items + warps - 1) / warps);
#define PYLON_LAUNCH_QK_WIDE(D_)                                                                                              \
        launch_dependent(qk_norm_rope_kv_write_wide_kernel<D_, PASSES>, dim3(wide_blocks), dim3(warps * 32), 0, stream, qkv, qw, kw, eps, \
                         cos_used, sin_t, table_positions, positions, token_row, block_table, table_width, page_size, k_pages,   \
                         v_pages, num_pages, nq, nkv, num_tokens, error)
        if (d == 64) PYLON_LAUNCH_QK_WIDE(64);
        else if (d == 128) PYLON_LAUNCH_QK_WIDE(128);
        else PYLON_LAUNCH_QK_WIDE(256);
#undef PYLON_LAUNCH_QK_WIDE
        PYLON_CHECK_LAUNCH("qk_norm_rope_kv_write");
      }
    }
    // Many tokens: four heads per warp (more bytes in flight); few: one, for as many warps as possible.
    const bool many = num_tokens >= 64;
    const long long vec_items = (long long)num_tokens * (many ? (nq + 2 * nkv + 3) / 4 : nq + 2 * nkv);
    const unsigned vec_blocks = (unsigned)((vec_items + warps - 1) / warps);
#define PYLON_LAUNCH_QK_VEC(C)                                                                                            \
    do {                                                                                                                  \
      if (many)                                                                                                           \
        launch_dependent(qk_norm_rope_kv_write_vec_kernel<T, C, 4>, dim3(vec_blocks), dim3(warps * 32), 0, stream, qkv, qkv_parts, parts, part_stride, q_out, qw, kw, eps,  \
                         cos_used, sin_t, table_positions, positions, token_row, block_table, table_width, page_size, k_pages, \
                         v_pages, num_pages, nq, nkv, num_tokens, error);                                                  \
      else                                                                                                                \
        launch_dependent(qk_norm_rope_kv_write_vec_kernel<T, C, 1>, dim3(vec_blocks), dim3(warps * 32), 0, stream, qkv, qkv_parts, parts, part_stride, q_out, qw, kw, eps,  \
                         cos_used, sin_t, table_positions, positions, token_row, block_table, table_width, page_size, k_pages, \
                         v_pages, num_pages, nq, nkv, num_tokens, error);                                                  \
    } while (0)
    if (d == 64) PYLON_LAUNCH_QK_VEC(2);
    else if (d == 128) PYLON_LAUNCH_QK_VEC(4);
    else PYLON_LAUNCH_QK_VEC(8);
#undef PYLON_LAUNCH_QK_VEC
    PYLON_CHECK_LAUNCH("qk_norm_rope_kv_write");
  }
#define PYLON_LAUNCH_QK(N)                                                                              \
  launch_dependent(qk_norm_rope_kv_write_kernel<T, N>, dim3(blocks), dim3(warps * 32), smem, stream,    \
      qkv, qw, kw, eps, cos_t, sin_t, rotary_dim, table_positions, positions, token_row, block_table,   \
      table_width, page_size, k_pages, v_pages, num_pages, nq, nkv, d, num_tokens, error)
  if (d <= 32) PYLON_LAUNCH_QK(1);
  else if (d <= 64) PYLON_LAUNCH_QK(2);
  else if (d <= 128) PYLON_LAUNCH_QK(4);
  else if (d <= 256) PYLON_LAUNCH_QK(8);
  else PYLON_LAUNCH_QK(16);
#undef PYLON_LAUNCH_QK
  PYLON_CHECK_LAUNCH("qk_norm_rope_kv_write");
}

extern "C" int pylon_qk_norm_rope_kv_write(void* qkv, const float* q_weight, const float* k_weight, float eps,
                                           const float* cos_table, const float* sin_table, int rotary_dim,
                                           int table_positions, const int* positions, const int* token_row,
                                           const int* block_table, int table_width, int page_size,
                                           void* k_pages, void* v_pages, int num_pages, int nq, int nkv, int d,
                                           int num_tokens, int dtype, int* error, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (d < 2 || d > 512) PYLON_REFUSE("qk_norm_rope_kv_write: head size %d is outside 2..512", d);
  if (rotary_dim < 0 || rotary_dim > d || (rotary_dim & 1))
    PYLON_REFUSE("qk_norm_rope_kv_write: rotary size %d must be even and at most the head size %d", rotary_dim, d);
  if (nq < 0 || nkv < 1 || page_size < 1 || table_width < 1)
    PYLON_REFUSE("qk_norm_rope_kv_write: heads %d/%d, page size %d, table width %d", nq, nkv, page_size, table_width);
  if (dtype == PYLON_DTYPE_F32)
    return launch_qk_norm_rope<float>((float*)qkv, nullptr, 0, 0, nullptr, q_weight, k_weight, eps, cos_table, sin_table, rotary_dim,
                                      table_positions, positions, token_row, block_table, table_width, page_size,
                                      (float*)k_pages, (float*)v_pages, num_pages, nq, nkv, d, num_tokens, error, stream);
  if (dtype == PYLON_DTYPE_BF16)
    return launch_qk_norm_rope<__nv_bfloat16>((__nv_bfloat16*)qkv, nullptr, 0, 0, nullptr, q_weight, k_weight, eps, cos_table, sin_table,
                                              rotary_dim, table_positions, positions, token_row, block_table,
                                              table_width, page_size, (__nv_bfloat16*)k_pages,
                                              (__nv_bfloat16*)v_pages, num_pages, nq, nkv, d, num_tokens, error, stream);
  PYLON_REFUSE("qk_norm_rope_kv_write: unknown dtype %d", dtype);
}

template <typename T>
static int launch_qk_norm(T* qkv, const float* qw, const float* kw, float eps, int nq, int nkv, int d, int num_tokens, cudaStream_t stream) {
  const int warps = 4;
  const long long items = (long long)num_tokens * (nq + nkv);
  const unsigned blocks = (unsigned)((items + warps - 1) / warps);
#define PYLON_LAUNCH_QK_NORM(N) launch_dependent(qk_norm_kernel<T, N>, dim3(blocks), dim3(warps * 32), 0, stream, qkv, qw, kw, eps, nq, nkv, d, num_tokens)
  if (d <= 32) PYLON_LAUNCH_QK_NORM(1);
  else if (d <= 64) PYLON_LAUNCH_QK_NORM(2);
  else if (d <= 128) PYLON_LAUNCH_QK_NORM(4);
  else if (d <= 256) PYLON_LAUNCH_QK_NORM(8);
  else PYLON_LAUNCH_QK_NORM(16);
#undef PYLON_LAUNCH_QK_NORM
  PYLON_CHECK_LAUNCH("qk_norm");
}

// RMSNorm of every q and k head of qkv [num_tokens, (nq + 2 nkv) * d], in place (a null weight leaves its heads alone).
extern "C" int pylon_qk_norm(void* qkv, const float* q_weight, const float* k_weight, float eps, int nq, int nkv, int d, int num_tokens,
                             int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || (!q_weight && !k_weight)) return 0;
  if (d < 1 || d > 512) PYLON_REFUSE("qk_norm: head size %d is outside 1..512", d);
  if (nq < 0 || nkv < 1) PYLON_REFUSE("qk_norm: heads %d/%d", nq, nkv);
  if (dtype == PYLON_DTYPE_F32) return launch_qk_norm<float>((float*)qkv, q_weight, k_weight, eps, nq, nkv, d, num_tokens, stream);
  if (dtype == PYLON_DTYPE_BF16) return launch_qk_norm<__nv_bfloat16>((__nv_bfloat16*)qkv, q_weight, k_weight, eps, nq, nkv, d, num_tokens, stream);
  PYLON_REFUSE("qk_norm: unknown dtype %d", dtype);
}

// The same for bfloat16 with the projections given as `parts` float32 partial sums [parts, num_tokens, (nq + 2 nkv) * d]
// (contiguous): they are added up, q goes to q_out [num_tokens, nq * d], k and v into the pages.  Head size 64, 128 or
// 256, rotary_dim 0 or d.
extern "C" int pylon_qk_norm_rope_kv_write_parts(const float* qkv_parts, int parts, void* q_out, const float* q_weight, const float* k_weight,
                                                 float eps, const float* cos_table, const float* sin_table, int rotary_dim,
                                                 int table_positions, const int* positions, const int* token_row,
                                                 const int* block_table, int table_width, int page_size, void* k_pages,
                                                 void* v_pages, int num_pages, int nq, int nkv, int d, int num_tokens,
                                                 int* error, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (!qkv_parts || parts < 1 || !q_out) PYLON_REFUSE("qk_norm_rope_kv_write_parts: %d parts", parts);
  if (nq < 0 || nkv < 1 || page_size < 1 || table_width < 1)
    PYLON_REFUSE("qk_norm_rope_kv_write_parts: heads %d/%d, page size %d, table width %d", nq, nkv, page_size, table_width);
  if (rotary_dim != 0 && rotary_dim != d) PYLON_REFUSE("qk_norm_rope_kv_write_parts: rotary size %d must be 0 or the head size %d", rotary_dim, d);
  return launch_qk_norm_rope<__nv_bfloat16>(nullptr, qkv_parts, parts, (long long)num_tokens * (nq + 2 * nkv) * d, (__nv_bfloat16*)q_out, q_weight,
                                            k_weight, eps, cos_table, sin_table, rotary_dim, table_positions, positions, token_row, block_table,
                                            table_width, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages, nq, nkv, d,
                                            num_tokens, error, stream);
}

extern "C" int pylon_swiglu(const void* gate_up, void* out, int num_tokens, int inter, int interleaved, int dtype,
                            cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (inter <= 0) PYLON_REFUSE("swiglu: intermediate size %d", inter);
  if (interleaved && inter % 8) PYLON_REFUSE("swiglu: the interleaved layout needs an intermediate size that is a multiple of 8, not %d", inter);
  const size_t total = (size_t)num_tokens * inter;
  const int threads = 256;
  const size_t most = (size_t)pylon::multiprocessors() * 32;
  auto grid = [&](size_t n) { size_t b = (n + threads - 1) / threads; return (int)(b < most ? b : most); };
  if (dtype == PYLON_DTYPE_BF16 && inter % 8 == 0 && ((uintptr_t)gate_up % 16 == 0) && ((uintptr_t)out % 16 == 0)) {
    launch_dependent(swiglu_bf16x8_kernel, dim3(grid(total / 8)), dim3(threads), 0, stream, (const uint4*)gate_up, (uint4*)out, inter / 8, total / 8, interleaved);
  } else if (dtype == PYLON_DTYPE_BF16) {
    swiglu_kernel<__nv_bfloat16><<<grid(total), threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total, interleaved);
  } else if (dtype == PYLON_DTYPE_F32) {
    swiglu_kernel<float><<<grid(total), threads, 0, stream>>>((const float*)gate_up, (float*)out, inter, total, interleaved);
  } else {
    PYLON_REFUSE("swiglu: unknown dtype %d", dtype);
  }
  PYLON_CHECK_LAUNCH("swiglu");
}
