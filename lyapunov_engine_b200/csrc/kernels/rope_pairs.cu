// Rotary positions on neighbouring pairs, for heads made of several segments,
// fused with the projection's bias, the layout the attention kernels read and
// the paged cache write.
//
// The projection's row of a token holds, in this order,
//   queries  [heads][segments][seg_dim]
//   keys     [kv_heads][segments][seg_dim]
//   values   [kv_heads][value_dim]
// and `bias` (float32, as wide as the row, or nullptr) is added first.  In each
// segment the entries (2i, 2i + 1), 2i + 1 < rot, turn by the angle
// position * rates[i]: (a, b) -> (a cos - b sin, b cos + a sin).  Angle, sine,
// cosine and rotation are 32-bit; the result is rounded once.
//
// Each (head, segment) becomes a query head of its own, `head_dim` wide, with
// the segment at columns [segment * seg_dim, (segment + 1) * seg_dim) and zeros
// elsewhere; a key head is the kv head's segments side by side.  So the dot
// product of such a query with such a key is the segment's own dot product,
// and segments * heads query heads share kv_heads key/value heads the way
// grouped queries do.  Values fill the first value_dim columns of their head;
// all padding columns are written as zeros.  With one segment this is plain
// rotary encoding in the interleaved layout.
#include "common.cuh"

namespace {

template <typename T>
__global__ void rope_pairs_store_kernel(const T *__restrict__ src, int64_t src_stride, const float *__restrict__ bias,
                                        T *__restrict__ q_out, int64_t q_stride, T *__restrict__ k_cache,
                                        T *__restrict__ v_cache, const float *__restrict__ rates,
                                        const int32_t *__restrict__ positions, const int32_t *__restrict__ request_of_token,
                                        const int32_t *__restrict__ block_table, int max_blocks, int heads, int kv_heads,
                                        int segments, int seg_dim, int value_dim, int rot, int head_dim, int page_size,
                                        int num_pages, int write_kv, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = static_cast<float>(pos);
  const T *row = src + static_cast<int64_t>(t) * src_stride;
  const int q_cols = heads * segments * seg_dim, k_cols = kv_heads * segments * seg_dim;

  // the rotated value of entry j of the segment that starts at column `col` of the row
  auto rotated = [&](int col, int j) -> float {
    float a = le::to_f32(row[col + j]);
    if (bias != nullptr) a += bias[col + j];
    if (j >= (rot & ~1)) return a;
    const int partner = j ^ 1;
    float b = le::to_f32(row[col + partner]);
    if (bias != nullptr) b += bias[col + partner];
    float s, c;
    sincosf(fpos * rates[j >> 1], &s, &c);
    return (j & 1) ? a * c + b * s : a * c - b * s;
  };

  T *q_row = q_out + static_cast<int64_t>(t) * q_stride;
  const int q_heads = heads * segments;
  for (int i = threadIdx.x; i < q_heads * head_dim; i += blockDim.x) {
    const int qh = i / head_dim, c = i - qh * head_dim;
    const int seg = qh % segments, j = c - seg * seg_dim;
    float v = 0.0f;
    if (j >= 0 && j < seg_dim) v = rotated(qh * seg_dim, j);
    q_row[i] = le::from_f32<T>(v);
  }
  if (!write_kv) return;
  const int b = request_of_token[t];
  const int page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
    return;
  }
  const int key_width = segments * seg_dim;
  for (int i = threadIdx.x; i < kv_heads * head_dim; i += blockDim.x) {
    const int g = i / head_dim, c = i - g * head_dim;
    const int64_t at = ((static_cast<int64_t>(page) * kv_heads + g) * page_size + pos % page_size) * head_dim + c;
    float k = 0.0f, v = 0.0f;
    if (c < key_width) {
      const int seg = c / seg_dim;
      k = rotated(q_cols + (g * segments + seg) * seg_dim, c - seg * seg_dim);
    }
    if (c < value_dim) {
      const int col = q_cols + k_cols + g * value_dim + c;
      v = le::to_f32(row[col]);
      if (bias != nullptr) v += bias[col];
    }
    k_cache[at] = le::from_f32<T>(k);
    v_cache[at] = le::from_f32<T>(v);
  }
}


// Eight consecutive elements as floats (16 bytes of bfloat16, 32 of float32).
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4 *>(p);
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16 *p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4 *>(p) = raw;
}
__device__ __forceinline__ void store8(float *p, const float (&v)[8]) {
  *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// The same in pieces of eight elements (seg_dim, value_dim and every offset multiples of 8, 16-byte aligned rows): a
// token's cosines and sines are computed once into shared memory, a thread moves 16 or 32 bytes at a time.
template <typename T>
__global__ void __launch_bounds__(256)
rope_pairs_store_vec_kernel(const T *__restrict__ src, int64_t src_stride, const float *__restrict__ bias,
                            T *__restrict__ q_out, int64_t q_stride, T *__restrict__ k_cache, T *__restrict__ v_cache,
                            const float *__restrict__ rates, const int32_t *__restrict__ positions,
                            const int32_t *__restrict__ request_of_token, const int32_t *__restrict__ block_table,
                            int max_blocks, int heads, int kv_heads, int segments, int seg_dim, int value_dim, int rot,
                            int head_dim, int page_size, int num_pages, int write_kv, int *__restrict__ status) {
  extern __shared__ float cs[];        // cos [rot / 2], sin [rot / 2]
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(static_cast<float>(pos) * rates[i], &cs[half + i], &cs[i]);
  __syncthreads();
  const T *row = src + static_cast<int64_t>(t) * src_stride;
  const int q_cols = heads * segments * seg_dim, k_cols = kv_heads * segments * seg_dim;

  // eight entries of a segment from column `col` of the row, entry j0 the first: bias added, pairs below `rot` turned
  auto turned = [&](int col, int j0, float (&v)[8]) {
    load8(row + col + j0, v);
    if (bias != nullptr) {
      float b[8];
      load8(bias + col + j0, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += b[i];
    }
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const int j = j0 + i;
      if (j + 1 < rot) {
        const float c = cs[j >> 1], s = cs[half + (j >> 1)];
        const float a = v[i], b = v[i + 1];
        v[i] = a * c - b * s;
        v[i + 1] = b * c + a * s;
      }
    }
  };

  T *q_row = q_out + static_cast<int64_t>(t) * q_stride;
  const int pieces = head_dim >> 3;
  const int q_heads = heads * segments;
  for (int i = threadIdx.x; i < q_heads * pieces; i += blockDim.x) {
    const int qh = i / pieces, c = (i - qh * pieces) << 3;
    const int seg = qh % segments, j = c - seg * seg_dim;
    float v[8] = {};
    if (j >= 0 && j < seg_dim) turned(qh * seg_dim, j, v);
    store8(q_row + qh * head_dim + c, v);
  }
  if (!write_kv) return;
  const int b = request_of_token[t];
  const int page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
    return;
  }
  const int key_width = segments * seg_dim;
  for (int i = threadIdx.x; i < kv_heads * pieces; i += blockDim.x) {
    const int g = i / pieces, c = (i - g * pieces) << 3;
    const int64_t at = ((static_cast<int64_t>(page) * kv_heads + g) * page_size + pos % page_size) * head_dim + c;
    float k[8] = {}, v[8] = {};
    if (c < key_width) {
      const int seg = c / seg_dim;
      turned(q_cols + (g * segments + seg) * seg_dim, c - seg * seg_dim, k);
    }
    if (c < value_dim) {
      const int col = q_cols + k_cols + g * value_dim + c;
      load8(row + col, v);
      if (bias != nullptr) {
        float bb[8];
        load8(bias + col, bb);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += bb[e];
      }
    }
    store8(k_cache + at, k);
    store8(v_cache + at, v);
  }
}

// Several attention maps of a head combined into one output, in 32 bits:
//   o = sum_m coef[m] * a_m   over the head's `segments` maps (each `head_dim`
// wide in `attn`, of which the first value_dim columns count), then, if
// eps >= 0, o / sqrt(mean(o^2) + eps), then times `post`.  One warp per
// (token, head).
// VEC (1, 2, 4 or 8) consecutive elements as floats, in one access where VEC > 1.
template <int VEC, typename T>
__device__ __forceinline__ void loadv(const T *p, float (&v)[VEC]) {
  struct __align__(sizeof(T) * VEC) Raw { T e[VEC]; };
  const Raw raw = *reinterpret_cast<const Raw *>(p);
#pragma unroll
  for (int i = 0; i < VEC; ++i) v[i] = le::to_f32(raw.e[i]);
}
template <int VEC, typename T>
__device__ __forceinline__ void storev(T *p, const float (&v)[VEC]) {
  struct __align__(sizeof(T) * VEC) Raw { T e[VEC]; };
  Raw raw;
#pragma unroll
  for (int i = 0; i < VEC; ++i) raw.e[i] = le::from_f32<T>(v[i]);
  *reinterpret_cast<Raw *>(p) = raw;
}

template <typename T, int VEC>
__global__ void maps_combine_kernel(T *__restrict__ out, int64_t out_stride, const T *__restrict__ attn, int64_t attn_stride,
                                    const float *__restrict__ coef, int tokens, int heads, int segments, int head_dim,
                                    int value_dim, float eps, float post) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens * heads) return;
  const int t = warp / heads, h = warp - t * heads;
  const T *a = attn + static_cast<int64_t>(t) * attn_stride + static_cast<int64_t>(h) * segments * head_dim;
  T *o = out + static_cast<int64_t>(t) * out_stride + static_cast<int64_t>(h) * value_dim;
  float sq = 0.0f;
  for (int c = lane * VEC; c < value_dim; c += 32 * VEC) {
    float v[VEC] = {};
    for (int m = 0; m < segments; ++m) {
      const float cm = coef[m];
      float x[VEC];
      loadv<VEC>(a + m * head_dim + c, x);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = fmaf(cm, x[i], v[i]);
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) sq += v[i] * v[i];
  }
  sq = le::warp_sum(sq);
  const float factor = eps >= 0.0f ? rsqrtf(sq / static_cast<float>(value_dim) + eps) * post : post;
  for (int c = lane * VEC; c < value_dim; c += 32 * VEC) {
    float v[VEC] = {};
    for (int m = 0; m < segments; ++m) {
      const float cm = coef[m];
      float x[VEC];
      loadv<VEC>(a + m * head_dim + c, x);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = fmaf(cm, x[i], v[i]);
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] *= factor;
    storev<VEC>(o + c, v);
  }
}

// x <- cap * tanh(x / cap), float32 in place.
__global__ void softcap_kernel(float *__restrict__ x, int64_t n, float cap) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace

LE_API int le_rope_pairs_store(const void *src, int64_t src_stride, int dtype, const float *bias, void *q_out, int64_t q_stride,
                               void *k_cache, void *v_cache, const float *rates, const int32_t *positions,
                               const int32_t *request_of_token, const int32_t *block_table, int max_blocks, int tokens,
                               int heads, int kv_heads, int segments, int seg_dim, int value_dim, int rot, int head_dim,
                               int page_size, int num_pages, int write_kv, int *status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (segments < 1 || segments * seg_dim > head_dim || value_dim > head_dim || rot > seg_dim || rot < 0)
    return le::invalid("le_rope_pairs_store: %d segments of %d (rotary width %d) and values of %d do not fit heads of %d",
                       segments, seg_dim, rot, value_dim, head_dim);
  const int threads = 256;
  const int elem = dtype == LE_BF16 ? 2 : 4;
  auto aligned = [&](const void *p) { return reinterpret_cast<uintptr_t>(p) % (8 * elem) == 0; };
  const bool vec = seg_dim % 8 == 0 && value_dim % 8 == 0 && head_dim % 8 == 0 && src_stride % 8 == 0 && q_stride % 8 == 0 &&
                   aligned(src) && aligned(q_out) && (!write_kv || (aligned(k_cache) && aligned(v_cache))) &&
                   reinterpret_cast<uintptr_t>(bias) % 32 == 0;
  const size_t smem = sizeof(float) * (rot > 0 ? rot : 2);
#define LE_ROPE_PAIRS(KERNEL, T, SMEM)                                                                                    \
  return le::launch_chained(KERNEL<T>, dim3(tokens), dim3(threads), SMEM, stream, static_cast<const T *>(src), src_stride, \
                            bias, static_cast<T *>(q_out), q_stride, static_cast<T *>(k_cache), static_cast<T *>(v_cache), \
                            rates, positions, request_of_token, block_table, max_blocks, heads, kv_heads, segments,       \
                            seg_dim, value_dim, rot, head_dim, page_size, num_pages, write_kv, status)
  if (dtype == LE_BF16) {
    if (vec) LE_ROPE_PAIRS(rope_pairs_store_vec_kernel, __nv_bfloat16, smem);
    LE_ROPE_PAIRS(rope_pairs_store_kernel, __nv_bfloat16, 0);
  }
  if (vec) LE_ROPE_PAIRS(rope_pairs_store_vec_kernel, float, smem);
  LE_ROPE_PAIRS(rope_pairs_store_kernel, float, 0);
#undef LE_ROPE_PAIRS
}

LE_API int le_maps_combine(void *out, int64_t out_stride, const void *attn, int64_t attn_stride, int dtype, const float *coef,
                           int tokens, int heads, int segments, int head_dim, int value_dim, float eps, float post,
                           cudaStream_t stream) {
  const int64_t warps = static_cast<int64_t>(tokens) * heads;
  if (warps <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  const int elem = dtype == LE_BF16 ? 2 : 4;
  // the widest piece (8, 4 or 2 elements) that divides everything and still gives each of a warp's lanes one
  int vec = 1;
  for (int v = 8; v > 1; v >>= 1)
    if (value_dim % v == 0 && head_dim % v == 0 && out_stride % v == 0 && attn_stride % v == 0 &&
        reinterpret_cast<uintptr_t>(out) % (v * elem) == 0 && reinterpret_cast<uintptr_t>(attn) % (v * elem) == 0 &&
        (value_dim / v >= 32 || v == 2)) {
      vec = v;
      break;
    }
#define LE_COMBINE(T, VEC)                                                                                                   \
  return le::launch_chained(maps_combine_kernel<T, VEC>, dim3(blocks), dim3(256), 0, stream, static_cast<T *>(out), out_stride, \
                            static_cast<const T *>(attn), attn_stride, coef, tokens, heads, segments, head_dim, value_dim, eps, \
                            post)
  if (dtype == LE_BF16) {
    if (vec == 8) LE_COMBINE(__nv_bfloat16, 8);
    if (vec == 4) LE_COMBINE(__nv_bfloat16, 4);
    if (vec == 2) LE_COMBINE(__nv_bfloat16, 2);
    LE_COMBINE(__nv_bfloat16, 1);
  }
  if (vec == 8) LE_COMBINE(float, 8);
  if (vec == 4) LE_COMBINE(float, 4);
  if (vec == 2) LE_COMBINE(float, 2);
  LE_COMBINE(float, 1);
#undef LE_COMBINE
}

LE_API int le_softcap(float *x, int64_t n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  softcap_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(x, n, cap);
  return le::launched();
}
