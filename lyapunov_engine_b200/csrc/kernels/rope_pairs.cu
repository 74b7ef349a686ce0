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

// Several attention maps of a head combined into one output, in 32 bits:
//   o = sum_m coef[m] * a_m   over the head's `segments` maps (each `head_dim`
// wide in `attn`, of which the first value_dim columns count), then, if
// eps >= 0, o / sqrt(mean(o^2) + eps), then times `post`.  One warp per
// (token, head).
template <typename T>
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
  for (int c = lane; c < value_dim; c += 32) {
    float v = 0.0f;
    for (int m = 0; m < segments; ++m) v = fmaf(coef[m], le::to_f32(a[m * head_dim + c]), v);
    sq += v * v;
  }
  sq = le::warp_sum(sq);
  const float factor = eps >= 0.0f ? rsqrtf(sq / static_cast<float>(value_dim) + eps) * post : post;
  for (int c = lane; c < value_dim; c += 32) {
    float v = 0.0f;
    for (int m = 0; m < segments; ++m) v = fmaf(coef[m], le::to_f32(a[m * head_dim + c]), v);
    o[c] = le::from_f32<T>(v * factor);
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
  if (dtype == LE_BF16)
    return le::launch_chained(rope_pairs_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                              static_cast<const __nv_bfloat16 *>(src), src_stride, bias, static_cast<__nv_bfloat16 *>(q_out),
                              q_stride, static_cast<__nv_bfloat16 *>(k_cache), static_cast<__nv_bfloat16 *>(v_cache), rates,
                              positions, request_of_token, block_table, max_blocks, heads, kv_heads, segments, seg_dim,
                              value_dim, rot, head_dim, page_size, num_pages, write_kv, status);
  return le::launch_chained(rope_pairs_store_kernel<float>, dim3(tokens), dim3(threads), 0, stream,
                            static_cast<const float *>(src), src_stride, bias, static_cast<float *>(q_out), q_stride,
                            static_cast<float *>(k_cache), static_cast<float *>(v_cache), rates, positions, request_of_token,
                            block_table, max_blocks, heads, kv_heads, segments, seg_dim, value_dim, rot, head_dim, page_size,
                            num_pages, write_kv, status);
}

LE_API int le_maps_combine(void *out, int64_t out_stride, const void *attn, int64_t attn_stride, int dtype, const float *coef,
                           int tokens, int heads, int segments, int head_dim, int value_dim, float eps, float post,
                           cudaStream_t stream) {
  const int64_t warps = static_cast<int64_t>(tokens) * heads;
  if (warps <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
  if (dtype == LE_BF16)
    return le::launch_chained(maps_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream,
                              static_cast<__nv_bfloat16 *>(out), out_stride, static_cast<const __nv_bfloat16 *>(attn),
                              attn_stride, coef, tokens, heads, segments, head_dim, value_dim, eps, post);
  return le::launch_chained(maps_combine_kernel<float>, dim3(blocks), dim3(256), 0, stream, static_cast<float *>(out),
                            out_stride, static_cast<const float *>(attn), attn_stride, coef, tokens, heads, segments, head_dim,
                            value_dim, eps, post);
}

LE_API int le_softcap(float *x, int64_t n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  softcap_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(x, n, cap);
  return le::launched();
}
