// Writes of a step's keys and values into the paged cache for mixers whose
// keys carry no position encoding.
//
// kv_store: keys and values are column ranges of the fused projection's rows;
// the token at position p of request b goes to page block_table[b][p / page]
// at offset p % page of pools laid out [pages, kv_heads, page, head_dim].
//
// latent_norm_store: one latent vector per token (a column range of the
// projection's rows, `rank` wide) is divided by its root mean square, times a
// weight, in 32 bits, rounded once, and stored as the single "head" of a pool
// [pages, 1, page, padded_rank]; columns from `rank` on are written as zeros.
// That pool serves as keys and as values of an attention over the latents.
#include "common.cuh"

namespace {

template <typename T>
__global__ void kv_store_kernel(const T *__restrict__ src, int64_t src_stride, int k_col, int v_col,
                                T *__restrict__ k_cache, T *__restrict__ v_cache,
                                const int32_t *__restrict__ positions, const int32_t *__restrict__ request_of_token,
                                const int32_t *__restrict__ block_table, int max_blocks, int num_kv_heads, int head_dim,
                                int page_size, int num_pages, int *__restrict__ status) {
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int b = request_of_token[t];
  const int page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
    return;
  }
  const T *row = src + static_cast<int64_t>(t) * src_stride;
  const int width = num_kv_heads * head_dim;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const int kvh = i / head_dim, d = i - kvh * head_dim;
    const int64_t at = ((static_cast<int64_t>(page) * num_kv_heads + kvh) * page_size + pos % page_size) * head_dim + d;
    k_cache[at] = row[k_col + i];
    v_cache[at] = row[v_col + i];
  }
}

template <typename T>
__global__ void latent_norm_store_kernel(const T *__restrict__ src, int64_t src_stride, int col, int rank, int padded_rank,
                                         const float *__restrict__ weight, float eps, T *__restrict__ cache,
                                         const int32_t *__restrict__ positions,
                                         const int32_t *__restrict__ request_of_token,
                                         const int32_t *__restrict__ block_table, int max_blocks, int page_size,
                                         int num_pages, int *__restrict__ status) {
  __shared__ float scratch[33];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int b = request_of_token[t];
  const int page = pos >= 0 ? block_table[static_cast<int64_t>(b) * max_blocks + pos / page_size] : -1;
  const bool bad = page < 0 || page >= num_pages;
  if (bad && threadIdx.x == 0) atomicOr(status, LE_STATUS_BAD_PAGE);
  const T *x = src + static_cast<int64_t>(t) * src_stride + col;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = le::to_f32(x[i]);
    ss += v * v;
  }
  ss = le::block_sum(ss, scratch);
  if (bad) return;
  const float inv = rsqrtf(ss / static_cast<float>(rank) + eps);
  T *dst = cache + (static_cast<int64_t>(page) * page_size + pos % page_size) * padded_rank;
  for (int i = threadIdx.x; i < padded_rank; i += blockDim.x)
    dst[i] = i < rank ? le::from_f32<T>(le::to_f32(x[i]) * inv * weight[i]) : le::from_f32<T>(0.0f);
}

}  // namespace

// src: rows of stride src_stride; keys start at column k_col, values at v_col, num_kv_heads * head_dim wide each.
LE_API int le_kv_store(const void *src, int64_t src_stride, int k_col, int v_col, void *k_cache, void *v_cache, int dtype,
                       const int32_t *positions, const int32_t *request_of_token, const int32_t *block_table,
                       int max_blocks, int num_tokens, int num_kv_heads, int head_dim, int page_size, int num_pages,
                       int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int width = num_kv_heads * head_dim;
  const int threads = width >= 512 ? 256 : 128;
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(kv_store_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream,
                                              static_cast<const T *>(src), src_stride, k_col, v_col,
                                              static_cast<T *>(k_cache), static_cast<T *>(v_cache), positions,
                                              request_of_token, block_table, max_blocks, num_kv_heads, head_dim,
                                              page_size, num_pages, status));
}

// src: rows of stride src_stride with the latent at columns col .. col + rank; cache: [pages, 1, page, padded_rank].
LE_API int le_latent_norm_store(const void *src, int64_t src_stride, int col, int rank, int padded_rank,
                                const float *weight, float eps, void *cache, int dtype, const int32_t *positions,
                                const int32_t *request_of_token, const int32_t *block_table, int max_blocks,
                                int num_tokens, int page_size, int num_pages, int *status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rank < 1 || padded_rank < rank) return le::invalid("le_latent_norm_store: rank %d, padded rank %d", rank, padded_rank);
  const int threads = rank >= 512 ? 256 : 128;
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(latent_norm_store_kernel<T>, dim3(num_tokens), dim3(threads), 0, stream,
                                              static_cast<const T *>(src), src_stride, col, rank, padded_rank, weight, eps,
                                              static_cast<T *>(cache), positions, request_of_token, block_table,
                                              max_blocks, page_size, num_pages, status));
}
