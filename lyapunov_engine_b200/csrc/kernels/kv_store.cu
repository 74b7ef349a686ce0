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
//
// latent_prepare (few rows, a decode step): latent_norm_store and the
// per-head products that carry each head's query into the latent space, in one
// launch: both read the projection's rows and neither reads the other's
// result.  Blocks whose blockIdx.y is below `heads` do the products, those at
// blockIdx.y == heads walk the tokens.
#include "common.cuh"
#include "gemm_heads_rows.cuh"

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

// One token's latent: norm and store (the whole block works on it).
template <typename T>
__device__ __forceinline__ void latent_norm_store_token(int t, float *scratch, const T *__restrict__ src, int64_t src_stride,
                                                        int col, int rank, int padded_rank, const float *__restrict__ weight,
                                                        float eps, T *__restrict__ cache, const int32_t *__restrict__ positions,
                                                        const int32_t *__restrict__ request_of_token,
                                                        const int32_t *__restrict__ block_table, int max_blocks, int page_size,
                                                        int num_pages, int *__restrict__ status) {
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
  latent_norm_store_token<T>(blockIdx.x, scratch, src, src_stride, col, rank, padded_rank, weight, eps, cache, positions,
                             request_of_token, block_table, max_blocks, page_size, num_pages, status);
}

template <typename T>
__global__ void __launch_bounds__(le_heads::GR_WARPS * 32)
latent_prepare_kernel(const T *__restrict__ src, int64_t src_stride, int num_tokens, int heads, int head_dim,
                      const T *__restrict__ w_into, T *__restrict__ q_latent, int64_t q_latent_stride, int col, int rank,
                      int padded_rank, const float *__restrict__ weight, float eps, T *__restrict__ cache,
                      const int32_t *__restrict__ positions, const int32_t *__restrict__ request_of_token,
                      const int32_t *__restrict__ block_table, int max_blocks, int page_size, int num_pages,
                      int *__restrict__ status) {
  __shared__ float scratch[33];
  le::let_successor_start();
  if (static_cast<int>(blockIdx.y) < heads) {
    le_heads::gemm_heads_rows_block<T>(q_latent, q_latent_stride, src, src_stride, w_into, static_cast<const T *>(nullptr), 0,
                                       num_tokens, padded_rank, head_dim);
    return;
  }
  le::wait_for_predecessor();
  if (cache == nullptr) return;
  for (int t = blockIdx.z * gridDim.x + blockIdx.x; t < num_tokens; t += gridDim.x * gridDim.z)
    latent_norm_store_token<T>(t, scratch, src, src_stride, col, rank, padded_rank, weight, eps, cache, positions,
                               request_of_token, block_table, max_blocks, page_size, num_pages, status);
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

// For at most 32 rows.  src: the projection's rows (stride src_stride, 16-byte aligned): head h's query at columns
// h * head_dim .., the latent at columns col .. col + rank.  q_latent[t, h, :] = w_into[h] @ query (w_into:
// [heads, padded_rank, head_dim]); the latent is normed and stored as le_latent_norm_store does (cache null: not stored).
LE_API int le_latent_prepare(const void *src, int64_t src_stride, int num_tokens, int heads, int head_dim, const void *w_into,
                             void *q_latent, int64_t q_latent_stride, int col, int rank, int padded_rank, const float *weight,
                             float eps, void *cache, int dtype, const int32_t *positions, const int32_t *request_of_token,
                             const int32_t *block_table, int max_blocks, int page_size, int num_pages, int *status,
                             cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int vec = dtype == LE_BF16 ? 8 : 4;
  if (num_tokens > 32 || head_dim % vec || src_stride % vec || heads < 1 || heads >= 65535 ||
      ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(w_into)) & 15))
    return le::invalid("le_latent_prepare: at most 32 rows, 16-byte aligned rows and head sizes");
  if (rank < 1 || padded_rank < rank) return le::invalid("le_latent_prepare: rank %d, padded rank %d", rank, padded_rank);
  const dim3 grid((padded_rank + le_heads::GR_WARPS * le_heads::GR_COLS - 1) / (le_heads::GR_WARPS * le_heads::GR_COLS), heads + 1,
                  (num_tokens + le_heads::GR_ROWS - 1) / le_heads::GR_ROWS);
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(latent_prepare_kernel<T>, grid, dim3(le_heads::GR_WARPS * 32), 0, stream,
                                              static_cast<const T *>(src), src_stride, num_tokens, heads, head_dim,
                                              static_cast<const T *>(w_into), static_cast<T *>(q_latent), q_latent_stride, col,
                                              rank, padded_rank, weight, eps, static_cast<T *>(cache), positions,
                                              request_of_token, block_table, max_blocks, page_size, num_pages, status));
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
