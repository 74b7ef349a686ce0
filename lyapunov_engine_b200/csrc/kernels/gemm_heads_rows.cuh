// The few-rows form of the per-head products (see gemm_heads.cu) as a block's
// work, for kernels that run it beside other work in one launch.
#pragma once

#include "common.cuh"

namespace le_heads {

constexpr int GR_ROWS = 8;      // rows of a a block takes (blockIdx.z walks the rest)
constexpr int GR_COLS = 4;      // output columns per warp
constexpr int GR_WARPS = 4;

// The work of one block of the few-rows form (blockIdx.x: 16 output columns, blockIdx.y: the head, blockIdx.z: 8 rows).
template <typename T>
__device__ __forceinline__ void gemm_heads_rows_block(T *__restrict__ out, int64_t out_stride, const T *__restrict__ a,
                                                      int64_t a_stride, const T *__restrict__ w, const T *__restrict__ gate,
                                                      int64_t gate_stride, int M, int N, int K) {
  constexpr int VEC = 16 / sizeof(T);
  const int head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * GR_WARPS + warp) * GR_COLS;
  const int m0 = blockIdx.z * GR_ROWS;
  const int rows = min(GR_ROWS, M - m0);
  if (n0 >= N) return;
  const T *wh = w + (static_cast<int64_t>(head) * N + n0) * K;
  float acc[GR_ROWS][GR_COLS] = {};
  // lanes take pieces of VEC consecutive k; K is a multiple of VEC (checked by the launcher).  The weights do not
  // depend on the kernel before this one: a lane's first pieces of them are asked for before the wait for it.
  auto load_weights = [&](float (&wv)[GR_COLS][VEC], int k) {
#pragma unroll
    for (int c = 0; c < GR_COLS; ++c) {
      if (n0 + c < N && k < K) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(wh + static_cast<int64_t>(c) * K + k);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int v = 0; v < VEC; ++v) wv[c][v] = le::to_f32(e[v]);
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) wv[c][v] = 0.0f;
      }
    }
  };
  float wv[GR_COLS][VEC];
  load_weights(wv, lane * VEC);
  le::wait_for_predecessor();
  for (int k = lane * VEC; k < K; k += 32 * VEC) {
    if (k != lane * VEC) load_weights(wv, k);
#pragma unroll
    for (int r = 0; r < GR_ROWS; ++r) {
      if (r < rows) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(a + (m0 + r) * a_stride + static_cast<int64_t>(head) * K + k);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          const float x = le::to_f32(e[v]);
#pragma unroll
          for (int c = 0; c < GR_COLS; ++c) acc[r][c] = fmaf(x, wv[c][v], acc[r][c]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < GR_ROWS; ++r)
#pragma unroll
    for (int c = 0; c < GR_COLS; ++c) acc[r][c] = le::warp_sum(acc[r][c]);
  if (lane < GR_COLS && n0 + lane < N) {
    for (int r = 0; r < rows; ++r) {
      float g = 1.0f;
      if (gate) g = 1.0f / (1.0f + expf(-le::to_f32(gate[(m0 + r) * gate_stride + head])));
      float v = acc[r][0];
#pragma unroll
      for (int c = 1; c < GR_COLS; ++c) v = lane == c ? acc[r][c] : v;
      out[(m0 + r) * out_stride + static_cast<int64_t>(head) * N + n0 + lane] = le::from_f32<T>(v * g);
    }
  }
}


}  // namespace le_heads
