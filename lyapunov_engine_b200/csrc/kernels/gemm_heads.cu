// One small matrix product per head, on the FP32 pipes:
//
//   out[t, h, n] = gate(t, h) * sum_k a[t, h, k] * w[h, n, k]
//
// a: rows of stride a_stride with head h at columns h * K ..; w: [heads, N, K]
// contiguous; out: rows of stride out_stride with head h at columns h * N ..
// gate(t, h) is sigmoid(gate[t, h]) when `gate` is given, else 1.
//
// A latent-attention mixer uses it twice: to carry each head's query into the
// latent space (w = that head's key map, transposed) and to carry each head's
// attended latent out of it (w = the head's value map), where the per-head
// output gate rides in the epilogue.
//
// Two forms.  Many rows: tiles of 32 rows x 64 columns through shared memory,
// every output one chain of fused multiply-adds over ascending k.  Few rows (a
// decode step): no shared memory and no block-wide barrier; a warp takes four
// output columns of a head, its lanes share out k (each reads 16-byte pieces of
// the weight rows, which lie contiguous in k), and the lanes' partial sums meet
// in a shuffle tree.  In both forms a row's result is the same whatever rows
// stand beside it.  Sums are 32-bit; inputs float32 or bfloat16; the result is
// rounded once.
#include "common.cuh"
#include "gemm_heads_rows.cuh"

namespace {

using le_heads::GR_COLS;
using le_heads::GR_ROWS;
using le_heads::GR_WARPS;

constexpr int GH_BM = 32, GH_BN = 64, GH_BK = 32, GH_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(GH_THREADS)
gemm_heads_kernel(T *__restrict__ out, int64_t out_stride, const T *__restrict__ a, int64_t a_stride,
                  const T *__restrict__ w, const T *__restrict__ gate, int64_t gate_stride, int M, int N, int K) {
  __shared__ float sa[GH_BK][GH_BM + 1];
  __shared__ float sw[GH_BK][GH_BN + 1];
  le::let_successor_start();
  le::wait_for_predecessor();
  const int head = blockIdx.z;
  const int m0 = blockIdx.x * GH_BM, n0 = blockIdx.y * GH_BN;
  const int tid = threadIdx.x;
  const int tm = tid / 16, tn = tid % 16;           // this thread: rows tm, tm + 16; columns tn + 16 j
  const T *wh = w + static_cast<int64_t>(head) * N * K;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += GH_BK) {
    __syncthreads();
    for (int i = tid; i < GH_BM * GH_BK; i += GH_THREADS) {
      const int r = i / GH_BK, k = i % GH_BK;
      sa[k][r] = (m0 + r < M && k0 + k < K) ? le::to_f32(a[(m0 + r) * a_stride + static_cast<int64_t>(head) * K + k0 + k]) : 0.0f;
    }
    for (int i = tid; i < GH_BN * GH_BK; i += GH_THREADS) {
      const int n = i / GH_BK, k = i % GH_BK;
      sw[k][n] = (n0 + n < N && k0 + k < K) ? le::to_f32(wh[static_cast<int64_t>(n0 + n) * K + k0 + k]) : 0.0f;
    }
    __syncthreads();
    const int kmax = min(GH_BK, K - k0);
    for (int k = 0; k < kmax; ++k) {
      const float a0 = sa[k][tm], a1 = sa[k][tm + 16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = sw[k][tn + 16 * j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = m0 + tm + 16 * i;
    if (m >= M) continue;
    float g = 1.0f;
    if (gate) g = 1.0f / (1.0f + expf(-le::to_f32(gate[m * gate_stride + head])));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + 16 * j;
      if (n < N) out[m * out_stride + static_cast<int64_t>(head) * N + n] = le::from_f32<T>(acc[i][j] * g);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(le_heads::GR_WARPS * 32)
gemm_heads_rows_kernel(T *__restrict__ out, int64_t out_stride, const T *__restrict__ a, int64_t a_stride,
                       const T *__restrict__ w, const T *__restrict__ gate, int64_t gate_stride, int M, int N, int K) {
  le::let_successor_start();
  le_heads::gemm_heads_rows_block<T>(out, out_stride, a, a_stride, w, gate, gate_stride, M, N, K);
}

}  // namespace

// Up to this many rows the form without shared memory runs (where the operands' rows can be read in 16-byte pieces).
constexpr int GEMM_HEADS_FEW_ROWS = 32;

LE_API int le_gemm_heads(void *out, int64_t out_stride, const void *a, int64_t a_stride, const void *w, const void *gate,
                         int64_t gate_stride, int dtype, int M, int heads, int N, int K, cudaStream_t stream) {
  if (M <= 0 || heads <= 0 || N <= 0) return 0;
  if (K <= 0) return le::invalid("le_gemm_heads: K must be positive");
  const int vec = dtype == LE_BF16 ? 8 : 4;
  if (M <= GEMM_HEADS_FEW_ROWS && K % vec == 0 && a_stride % vec == 0 && heads <= 65535 &&
      ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) & 15) == 0) {
    const dim3 few((N + GR_WARPS * GR_COLS - 1) / (GR_WARPS * GR_COLS), heads, (M + GR_ROWS - 1) / GR_ROWS);
    LE_DISPATCH_DTYPE(dtype, T,
                      return le::launch_chained(gemm_heads_rows_kernel<T>, few, dim3(GR_WARPS * 32), 0, stream,
                                                static_cast<T *>(out), out_stride, static_cast<const T *>(a), a_stride,
                                                static_cast<const T *>(w), static_cast<const T *>(gate), gate_stride, M, N, K));
  }
  const dim3 grid((M + GH_BM - 1) / GH_BM, (N + GH_BN - 1) / GH_BN, heads);
  if (grid.y > 65535 || grid.z > 65535) return le::invalid("le_gemm_heads: too many columns or heads for one launch");
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(gemm_heads_kernel<T>, grid, dim3(GH_THREADS), 0, stream,
                                              static_cast<T *>(out), out_stride, static_cast<const T *>(a), a_stride,
                                              static_cast<const T *>(w), static_cast<const T *>(gate), gate_stride, M, N, K));
}
