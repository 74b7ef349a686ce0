// A residual stream kept as S parallel copies ("hyper-connections"), and the
// norm that reads it, as one kernel.
//
// For a row t with copies x_0 .. x_{S-1} (float32 [T, S, W]) one launch does,
// in 32 bits throughout:
//   1. the pending update of the sub-layer before it, whose output is y:
//        x'_j = sum_s M[s][j] x_s + post[j] * y         (all j from the old x)
//      (y in the activations' type, or float32 partial sums of a split-K
//      product, added in order); without y the copies stay as they are; with
//      `init` (float32 [T, W]) every copy starts as that row;
//   2. the read of the next sub-layer: u = sum_s pre[s] x'_s (pre == nullptr:
//      the plain sum of the copies, what the model's last norm reads);
//   3. a norm of u: layer norm ((u - mean) / sqrt(var + eps) * w + b, var the
//      mean of squared deviations, two passes) or, without b, RMS norm.
// With `rows` only the listed rows are read and normed (into out[0 .. n)) and
// the copies are left as they are in memory.  S = 1 with M, post and pre all
// nullptr is the ordinary residual addition x += y before a norm.
#include "common.cuh"

namespace {

constexpr int MOST_STREAMS = 8;

template <typename T, int VEC> struct Pack;
template <> struct Pack<float, 1> { float v; __device__ float get(int) const { return v; } __device__ void set(int, float x) { v = x; } };
template <> struct Pack<__nv_bfloat16, 1> {
  __nv_bfloat16 v;
  __device__ float get(int) const { return __bfloat162float(v); }
  __device__ void set(int, float x) { v = __float2bfloat16_rn(x); }
};
template <> struct __align__(16) Pack<float, 4> { float v[4]; __device__ float get(int i) const { return v[i]; } __device__ void set(int i, float x) { v[i] = x; } };
template <> struct __align__(8) Pack<__nv_bfloat16, 4> {
  __nv_bfloat16 v[4];
  __device__ float get(int i) const { return __bfloat162float(v[i]); }
  __device__ void set(int i, float x) { v[i] = __float2bfloat16_rn(x); }
};

// VEC consecutive columns a thread and step (4: 16-byte accesses; the launcher sizes the block so that a row of up to
// 2,048 columns is one step, every load of a thread in flight before its first store).
template <typename TOut, typename TDelta, int VEC, int MAX_STREAMS>
__global__ void __launch_bounds__(512)
stream_norm_kernel(TOut *__restrict__ out, float *__restrict__ streams, const float *__restrict__ init,
                   const TDelta *__restrict__ delta, int parts, int64_t part_stride, const float *__restrict__ mix,
                   const float *__restrict__ post, const float *__restrict__ pre, const float *__restrict__ weight,
                   const float *__restrict__ bias, const int32_t *__restrict__ rows, float eps, int W, int S) {
  extern __shared__ float smem[];
  float *u_row = smem;               // [W]
  float *scratch = smem + W;         // [33]
  float *coef = scratch + 33;        // mix [S * S], post [S], pre [S]
  le::let_successor_start();
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) coef[i] = mix != nullptr ? mix[i] : (i / S == i % S ? 1.0f : 0.0f);
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    coef[S * S + i] = post != nullptr ? post[i] : 1.0f;
    coef[S * S + S + i] = pre != nullptr ? pre[i] : 1.0f;
  }
  le::wait_for_predecessor();
  __syncthreads();
  const int r = blockIdx.x;
  const int64_t t = rows != nullptr ? rows[r] : r;
  const bool write_back = rows == nullptr && (delta != nullptr || init != nullptr);
  float *x_row = streams + t * S * W;
  using F = Pack<float, VEC>;
  using D = Pack<TDelta, VEC>;
  float sum = 0.0f;
  for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
    F x[MAX_STREAMS];
    if (init != nullptr) {
      const F v = *reinterpret_cast<const F *>(init + t * W + c);
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s) x[s] = v;
    } else {
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) x[s] = *reinterpret_cast<const F *>(x_row + static_cast<int64_t>(s) * W + c);
    }
    if (delta != nullptr) {
      float y[VEC] = {};
      for (int p = 0; p < parts; ++p) {
        const D d = *reinterpret_cast<const D *>(delta + p * part_stride + t * W + c);
#pragma unroll
        for (int i = 0; i < VEC; ++i) y[i] += d.get(i);
      }
      F nx[MAX_STREAMS];
#pragma unroll
      for (int j = 0; j < MAX_STREAMS; ++j) {
        if (j < S) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            float acc = 0.0f;
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
              if (s < S) acc = fmaf(coef[s * S + j], x[s].get(i), acc);
            nx[j].set(i, fmaf(coef[S * S + j], y[i], acc));
          }
        }
      }
#pragma unroll
      for (int j = 0; j < MAX_STREAMS; ++j)
        if (j < S) x[j] = nx[j];
    }
    if (write_back) {
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) *reinterpret_cast<F *>(x_row + static_cast<int64_t>(s) * W + c) = x[s];
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float u = 0.0f;
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) u = fmaf(coef[S * S + S + s], x[s].get(i), u);
      u_row[c + i] = u;
      sum += u;
    }
  }
  float mean = 0.0f;
  if (bias != nullptr) mean = le::block_sum(sum, scratch) / static_cast<float>(W);
  float sq = 0.0f;
  for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float d = u_row[c + i] - mean;
      sq += d * d;
    }
  }
  const float inv = rsqrtf(le::block_sum(sq, scratch) / static_cast<float>(W) + eps);
  TOut *o = out + static_cast<int64_t>(r) * W;
  for (int c = threadIdx.x * VEC; c < W; c += blockDim.x * VEC) {
    const F wv = *reinterpret_cast<const F *>(weight + c);
    F bv;
    if (bias != nullptr) bv = *reinterpret_cast<const F *>(bias + c);
    Pack<TOut, VEC> res;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float v = (u_row[c + i] - mean) * inv * wv.get(i);
      if (bias != nullptr) v += bv.get(i);
      res.set(i, v);
    }
    *reinterpret_cast<Pack<TOut, VEC> *>(o + c) = res;
  }
}

// sum of the copies of every row, float32 [T, W] (what a caller that wants the
// stream itself, not its norm, reads)
__global__ void stream_sum_kernel(float *__restrict__ out, const float *__restrict__ streams, int64_t n, int W, int S) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t t = i / W, c = i - t * W;
  float acc = 0.0f;
  for (int s = 0; s < S; ++s) acc += streams[(t * S + s) * W + c];
  out[i] = acc;
}

template <typename TOut, typename TDelta>
int launch_stream_norm(void *out, float *streams, const float *init, const void *delta, int parts, int64_t part_stride,
                       const float *mix, const float *post, const float *pre, const float *weight, const float *bias,
                       const int32_t *rows, float eps, int n, int W, int S, cudaStream_t stream) {
  const size_t smem = sizeof(float) * (W + 33 + S * S + 2 * S);
  auto aligned = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = W % 4 == 0 && aligned(out) && aligned(streams) && aligned(init) && aligned(delta) && aligned(weight) &&
                   aligned(bias) && part_stride % 4 == 0;
  // few rows (a decode step): a thread per 16 bytes, so that a row is one round of loads; many rows: smaller blocks,
  // several to a multiprocessor, which hide each other's rounds
  int threads = vec ? (W / 4 + 31) / 32 * 32 : (W >= 1024 ? 256 : 128);
  const int most = n <= 64 ? 512 : 256;
  threads = threads > most ? most : threads;
#define LE_STREAM_NORM(VEC, BOUND)                                                                                          \
  return le::launch_chained(stream_norm_kernel<TOut, TDelta, VEC, BOUND>, dim3(n), dim3(threads), smem, stream,             \
                            static_cast<TOut *>(out), streams, init, static_cast<const TDelta *>(delta), parts, part_stride, \
                            mix, post, pre, weight, bias, rows, eps, W, S)
  if (vec) {
    if (S == 1) LE_STREAM_NORM(4, 1);
    if (S == 2) LE_STREAM_NORM(4, 2);
    if (S <= 4) LE_STREAM_NORM(4, 4);
    LE_STREAM_NORM(4, 8);
  }
  if (S <= 4) LE_STREAM_NORM(1, 4);
  LE_STREAM_NORM(1, 8);
#undef LE_STREAM_NORM
}

}  // namespace

LE_API int le_stream_norm(void *out, int out_dtype, float *streams, const float *init, const void *delta, int delta_dtype,
                          int parts, int64_t part_stride, const float *mix, const float *post, const float *pre,
                          const float *weight, const float *bias, const int32_t *rows, float eps, int n, int W, int S,
                          cudaStream_t stream) {
  if (n <= 0) return 0;
  if (S < 1 || S > MOST_STREAMS) return le::invalid("le_stream_norm: 1 to %d copies of the stream, got %d", MOST_STREAMS, S);
  if (W < 1 || W > 11000) return le::invalid("le_stream_norm: rows of up to 11000 values, got %d", W);
  if (delta == nullptr) parts = 0;
  if (out_dtype == LE_BF16 && (delta == nullptr || delta_dtype == LE_BF16))
    return launch_stream_norm<__nv_bfloat16, __nv_bfloat16>(out, streams, init, delta, parts, part_stride, mix, post, pre,
                                                            weight, bias, rows, eps, n, W, S, stream);
  if (out_dtype == LE_BF16)
    return launch_stream_norm<__nv_bfloat16, float>(out, streams, init, delta, parts, part_stride, mix, post, pre, weight,
                                                    bias, rows, eps, n, W, S, stream);
  if (delta != nullptr && delta_dtype != LE_F32) return le::invalid("le_stream_norm: float32 rows take a float32 update");
  return launch_stream_norm<float, float>(out, streams, init, delta, parts, part_stride, mix, post, pre, weight, bias, rows,
                                          eps, n, W, S, stream);
}

LE_API int le_stream_sum(float *out, const float *streams, int T, int W, int S, cudaStream_t stream) {
  const int64_t n = static_cast<int64_t>(T) * W;
  if (n <= 0) return 0;
  stream_sum_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(out, streams, n, W, S);
  return le::launched();
}
