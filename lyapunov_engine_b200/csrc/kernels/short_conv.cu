// Causal convolution over time on every channel, added to its own input, with
// the last inputs of each request kept as per-request state between steps:
//
//   out[t] = h[t] + sum_{j < taps} w[j] * h[t - (taps - 1 - j)]        (per channel)
//
// where h before the start of a request is zero.  A step brings any cut of a
// request's tokens (a whole prompt, a portion of two tokens, one decoded
// token); inputs from before the step come from the request's state row
// [taps - 1, channels], which holds the inputs at the taps - 1 positions before
// the step, oldest first, and is brought up to date here.
//
// Work is cut into tiles of TILE consecutive tokens of one request (the
// step's tile lists) times slices of channels; a thread owns VEC neighbouring
// channels of its tile (one 16-byte access where the sizes allow it).  Only a
// request's first tile reads the state, and the thread that read a channel's
// state is the one that writes it, after its reads, from the step's inputs
// (which this kernel only reads): no other block touches that state, so one
// launch serves every cut.  Rows that stand for no request (slot < 0) see
// zeros before them and keep nothing.  In a step whose requests all bring one
// token (`tile_request` null) request b is tile b: no list is read.
//
// Sums are 32-bit, rounded once.
#include "common.cuh"

namespace {

constexpr int CONV_THREADS = 128;
constexpr int CONV_MAX_TAPS = 17;   // a tile of 16 tokens must hold the taps - 1 inputs before the next tile

// VEC values at p as floats / from floats, in 16-byte accesses where VEC > 1 (p is then 16-byte aligned and VEC a
// multiple of the values one access holds).
template <typename T, int VEC>
__device__ __forceinline__ void load_channels(float (&dst)[VEC], const T *p) {
  if constexpr (VEC == 1) {
    dst[0] = le::to_f32(*p);
  } else {
    constexpr int PER = 16 / sizeof(T);
    static_assert(VEC % PER == 0, "whole 16-byte accesses");
#pragma unroll
    for (int i = 0; i < VEC; i += PER) {
      const uint4 raw = *reinterpret_cast<const uint4 *>(p + i);
      const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
      for (int v = 0; v < PER; ++v) dst[i + v] = le::to_f32(e[v]);
    }
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void store_channels(T *p, const float (&src)[VEC]) {
  if constexpr (VEC == 1) {
    *p = le::from_f32<T>(src[0]);
  } else {
    constexpr int PER = 16 / sizeof(T);
    static_assert(VEC % PER == 0, "whole 16-byte accesses");
#pragma unroll
    for (int i = 0; i < VEC; i += PER) {
      uint4 raw;
      T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
      for (int v = 0; v < PER; ++v) e[v] = le::from_f32<T>(src[i + v]);
      *reinterpret_cast<uint4 *>(p + i) = raw;
    }
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_kernel(T *__restrict__ out, const T *__restrict__ h, const float *__restrict__ w, float *__restrict__ state,
                  int num_state_rows, const int32_t *__restrict__ state_slots, const int32_t *__restrict__ cu_q,
                  const int32_t *__restrict__ tile_request, const int32_t *__restrict__ tile_q0, int tile, int channels,
                  int taps) {
  le::let_successor_start();
  const int c = (blockIdx.y * CONV_THREADS + threadIdx.x) * VEC;
  if (c >= channels) return;
  const int keep = taps - 1;
  // (weights and the step's integers do not depend on the kernel before this one)
  float wt[CONV_MAX_TAPS][VEC];
  for (int j = 0; j < taps; ++j) load_channels<float, VEC>(wt[j], w + static_cast<int64_t>(j) * channels + c);
  int b, q0, first, q_len;
  if (tile_request) {
    b = tile_request[blockIdx.x], q0 = tile_q0[blockIdx.x];
    first = cu_q[b], q_len = cu_q[b + 1] - first;
  } else {
    b = blockIdx.x, q0 = 0, first = b, q_len = 1;
  }
  const int slot = state_slots[b];
  float *mine = (slot >= 0 && slot < num_state_rows && keep > 0)
                    ? state + (static_cast<int64_t>(slot) * keep) * channels + c
                    : nullptr;
  float before[CONV_MAX_TAPS][VEC];   // the inputs at the `keep` positions before the step, oldest first
  if (q0 == 0) {
    for (int s = 0; s < keep; ++s) {
      if (mine) {
        load_channels<float, VEC>(before[s], mine + static_cast<int64_t>(s) * channels);
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) before[s][v] = 0.0f;
      }
    }
  }
  le::wait_for_predecessor();
  const int rows = min(tile, q_len - q0);
  const T *hx = h + static_cast<int64_t>(first) * channels + c;
  for (int r = 0; r < rows; ++r) {
    const int q = q0 + r;          // index of this token among the request's tokens in the step
    float acc[VEC];
    load_channels<T, VEC>(acc, hx + static_cast<int64_t>(q) * channels);
    for (int j = 0; j < taps; ++j) {
      const int src = q - (keep - j);
      // (src < 0 only happens in the request's first tile: a tile holds at least `keep` tokens)
      float v[VEC];
      if (src >= 0) {
        load_channels<T, VEC>(v, hx + static_cast<int64_t>(src) * channels);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = before[keep + src][e];
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wt[j][e], v[e], acc[e]);
    }
    store_channels<T, VEC>(out + (static_cast<int64_t>(first) + q) * channels + c, acc);
  }

  if (q0 == 0 && mine) {
    for (int s = 0; s < keep; ++s) {
      const int src = q_len - keep + s;
      float v[VEC];
      if (src >= 0) {
        load_channels<T, VEC>(v, hx + static_cast<int64_t>(src) * channels);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[e] = before[keep + src][e];
      }
      store_channels<float, VEC>(mine + static_cast<int64_t>(s) * channels, v);
    }
  }
}

}  // namespace

// out, h: [tokens, channels] contiguous (different buffers); w: [taps, channels] float32; state:
// [num_state_rows, taps - 1, channels] float32 (may be null when taps is 1); the tiles list `tile` tokens each.
// tile_request and tile_q0 null: every request of the step brings one token, and there are `num_tiles` of them.
LE_API int le_short_conv(void *out, const void *h, int dtype, const float *w, float *state, int num_state_rows,
                         const int32_t *state_slots, const int32_t *cu_q, const int32_t *tile_request,
                         const int32_t *tile_q0, int num_tiles, int tile, int channels, int taps, cudaStream_t stream) {
  if (num_tiles <= 0 || channels <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS) return le::invalid("le_short_conv: taps must be 1..%d, got %d", CONV_MAX_TAPS, taps);
  if (tile < taps - 1) return le::invalid("le_short_conv: tiles of %d tokens cannot hold %d earlier inputs", tile, taps - 1);
  if (out == h) return le::invalid("le_short_conv: out and h must be different buffers");
  if ((tile_request == nullptr) != (tile_q0 == nullptr)) return le::invalid("le_short_conv: both tile lists or neither");
  const int vec = dtype == LE_BF16 ? 8 : 4;
  // 16-byte accesses to the rows (vec values of the type) and to weights and state (two or one of them per access)
  const bool wide = channels % 8 == 0 && taps <= 5 &&
                    ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w) |
                      reinterpret_cast<uintptr_t>(state)) & 15) == 0;
  const int per_block = CONV_THREADS * (wide ? vec : 1);
  const dim3 grid(num_tiles, (channels + per_block - 1) / per_block);
  if (grid.y > 65535) return le::invalid("le_short_conv: too many channels for one launch");
#define LE_GO(T, V)                                                                                                  \
  return le::launch_chained(short_conv_kernel<T, V>, grid, dim3(CONV_THREADS), 0, stream, static_cast<T *>(out),     \
                            static_cast<const T *>(h), w, state, num_state_rows, state_slots, cu_q, tile_request,    \
                            tile_q0, tile, channels, taps)
  if (dtype == LE_BF16) { if (wide) LE_GO(__nv_bfloat16, 8); LE_GO(__nv_bfloat16, 1); }
  if (dtype == LE_F32) { if (wide) LE_GO(float, 4); LE_GO(float, 1); }
#undef LE_GO
  return le::invalid("le_short_conv: unknown dtype code %d", dtype);
}
