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
// step's tile lists) times slices of channels; a thread owns one channel of
// its tile.  Only a request's first tile reads the state, and the thread that
// read a channel's state is the one that writes it, after its reads, from the
// step's inputs (which this kernel only reads): no other block touches that
// state, so one launch serves every cut.  Rows that stand for no request
// (slot < 0) see zeros before them and keep nothing.
//
// Sums are 32-bit, rounded once.
#include "common.cuh"

namespace {

constexpr int CONV_THREADS = 128;
constexpr int CONV_MAX_TAPS = 17;   // a tile of 16 tokens must hold the taps - 1 inputs before the next tile

template <typename T>
__global__ void __launch_bounds__(CONV_THREADS)
short_conv_kernel(T *__restrict__ out, const T *__restrict__ h, const float *__restrict__ w, float *__restrict__ state,
                  int num_state_rows, const int32_t *__restrict__ state_slots, const int32_t *__restrict__ cu_q,
                  const int32_t *__restrict__ tile_request, const int32_t *__restrict__ tile_q0, int tile, int channels,
                  int taps) {
  le::let_successor_start();
  const int c = blockIdx.y * CONV_THREADS + threadIdx.x;
  const int b = tile_request[blockIdx.x];
  const int q0 = tile_q0[blockIdx.x];
  float wt[CONV_MAX_TAPS];
  if (c < channels)
    for (int j = 0; j < taps; ++j) wt[j] = w[static_cast<int64_t>(j) * channels + c];
  le::wait_for_predecessor();
  if (c >= channels) return;
  const int first = cu_q[b];
  const int q_len = cu_q[b + 1] - first;
  const int rows = min(tile, q_len - q0);
  const int keep = taps - 1;
  const int slot = state_slots[b];
  float *mine = (slot >= 0 && slot < num_state_rows && keep > 0)
                    ? state + (static_cast<int64_t>(slot) * keep) * channels + c
                    : nullptr;
  float before[CONV_MAX_TAPS];   // the inputs at the `keep` positions before the step, oldest first
  if (q0 == 0)
    for (int s = 0; s < keep; ++s) before[s] = mine ? mine[static_cast<int64_t>(s) * channels] : 0.0f;

  const T *hx = h + static_cast<int64_t>(first) * channels + c;
  for (int r = 0; r < rows; ++r) {
    const int q = q0 + r;          // index of this token among the request's tokens in the step
    float acc = le::to_f32(hx[static_cast<int64_t>(q) * channels]);
    for (int j = 0; j < taps; ++j) {
      const int src = q - (keep - j);
      // (src < 0 only happens in the request's first tile: a tile holds at least `keep` tokens)
      const float v = src >= 0 ? le::to_f32(hx[static_cast<int64_t>(src) * channels]) : before[keep + src];
      acc = fmaf(wt[j], v, acc);
    }
    out[(static_cast<int64_t>(first) + q) * channels + c] = le::from_f32<T>(acc);
  }

  if (q0 == 0 && mine) {
    for (int s = 0; s < keep; ++s) {
      const int src = q_len - keep + s;
      mine[static_cast<int64_t>(s) * channels] =
          src >= 0 ? le::to_f32(hx[static_cast<int64_t>(src) * channels]) : before[keep + src];
    }
  }
}

}  // namespace

// out, h: [tokens, channels] contiguous (different buffers); w: [taps, channels] float32; state:
// [num_state_rows, taps - 1, channels] float32 (may be null when taps is 1); the tiles list `tile` tokens each.
LE_API int le_short_conv(void *out, const void *h, int dtype, const float *w, float *state, int num_state_rows,
                         const int32_t *state_slots, const int32_t *cu_q, const int32_t *tile_request,
                         const int32_t *tile_q0, int num_tiles, int tile, int channels, int taps, cudaStream_t stream) {
  if (num_tiles <= 0 || channels <= 0) return 0;
  if (taps < 1 || taps > CONV_MAX_TAPS) return le::invalid("le_short_conv: taps must be 1..%d, got %d", CONV_MAX_TAPS, taps);
  if (tile < taps - 1) return le::invalid("le_short_conv: tiles of %d tokens cannot hold %d earlier inputs", tile, taps - 1);
  if (out == h) return le::invalid("le_short_conv: out and h must be different buffers");
  const dim3 grid(num_tiles, (channels + CONV_THREADS - 1) / CONV_THREADS);
  if (grid.y > 65535) return le::invalid("le_short_conv: too many channels for one launch");
  LE_DISPATCH_DTYPE(dtype, T,
                    return le::launch_chained(short_conv_kernel<T>, grid, dim3(CONV_THREADS), 0, stream,
                                              static_cast<T *>(out), static_cast<const T *>(h), w, state, num_state_rows,
                                              state_slots, cu_q, tile_request, tile_q0, tile, channels, taps));
}
