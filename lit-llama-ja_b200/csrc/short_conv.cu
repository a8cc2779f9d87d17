// Short causal convolution over time, one filter per channel, with the last taps-1 inputs of every sequence kept as
// state between steps:
//
//   y[b][t][c] = (residual ? x[b][t][c] : 0) + bias[c] + sum_{j < taps} w[c][j] * x[b][t - (taps-1) + j][c]      (then silu)
//
// w's last column weighs the current token.  Inputs before the step's first token come from state[b][taps-1][C] (fp32,
// oldest first); a sequence at position 0 has no past, whatever the state holds (a slot that another request used needs
// no clearing).  The input is a column slice of a wider matrix (a projection's output), any of the activation dtypes.
#include "common.cuh"

namespace llb {

constexpr int SC_THREADS = 128;
constexpr int SC_MAX_TAPS = 8;

// grid (channel tiles, time tiles, B).  A thread owns one channel and slides a window of taps inputs over its time tile.
// fuse_state: the launch has ONE time tile and the thread also writes the new state (it has read the old one already).
template <typename TX, typename TY>
__global__ void __launch_bounds__(SC_THREADS) short_conv_kernel(const TX* __restrict__ x, int x_stride, int col0,
                                                                const float* __restrict__ w, const float* __restrict__ bias,
                                                                float* __restrict__ state, const int32_t* __restrict__ pos_ids,
                                                                TY* __restrict__ y, int y_stride, int T, int C, int taps,
                                                                int t_tile, int residual, int act_silu, int fuse_state) {
  const int c = blockIdx.x * SC_THREADS + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * t_tile, t1 = min(T, t0 + t_tile);
  const bool fresh = pos_ids[0] == 0;
  const int hist = taps - 1;
  float wr[SC_MAX_TAPS], win[SC_MAX_TAPS];
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS; ++j) wr[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
  const float bs = bias ? bias[c] : 0.f;
  const TX* xb = x + (size_t)b * T * x_stride + col0 + c;
  float* sb = state + (size_t)b * hist * C + c;
  // win[j] = input at time t - hist + j; filled for t = t0 (slot hist is loaded in the loop)
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS - 1; ++j) {
    float v = 0.f;
    if (j < hist) {
      const int s = t0 - hist + j;
      if (s >= 0) v = dt<TX>::ld(xb, (size_t)s * x_stride);
      else if (!fresh) v = sb[(size_t)(hist + s) * C];
    }
    win[j] = v;
  }
#pragma unroll 8
  for (int t = t0; t < t1; ++t) {          // unrolled: the loads of eight tokens are in flight together
    const float cur = dt<TX>::ld(xb, (size_t)t * x_stride);
    float acc = bs;
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; ++j) {
      if (j < hist) acc += wr[j] * win[j];
      else if (j == hist) acc += wr[j] * cur;
    }
    if (residual) acc += cur;
    if (act_silu) acc = acc / (1.f + expf(-acc));
    dt<TY>::st(y, ((size_t)b * T + t) * y_stride + c, acc);
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS - 1; ++j)
      if (j < hist) win[j] = (j + 1 < hist) ? win[j + 1] : cur;
  }
  if (fuse_state) {
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS - 1; ++j)
      if (j < hist) sb[(size_t)j * C] = win[j];
  }
}

// The new state after a step of T tokens: the last taps-1 inputs (old state entries where the step is shorter).  One thread
// per (sequence, channel) reads everything it needs before it writes.
template <typename TX>
__global__ void short_conv_state_kernel(const TX* __restrict__ x, int x_stride, int col0, float* __restrict__ state,
                                        const int32_t* __restrict__ pos_ids, int T, int C, int taps) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.y;
  const bool fresh = pos_ids[0] == 0;
  const int hist = taps - 1;
  const TX* xb = x + (size_t)b * T * x_stride + col0 + c;
  float* sb = state + (size_t)b * hist * C + c;
  float nv[SC_MAX_TAPS - 1];
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS - 1; ++j) {
    float v = 0.f;
    if (j < hist) {
      const int s = T - hist + j;
      if (s >= 0) v = dt<TX>::ld(xb, (size_t)s * x_stride);
      else if (!fresh) v = sb[(size_t)(hist + s) * C];
    }
    nv[j] = v;
  }
#pragma unroll
  for (int j = 0; j < SC_MAX_TAPS - 1; ++j)
    if (j < hist) sb[(size_t)j * C] = nv[j];
}

template <typename TX, typename TY>
static int short_conv_launch(const void* x, int x_stride, int col0, const float* w, const float* bias, float* state,
                             const int32_t* pos_ids, void* y, int y_stride, int B, int T, int C, int taps, int flags,
                             cudaStream_t st) {
  // time tiles: enough blocks to fill the device, at least 32 tokens each (every tile re-reads taps-1 inputs)
  const int ctiles = (C + SC_THREADS - 1) / SC_THREADS;
  int tiles = max(1, min((T + 31) / 32, (8 * sm_count() + ctiles * B - 1) / (ctiles * B)));
  const int t_tile = (T + tiles - 1) / tiles;
  tiles = (T + t_tile - 1) / t_tile;
  const int fuse = tiles == 1 && state != nullptr;
  short_conv_kernel<TX, TY><<<dim3(ctiles, tiles, B), SC_THREADS, 0, st>>>((const TX*)x, x_stride, col0, w, bias, state, pos_ids,
                                                                          (TY*)y, y_stride, T, C, taps, t_tile, flags & 1,
                                                                          (flags >> 1) & 1, fuse);
  LL_LAUNCH_OK("short_conv_kernel");
  if (!fuse && taps > 1) {
    short_conv_state_kernel<TX><<<dim3((C + 127) / 128, B), 128, 0, st>>>((const TX*)x, x_stride, col0, state, pos_ids, T, C, taps);
    LL_LAUNCH_OK("short_conv_state_kernel");
  }
  return LL_OK;
}

}  // namespace llb

using namespace llb;

extern "C" {

int ll_short_conv(const void* x, int x_dtype, int x_stride, int col0, const float* w, const float* bias, float* state,
                  const int32_t* pos_ids, void* y, int y_dtype, int y_stride, int B, int T, int C, int taps, int flags,
                  ll_stream stream) {
  LL_CHECK_ARG(x && w && state && pos_ids && y, "short_conv: null pointer");
  LL_CHECK_ARG(B >= 0 && T >= 0 && C > 0 && taps >= 1 && taps <= SC_MAX_TAPS && x_stride >= col0 + C && y_stride >= C,
               "bad short_conv arguments (taps up to %d)", SC_MAX_TAPS);
  if (B == 0 || T == 0) return LL_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define LL_SC(TX, TY) return short_conv_launch<TX, TY>(x, x_stride, col0, w, bias, state, pos_ids, y, y_stride, B, T, C, taps, flags, st)
  if (x_dtype == LL_F32 && y_dtype == LL_F32) LL_SC(float, float);
  if (x_dtype == LL_F32 && y_dtype == LL_BF16) LL_SC(float, __nv_bfloat16);
  if (x_dtype == LL_BF16 && y_dtype == LL_BF16) LL_SC(__nv_bfloat16, __nv_bfloat16);
#undef LL_SC
  set_error("short_conv: unsupported dtypes %d -> %d", x_dtype, y_dtype);
  return LL_ERR_UNSUPPORTED;
}

}  // extern "C"
