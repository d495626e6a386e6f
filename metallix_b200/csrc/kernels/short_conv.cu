// A causal convolution over time on each channel, a few taps long, over the
// packed tokens of a step, with the inputs it still needs from earlier steps
// kept per request.
//
//   y_t[c] = bias[c] + sum_j w[c, j] * x_(t - taps + 1 + j)[c]        (zeros before the sequence's start)
//
// and then, by choice, out = x + y (the convolution as a correction of its
// own input) and / or out = silu(out). The last column of w is the current
// token's. A request row's tokens are consecutive; what lies before the first
// of them comes from `state` [slots, taps - 1, channels] (float32; entry k is
// the input taps - 1 - k tokens before the row's first), which a second
// kernel then moves on by the row's tokens. A row of length 0 (a padding row
// of a captured step) reads and writes no state.
#include "common.cuh"

namespace mxb {

constexpr int kConvThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
short_conv_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w, const float* __restrict__ bias,
                  const float* __restrict__ state, const int* __restrict__ token_request,
                  const int* __restrict__ row_start, const int* __restrict__ row_length,
                  const int* __restrict__ request_slots, T* __restrict__ out, int tokens, int channels, int taps,
                  int num_slots, int residual, int activation, int* status) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= static_cast<long long>(tokens) * channels) return;
  const int t = static_cast<int>(index / channels), c = static_cast<int>(index - static_cast<long long>(t) * channels);
  const int row = token_request[t];
  const int n = row_length[row];
  T* dst = out + static_cast<size_t>(t) * channels + c;
  if (n <= 0) {
    *dst = from_float<T>(0.0f);
    return;
  }
  const int start = row_start[row], i = t - start, slot = request_slots[row];
  if (slot < 0 || slot >= num_slots) {
    if (c == 0) atomicOr(status, kStatusBadSlot);
    *dst = from_float<T>(0.0f);
    return;
  }
  const int before = taps - 1;
  const float* held = state + static_cast<size_t>(slot) * before * channels + c;
  const float* wc = w + static_cast<size_t>(c) * taps;
  float acc = bias != nullptr ? bias[c] : 0.0f;
  for (int j = 0; j < taps; ++j) {
    const int rel = i - before + j;
    const float v = rel >= 0 ? to_float(x[static_cast<size_t>(start + rel) * ldx + c])
                             : held[static_cast<size_t>(before + rel) * channels];
    acc = fmaf(wc[j], v, acc);
  }
  if (residual) acc += to_float(x[static_cast<size_t>(t) * ldx + c]);
  if (activation == 1) acc = acc / (1.0f + expf(-acc));
  *dst = from_float<T>(acc);
}

// The state after the row's n tokens: entry k is the input n - (taps - 1) + k
// of the row if that is one of its tokens, else what entry k + n held. One
// thread owns a channel's entries and walks them upwards, so an entry is
// read before it is overwritten.
template <typename T>
__global__ void __launch_bounds__(kConvThreads)
short_conv_state_kernel(const T* __restrict__ x, long long ldx, float* __restrict__ state,
                        const int* __restrict__ row_start, const int* __restrict__ row_length,
                        const int* __restrict__ request_slots, int channels, int taps, int num_slots) {
  const int row = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = row_length[row];
  if (c >= channels || n <= 0) return;
  const int slot = request_slots[row];
  if (slot < 0 || slot >= num_slots) return;
  const int start = row_start[row], before = taps - 1;
  float* held = state + static_cast<size_t>(slot) * before * channels + c;
  for (int k = 0; k < before; ++k) {
    const int rel = n - before + k;
    held[static_cast<size_t>(k) * channels] =
        rel >= 0 ? to_float(x[static_cast<size_t>(start + rel) * ldx + c]) : held[static_cast<size_t>(k + n) * channels];
  }
}

template <typename T>
static int launch_short_conv(const void* x, long long ldx, const float* w, const float* bias, float* state,
                             const int* token_request, const int* row_start, const int* row_length,
                             const int* request_slots, void* out, int tokens, int rows, int channels, int taps,
                             int num_slots, int residual, int activation, int* status, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * channels;
  const unsigned blocks = static_cast<unsigned>((total + kConvThreads - 1) / kConvThreads);
  short_conv_kernel<T><<<blocks, kConvThreads, 0, stream>>>(
      static_cast<const T*>(x), ldx, w, bias, state, token_request, row_start, row_length, request_slots,
      static_cast<T*>(out), tokens, channels, taps, num_slots, residual, activation, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || taps <= 1) return static_cast<int>(e);
  dim3 grid(ceil_div(channels, kConvThreads), rows);
  short_conv_state_kernel<T><<<grid, kConvThreads, 0, stream>>>(static_cast<const T*>(x), ldx, state, row_start,
                                                               row_length, request_slots, channels, taps, num_slots);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// x: [tokens, channels] with row stride ldx; w: [channels, taps]; bias: [channels] or null;
// state: [num_slots, taps - 1, channels]; out: [tokens, channels] contiguous, must not overlap x.
MXB_API int mxb_short_conv(const void* x, long long ldx, const float* w, const float* bias, float* state,
                           const int* token_request, const int* row_start, const int* row_length,
                           const int* request_slots, void* out, int tokens, int rows, int channels, int taps,
                           int num_slots, int residual, int activation, int dtype, int* status, cudaStream_t stream) {
  if (tokens <= 0 || rows <= 0) return 0;
  if (channels <= 0 || taps < 1 || taps > 64) return static_cast<int>(cudaErrorInvalidValue);
#define ARGS x, ldx, w, bias, state, token_request, row_start, row_length, request_slots, out, tokens, rows, channels, \
             taps, num_slots, residual, activation, status, stream
  if (dtype == kF32) return launch_short_conv<float>(ARGS);
  if (dtype == kBF16) return launch_short_conv<__nv_bfloat16>(ARGS);
#undef ARGS
  return static_cast<int>(cudaErrorInvalidValue);
}
