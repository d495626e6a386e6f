// A causal convolution over time on each channel, a few taps long, over the
// packed tokens of a step, with the inputs it still needs from earlier steps
// kept per request.
//
//   y_t[c] = bias[c] + sum_j w[j, c] * x_(t - taps + 1 + j)[c]        (zeros before the sequence's start)
//
// and then, by choice, out = x + y (the convolution as a correction of its
// own input) and / or out = silu(out). w is tap-major, [taps, channels], so
// that neighbouring channels' weights lie side by side; its last row is the
// current token's. A request row's tokens are consecutive; what lies before the first
// of them comes from `state` [slots, taps - 1, channels] (float32; entry k is
// the input taps - 1 - k tokens before the row's first), which a second
// kernel then moves on by the row's tokens; in a step of single tokens the
// thread that has just read a channel's entries moves them on itself (`fold`). A row of length 0 (a padding row
// of a captured step) reads and writes no state.
#include "common.cuh"

namespace mxb {

constexpr int kConvThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
short_conv_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w, const float* __restrict__ bias,
                  const float* state, const int* __restrict__ token_request,
                  const int* __restrict__ row_start, const int* __restrict__ row_length,
                  const int* __restrict__ request_slots, T* __restrict__ out, int tokens, int channels, int taps,
                  int num_slots, int residual, int activation, int fold, float* state_out, int* status) {
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
  float acc = bias != nullptr ? bias[c] : 0.0f;
  for (int j = 0; j < taps; ++j) {
    const int rel = i - before + j;
    const float v = rel >= 0 ? to_float(x[static_cast<size_t>(start + rel) * ldx + c])
                             : held[static_cast<size_t>(before + rel) * channels];
    acc = fmaf(w[static_cast<size_t>(j) * channels + c], v, acc);
  }
  if (residual) acc += to_float(x[static_cast<size_t>(t) * ldx + c]);
  if (activation == 1) acc = acc / (1.0f + expf(-acc));
  *dst = from_float<T>(acc);
  if (fold && n == 1) {     // the row's only token: this thread alone has read these entries
    float* moved = state_out + static_cast<size_t>(slot) * before * channels + c;
    for (int k = 0; k < before; ++k)
      moved[static_cast<size_t>(k) * channels] = k + 1 < before ? moved[static_cast<size_t>(k + 1) * channels]
                                                                : to_float(x[static_cast<size_t>(t) * ldx + c]);
  }
}

// The same for whole vectors of 16 bytes: a thread owns V neighbouring
// channels (their weights in registers, up to kConvRegisterTaps taps) and a
// run of kConvRun consecutive tokens, whose taps overlap. Needs channels and
// ldx to be multiples of V and 16-byte aligned x, w and out.
constexpr int kConvRegisterTaps = 4;

template <typename T> struct ConvVector;
template <> struct ConvVector<float> {
  static constexpr int V = 4;
  using Packed = float4;
  static __device__ __forceinline__ void unpack(const float4& q, float (&v)[4]) {
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct ConvVector<__nv_bfloat16> {
  static constexpr int V = 8;
  using Packed = uint4;
  static __device__ __forceinline__ void unpack(const uint4& q, float (&v)[8]) {
    const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(words[i] << 16);
      v[2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t words[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 pair = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      words[i] = *reinterpret_cast<uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(words[0], words[1], words[2], words[3]);
  }
};

constexpr int kConvRun = 4;     // consecutive tokens a thread of the vector kernel works through

template <typename T, int TAPS>
__global__ void __launch_bounds__(kConvThreads, 3)
short_conv_vector_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w,
                         const float* __restrict__ bias, const float* state,
                         const int* __restrict__ token_request, const int* __restrict__ row_start,
                         const int* __restrict__ row_length, const int* __restrict__ request_slots,
                         T* __restrict__ out, int tokens, int channels, int num_slots, int residual,
                         int activation, int fold, float* state_out, int* status) {
  constexpr int V = ConvVector<T>::V, MAXT = kConvRegisterTaps, WINDOW = kConvRun + MAXT - 1, taps = TAPS;
  const int c = (blockIdx.x * kConvThreads + threadIdx.x) * V;
  if (c >= channels) return;
  constexpr int before = taps - 1;
  const int first = blockIdx.y * kConvRun;
  // Tap j of token t is row t - before + j of x wherever that row is the same
  // request's. So the rows first - before ... first + kConvRun - 1 are all
  // the run needs of x; they and the weights are asked for at once, before
  // the requests are looked up, and only a request's first tokens go to the
  // state instead. window[m] is row first - (MAXT - 1) + m.
  typename ConvVector<T>::Packed window[WINDOW];     // as loaded: 16 bytes a row
#pragma unroll
  for (int m = 0; m < WINDOW; ++m) {
    const int at = first - (MAXT - 1) + m;
    if (m >= MAXT - 1 - before && at >= 0 && at < tokens)
      window[m] = *reinterpret_cast<const typename ConvVector<T>::Packed*>(x + static_cast<size_t>(at) * ldx + c);
  }
  float wr[MAXT][V], base[V];
#pragma unroll
  for (int j = 0; j < MAXT; ++j) {
    if (j < taps) {
#pragma unroll
      for (int v = 0; v < V; v += 4) {
        const float4 q = *reinterpret_cast<const float4*>(w + static_cast<size_t>(j) * channels + c + v);
        wr[j][v] = q.x; wr[j][v + 1] = q.y; wr[j][v + 2] = q.z; wr[j][v + 3] = q.w;
      }
    }
  }
#pragma unroll
  for (int v = 0; v < V; ++v) base[v] = bias != nullptr ? bias[c + v] : 0.0f;
  int row = -1, n = 0, slot = 0, start = 0;     // the request row of the token before, and what was looked up for it
#pragma unroll
  for (int r = 0; r < kConvRun; ++r) {
    const int t = first + r;
    if (t >= tokens) break;
    const int now = token_request[t];
    if (now != row) {
      row = now;
      n = row_length[row];
      slot = n > 0 ? request_slots[row] : 0;
      start = row_start[row];
    }
    T* dst = out + static_cast<size_t>(t) * channels + c;
    float acc[V];
    if (n <= 0 || slot < 0 || slot >= num_slots) {
      if (n > 0 && c == 0) atomicOr(status, kStatusBadSlot);
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = 0.0f;
      ConvVector<T>::store(dst, acc);
      continue;
    }
    const int i = t - start;
    const float* held = state + static_cast<size_t>(slot) * before * channels + c;
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = base[v];
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
      if (j < taps) {
        const int rel = i - before + j;
        float value[V];
        if (rel < 0) {
#pragma unroll
          for (int v = 0; v < V; ++v) value[v] = held[static_cast<size_t>(before + rel) * channels + v];
        } else {
          // row t - before + j = first - (MAXT - 1) + m: a constant m once the loops are unrolled
#pragma unroll
          for (int m = 0; m < WINDOW; ++m)
            if (m == r - before + j + MAXT - 1) ConvVector<T>::unpack(window[m], value);
        }
        if (fold && n == 1 && j >= 1) {    // the row's only token: entry j - 1 has been read, entry j is what it becomes
          float* moved = state_out + static_cast<size_t>(slot) * before * channels + c + static_cast<size_t>(j - 1) * channels;
#pragma unroll
          for (int v = 0; v < V; v += 4) *reinterpret_cast<float4*>(moved + v) = make_float4(value[v], value[v + 1], value[v + 2], value[v + 3]);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = fmaf(wr[j][v], value[v], acc[v]);
        if (residual && j == taps - 1) {
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] += value[v];    // the last tap's input is the token's own
        }
      }
    }
    if (activation == 1) {
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = acc[v] / (1.0f + expf(-acc[v]));
    }
    ConvVector<T>::store(dst, acc);
  }
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
                             int num_slots, int residual, int activation, int longest, int* status,
                             cudaStream_t stream) {
  constexpr int V = ConvVector<T>::V;
  const int fold = longest == 1 && taps > 1;     // single tokens: the state is moved on by the same launch
  if (taps <= kConvRegisterTaps && channels % V == 0 && ldx % V == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(w) & 15) == 0 && ceil_div(tokens, kConvRun) <= 65535 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    dim3 grid(ceil_div(channels / V, kConvThreads), ceil_div(tokens, kConvRun));
#define VECTOR(TAPS)                                                                                               \
  short_conv_vector_kernel<T, TAPS><<<grid, kConvThreads, 0, stream>>>(                                           \
      static_cast<const T*>(x), ldx, w, bias, state, token_request, row_start, row_length, request_slots,         \
      static_cast<T*>(out), tokens, channels, num_slots, residual, activation, fold, state, status)
    if (taps == 1) VECTOR(1); else if (taps == 2) VECTOR(2); else if (taps == 3) VECTOR(3); else VECTOR(4);
#undef VECTOR
  } else {
    const long long total = static_cast<long long>(tokens) * channels;
    const unsigned blocks = static_cast<unsigned>((total + kConvThreads - 1) / kConvThreads);
    short_conv_kernel<T><<<blocks, kConvThreads, 0, stream>>>(
        static_cast<const T*>(x), ldx, w, bias, state, token_request, row_start, row_length, request_slots,
        static_cast<T*>(out), tokens, channels, taps, num_slots, residual, activation, fold, state, status);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || taps <= 1 || fold) return static_cast<int>(e);
  dim3 grid(ceil_div(channels, kConvThreads), rows);
  short_conv_state_kernel<T><<<grid, kConvThreads, 0, stream>>>(static_cast<const T*>(x), ldx, state, row_start,
                                                               row_length, request_slots, channels, taps, num_slots);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// x: [tokens, channels] with row stride ldx; w: [taps, channels]; bias: [channels] or null;
// state: [num_slots, taps - 1, channels]; out: [tokens, channels] contiguous, must not overlap x.
// longest: the most tokens of a row (0 if not known; 1: a step of single tokens).
MXB_API int mxb_short_conv(const void* x, long long ldx, const float* w, const float* bias, float* state,
                           const int* token_request, const int* row_start, const int* row_length,
                           const int* request_slots, void* out, int tokens, int rows, int channels, int taps,
                           int num_slots, int residual, int activation, int longest, int dtype, int* status,
                           cudaStream_t stream) {
  if (tokens <= 0 || rows <= 0) return 0;
  if (channels <= 0 || taps < 1 || taps > 64) return static_cast<int>(cudaErrorInvalidValue);
#define ARGS x, ldx, w, bias, state, token_request, row_start, row_length, request_slots, out, tokens, rows, channels, \
             taps, num_slots, residual, activation, longest, status, stream
  if (dtype == kF32) return launch_short_conv<float>(ARGS);
  if (dtype == kBF16) return launch_short_conv<__nv_bfloat16>(ARGS);
#undef ARGS
  return static_cast<int>(cudaErrorInvalidValue);
}
