// The selective state-space recurrence (Mamba's scan) over the packed tokens
// of a step, with the state kept per request.
//
// Per channel c and state n, with a step size d_t[c] = softplus(p_t[c] + b[c])
// that depends on the token:
//
//   S[c, n] <- exp(d_t[c] A[c, n]) S[c, n] + d_t[c] x_t[c] B_t[n]
//   y_t[c]  =  sum_n S[c, n] C_t[n] + D[c] x_t[c]
//   out_t[c] = y_t[c] * silu(z_t[c])
//
// Step sizes, decays, exponentials, the state and the sums are float32 in
// both precisions; x, B, C and z arrive in the compute type. Four lanes share
// a channel, each owning every fourth state in registers; a request row's
// tokens are walked in order, so what a position gets does not depend on how
// the sequence was cut into steps. `state` is [slots, channels, states]
// float32; a row of length 0 touches no slot.
#include "common.cuh"

namespace mxb {

constexpr int kScanLanes = 4;          // lanes that share a channel
constexpr int kScanThreads = 128;      // 32 channels a block

__device__ __forceinline__ float softplus_of(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

template <typename T, int PER, int AHEAD>
__global__ void __launch_bounds__(kScanThreads)
selective_scan_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ step, long long ld_step,
                      const float* __restrict__ step_bias, const float* __restrict__ a, const T* __restrict__ b,
                      const T* __restrict__ c, long long ldbc, const float* __restrict__ d, const T* __restrict__ z,
                      long long ldz, float* __restrict__ state, const int* __restrict__ row_start,
                      const int* __restrict__ row_length, const int* __restrict__ request_slots,
                      T* __restrict__ out, int channels, int states, int num_slots, int* status) {
  const int row = blockIdx.y;
  const int n = row_length[row];
  if (n <= 0) return;
  const int slot = request_slots[row];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  const int lane = threadIdx.x & (kScanLanes - 1);
  const int ch = blockIdx.x * (kScanThreads / kScanLanes) + (threadIdx.x / kScanLanes);
  const bool live = ch < channels;
  const int cc = live ? ch : channels - 1;      // idle lanes of the last block shadow a real channel and write nothing
  const int start = row_start[row];
  float* held = state + (static_cast<size_t>(slot) * channels + cc) * states;
  float s[PER], decay[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int k = lane + kScanLanes * j;
    s[j] = k < states ? held[k] : 0.0f;
    decay[j] = k < states ? a[static_cast<size_t>(cc) * states + k] : 0.0f;
  }
  const float bias = step_bias[cc], skip = d[cc];
  // The recurrence ties a token to the one before it only through one
  // multiply-add per state; everything else about a token (its loads, step
  // size, decays, increments, gate) does not wait for the token before. So
  // AHEAD tokens are fetched and prepared side by side, then stepped through.
  // A token past the row's end repeats the last one's loads with a decay of
  // one and an increment of zero, which leaves the state as it is. A step of
  // single tokens (a decode step) takes AHEAD = 1.
  if constexpr (AHEAD >= kScanLanes) {
    // What belongs to a token and not to a state (its step size, its input
    // times the step size, its gate) is the same for the lanes that share a
    // channel: lane l works it out for the tokens l, l + 4, ... of the batch
    // and hands it round; it also writes those tokens' outputs.
    constexpr int OWN = AHEAD / kScanLanes;
    for (int i0 = 0; i0 < n; i0 += AHEAD) {
      float own_dt[OWN], own_dx[OWN], own_x[OWN], own_gate[OWN];
      T bs[AHEAD][PER], cs[AHEAD][PER];
#pragma unroll
      for (int h = 0; h < OWN; ++h) {
        const int i = i0 + lane + kScanLanes * h;
        const size_t t = static_cast<size_t>(start + (i < n ? i : n - 1));
        own_dt[h] = step[t * ld_step + cc];
        own_x[h] = to_float(x[t * ldx + cc]);
        own_gate[h] = to_float(z[t * ldz + cc]);
      }
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const size_t t = static_cast<size_t>(start + (i0 + u < n ? i0 + u : n - 1));
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int k = lane + kScanLanes * j;
          bs[u][j] = k < states ? b[t * ldbc + k] : from_float<T>(0.0f);   // a state that is not there stays at zero
          cs[u][j] = k < states ? c[t * ldbc + k] : from_float<T>(0.0f);
        }
      }
#pragma unroll
      for (int h = 0; h < OWN; ++h) {
        own_dt[h] = softplus_of(own_dt[h] + bias);
        own_dx[h] = own_dt[h] * own_x[h];
        own_gate[h] = own_gate[h] / (1.0f + expf(-own_gate[h]));
      }
      float keep[AHEAD][PER], add[AHEAD][PER], y[AHEAD];
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const bool valid = i0 + u < n;
        const float dt = __shfl_sync(0xffffffffu, own_dt[u / kScanLanes], u % kScanLanes, kScanLanes);
        const float dx = __shfl_sync(0xffffffffu, own_dx[u / kScanLanes], u % kScanLanes, kScanLanes);
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          keep[u][j] = valid ? expf(dt * decay[j]) : 1.0f;
          add[u][j] = valid ? dx * to_float(bs[u][j]) : 0.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
          s[j] = fmaf(keep[u][j], s[j], add[u][j]);
          sum = fmaf(s[j], to_float(cs[u][j]), sum);
        }
        y[u] = sum;
      }
#pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        y[u] += __shfl_xor_sync(0xffffffffu, y[u], 1);
        y[u] += __shfl_xor_sync(0xffffffffu, y[u], 2);
        if (lane == u % kScanLanes && live && i0 + u < n)
          out[static_cast<size_t>(start + i0 + u) * channels + cc] =
              from_float<T>(fmaf(skip, own_x[u / kScanLanes], y[u]) * own_gate[u / kScanLanes]);
      }
    }
  } else {
    for (int i0 = 0; i0 < n; i0 += AHEAD) {
      float pv[AHEAD], xs[AHEAD], zs[AHEAD];
      T bs[AHEAD][PER], cs[AHEAD][PER];
  #pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const size_t t = static_cast<size_t>(start + (i0 + u < n ? i0 + u : n - 1));
        pv[u] = step[t * ld_step + cc];
        xs[u] = to_float(x[t * ldx + cc]);
        zs[u] = to_float(z[t * ldz + cc]);
  #pragma unroll
        for (int j = 0; j < PER; ++j) {
          const int k = lane + kScanLanes * j;
          bs[u][j] = k < states ? b[t * ldbc + k] : from_float<T>(0.0f);   // a state that is not there stays at zero
          cs[u][j] = k < states ? c[t * ldbc + k] : from_float<T>(0.0f);
        }
      }
      float keep[AHEAD][PER], add[AHEAD][PER], gate[AHEAD], y[AHEAD];
  #pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        const bool valid = i0 + u < n;
        const float dt = softplus_of(pv[u] + bias);
        const float dx = dt * xs[u];
  #pragma unroll
        for (int j = 0; j < PER; ++j) {
          keep[u][j] = valid ? expf(dt * decay[j]) : 1.0f;
          add[u][j] = valid ? dx * to_float(bs[u][j]) : 0.0f;
        }
        gate[u] = zs[u] / (1.0f + expf(-zs[u]));
      }
  #pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        float sum = 0.0f;
  #pragma unroll
        for (int j = 0; j < PER; ++j) {
          s[j] = fmaf(keep[u][j], s[j], add[u][j]);
          sum = fmaf(s[j], to_float(cs[u][j]), sum);
        }
        y[u] = sum;
      }
  #pragma unroll
      for (int u = 0; u < AHEAD; ++u) {
        y[u] += __shfl_xor_sync(0xffffffffu, y[u], 1);
        y[u] += __shfl_xor_sync(0xffffffffu, y[u], 2);
        if (lane == 0 && live && i0 + u < n)
          out[static_cast<size_t>(start + i0 + u) * channels + cc] = from_float<T>(fmaf(skip, xs[u], y[u]) * gate[u]);
      }
    }
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int k = lane + kScanLanes * j;
      if (k < states) held[k] = s[j];
    }
  }
}

template <typename T, int PER>
static int launch_scan(const void* x, long long ldx, const float* step, long long ld_step, const float* step_bias,
                       const float* a, const void* b, const void* c, long long ldbc, const float* d, const void* z,
                       long long ldz, float* state, const int* row_start, const int* row_length,
                       const int* request_slots, void* out, int rows, int channels, int states, int num_slots,
                       int longest, int* status, cudaStream_t stream) {
  dim3 grid(ceil_div(channels, kScanThreads / kScanLanes), rows);
  constexpr int ahead = PER <= 4 ? 8 : (PER <= 16 ? 2 : 1);
#define SCAN(AHEAD)                                                                                                  \
  selective_scan_kernel<T, PER, AHEAD><<<grid, kScanThreads, 0, stream>>>(                                          \
      static_cast<const T*>(x), ldx, step, ld_step, step_bias, a, static_cast<const T*>(b), static_cast<const T*>(c), \
      ldbc, d, static_cast<const T*>(z), ldz, state, row_start, row_length, request_slots, static_cast<T*>(out),    \
      channels, states, num_slots, status)
  if (longest == 1 || ahead == 1) SCAN(1); else SCAN(ahead);
#undef SCAN
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// x, z: [tokens, channels] (row strides ldx, ldz); step: float32 [tokens, channels] ahead of its bias and softplus;
// a: float32 [channels, states] (negative); b, c: [tokens, states] with row stride ldbc; d: [channels];
// out: [tokens, channels] contiguous. Up to 256 states. longest: the most tokens of a row (0 if not known).
MXB_API int mxb_selective_scan(const void* x, long long ldx, const float* step, long long ld_step,
                               const float* step_bias, const float* a, const void* b, const void* c, long long ldbc,
                               const float* d, const void* z, long long ldz, float* state, const int* row_start,
                               const int* row_length, const int* request_slots, void* out, int rows, int channels,
                               int states, int num_slots, int longest, int dtype, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (channels <= 0 || states <= 0 || states > 64 * kScanLanes) return static_cast<int>(cudaErrorInvalidValue);
  const int per = ceil_div(states, kScanLanes);
#define ARGS x, ldx, step, ld_step, step_bias, a, b, c, ldbc, d, z, ldz, state, row_start, row_length, request_slots, \
             out, rows, channels, states, num_slots, longest, status, stream
#define DISPATCH(T)                                    \
  if (per <= 1) return launch_scan<T, 1>(ARGS);        \
  if (per <= 2) return launch_scan<T, 2>(ARGS);        \
  if (per <= 4) return launch_scan<T, 4>(ARGS);        \
  if (per <= 8) return launch_scan<T, 8>(ARGS);        \
  if (per <= 16) return launch_scan<T, 16>(ARGS);      \
  if (per <= 32) return launch_scan<T, 32>(ARGS);      \
  return launch_scan<T, 64>(ARGS);
  if (dtype == kF32) { DISPATCH(float) }
  if (dtype == kBF16) { DISPATCH(__nv_bfloat16) }
#undef DISPATCH
#undef ARGS
  return static_cast<int>(cudaErrorInvalidValue);
}
