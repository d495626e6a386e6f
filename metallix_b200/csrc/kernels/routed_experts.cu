// A feed-forward made of many small experts of which every token uses a few.
//
// Router (float32 throughout): s = softmax(z) over all R = experts + identity
// outputs; the `top` outputs with the largest s + correction are chosen (ties
// go to the lower index); their weights are their s, divided by the sum of
// the chosen s (+ 1e-20). The sum s + correction is formed and compared in
// double precision: where the correction is the same for several outputs and
// their scores are tiny beside it, the float32 sum would round the scores
// away and leave the choice to the tie rule instead of to the scores. The
// last `identity` outputs stand for experts that return their input.
// route_kernel leaves, per token, the chosen indices and weights, a dense row
// of weights over the real experts (zeros for those not chosen) and the sum of
// the weights that fell on identity experts.
//
// Two ways through the experts W_down act(W_up h), act(u) = relu(u)^2:
// * all experts at once, for steps of many tokens: one product with the
//   stacked W_up [experts * ff, hidden], dense_act_kernel squares, and
//   multiplies column e * ff + f by the token's weight for expert e (zero for
//   most), one product with W_down [hidden, experts * ff];
// * only the chosen ones, for steps of few tokens: routed_up_kernel (a warp
//   per row of a chosen expert's W_up) and routed_down_kernel (a warp per
//   output value, over the chosen experts' column blocks of W_down), so that
//   a decode step reads `top` experts' weights and not all of them.
// Both add weight_identity * h at the end (add_identity_kernel, or inside
// routed_down_kernel).
#include "common.cuh"

namespace mxb {

constexpr int kRouteThreads = 128;   // four tokens a block, a warp each

__global__ void __launch_bounds__(kRouteThreads)
route_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ chosen,
             float* __restrict__ weights, float* __restrict__ dense, float* __restrict__ identity_weight,
             int tokens, int outputs, int experts, int top) {
  extern __shared__ double shared[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kRouteThreads / 32) + warp;
  if (t >= tokens) return;
  double* choice = reinterpret_cast<double*>(shared) + static_cast<size_t>(warp) * outputs;   // s + correction, minus infinity once taken
  float* score = reinterpret_cast<float*>(reinterpret_cast<double*>(shared) + static_cast<size_t>(kRouteThreads / 32) * outputs) +
                 static_cast<size_t>(warp) * outputs;                                        // s
  const float* z = logits + static_cast<size_t>(t) * outputs;
  float peak = -INFINITY;
  for (int r = lane; r < outputs; r += 32) peak = fmaxf(peak, z[r]);
  peak = warp_max(peak);
  float total = 0.0f;
  for (int r = lane; r < outputs; r += 32) {
    const float e = expf(z[r] - peak);
    score[r] = e;
    total += e;
  }
  total = warp_sum(total);
  for (int r = lane; r < outputs; r += 32) {
    const float s = score[r] / total;
    score[r] = s;
    choice[r] = static_cast<double>(s) + static_cast<double>(correction[r]);
  }
  for (int e = lane; e < experts; e += 32) dense[static_cast<size_t>(t) * experts + e] = 0.0f;
  __syncwarp();
  float picked_sum = 0.0f;
  for (int k = 0; k < top; ++k) {
    double best = -INFINITY;
    int where = 0x7fffffff;
    for (int r = lane; r < outputs; r += 32) {
      const double v = choice[r];
      if (v > best) { best = v; where = r; }     // ascending r: the lower index stays on a tie
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const double other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
      if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
    }
    if (where >= outputs) where = k < outputs ? k : 0;   // nothing comparable left (non-finite logits)
    if (lane == 0) {
      chosen[static_cast<size_t>(t) * top + k] = where;
      choice[where] = -INFINITY;
    }
    picked_sum += score[where];
    __syncwarp();
  }
  const float scale = 1.0f / (picked_sum + 1e-20f);
  if (lane == 0) {
    float on_identity = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int where = chosen[static_cast<size_t>(t) * top + k];
      const float w = score[where] * scale;
      weights[static_cast<size_t>(t) * top + k] = w;
      if (where < experts) dense[static_cast<size_t>(t) * experts + where] = w;
      else on_identity += w;
    }
    identity_weight[t] = on_identity;
  }
}

// act[t, e * ff + f] = relu(up[t, e * ff + f])^2 * dense[t, e]
template <typename T>
__global__ void dense_act_kernel(const T* __restrict__ up, const float* __restrict__ dense, T* __restrict__ act,
                                 long long total, int experts, int ff) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const long long width = static_cast<long long>(experts) * ff;
  const long long t = index / width;
  const int e = static_cast<int>((index - t * width) / ff);
  const float w = dense[t * experts + e];
  float u = w != 0.0f ? to_float(up[index]) : 0.0f;
  u = fmaxf(u, 0.0f);
  act[index] = from_float<T>(u * u * w);
}

// y[t, :] += identity_weight[t] * h[t, :]   (y float32)
template <typename T>
__global__ void add_identity_kernel(float* __restrict__ y, const T* __restrict__ h,
                                    const float* __restrict__ identity_weight, long long total, int hidden) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const float w = identity_weight[index / hidden];
  if (w != 0.0f) y[index] = fmaf(w, to_float(h[index]), y[index]);
}

constexpr int kRoutedThreads = 256;   // eight warps, a row of a weight each

// act[(t, k), f] = relu(W_up[e * ff + f, :] . h[t, :])^2 * weight[t, k] for e = chosen[t, k] < experts
template <typename T>
__global__ void __launch_bounds__(kRoutedThreads)
routed_up_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ chosen,
                 const float* __restrict__ weights, float* __restrict__ act, int hidden, int experts, int ff, int top) {
  const int pair = blockIdx.x;                    // token * top + k
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = blockIdx.y * (kRoutedThreads / 32) + warp;
  const int e = chosen[pair];
  if (f >= ff || e >= experts || e < 0) return;
  const T* x = h + static_cast<size_t>(pair / top) * hidden;
  const T* row = w_up + (static_cast<size_t>(e) * ff + f) * hidden;
  float sum = 0.0f;
  for (int i = lane; i < hidden; i += 32) sum = fmaf(to_float(row[i]), to_float(x[i]), sum);
  sum = warp_sum(sum);
  if (lane == 0) {
    const float u = fmaxf(sum, 0.0f);
    act[static_cast<size_t>(pair) * ff + f] = u * u * weights[pair];
  }
}

// y[t, c] = sum_k W_down[c, e_k * ff : (e_k + 1) * ff] . act[(t, k), :]  +  (sum of identity weights) * h[t, c]
template <typename T>
__global__ void __launch_bounds__(kRoutedThreads)
routed_down_kernel(const float* __restrict__ act, const T* __restrict__ w_down, const T* __restrict__ h,
                   const int* __restrict__ chosen, const float* __restrict__ weights, float* __restrict__ y,
                   int hidden, int experts, int ff, int top) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.y * (kRoutedThreads / 32) + warp;
  if (c >= hidden) return;
  const size_t width = static_cast<size_t>(experts) * ff;
  float sum = 0.0f, on_identity = 0.0f;
  for (int k = 0; k < top; ++k) {
    const int e = chosen[static_cast<size_t>(t) * top + k];
    if (e < 0) continue;
    if (e >= experts) {
      on_identity += weights[static_cast<size_t>(t) * top + k];
      continue;
    }
    const T* row = w_down + static_cast<size_t>(c) * width + static_cast<size_t>(e) * ff;
    const float* a = act + (static_cast<size_t>(t) * top + k) * ff;
    for (int i = lane; i < ff; i += 32) sum = fmaf(to_float(row[i]), a[i], sum);
  }
  sum = warp_sum(sum);
  if (lane == 0) y[static_cast<size_t>(t) * hidden + c] = fmaf(on_identity, to_float(h[static_cast<size_t>(t) * hidden + c]), sum);
}

}  // namespace mxb

using namespace mxb;

// logits: float32 [tokens, outputs]; correction: float32 [outputs]; chosen: int32 [tokens, top];
// weights: float32 [tokens, top]; dense: float32 [tokens, experts]; identity_weight: float32 [tokens].
MXB_API int mxb_route_experts(const float* logits, const float* correction, int* chosen, float* weights, float* dense,
                              float* identity_weight, int tokens, int outputs, int experts, int top,
                              cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (outputs <= 0 || experts < 0 || experts > outputs || top <= 0 || top > outputs)
    return static_cast<int>(cudaErrorInvalidValue);
  const size_t shared = (sizeof(float) + sizeof(double)) * outputs * (kRouteThreads / 32);
  if (shared > 48 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  route_kernel<<<ceil_div(tokens, kRouteThreads / 32), kRouteThreads, shared, stream>>>(
      logits, correction, chosen, weights, dense, identity_weight, tokens, outputs, experts, top);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_experts_dense_act(const void* up, const float* dense, void* act, int tokens, int experts, int ff,
                                  int dtype, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * experts * ff;
  if (total <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == kF32)
    dense_act_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(up), dense,
                                                       static_cast<float*>(act), total, experts, ff);
  else if (dtype == kBF16)
    dense_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(up), dense,
                                                               static_cast<__nv_bfloat16*>(act), total, experts, ff);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_experts_add_identity(float* y, const void* h, const float* identity_weight, int tokens, int hidden,
                                     int dtype, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * hidden;
  if (total <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == kF32)
    add_identity_kernel<float><<<blocks, 256, 0, stream>>>(y, static_cast<const float*>(h), identity_weight, total, hidden);
  else if (dtype == kBF16)
    add_identity_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(y, static_cast<const __nv_bfloat16*>(h),
                                                                  identity_weight, total, hidden);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

// h: [tokens, hidden]; w_up: [experts * ff, hidden]; w_down: [hidden, experts * ff]; act: float32 scratch
// [tokens * top, ff]; y: float32 [tokens, hidden].
MXB_API int mxb_experts_routed(const void* h, const void* w_up, const void* w_down, const int* chosen,
                               const float* weights, float* act, float* y, int tokens, int hidden, int experts, int ff,
                               int top, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden <= 0 || ff <= 0 || top <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const int per_block = kRoutedThreads / 32;
  dim3 up_grid(tokens * top, ceil_div(ff, per_block)), down_grid(tokens, ceil_div(hidden, per_block));
  if (dtype == kF32) {
    routed_up_kernel<float><<<up_grid, kRoutedThreads, 0, stream>>>(
        static_cast<const float*>(h), static_cast<const float*>(w_up), chosen, weights, act, hidden, experts, ff, top);
    routed_down_kernel<float><<<down_grid, kRoutedThreads, 0, stream>>>(
        act, static_cast<const float*>(w_down), static_cast<const float*>(h), chosen, weights, y, hidden, experts, ff, top);
  } else if (dtype == kBF16) {
    routed_up_kernel<__nv_bfloat16><<<up_grid, kRoutedThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w_up), chosen, weights, act, hidden,
        experts, ff, top);
    routed_down_kernel<__nv_bfloat16><<<down_grid, kRoutedThreads, 0, stream>>>(
        act, static_cast<const __nv_bfloat16*>(w_down), static_cast<const __nv_bfloat16*>(h), chosen, weights, y,
        hidden, experts, ff, top);
  } else {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return static_cast<int>(cudaGetLastError());
}
