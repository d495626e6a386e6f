// A feed-forward made of many small experts of which every token uses a few.
//
// Router (float32 throughout): s = softmax(z) over all R = experts + identity
// outputs (or, as a switch, s = sigmoid(z) for each output on its own; the
// outputs may also form equal groups of neighbours of which only the best few,
// by the sum of a group's two largest s + correction, can be chosen from; and
// the weights may be multiplied by a constant); the `top` outputs with the largest s + correction are chosen (ties
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
// Two ways through the experts W_down act(W_up h), act(u) = relu(u)^2, with
// W_up stacked [experts * ff, hidden] and W_down stacked [experts * hidden, ff]:
// * grouped, for steps of many tokens: expert_rows_kernel gives every
//   (token, choice) pair a row in an array sorted by expert, each expert's
//   rows padded to whole tiles of kGroupTile, and names each tile's expert;
//   gather_rows_kernel copies the tokens' inputs there; two grouped
//   tensor-core products (the first with relu^2 in its epilogue) run each
//   tile against its expert's matrices; combine_rows_kernel sums a token's
//   rows with their weights. Every pair costs one row of each product, so
//   the work is `top` experts per token however many experts there are.
// * row by row, for steps of few tokens and for float32: routed_up_kernel (a
//   warp per row of a chosen expert's W_up) and routed_down_kernel (a warp
//   per output value, over the chosen experts' W_down), so that a decode step
//   reads `top` experts' weights and not all of them.
// Both add weight_identity * h at the end (combine_rows_kernel, or inside
// routed_down_kernel).
#include "common.cuh"

namespace mxb {

constexpr int kRouteThreads = 128;   // four tokens a block, a warp each

__global__ void __launch_bounds__(kRouteThreads)
route_kernel(const float* __restrict__ logits, const float* __restrict__ correction, int* __restrict__ chosen,
             float* __restrict__ weights, float* __restrict__ dense, float* __restrict__ identity_weight,
             int tokens, int outputs, int experts, int top, int sigmoid_scores, int group_count, int group_keep,
             float weight_scale, long long ld) {
  extern __shared__ double shared[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kRouteThreads / 32) + warp;
  if (t >= tokens) return;
  double* choice = reinterpret_cast<double*>(shared) + static_cast<size_t>(warp) * outputs;   // s + correction, minus infinity once taken
  float* score = reinterpret_cast<float*>(reinterpret_cast<double*>(shared) + static_cast<size_t>(kRouteThreads / 32) * outputs) +
                 static_cast<size_t>(warp) * outputs;                                        // s
  const float* z = logits + static_cast<long long>(t) * ld;   // rows may be further apart than they are long
  if (sigmoid_scores) {   // every output's score on its own: s = 1 / (1 + e^-z)
    for (int r = lane; r < outputs; r += 32) {
      const float s = 1.0f / (1.0f + expf(-z[r]));
      score[r] = s;
      choice[r] = static_cast<double>(s) + static_cast<double>(correction[r]);
    }
  } else {
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
  }
  for (int e = lane; e < experts; e += 32) dense[static_cast<size_t>(t) * experts + e] = 0.0f;
  __syncwarp();
  if (group_count > 1 && group_keep < group_count) {
    // Outputs form group_count equal groups of neighbours; a group's score is the sum of its two largest
    // s + correction (of its only one, where a group is a single output); outside the group_keep best groups
    // (ties to the lower index) nothing can be chosen: those outputs count as minus infinity.
    double* group_score = reinterpret_cast<double*>(score + static_cast<size_t>(kRouteThreads / 32 - warp) * outputs) +
                          static_cast<size_t>(warp) * outputs;
    const int size = outputs / group_count;
    for (int g = lane; g < group_count; g += 32) {
      double best = -INFINITY, second = -INFINITY;
      for (int i = 0; i < size; ++i) {
        const double v = choice[g * size + i];
        if (v > best) { second = best; best = v; }
        else if (v > second) second = v;
      }
      group_score[g] = size > 1 ? best + second : best;
    }
    __syncwarp();
    for (int k = 0; k < group_keep; ++k) {
      double best = -INFINITY;
      int where = 0x7fffffff;
      for (int g = lane; g < group_count; g += 32) {
        const double v = group_score[g];
        if (v > best) { best = v; where = g; }
      }
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) {
        const double other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
        if (other > best || (other == best && other_where < where)) { best = other; where = other_where; }
      }
      if (where >= group_count) break;   // nothing comparable left
      if (lane == 0) group_score[where] = nan("");   // kept: no comparison picks it again
      __syncwarp();
    }
    for (int r = lane; r < outputs; r += 32)
      if (!isnan(group_score[r / size])) choice[r] = -INFINITY;
    __syncwarp();
  }
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
  const float scale = weight_scale / (picked_sum + 1e-20f);
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

// y[t, :] += identity_weight[t] * h[t, :]   (y float32)
template <typename T>
__global__ void add_identity_kernel(float* __restrict__ y, const T* __restrict__ h,
                                    const float* __restrict__ identity_weight, long long total, int hidden) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const float w = identity_weight[index / hidden];
  if (w != 0.0f) y[index] = fmaf(w, to_float(h[index]), y[index]);
}

// y[t, :] += sigmoid(gate[t * ldg]) * x[t, :]   (y float32): an expert that every token uses, behind a gate of one
// number per token
template <typename T>
__global__ void add_gated_rows_kernel(float* __restrict__ y, const T* __restrict__ x, const float* __restrict__ gate,
                                      long long ldg, long long total, int hidden) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const float g = gate[(index / hidden) * ldg];
  y[index] = fmaf(1.0f / (1.0f + expf(-g)), to_float(x[index]), y[index]);
}

constexpr int kGroupTile = 128;      // rows of a tile of the grouped products
constexpr int kGroupThreads = 1024;
constexpr int kGroupExperts = 1024;  // the most experts expert_rows_kernel counts in shared memory

// One block. position[p] = the row of pair p = (token, choice) in the array
// sorted by expert (-1 for an identity expert); tile_group[i] = the expert of
// row tile i (-1 for the tiles that stay empty). Expert e's rows start at the
// sum of the experts' before it, each rounded up to whole tiles. Which of an
// expert's rows a pair gets depends on the order the threads arrive in; the
// products treat every row alike, so the result does not.
__global__ void __launch_bounds__(kGroupThreads)
expert_rows_kernel(const int* __restrict__ chosen, int* __restrict__ position, int* __restrict__ tile_group,
                   int pairs, int experts, int tiles) {
  __shared__ int count[kGroupExperts], start[kGroupExperts], cursor[kGroupExperts];
  __shared__ int used_tiles;
  for (int e = threadIdx.x; e < experts; e += kGroupThreads) { count[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += kGroupThreads) {
    const int e = chosen[p];
    if (e >= 0 && e < experts) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tile = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = tile;
      tile += (count[e] + kGroupTile - 1) / kGroupTile;
    }
    used_tiles = tile;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += kGroupThreads) {
    const int first = start[e], last = first + (count[e] + kGroupTile - 1) / kGroupTile;
    for (int tile = first; tile < last && tile < tiles; ++tile) tile_group[tile] = e;
  }
  for (int tile = used_tiles + threadIdx.x; tile < tiles; tile += kGroupThreads) tile_group[tile] = -1;
  for (int p = threadIdx.x; p < pairs; p += kGroupThreads) {
    const int e = chosen[p];
    position[p] = e >= 0 && e < experts ? start[e] * kGroupTile + atomicAdd(&cursor[e], 1) : -1;
  }
}

// sorted[position[p], :] = h[p / top, :], 16 bytes a thread at a time (hidden * sizeof(T) a multiple of 16)
template <typename T>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ h, const int* __restrict__ position, T* __restrict__ sorted, int pairs,
                   int hidden, int top) {
  const int p = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (p >= pairs) return;
  const int row = position[p];
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(h + static_cast<size_t>(p / top) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(sorted + static_cast<size_t>(row) * hidden);
  const int vectors = hidden * static_cast<int>(sizeof(T)) / 16;
  for (int i = lane; i < vectors; i += 32) dst[i] = src[i];
}

// y[t, c] = sum_k weights[t, k] * rows[position[t, k], c] + identity_weight[t] * h[t, c]; four columns a thread
template <typename T>
__global__ void __launch_bounds__(256)
combine_rows_kernel(const float* __restrict__ rows, const int* __restrict__ position,
                    const float* __restrict__ weights, const float* __restrict__ identity_weight,
                    const T* __restrict__ h, float* __restrict__ y, int hidden, int top) {
  const int t = blockIdx.x;
  const float on_identity = identity_weight[t];
  for (int c = threadIdx.x * 4; c < hidden; c += 256 * 4) {
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int k = 0; k < top; ++k) {
      const int row = position[static_cast<size_t>(t) * top + k];
      if (row < 0) continue;
      const float w = weights[static_cast<size_t>(t) * top + k];
      const float4 v = *reinterpret_cast<const float4*>(rows + static_cast<size_t>(row) * hidden + c);
      sum[0] = fmaf(w, v.x, sum[0]); sum[1] = fmaf(w, v.y, sum[1]);
      sum[2] = fmaf(w, v.z, sum[2]); sum[3] = fmaf(w, v.w, sum[3]);
    }
    if (on_identity != 0.0f) {
#pragma unroll
      for (int i = 0; i < 4; ++i) sum[i] = fmaf(on_identity, to_float(h[static_cast<size_t>(t) * hidden + c + i]), sum[i]);
    }
    *reinterpret_cast<float4*>(y + static_cast<size_t>(t) * hidden + c) = make_float4(sum[0], sum[1], sum[2], sum[3]);
  }
}

// A lane's share of the dot product of a weight row with a vector: 16 bytes
// of the row at a time where the row starts on such a boundary and its length
// allows it, one value at a time otherwise.
template <typename T, typename U>
__device__ __forceinline__ float dot_rows(const T* __restrict__ row, const U* __restrict__ x, int length, int lane) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  float sum = 0.0f;
  if (length % V == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    float partial[4] = {0.0f, 0.0f, 0.0f, 0.0f};     // independent chains: the loads of a row are all in flight
    int lap = 0;
    for (int i = lane * V; i < length; i += 32 * V, ++lap) {
      const uint4 q = *reinterpret_cast<const uint4*>(row + i);
      const T* w = reinterpret_cast<const T*>(&q);
      float s = 0.0f;
#pragma unroll
      for (int v = 0; v < V; ++v) s = fmaf(to_float(w[v]), to_float(x[i + v]), s);
      partial[lap & 3] += s;
    }
    sum = (partial[0] + partial[1]) + (partial[2] + partial[3]);
  } else {
    for (int i = lane; i < length; i += 32) sum = fmaf(to_float(row[i]), to_float(x[i]), sum);
  }
  return sum;
}

constexpr int kRoutedThreads = 256;   // eight warps, a row of a weight each

// act[(t, k), f] = relu(W_up[e * ff + f, :] . h[t, :])^2 * weight[t, k] for e = chosen[t, k] < experts; or, `gated`,
// with an expert's matrix [2 * ff, hidden] holding gate rows and then up rows,
// silu(W_gate[f, :] . h) * (W_up[f, :] . h) * weight
template <typename T>
__global__ void __launch_bounds__(kRoutedThreads)
routed_up_kernel(const T* __restrict__ h, const T* __restrict__ w_up, const int* __restrict__ chosen,
                 const float* __restrict__ weights, float* __restrict__ act, int hidden, int experts, int ff, int top,
                 int gated) {
  const int pair = blockIdx.x;                    // token * top + k
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f = blockIdx.y * (kRoutedThreads / 32) + warp;
  const int e = chosen[pair];
  if (f >= ff || e >= experts || e < 0) return;
  const T* x = h + static_cast<size_t>(pair / top) * hidden;
  if (gated) {
    const T* gate_row = w_up + (static_cast<size_t>(e) * 2 * ff + f) * hidden;
    const float gate = warp_sum(dot_rows(gate_row, x, hidden, lane));
    const float up = warp_sum(dot_rows(gate_row + static_cast<size_t>(ff) * hidden, x, hidden, lane));
    if (lane == 0) act[static_cast<size_t>(pair) * ff + f] = gate / (1.0f + expf(-gate)) * up * weights[pair];
    return;
  }
  const T* row = w_up + (static_cast<size_t>(e) * ff + f) * hidden;
  float sum = dot_rows(row, x, hidden, lane);
  sum = warp_sum(sum);
  if (lane == 0) {
    const float u = fmaxf(sum, 0.0f);
    act[static_cast<size_t>(pair) * ff + f] = u * u * weights[pair];
  }
}

// y[t, c] = sum_k W_down[e_k * hidden + c, :] . act[(t, k), :]  +  (sum of identity weights) * h[t, c]
template <typename T>
__global__ void __launch_bounds__(kRoutedThreads)
routed_down_kernel(const float* __restrict__ act, const T* __restrict__ w_down, const T* __restrict__ h,
                   const int* __restrict__ chosen, const float* __restrict__ weights, float* __restrict__ y,
                   int hidden, int experts, int ff, int top) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.y * (kRoutedThreads / 32) + warp;
  if (c >= hidden) return;
  float sum = 0.0f, on_identity = 0.0f;
  for (int k = 0; k < top; ++k) {
    const int e = chosen[static_cast<size_t>(t) * top + k];
    if (e < 0) continue;
    if (e >= experts) {
      on_identity += weights[static_cast<size_t>(t) * top + k];
      continue;
    }
    const T* row = w_down + (static_cast<size_t>(e) * hidden + c) * ff;
    const float* a = act + (static_cast<size_t>(t) * top + k) * ff;
    sum += dot_rows(row, a, ff, lane);
  }
  sum = warp_sum(sum);
  if (lane == 0) y[static_cast<size_t>(t) * hidden + c] = fmaf(on_identity, to_float(h[static_cast<size_t>(t) * hidden + c]), sum);
}

}  // namespace mxb

using namespace mxb;

// logits: float32 [tokens, outputs]; correction: float32 [outputs]; chosen: int32 [tokens, top];
// weights: float32 [tokens, top]; dense: float32 [tokens, experts]; identity_weight: float32 [tokens].
// sigmoid_scores: s = sigmoid(z) instead of softmax(z). group_count > 1: the outputs form that many equal groups of
// neighbours, and only outputs of the group_keep best groups can be chosen. weight_scale multiplies the weights.
MXB_API int mxb_route_experts(const float* logits, const float* correction, int* chosen, float* weights, float* dense,
                              float* identity_weight, int tokens, int outputs, int experts, int top,
                              int sigmoid_scores, int group_count, int group_keep, float weight_scale,
                              long long ld, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (outputs <= 0 || experts < 0 || experts > outputs || top <= 0 || top > outputs)
    return static_cast<int>(cudaErrorInvalidValue);
  if (group_count > 1 && (outputs % group_count != 0 || group_keep < 1 || group_keep > group_count ||
                          static_cast<long long>(group_keep) * (outputs / group_count) < top))
    return static_cast<int>(cudaErrorInvalidValue);
  // per warp: s + correction (double), s (float) and, with groups, the groups' scores (double)
  const size_t shared = (sizeof(float) + (group_count > 1 ? 2 : 1) * sizeof(double)) * outputs * (kRouteThreads / 32);
  if (shared > 48 * 1024) return static_cast<int>(cudaErrorInvalidValue);
  route_kernel<<<ceil_div(tokens, kRouteThreads / 32), kRouteThreads, shared, stream>>>(
      logits, correction, chosen, weights, dense, identity_weight, tokens, outputs, experts, top, sigmoid_scores,
      group_count, group_keep, weight_scale, ld < outputs ? outputs : ld);
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

// h: [tokens, hidden]; w_up: [experts * ff, hidden] (gated: [experts * 2 * ff, hidden], every expert's gate rows
// and then its up rows, the activation silu instead of relu^2); w_down: [experts * hidden, ff]; act: float32
// scratch [tokens * top, ff]; y: float32 [tokens, hidden].
MXB_API int mxb_experts_routed(const void* h, const void* w_up, const void* w_down, const int* chosen,
                               const float* weights, float* act, float* y, int tokens, int hidden, int experts, int ff,
                               int top, int dtype, int gated, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden <= 0 || ff <= 0 || top <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const int per_block = kRoutedThreads / 32;
  dim3 up_grid(tokens * top, ceil_div(ff, per_block)), down_grid(tokens, ceil_div(hidden, per_block));
  if (dtype == kF32) {
    routed_up_kernel<float><<<up_grid, kRoutedThreads, 0, stream>>>(
        static_cast<const float*>(h), static_cast<const float*>(w_up), chosen, weights, act, hidden, experts, ff, top, gated);
    routed_down_kernel<float><<<down_grid, kRoutedThreads, 0, stream>>>(
        act, static_cast<const float*>(w_down), static_cast<const float*>(h), chosen, weights, y, hidden, experts, ff, top);
  } else if (dtype == kBF16) {
    routed_up_kernel<__nv_bfloat16><<<up_grid, kRoutedThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(w_up), chosen, weights, act, hidden,
        experts, ff, top, gated);
    routed_down_kernel<__nv_bfloat16><<<down_grid, kRoutedThreads, 0, stream>>>(
        act, static_cast<const __nv_bfloat16*>(w_down), static_cast<const __nv_bfloat16*>(h), chosen, weights, y,
        hidden, experts, ff, top);
  } else {
    return static_cast<int>(cudaErrorInvalidValue);
  }
  return static_cast<int>(cudaGetLastError());
}

// y: float32 [tokens, hidden], in place; x: [tokens, hidden]; gate: float32, one value per token, ldg apart.
MXB_API int mxb_add_gated_rows(float* y, const void* x, const float* gate, long long ldg, int tokens, int hidden,
                               int dtype, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * hidden;
  if (total <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == kF32)
    add_gated_rows_kernel<float><<<blocks, 256, 0, stream>>>(y, static_cast<const float*>(x), gate, ldg, total, hidden);
  else if (dtype == kBF16)
    add_gated_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(y, static_cast<const __nv_bfloat16*>(x), gate, ldg,
                                                                    total, hidden);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

// The rows of a tile of the grouped products, and the most experts mxb_expert_rows takes.
MXB_API int mxb_expert_rows_tile() { return kGroupTile; }
MXB_API int mxb_expert_rows_experts() { return kGroupExperts; }

// chosen: int32 [pairs]; position: int32 [pairs]; tile_group: int32 [tiles], tiles >= (pairs + experts *
// (tile - 1)) / tile rounded up, which holds every expert's rows however they fall.
MXB_API int mxb_expert_rows(const int* chosen, int* position, int* tile_group, int pairs, int experts, int tiles,
                            cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (experts < 1 || experts > kGroupExperts ||
      static_cast<long long>(tiles) * kGroupTile < static_cast<long long>(pairs) + static_cast<long long>(experts) * (kGroupTile - 1))
    return static_cast<int>(cudaErrorInvalidValue);
  expert_rows_kernel<<<1, kGroupThreads, 0, stream>>>(chosen, position, tile_group, pairs, experts, tiles);
  return static_cast<int>(cudaGetLastError());
}

// sorted[position[p], :] = h[p / top, :] for the pairs with a position; hidden * the element's size a multiple of 16.
MXB_API int mxb_expert_gather_rows(const void* h, const int* position, void* sorted, int pairs, int hidden, int top,
                                   int dtype, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  const int size = dtype == kF32 ? 4 : 2;
  if (hidden <= 0 || top <= 0 || (hidden * size) % 16 != 0 || (reinterpret_cast<uintptr_t>(h) & 15) ||
      (reinterpret_cast<uintptr_t>(sorted) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  const unsigned blocks = static_cast<unsigned>(ceil_div(pairs, 8));
  if (dtype == kF32)
    gather_rows_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(h), position,
                                                         static_cast<float*>(sorted), pairs, hidden, top);
  else if (dtype == kBF16)
    gather_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h), position,
                                                                 static_cast<__nv_bfloat16*>(sorted), pairs, hidden, top);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

// rows: float32 [sorted rows, hidden]; y: float32 [tokens, hidden]; hidden a multiple of 4.
MXB_API int mxb_expert_combine_rows(const float* rows, const int* position, const float* weights,
                                    const float* identity_weight, const void* h, float* y, int tokens, int hidden,
                                    int top, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden <= 0 || hidden % 4 != 0 || top <= 0 || (reinterpret_cast<uintptr_t>(rows) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  if (dtype == kF32)
    combine_rows_kernel<float><<<tokens, 256, 0, stream>>>(rows, position, weights, identity_weight,
                                                          static_cast<const float*>(h), y, hidden, top);
  else if (dtype == kBF16)
    combine_rows_kernel<__nv_bfloat16><<<tokens, 256, 0, stream>>>(rows, position, weights, identity_weight,
                                                                  static_cast<const __nv_bfloat16*>(h), y, hidden, top);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}
