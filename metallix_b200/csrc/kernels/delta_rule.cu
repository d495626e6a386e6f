// The gated delta rule with one decay per head and key channel, state per
// request in the cache's slots, float32 throughout.
//
// Per head, with key width D and value width V, a request carries a matrix
// S [D, V]. A token brings q, k (D values each, from one of G groups that
// several heads may share), v (V values), a write strength beta and a decay
// g (D values in (0, 1)):
//
//   qn = q / sqrt(sum q^2 + 1e-6) * D^-1/2,   kn = k / sqrt(sum k^2 + 1e-6)
//   beta = sigmoid(b),   g_d = exp(-a_h * softplus(s_d + bias_d))
//   S <- g (rows) * S;  u = beta (v - S^T kn);  S <- S + kn u^T;  o = S^T qn
//
// Every value column of S goes its own way: column j needs only v_j and what
// all columns share (qn, kn, g, beta). A block owns up to 64 columns of one
// head of one request; four lanes share a column, each with a quarter of its
// D channels in registers. Tokens are taken in batches of one per warp: each
// warp prepares what the columns share for one token (unit norms, decay,
// beta and qn . kn) into shared memory, then all threads walk through the
// batch. With r = g * S (the decayed column) the two dot products kn . r and
// qn . r are taken in one pass and o = qn . r + (qn . kn) u, which equals
// S'^T qn for the updated S' = r + kn u and leaves the update off the chain
// to the output.
#include "common.cuh"

namespace mxb {

constexpr int kDeltaLanes = 4;        // lanes that share a value column
constexpr int kDeltaMaxWarps = 8;     // warps of a block = tokens of a batch

// Where channel d of a shared vector lies: every lane's quarter starts 4 floats further than a
// multiple of its length, so that the four lanes' 16-byte reads fall on different banks.
template <int DPT>
__device__ __forceinline__ int delta_slot(int d) { return d + (d / DPT) * 4; }

template <typename T, int DPT>
__global__ void __launch_bounds__(kDeltaMaxWarps * 32)
delta_rule_kernel(const T* __restrict__ qkv, long long ld, int q_off, int k_off, int v_off,
                  const float* __restrict__ beta_pre, long long ldb, int b_off,
                  const float* __restrict__ step_pre, long long lds, const float* __restrict__ step_bias,
                  const float* __restrict__ rate, float* __restrict__ state, long long slot_stride, int num_slots,
                  const int* __restrict__ row_start, const int* __restrict__ row_length,
                  const int* __restrict__ request_slots, float* __restrict__ out, int heads, int groups, int dim,
                  int vdim, int* status) {
  constexpr int PITCH = kDeltaLanes * (DPT + 4);
  __shared__ __align__(16) float s_q[kDeltaMaxWarps][PITCH], s_k[kDeltaMaxWarps][PITCH], s_g[kDeltaMaxWarps][PITCH];
  __shared__ float s_beta[kDeltaMaxWarps], s_qk[kDeltaMaxWarps];
  const int row = blockIdx.x, head = blockIdx.y;
  const int length = row_length[row];
  if (length <= 0) return;   // a padding row owns no state
  const int slot = request_slots[row];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  const int first = row_start[row];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int columns = blockDim.x / kDeltaLanes;
  const int column = blockIdx.z * columns + threadIdx.x / kDeltaLanes, part = threadIdx.x % kDeltaLanes;
  const bool live = column < vdim;
  const int group = head / (heads / groups);
  const float q_scale = rsqrtf(static_cast<float>(dim));
  const float head_rate = rate[head];
  // zeros in the shared vectors' padding channels (dim .. 4 * DPT), once: they are never written again
  for (int i = threadIdx.x; i < kDeltaMaxWarps * PITCH; i += blockDim.x) {
    (&s_q[0][0])[i] = 0.0f; (&s_k[0][0])[i] = 0.0f; (&s_g[0][0])[i] = 0.0f;
  }
  // this thread's quarter of its column of S
  float s[DPT];
  float* column_state = state + static_cast<long long>(slot) * slot_stride +
                        (static_cast<long long>(head) * dim) * vdim + column;
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = part * DPT + i;
    s[i] = live && d < dim ? column_state[static_cast<long long>(d) * vdim] : 0.0f;
  }
  for (int base = 0; base < length; base += warps) {
    const int batch = min(warps, length - base);
    __syncthreads();   // the batch before this one has been read
    if (warp < batch) {
      const long long t = first + base + warp;
      const T* q_row = qkv + t * ld + q_off + group * dim;
      const T* k_row = qkv + t * ld + k_off + group * dim;
      const float* step_row = step_pre + t * lds + head * dim;
      float qq = 0.0f, kk = 0.0f, qk = 0.0f;
      for (int d = lane; d < dim; d += 32) {
        const float qv = to_float(q_row[d]), kv = to_float(k_row[d]);
        qq = fmaf(qv, qv, qq); kk = fmaf(kv, kv, kk); qk = fmaf(qv, kv, qk);
      }
      qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
      const float q_unit = rsqrtf(qq + 1e-6f) * q_scale, k_unit = rsqrtf(kk + 1e-6f);
      for (int d = lane; d < dim; d += 32) {
        const float z = step_row[d] + step_bias[head * dim + d];
        const float softplus = z > 20.0f ? z : log1pf(expf(z));
        const int at = delta_slot<DPT>(d);
        s_q[warp][at] = to_float(q_row[d]) * q_unit;
        s_k[warp][at] = to_float(k_row[d]) * k_unit;
        s_g[warp][at] = expf(-head_rate * softplus);
      }
      if (lane == 0) {
        s_beta[warp] = sigmoid_of(beta_pre[t * ldb + b_off + head]);
        s_qk[warp] = qk * q_unit * k_unit;
      }
    }
    float v[kDeltaMaxWarps];
#pragma unroll
    for (int j = 0; j < kDeltaMaxWarps; ++j)
      v[j] = live && j < batch ? to_float(qkv[(static_cast<long long>(first + base + j)) * ld + v_off + head * vdim + column])
                               : 0.0f;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kDeltaMaxWarps; ++j) {
      if (j >= batch) break;
      const float4* q4 = reinterpret_cast<const float4*>(&s_q[j][part * (DPT + 4)]);
      const float4* k4 = reinterpret_cast<const float4*>(&s_k[j][part * (DPT + 4)]);
      const float4* g4 = reinterpret_cast<const float4*>(&s_g[j][part * (DPT + 4)]);
      float k_dot = 0.0f, q_dot = 0.0f;
      float kept[DPT];
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
        const float4 g = g4[i / 4], k = k4[i / 4], q = q4[i / 4];
        s[i] *= g.x; s[i + 1] *= g.y; s[i + 2] *= g.z; s[i + 3] *= g.w;
        k_dot = fmaf(k.x, s[i], k_dot); k_dot = fmaf(k.y, s[i + 1], k_dot);
        k_dot = fmaf(k.z, s[i + 2], k_dot); k_dot = fmaf(k.w, s[i + 3], k_dot);
        q_dot = fmaf(q.x, s[i], q_dot); q_dot = fmaf(q.y, s[i + 1], q_dot);
        q_dot = fmaf(q.z, s[i + 2], q_dot); q_dot = fmaf(q.w, s[i + 3], q_dot);
        kept[i] = k.x; kept[i + 1] = k.y; kept[i + 2] = k.z; kept[i + 3] = k.w;
      }
      k_dot += __shfl_xor_sync(0xffffffffu, k_dot, 1); q_dot += __shfl_xor_sync(0xffffffffu, q_dot, 1);
      k_dot += __shfl_xor_sync(0xffffffffu, k_dot, 2); q_dot += __shfl_xor_sync(0xffffffffu, q_dot, 2);
      const float u = s_beta[j] * (v[j] - k_dot);
#pragma unroll
      for (int i = 0; i < DPT; ++i) s[i] = fmaf(kept[i], u, s[i]);
      if (live && part == 0)
        out[(static_cast<long long>(first + base + j)) * (static_cast<long long>(heads) * vdim) + head * vdim + column] =
            fmaf(s_qk[j], u, q_dot);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = part * DPT + i;
      if (d < dim) column_state[static_cast<long long>(d) * vdim] = s[i];
    }
  }
}

}  // namespace mxb

using namespace mxb;

// The most key channels a head may have: four lanes of 64 registers each.
MXB_API int mxb_delta_rule_max_dim() { return kDeltaLanes * 64; }

// qkv: [tokens, ld] of `dtype`, holding from the column offsets on groups * dim queries, groups * dim keys and
// heads * vdim values (after their convolution and activation). beta_pre: float32 [tokens, ldb], one
// pre-activation per head from column b_off on. step_pre: float32 [tokens, lds] with heads * dim step
// pre-activations; step_bias: float32 [heads * dim]; rate: float32 [heads] (positive). state: float32
// [num_slots, heads, dim, vdim], rows slot_stride values apart, advanced in place. Row r brings row_length[r]
// tokens (0: a padding row, nothing is read or written) from packed token row_start[r] on and owns slot
// request_slots[r]. out: float32 [tokens, heads * vdim].
MXB_API int mxb_delta_rule(const void* qkv, long long ld, int q_off, int k_off, int v_off, const float* beta_pre,
                           long long ldb, int b_off, const float* step_pre, long long lds, const float* step_bias,
                           const float* rate, float* state, long long slot_stride, int num_slots,
                           const int* row_start, const int* row_length, const int* request_slots, float* out,
                           int rows, int heads, int groups, int dim, int vdim, int dtype, int* status,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups != 0 || dim <= 0 || dim > mxb_delta_rule_max_dim() || vdim <= 0)
    return static_cast<int>(cudaErrorInvalidValue);
  // as many columns a block as the head has, in whole warps (8 columns), up to 64
  int columns = ((vdim + 7) / 8) * 8;
  if (columns > 64) columns = 64;
  const dim3 grid(rows, heads, (vdim + columns - 1) / columns), block(columns * kDeltaLanes);
  const int per_lane = (dim + kDeltaLanes - 1) / kDeltaLanes;
#define LAUNCH(T, DPT)                                                                                            \
  delta_rule_kernel<T, DPT><<<grid, block, 0, stream>>>(static_cast<const T*>(qkv), ld, q_off, k_off, v_off,      \
      beta_pre, ldb, b_off, step_pre, lds, step_bias, rate, state, slot_stride, num_slots, row_start, row_length, \
      request_slots, out, heads, groups, dim, vdim, status)
#define BY_DIM(T)                                  \
  if (per_lane <= 8) LAUNCH(T, 8);                 \
  else if (per_lane <= 16) LAUNCH(T, 16);          \
  else if (per_lane <= 32) LAUNCH(T, 32);          \
  else LAUNCH(T, 64);
  if (dtype == kF32) { BY_DIM(float) }
  else if (dtype == kBF16) { BY_DIM(__nv_bfloat16) }
  else return static_cast<int>(cudaErrorInvalidValue);
#undef BY_DIM
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}
