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
// all columns share (qn, kn, g, beta). A block owns some of the columns of
// one head of one request; 4 to 16 lanes share a column, each with its share
// of the D channels in registers (4 to 16 of them: a token is a chain of
// dependent steps, so what hides its latency is many warps with little work
// each, not few with much). Tokens are taken in batches of up to eight: a
// warp prepares what the columns share for one token (unit norms, decay,
// beta and qn . kn) into shared memory, then all threads walk through the
// batch; what the batch after it needs from memory is asked for before the
// walk, so that it arrives while the walk runs. With r = g * S (the decayed
// column) the two dot products kn . r and qn . r are taken in one pass and
// o = qn . r + (qn . kn) u, which equals S'^T qn for the updated S' = r + kn u
// and leaves the update off the chain to the output.
#include "common.cuh"

namespace mxb {

constexpr int kDeltaMaxWarps = 8;     // tokens of a batch: one warp prepares each (a block of fewer warps takes fewer)

// Where channel d of a shared vector lies: every lane's quarter starts 4 floats further than a
// multiple of its length, so that the four lanes' 16-byte reads fall on different banks.
template <int DPT>
__device__ __forceinline__ int delta_slot(int d) { return d + (d / DPT) * 4; }

// LANES lanes share a value column, each with DPT of its key channels; COLS neighbouring columns a thread.
template <typename T, int DPT, int LANES, int COLS>
__global__ void __launch_bounds__(512)
delta_rule_kernel(const T* __restrict__ qkv, long long ld, int q_off, int k_off, int v_off,
                  const T* __restrict__ beta_pre, long long ldb, int b_off,
                  const float* __restrict__ step_pre, long long lds, const float* __restrict__ step_bias,
                  const float* __restrict__ rate, float* __restrict__ state, long long slot_stride, int num_slots,
                  const int* __restrict__ row_start, const int* __restrict__ row_length,
                  const int* __restrict__ request_slots, float* __restrict__ out, int heads, int groups, int dim,
                  int vdim, int* status) {
  constexpr int PITCH = LANES * (DPT + 4);
  constexpr int NL = (LANES * DPT + 31) / 32;   // channels a lane prepares for its warp's token
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
  const int warps = min(static_cast<int>(blockDim.x >> 5), kDeltaMaxWarps);   // tokens of a batch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int columns = blockDim.x / LANES * COLS;   // of a block; a thread's COLS columns are neighbours
  const int column = blockIdx.z * columns + threadIdx.x / LANES * COLS, part = threadIdx.x % LANES;
  bool live[COLS];
#pragma unroll
  for (int c = 0; c < COLS; ++c) live[c] = column + c < vdim;
  const int group = head / (heads / groups);
  const float q_scale = rsqrtf(static_cast<float>(dim));
  const float head_rate = rate[head];
  // zeros in the shared vectors' padding channels (dim .. 4 * DPT), once: they are never written again
  for (int i = threadIdx.x; i < kDeltaMaxWarps * PITCH; i += blockDim.x) {
    (&s_q[0][0])[i] = 0.0f; (&s_k[0][0])[i] = 0.0f; (&s_g[0][0])[i] = 0.0f;
  }
  float bias[NL];
#pragma unroll
  for (int i = 0; i < NL; ++i) {
    const int d = lane + 32 * i;
    bias[i] = d < dim ? step_bias[head * dim + d] : 0.0f;
  }
  // this thread's quarter of its columns of S
  float s[COLS][DPT];
  // In memory a column's channels lie side by side ([heads, vdim, dim]): a lane's share is one run of DPT values.
  float* column_state = state + static_cast<long long>(slot) * slot_stride +
                        (static_cast<long long>(head) * vdim + column) * dim + part * DPT;
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = part * DPT + i;
#pragma unroll
    for (int c = 0; c < COLS; ++c) s[c][i] = live[c] && d < dim ? column_state[static_cast<long long>(c) * dim + i] : 0.0f;
  }
  // What the next batch needs from memory, asked for a batch ahead: the raw q, k and step size of the token
  // this warp prepares, its write strength, and this thread's value of every token of the batch.
  float raw_q[NL], raw_k[NL], raw_step[NL], raw_beta = 0.0f, next_v[kDeltaMaxWarps][COLS];
  auto fetch = [&](int base) {
    const int batch = min(warps, length - base);
    if (warp < batch) {
      const long long t = first + base + warp;
      const T* q_row = qkv + t * ld + q_off + group * dim;
      const T* k_row = qkv + t * ld + k_off + group * dim;
      const float* step_row = step_pre + t * lds + head * dim;
#pragma unroll
      for (int i = 0; i < NL; ++i) {
        const int d = lane + 32 * i;
        raw_q[i] = d < dim ? to_float(q_row[d]) : 0.0f;
        raw_k[i] = d < dim ? to_float(k_row[d]) : 0.0f;
        raw_step[i] = d < dim ? step_row[d] : 0.0f;
      }
      raw_beta = to_float(beta_pre[t * ldb + b_off + head]);
    }
#pragma unroll
    for (int j = 0; j < kDeltaMaxWarps; ++j)
#pragma unroll
      for (int c = 0; c < COLS; ++c)
        next_v[j][c] = live[c] && j < batch
                           ? to_float(qkv[(static_cast<long long>(first + base + j)) * ld + v_off + head * vdim + column + c])
                           : 0.0f;
  };
  fetch(0);
  for (int base = 0; base < length; base += warps) {
    const int batch = min(warps, length - base);
    __syncthreads();   // the batch before this one has been read
    if (warp < batch) {   // unit norms, decay, write strength and qn . kn of this warp's token, from what was fetched
      float qq = 0.0f, kk = 0.0f, qk = 0.0f;
#pragma unroll
      for (int i = 0; i < NL; ++i) {
        qq = fmaf(raw_q[i], raw_q[i], qq); kk = fmaf(raw_k[i], raw_k[i], kk); qk = fmaf(raw_q[i], raw_k[i], qk);
      }
      qq = warp_sum(qq); kk = warp_sum(kk); qk = warp_sum(qk);
      const float q_unit = rsqrtf(qq + 1e-6f) * q_scale, k_unit = rsqrtf(kk + 1e-6f);
#pragma unroll
      for (int i = 0; i < NL; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) {
          const float z = raw_step[i] + bias[i];
          const float softplus = z > 20.0f ? z : log1pf(expf(z));
          const int at = delta_slot<DPT>(d);
          s_q[warp][at] = raw_q[i] * q_unit;
          s_k[warp][at] = raw_k[i] * k_unit;
          s_g[warp][at] = expf(-head_rate * softplus);
        }
      }
      if (lane == 0) {
        s_beta[warp] = sigmoid_of(raw_beta);
        s_qk[warp] = qk * q_unit * k_unit;
      }
    }
    float v[kDeltaMaxWarps][COLS];
#pragma unroll
    for (int j = 0; j < kDeltaMaxWarps; ++j)
#pragma unroll
      for (int c = 0; c < COLS; ++c) v[j][c] = next_v[j][c];
    __syncthreads();
    if (base + warps < length) fetch(base + warps);   // on its way while this batch is walked through
#pragma unroll
    for (int j = 0; j < kDeltaMaxWarps; ++j) {
      if (j >= batch) break;
      const float4* q4 = reinterpret_cast<const float4*>(&s_q[j][part * (DPT + 4)]);
      const float4* k4 = reinterpret_cast<const float4*>(&s_k[j][part * (DPT + 4)]);
      const float4* g4 = reinterpret_cast<const float4*>(&s_g[j][part * (DPT + 4)]);
      // Shared memory's read rate paces the walk: what is read once (decay, key, query) serves all of the
      // thread's columns, and the key stays in registers for the write where there is room for it.
      constexpr bool KEEP = DPT * COLS <= 32;
      float k_dot[COLS], q_dot[COLS], kept[KEEP ? DPT : 1];
#pragma unroll
      for (int c = 0; c < COLS; ++c) k_dot[c] = q_dot[c] = 0.0f;
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
        const float4 g = g4[i / 4], k = k4[i / 4], q = q4[i / 4];
        if (KEEP) { kept[i] = k.x; kept[i + 1] = k.y; kept[i + 2] = k.z; kept[i + 3] = k.w; }
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          s[c][i] *= g.x; s[c][i + 1] *= g.y; s[c][i + 2] *= g.z; s[c][i + 3] *= g.w;
          k_dot[c] = fmaf(k.x, s[c][i], k_dot[c]); k_dot[c] = fmaf(k.y, s[c][i + 1], k_dot[c]);
          k_dot[c] = fmaf(k.z, s[c][i + 2], k_dot[c]); k_dot[c] = fmaf(k.w, s[c][i + 3], k_dot[c]);
          q_dot[c] = fmaf(q.x, s[c][i], q_dot[c]); q_dot[c] = fmaf(q.y, s[c][i + 1], q_dot[c]);
          q_dot[c] = fmaf(q.z, s[c][i + 2], q_dot[c]); q_dot[c] = fmaf(q.w, s[c][i + 3], q_dot[c]);
        }
      }
      float u[COLS];
#pragma unroll
      for (int c = 0; c < COLS; ++c) {
#pragma unroll
        for (int offset = 1; offset < LANES; offset <<= 1) {   // over the lanes that share the column
          k_dot[c] += __shfl_xor_sync(0xffffffffu, k_dot[c], offset);
          q_dot[c] += __shfl_xor_sync(0xffffffffu, q_dot[c], offset);
        }
        u[c] = s_beta[j] * (v[j][c] - k_dot[c]);
      }
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {   // the write
        float4 k;
        if (KEEP) k = make_float4(kept[i], kept[i + 1], kept[i + 2], kept[i + 3]);
        else k = k4[i / 4];
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
          s[c][i] = fmaf(k.x, u[c], s[c][i]); s[c][i + 1] = fmaf(k.y, u[c], s[c][i + 1]);
          s[c][i + 2] = fmaf(k.z, u[c], s[c][i + 2]); s[c][i + 3] = fmaf(k.w, u[c], s[c][i + 3]);
        }
      }
      if (part == 0) {
#pragma unroll
        for (int c = 0; c < COLS; ++c)
          if (live[c])
            out[(static_cast<long long>(first + base + j)) * (static_cast<long long>(heads) * vdim) + head * vdim + column + c] =
                fmaf(s_qk[j], u[c], q_dot[c]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = part * DPT + i;
#pragma unroll
    for (int c = 0; c < COLS; ++c)
      if (live[c] && d < dim) column_state[static_cast<long long>(c) * dim + i] = s[c][i];
  }
}

}  // namespace mxb

using namespace mxb;

// The most key channels a head may have: sixteen lanes of sixteen registers each.
MXB_API int mxb_delta_rule_max_dim() { return 256; }

// qkv: [tokens, ld] of `dtype`, holding from the column offsets on groups * dim queries, groups * dim keys and
// heads * vdim values (after their convolution and activation). beta_pre: [tokens, ldb] of `dtype`, one
// pre-activation per head from column b_off on. step_pre: float32 [tokens, lds] with heads * dim step
// pre-activations; step_bias: float32 [heads * dim]; rate: float32 [heads] (positive). state: float32
// [num_slots, heads, vdim, dim] (S transposed: a value column's key channels side by side), rows slot_stride
// values apart, advanced in place. Row r brings row_length[r]
// tokens (0: a padding row, nothing is read or written) from packed token row_start[r] on and owns slot
// request_slots[r]. out: float32 [tokens, heads * vdim]. longest: the most tokens any row brings, 0 if unknown.
MXB_API int mxb_delta_rule(const void* qkv, long long ld, int q_off, int k_off, int v_off, const void* beta_pre,
                           long long ldb, int b_off, const float* step_pre, long long lds, const float* step_bias,
                           const float* rate, float* state, long long slot_stride, int num_slots,
                           const int* row_start, const int* row_length, const int* request_slots, float* out,
                           int rows, int heads, int groups, int dim, int vdim, int dtype, int longest, int* status,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups != 0 || dim <= 0 || dim > mxb_delta_rule_max_dim() || vdim <= 0)
    return static_cast<int>(cudaErrorInvalidValue);
  // Lanes a column and channels a lane by the key width; a block has up to 512 threads and as many columns as
  // make whole warps, but not so many that a step of few (request, head) pairs leaves SMs without a block.
  const int lanes = dim <= 32 ? 4 : (dim <= 64 ? 8 : 16);
  const int per_lane = dim <= 16 ? 4 : (dim <= 128 ? 8 : 16);
  const int step = 32 / lanes;                                   // columns of a warp
  int columns = ((vdim + step - 1) / step) * step;
  // A step of single tokens (`longest`, the most tokens of any row, if the caller knows it; 0: unknown) is one
  // chain of trips to memory per block: small blocks, several of them resident on an SM, overlap their chains.
  const int most = (longest > 0 && longest < 8 ? 128 : 512) / lanes;
  if (columns > most) columns = most;
  while (columns > 2 * step && columns >= 32 &&
         static_cast<long long>(rows) * heads * ((vdim + columns - 1) / columns) < 128)
    columns /= 2;
  columns = ((columns + step - 1) / step) * step;
  const dim3 grid(rows, heads, (vdim + columns - 1) / columns), block(columns * lanes);
#define LAUNCH(T, DPT, LANES)                                                                                       \
  delta_rule_kernel<T, DPT, LANES, 1><<<grid, block, 0, stream>>>(static_cast<const T*>(qkv), ld, q_off, k_off,      \
      v_off, static_cast<const T*>(beta_pre), ldb, b_off, step_pre, lds, step_bias, rate, state, slot_stride,       \
      num_slots, row_start, row_length, request_slots, out, heads, groups, dim, vdim, status)
#define BY_DIM(T)                                                   \
  if (lanes == 4 && per_lane == 4) LAUNCH(T, 4, 4);                 \
  else if (lanes == 4) LAUNCH(T, 8, 4);                             \
  else if (lanes == 8) LAUNCH(T, 8, 8);                             \
  else if (per_lane == 8) LAUNCH(T, 8, 16);                         \
  else LAUNCH(T, 16, 16);
  if (dtype == kF32) { BY_DIM(float) }
  else if (dtype == kBF16) { BY_DIM(__nv_bfloat16) }
  else return static_cast<int>(cudaErrorInvalidValue);
#undef BY_DIM
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}
