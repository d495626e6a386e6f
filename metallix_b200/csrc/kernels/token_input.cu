// A per-layer input from the token itself, gated by the residual stream:
//
//   g = gelu_tanh(x W_gate^T) * e,   e = table[token, offset : offset + dim]
//
// with gelu_tanh(v) = 0.5 v (1 + tanh(sqrt(2 / pi) (v + 0.044715 v^3))). The two
// products around it are ordinary matrix products; here are the pieces
// between them: the residual stream taking what is still pending and leaving
// in the compute type (add_cast), and the gate with the gathered table row
// (gelu_gate_rows).
#include "common.cuh"

namespace mxb {

template <typename TDelta, typename TOut>
__global__ void add_cast_kernel(float* __restrict__ x, const TDelta* __restrict__ delta, TOut* __restrict__ out,
                                long long total) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  float v = x[index];
  if (delta != nullptr) {
    v += to_float(delta[index]);
    x[index] = v;
  }
  out[index] = from_float<TOut>(v);
}

__device__ __forceinline__ float gelu_tanh_of(float v) {
  return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

template <typename T>
__global__ void gelu_gate_rows_kernel(const T* __restrict__ gate, const T* __restrict__ table,
                                      const int* __restrict__ ids, T* __restrict__ out, long long total, int dim,
                                      int table_width, int offset, int vocab, int* status) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const long long t = index / dim;
  const int j = static_cast<int>(index - t * dim);
  const int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (j == 0) atomicOr(status, kStatusBadTokenId);
    out[index] = from_float<T>(0.0f);
    return;
  }
  const float e = to_float(table[static_cast<size_t>(id) * table_width + offset + j]);
  out[index] = from_float<T>(gelu_tanh_of(to_float(gate[index])) * e);
}

}  // namespace mxb

using namespace mxb;

// x (float32, in place) += delta (may be null); out = x in out_dtype.
MXB_API int mxb_add_cast(float* x, const void* delta, int delta_dtype, void* out, int out_dtype, long long total,
                         cudaStream_t stream) {
  if (total <= 0) return 0;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
#define LAUNCH(TD, TO)                                                                                              \
  add_cast_kernel<TD, TO><<<blocks, 256, 0, stream>>>(x, static_cast<const TD*>(delta), static_cast<TO*>(out), total)
  if (delta_dtype == kF32 && out_dtype == kF32) LAUNCH(float, float);
  else if (delta_dtype == kF32 && out_dtype == kBF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == kBF16 && out_dtype == kF32) LAUNCH(__nv_bfloat16, float);
  else if (delta_dtype == kBF16 && out_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// gate, out: [tokens, dim]; table: [vocab, table_width]; the row's values offset .. offset + dim - 1 are taken.
MXB_API int mxb_gelu_gate_rows(const void* gate, const void* table, const int* ids, void* out, int tokens, int dim,
                               int table_width, int offset, int vocab, int dtype, int* status, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * dim;
  if (total <= 0) return 0;
  if (offset < 0 || offset + dim > table_width) return static_cast<int>(cudaErrorInvalidValue);
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == kF32)
    gelu_gate_rows_kernel<float><<<blocks, 256, 0, stream>>>(
        static_cast<const float*>(gate), static_cast<const float*>(table), ids, static_cast<float*>(out), total, dim,
        table_width, offset, vocab, status);
  else if (dtype == kBF16)
    gelu_gate_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(table), ids,
        static_cast<__nv_bfloat16*>(out), total, dim, table_width, offset, vocab, status);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}
