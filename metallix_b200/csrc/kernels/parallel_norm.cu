// A layer whose two sublayers read the same input: x <- x + m (a + b), then
// both sublayers' norms of the new x in one pass over the row. The two norms
// share the row's mean square (they differ in their weights only):
//
//   x += m * (a + b)                    float32, in place (a, b optional)
//   r = rsqrt(mean(x^2) + eps)
//   y1 = x r w1,   y2 = x r w2          (y2 optional)
//
// a and b are what the previous layer's mixer and feed-forward left (float32
// or bfloat16, each in its own type); the sum a + b is formed in float32
// before it is scaled. One block per row, four values a thread at a time; the
// thread's first four values stay in registers between the two passes.
#include "common.cuh"

namespace mxb {

__device__ __forceinline__ float4 pn_load4(const void* p, int code, size_t index) {
  if (code == kF32) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + index);
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p) + index);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

__device__ __forceinline__ void pn_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void pn_store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <typename TOut>
__global__ void __launch_bounds__(256)
pair_add_rmsnorm_kernel(float* __restrict__ x, const void* __restrict__ a, int a_code, const void* __restrict__ b,
                        int b_code, float m, const float* __restrict__ w1, const float* __restrict__ w2,
                        TOut* __restrict__ y1, TOut* __restrict__ y2, const int* __restrict__ rows_index, int size,
                        float eps) {
  __shared__ float scratch[33];
  chain_release();
  const size_t src = rows_index ? static_cast<size_t>(rows_index[blockIdx.x]) : static_cast<size_t>(blockIdx.x);
  const int first = threadIdx.x * 4;
  float4 held = make_float4(0.0f, 0.0f, 0.0f, 0.0f), gain1 = held, gain2 = held;
  if (first < size && w1 != nullptr) {   // the norm weights come before the wait for the kernels that produce x, a and b
    gain1 = *reinterpret_cast<const float4*>(w1 + first);
    if (w2 != nullptr) gain2 = *reinterpret_cast<const float4*>(w2 + first);
  }
  chain_wait();
  float* row = behind_wait(x) + src * size;
  a = behind_wait(a);
  b = behind_wait(b);
  float sum = 0.0f;
  for (int i = first; i < size; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(row + i);
    if (a != nullptr || b != nullptr) {
      float4 d = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (a != nullptr) d = pn_load4(a, a_code, src * size + i);
      if (b != nullptr) {
        const float4 e = pn_load4(b, b_code, src * size + i);
        d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
      }
      v.x = fmaf(m, d.x, v.x); v.y = fmaf(m, d.y, v.y); v.z = fmaf(m, d.z, v.z); v.w = fmaf(m, d.w, v.w);
      *reinterpret_cast<float4*>(row + i) = v;
    }
    if (i == first) held = v;
    sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (y1 == nullptr) return;   // the sum alone was wanted
  sum = block_sum(sum, scratch);
  const float scale = rsqrtf(sum / static_cast<float>(size) + eps);
  for (int i = first; i < size; i += blockDim.x * 4) {
    const float4 v = i == first ? held : *reinterpret_cast<const float4*>(row + i);
    const float4 g = i == first ? gain1 : *reinterpret_cast<const float4*>(w1 + i);
    pn_store4(y1 + static_cast<size_t>(blockIdx.x) * size + i,
              make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w));
    if (y2 != nullptr) {
      const float4 h = i == first ? gain2 : *reinterpret_cast<const float4*>(w2 + i);
      pn_store4(y2 + static_cast<size_t>(blockIdx.x) * size + i,
                make_float4(v.x * scale * h.x, v.y * scale * h.y, v.z * scale * h.z, v.w * scale * h.w));
    }
  }
}

// out[t, c] = in[t, c] + bias[c] with `in` float32 (a product's unrounded result) or the output's own type:
// the bias of a projection, added before the one rounding to the output's type.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
add_bias_kernel(const TIn* __restrict__ in, long long ldi, const float* __restrict__ bias, TOut* __restrict__ out,
                long long ldo, int width, long long total) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= total) return;
  const long long t = index / width;
  const int c = static_cast<int>(index - t * width);
  out[t * ldo + c] = from_float<TOut>(to_float(in[t * ldi + c]) + bias[c]);
}

// The same, eight columns a thread (width a multiple of 8, rows and bias on 16-byte boundaries).
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
add_bias_by8_kernel(const TIn* __restrict__ in, long long ldi, const float* __restrict__ bias, TOut* __restrict__ out,
                    long long ldo, int width, long long groups) {
  const long long index = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (index >= groups) return;
  const int per_row = width / 8;
  const long long t = index / per_row;
  const int c = static_cast<int>(index - t * per_row) * 8;
  const float4 lo = pn_load4(in + t * ldi + c, sizeof(TIn) == 4 ? kF32 : kBF16, 0);
  const float4 hi = pn_load4(in + t * ldi + c + 4, sizeof(TIn) == 4 ? kF32 : kBF16, 0);
  const float4 b_lo = *reinterpret_cast<const float4*>(bias + c), b_hi = *reinterpret_cast<const float4*>(bias + c + 4);
  pn_store4(out + t * ldo + c, make_float4(lo.x + b_lo.x, lo.y + b_lo.y, lo.z + b_lo.z, lo.w + b_lo.w));
  pn_store4(out + t * ldo + c + 4, make_float4(hi.x + b_hi.x, hi.y + b_hi.y, hi.z + b_hi.z, hi.w + b_hi.w));
}

}  // namespace mxb

using namespace mxb;

// x: float32 [rows_of_x, size], updated in place when a or b is given (then rows_index must be null and the
// grid covers every row). a, b: [rows, size] of their own types (kF32 / kBF16), or null. y1, y2: [rows, size] of
// y_dtype; y2 with w2 or neither; y1 null: only the sum is made. size a multiple of 4 (8 for a bfloat16 operand),
// everything 16-byte aligned.
MXB_API int mxb_pair_add_rmsnorm(float* x, const void* a, int a_dtype, const void* b, int b_dtype, float m,
                                 const float* w1, const float* w2, void* y1, void* y2, int y_dtype,
                                 const int* rows_index, int rows, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool halves = (a != nullptr && a_dtype == kBF16) || (b != nullptr && b_dtype == kBF16) || y_dtype == kBF16;
  if (size <= 0 || size % (halves ? 8 : 4) != 0 || !aligned(x) || !aligned(a) || !aligned(b) || !aligned(w1) ||
      !aligned(w2) || !aligned(y1) || !aligned(y2) || (y1 != nullptr && w1 == nullptr) ||
      ((y2 != nullptr) != (w2 != nullptr)) || (rows_index != nullptr && (a != nullptr || b != nullptr)))
    return static_cast<int>(cudaErrorInvalidValue);
  int threads = ((size / 4 + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  if (y_dtype == kF32)
    return static_cast<int>(launch_chained(pair_add_rmsnorm_kernel<float>, dim3(rows), dim3(threads), 0, stream, x, a,
                                           a_dtype, b, b_dtype, m, w1, w2, static_cast<float*>(y1),
                                           static_cast<float*>(y2), rows_index, size, eps));
  if (y_dtype == kBF16)
    return static_cast<int>(launch_chained(pair_add_rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream,
                                           x, a, a_dtype, b, b_dtype, m, w1, w2, static_cast<__nv_bfloat16*>(y1),
                                           static_cast<__nv_bfloat16*>(y2), rows_index, size, eps));
  return static_cast<int>(cudaErrorInvalidValue);
}

// in: [tokens, width] rows ldi apart, float32 or the output's type; out: [tokens, width] rows ldo apart.
MXB_API int mxb_add_bias(const void* in, long long ldi, int in_dtype, const float* bias, void* out, long long ldo,
                         int out_dtype, int tokens, int width, cudaStream_t stream) {
  const long long total = static_cast<long long>(tokens) * width;
  if (total <= 0) return 0;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (width % 8 == 0 && ldi % 8 == 0 && ldo % 8 == 0 && aligned(in) && aligned(out) && aligned(bias)) {
    const long long groups = total / 8;
    const unsigned by8 = static_cast<unsigned>((groups + 255) / 256);
#define BY8(TI, TO) add_bias_by8_kernel<TI, TO><<<by8, 256, 0, stream>>>(static_cast<const TI*>(in), ldi, bias, \
                                                                          static_cast<TO*>(out), ldo, width, groups)
    if (in_dtype == kF32 && out_dtype == kF32) BY8(float, float);
    else if (in_dtype == kF32 && out_dtype == kBF16) BY8(float, __nv_bfloat16);
    else if (in_dtype == kBF16 && out_dtype == kBF16) BY8(__nv_bfloat16, __nv_bfloat16);
    else return static_cast<int>(cudaErrorInvalidValue);
#undef BY8
    return static_cast<int>(cudaGetLastError());
  }
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
#define LAUNCH(TI, TO) add_bias_kernel<TI, TO><<<blocks, 256, 0, stream>>>(static_cast<const TI*>(in), ldi, bias, \
                                                                             static_cast<TO*>(out), ldo, width, total)
  if (in_dtype == kF32 && out_dtype == kF32) LAUNCH(float, float);
  else if (in_dtype == kF32 && out_dtype == kBF16) LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == kBF16 && out_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}
