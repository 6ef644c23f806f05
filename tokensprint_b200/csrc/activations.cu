// Element-wise activations of feed-forward layers that are not SwiGLU, evaluated in float32 with
// one rounding at the store.
//
//   gelu_tanh(z)  = z/2 * (1 + tanh(sqrt(2/pi) * (z + 0.044715 z^3)))
//   capped_glu    : a = min(gate, limit), b = clamp(up, -limit, limit), out = a * sigmoid(alpha a) * (b + 1)
//                   on a stacked product [T, 2 I] (all gates, then all ups)
//   gelu_gate_rows: x[t, j] = gelu_tanh(x[t, j]) * table[ids[t], col0 + j]: a small gate that is
//                   multiplied by a slice of the token's row in a table (a per-layer token input)
#include "common.cuh"

__device__ __forceinline__ float ts_gelu_tanh(float z) {
  const float k = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * z * (1.f + tanhf(k * (z + 0.044715f * z * z * z)));
}

template <typename TA>
__global__ void gelu_tanh_kernel(const TA* __restrict__ x, TA* __restrict__ out, size_t n) {
  ts_pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = ts_from_float<TA>(ts_gelu_tanh(ts_to_float(x[i])));
}

TS_EXPORT int ts_gelu_tanh(const void* x, void* out, int act_dtype, long long n, void* stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32) return ts_launch(gelu_tanh_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)x, (float*)out, (size_t)n);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(gelu_tanh_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, (size_t)n);
  return TS_ERR_BAD_ARGUMENT;
}

template <typename TA>
__global__ void capped_glu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int I, size_t total, float limit, float alpha) {
  ts_pdl_prologue();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / I;
  const int i = (int)(idx - t * I);
  const TA* row = gu + t * (size_t)(2 * I);
  const float a = fminf(ts_to_float(row[i]), limit);
  const float b = fminf(fmaxf(ts_to_float(row[I + i]), -limit), limit);
  out[idx] = ts_from_float<TA>(a / (1.f + expf(-alpha * a)) * (b + 1.f));
}

TS_EXPORT int ts_capped_glu(const void* gu, void* out, int act_dtype, int T, int I, float limit, float alpha, void* stream) {
  if (T <= 0) return 0;
  if (I <= 0) return TS_ERR_BAD_ARGUMENT;
  const size_t total = (size_t)T * I;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(capped_glu_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gu, (float*)out, I, total, limit, alpha);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(capped_glu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I, total, limit, alpha);
  return TS_ERR_BAD_ARGUMENT;
}

template <typename TA>
__global__ void gelu_gate_rows_kernel(TA* __restrict__ x, const TA* __restrict__ table, const int* __restrict__ ids, int D, long long ld,
                                      int col0, int V, size_t total) {
  ts_pdl_prologue();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / D;
  const int j = (int)(idx - t * D);
  const int id = ids[t];
  const float e = (id >= 0 && id < V) ? ts_to_float(table[(size_t)id * ld + col0 + j]) : __int_as_float(0x7fc00000);
  x[idx] = ts_from_float<TA>(ts_gelu_tanh(ts_to_float(x[idx])) * e);
}

TS_EXPORT int ts_gelu_gate_rows(void* x, const void* table, int act_dtype, const int* ids, int T, int D, long long ld, int col0, int V,
                                void* stream) {
  if (T <= 0 || D <= 0) return 0;
  if (col0 < 0 || col0 + D > ld || V <= 0) return TS_ERR_BAD_ARGUMENT;
  const size_t total = (size_t)T * D;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(gelu_gate_rows_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)x, (const float*)table, ids, D, ld, col0, V, total);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(gelu_gate_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (__nv_bfloat16*)x, (const __nv_bfloat16*)table, ids, D,
                     ld, col0, V, total);
  return TS_ERR_BAD_ARGUMENT;
}

// weighted_sum: out[i] = sum_j scale[j] * in_j[i] over up to four inputs of the activation type,
// summed in float32 and rounded once (branches of a layer that run side by side).
struct WeightedInputs {
  const void* in[4];
  float scale[4];
  int count;
};

template <typename TA>
__global__ void weighted_sum_kernel(WeightedInputs w, TA* __restrict__ out, size_t n) {
  ts_pdl_prologue();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (j < w.count) acc = fmaf(w.scale[j], ts_to_float(static_cast<const TA*>(w.in[j])[i]), acc);
    out[i] = ts_from_float<TA>(acc);
  }
}

TS_EXPORT int ts_weighted_sum(const void* a, const void* b, const void* c, const void* d, float sa, float sb, float sc, float sd, int count,
                              void* out, int act_dtype, long long n, void* stream) {
  if (n <= 0) return 0;
  if (count < 1 || count > 4) return TS_ERR_BAD_ARGUMENT;
  WeightedInputs w = {{a, b, c, d}, {sa, sb, sc, sd}, count};
  for (int j = 0; j < count; ++j)
    if (w.in[j] == nullptr) return TS_ERR_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)min((n + 255) / 256, (long long)148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32) return ts_launch(weighted_sum_kernel<float>, dim3(blocks), dim3(256), 0, s, w, (float*)out, (size_t)n);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(weighted_sum_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, w, (__nv_bfloat16*)out, (size_t)n);
  return TS_ERR_BAD_ARGUMENT;
}
