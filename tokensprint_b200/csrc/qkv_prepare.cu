// What stands between a stacked q/k/v projection and attention when the mixer has more to it than
// the fused q/k kernels know: projection biases, a rotation whose cosines and sines carry a
// magnitude, a unit RMS norm of q and k AFTER the rotation, values narrower or wider than keys;
// and, behind attention, an output gate.
//
// rope_table:   table[t, j] = magnitude * (cos, sin)(positions[t] * inv_freq[j]); the angle is
//               formed and reduced in float64 (inv_freq arrives in float64), the result is float32.
// qkv_prepare:  one warp per (token, head).  For a query head: x = proj + bias, pair (i, i + rot/2)
//               of the first `rot` entries turns by the table's angle j = i, the rest stays; with
//               `unit_norm` the head is then divided by sqrt(mean(x^2) + eps) over its d entries; with a
//               query temperature (`qt_every` > 0) a query head is multiplied by
//               1 + qt_coef * ln(floor((position + 1) / qt_every) + 1): queries grow with the logarithm of
//               the position, in steps of `qt_every` positions;
//               written to q_out [T, nq, D], entries d..D-1 zero.  For a key head the same, stored
//               at the token's cache slot in k_dst [slots, nkv, D]; the value head of the same index
//               (e entries, bias, nothing else) goes to v_dst [slots, nkv, D], entries e..D-1 zero.
//               D >= max(d, e): a kernel compiled for heads of D entries then runs heads whose keys
//               and values differ in width (zeros add nothing to a score and are never read back).
//               All arithmetic is float32; inputs and outputs are in the activation type.
// gate_rows:    y[t, h*e + i] = a[t, h, i] * sigmoid(g[t, h*e + i]) (a has rows of D >= e entries per
//               head; g null: a plain compaction), the gate in float32.
#include "common.cuh"

#define QP_WARPS 4
#define QP_MAX_DIM 512

__global__ void rope_table_kernel(const int* __restrict__ positions, const double* __restrict__ inv_freq, float magnitude, int T, int half,
                                  float2* __restrict__ out) {
  ts_pdl_prologue();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i - t * half;
  double sn, cs;
  sincos((double)positions[t] * inv_freq[j], &sn, &cs);
  out[i] = make_float2((float)(cs * (double)magnitude), (float)(sn * (double)magnitude));
}

TS_EXPORT int ts_rope_table(const int* positions, const double* inv_freq, float magnitude, int T, int half, float* out, void* stream) {
  if (T <= 0 || half <= 0) return 0;
  if (positions == nullptr || inv_freq == nullptr || out == nullptr || ((uintptr_t)out % 8)) return TS_ERR_BAD_ARGUMENT;
  const int n = T * half;
  return ts_launch(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, (cudaStream_t)stream, positions, inv_freq, magnitude, T, half,
                   reinterpret_cast<float2*>(out));
}

template <typename TA>
__global__ void __launch_bounds__(QP_WARPS * 32) qkv_prepare_kernel(
    const TA* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, const float* __restrict__ q_bias,
    const float* __restrict__ k_bias, const float* __restrict__ v_bias, const float2* __restrict__ table, int rot, int unit_norm, float eps,
    TA* __restrict__ q_out, TA* __restrict__ k_dst, TA* __restrict__ v_dst, const int* __restrict__ slot_mapping, int T, int nq, int nkv,
    int d, int e, int D, const int* __restrict__ positions, float qt_coef, int qt_every) {
  ts_pdl_prologue();
  __shared__ float buf[QP_WARPS][QP_MAX_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * QP_WARPS + warp;
  const int heads = nq + nkv;
  if (item >= (long long)T * heads) return;
  const int t = (int)(item / heads), hh = (int)(item - (long long)t * heads);
  const bool is_q = hh < nq;
  const int h = is_q ? hh : hh - nq;
  long long slot = t;
  if (!is_q && slot_mapping != nullptr) {
    slot = slot_mapping[t];
    if (slot < 0) return;  // a token whose keys are not kept
  }
  const TA* row = proj + (size_t)t * ld + (is_q ? q_off : k_off) + (size_t)h * d;
  const float* bias = is_q ? q_bias : k_bias;
  if (bias != nullptr) bias += (size_t)h * d;
  const int half = rot >> 1;
  float* x = buf[warp];
  float ss = 0.f;
  for (int j = lane; j < half; j += 32) {
    const float u = ts_to_float(row[j]) + (bias ? bias[j] : 0.f);
    const float v = ts_to_float(row[j + half]) + (bias ? bias[j + half] : 0.f);
    const float2 cs = table[(size_t)t * half + j];
    const float a = u * cs.x - v * cs.y, b = v * cs.x + u * cs.y;
    x[j] = a, x[j + half] = b;
    ss += a * a + b * b;
  }
  for (int i = rot + lane; i < d; i += 32) {
    const float u = ts_to_float(row[i]) + (bias ? bias[i] : 0.f);
    x[i] = u;
    ss += u * u;
  }
  __syncwarp();
  float mul = 1.f;
  if (unit_norm) mul = 1.f / sqrtf(ts_warp_sum(ss) / (float)d + eps);
  if (is_q && qt_every > 0) mul *= 1.f + qt_coef * logf((float)((positions[t] + 1) / qt_every) + 1.f);
  TA* dst = is_q ? q_out + ((size_t)t * nq + h) * D : k_dst + ((size_t)slot * nkv + h) * D;
  for (int i = lane; i < D; i += 32) dst[i] = ts_from_float<TA>(i < d ? x[i] * mul : 0.f);
  if (!is_q && v_dst != nullptr) {
    const TA* vrow = proj + (size_t)t * ld + v_off + (size_t)h * e;
    const float* vb = v_bias ? v_bias + (size_t)h * e : nullptr;
    TA* vd = v_dst + ((size_t)slot * nkv + h) * D;
    for (int i = lane; i < D; i += 32) vd[i] = ts_from_float<TA>(i < e ? ts_to_float(vrow[i]) + (vb ? vb[i] : 0.f) : 0.f);
  }
}

TS_EXPORT int ts_qkv_prepare(const void* proj, int act_dtype, long long ld, int q_off, int k_off, int v_off, const float* q_bias,
                             const float* k_bias, const float* v_bias, const float* table, int rot, int unit_norm, float eps, void* q_out,
                             void* k_dst, void* v_dst, const int* slot_mapping, int T, int nq, int nkv, int d, int e, int D, const int* positions,
                             float qt_coef, int qt_every, void* stream) {
  if (T <= 0) return 0;
  if (nq < 0 || nkv < 0 || nq + nkv <= 0 || d <= 0 || e <= 0 || D < d || D < e || rot < 0 || rot > d || (rot & 1) || (rot > 0 && table == nullptr) ||
      qt_every < 0 || (qt_every > 0 && positions == nullptr))
    return TS_ERR_BAD_ARGUMENT;
  if (D > QP_MAX_DIM) return TS_ERR_UNSUPPORTED_SIZE;
  const long long items = (long long)T * (nq + nkv);
  const unsigned blocks = (unsigned)((items + QP_WARPS - 1) / QP_WARPS);
  cudaStream_t s = (cudaStream_t)stream;
  const float2* tb = reinterpret_cast<const float2*>(table);
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(qkv_prepare_kernel<float>, dim3(blocks), dim3(QP_WARPS * 32), 0, s, (const float*)proj, ld, q_off, k_off, v_off, q_bias,
                     k_bias, v_bias, tb, rot, unit_norm, eps, (float*)q_out, (float*)k_dst, (float*)v_dst, slot_mapping, T, nq, nkv, d, e, D, positions, qt_coef, qt_every);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(qkv_prepare_kernel<__nv_bfloat16>, dim3(blocks), dim3(QP_WARPS * 32), 0, s, (const __nv_bfloat16*)proj, ld, q_off, k_off,
                     v_off, q_bias, k_bias, v_bias, tb, rot, unit_norm, eps, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_dst,
                     (__nv_bfloat16*)v_dst, slot_mapping, T, nq, nkv, d, e, D, positions, qt_coef, qt_every);
  return TS_ERR_BAD_ARGUMENT;
}

template <typename TA>
__global__ void gate_rows_kernel(const TA* __restrict__ a, const TA* __restrict__ g, long long ld_g, TA* __restrict__ y, long long n, int H, int e,
                                 int D) {
  ts_pdl_prologue();
  const int He = H * e;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / He;
    const int c = (int)(i - t * He), h = c / e, j = c - h * e;
    float v = ts_to_float(a[((size_t)t * H + h) * D + j]);
    if (g != nullptr) v *= 1.f / (1.f + expf(-ts_to_float(g[(size_t)t * ld_g + c])));
    y[i] = ts_from_float<TA>(v);
  }
}

TS_EXPORT int ts_gate_rows(const void* a, const void* g, long long ld_g, int act_dtype, void* y, int T, int H, int e, int D, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || e <= 0 || D < e) return TS_ERR_BAD_ARGUMENT;
  const long long n = (long long)T * H * e;
  const unsigned blocks = (unsigned)min((n + 255) / 256, (long long)148 * 16);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(gate_rows_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)a, (const float*)g, ld_g, (float*)y, n, H, e, D);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(gate_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)a, (const __nv_bfloat16*)g, ld_g,
                     (__nv_bfloat16*)y, n, H, e, D);
  return TS_ERR_BAD_ARGUMENT;
}
