// What stands around the linear recurrence (gla.cu, ts_linear_scan) in mixers whose decay is one
// number per (token, head): a matrix memory with exponential gates and a selective state-space
// layer.  Everything here is float32 inside; only projections are read, and finished rows written,
// in the activation type.
//
// rows_dot_f32:      out[t, r] = x[t, :] . w[r, :] + bias[r] with float32 weights and sums: the few
//                    rows of a projection that feed gates or step sizes (a bfloat16 result would
//                    carry three digits into an exponential).  One warp per (token, row).
// mlstm_gate_scan:   per (sequence, head), from the gates' pre-activations pre[t] = (i~, f~) (+ a bias [2 heads]):
//                      log_i = cap tanh(i~ / cap),  log_f = logsigmoid(cap tanh(f~ / cap))
//                      m_t = max(log_f + m_(t-1), log_i)        m before a request's first token is 0
//                      decay_t = exp(log_f + m_(t-1) - m_t),  kscale_t = exp(log_i - m_t)
//                    m is carried in the request's state.  One warp per (sequence, head) scans 32
//                    tokens at a time: the step m -> max(m + a, b) composes associatively,
//                    (a2, b2) o (a1, b1) = (a1 + a2, max(b1 + a2, b2)), so no difference of large
//                    prefix sums is ever formed.
// mlstm_norm_gate:   per (token, head), o' = [S^T q ; n . q] from the scan (e + 1 entries):
//                      o = o'[:e] / (max(|o'[e]|, exp(-m_t)) + 1e-6);  o / sqrt(mean(o^2) + eps) * w[h, :] * sigmoid(g)
// ssm_conv:          causal convolution per channel over the last `taps` inputs (the current token's
//                    weight is the last), bias, silu; inputs before a portion's first token come from
//                    the request's state (the last taps - 1 inputs, zeros at first).  The same launch
//                    turns the step-size rows into dt = softplus(raw + dt_bias) and the decay
//                    exp(-exp(A_log) dt).
// ssm_conv_state:    the last taps - 1 inputs of every sequence go into its state (after ssm_conv).
// ssm_gate_norm:     y = (o + D_h x) * silu(z), RMS-normed in `parts` equal parts of the row, times w.
#include "common.cuh"

__device__ __forceinline__ float rg_log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float rg_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float rg_silu(float z) { return z / (1.f + expf(-z)); }

template <typename TA>
__global__ void rows_dot_f32_kernel(const TA* __restrict__ x, long long ld_x, const float* __restrict__ w, const float* __restrict__ bias,
                                    float* __restrict__ out, int T, int R, int W) {
  ts_pdl_prologue();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * R) return;
  const int t = (int)(item / R), r = (int)(item - (long long)t * R);
  const TA* xr = x + (size_t)t * ld_x;
  const float* wr = w + (size_t)r * W;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int i = lane;
  for (; i + 96 < W; i += 128) {
    acc[0] = fmaf(ts_to_float(xr[i]), wr[i], acc[0]);
    acc[1] = fmaf(ts_to_float(xr[i + 32]), wr[i + 32], acc[1]);
    acc[2] = fmaf(ts_to_float(xr[i + 64]), wr[i + 64], acc[2]);
    acc[3] = fmaf(ts_to_float(xr[i + 96]), wr[i + 96], acc[3]);
  }
  for (; i < W; i += 32) acc[0] = fmaf(ts_to_float(xr[i]), wr[i], acc[0]);
  const float sum = ts_warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
  if (lane == 0) out[(size_t)t * R + r] = sum + (bias ? bias[r] : 0.f);
}

TS_EXPORT int ts_rows_dot_f32(const void* x, int act_dtype, long long ld_x, const float* w, const float* bias, float* out, int T, int R, int W,
                              void* stream) {
  if (T <= 0 || R <= 0) return 0;
  if (W <= 0) return TS_ERR_BAD_ARGUMENT;
  const long long items = (long long)T * R;
  const unsigned blocks = (unsigned)((items + 3) / 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(rows_dot_f32_kernel<float>, dim3(blocks), dim3(128), 0, s, (const float*)x, ld_x, w, bias, out, T, R, W);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(rows_dot_f32_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, s, (const __nv_bfloat16*)x, ld_x, w, bias, out, T, R, W);
  return TS_ERR_BAD_ARGUMENT;
}

__global__ void mlstm_gate_scan_kernel(const float* __restrict__ pre, const float* __restrict__ bias, float cap, float* __restrict__ m_state, long long slot_stride,
                                       const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens, float* __restrict__ decay,
                                       float* __restrict__ kscale, float* __restrict__ m_out, int B, int H) {
  ts_pdl_prologue();
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= B * H) return;
  const int b = item / H, h = item - b * H;
  const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1];
  if (t_end <= t_begin) return;  // a lane of a fixed-size batch without a request
  float* mp = m_state + (size_t)state_slots[b] * slot_stride + h;
  float carry = *mp;
  const float inv_cap = 1.f / cap;
  for (int base = t_begin; base < t_end; base += 32) {
    const int t = base + lane;
    const bool valid = t < t_end;
    float log_i = -INFINITY, log_f = 0.f;
    if (valid) {
      log_i = cap * tanhf((pre[(size_t)t * 2 * H + h] + (bias ? bias[h] : 0.f)) * inv_cap);
      log_f = rg_log_sigmoid(cap * tanhf((pre[(size_t)t * 2 * H + H + h] + (bias ? bias[H + h] : 0.f)) * inv_cap));
    }
    float a = log_f, bb = log_i;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float a1 = __shfl_up_sync(0xffffffffu, a, off), b1 = __shfl_up_sync(0xffffffffu, bb, off);
      if (lane >= off) {
        bb = fmaxf(b1 + a, bb);  // the earlier steps first, then this lane's
        a = a1 + a;
      }
    }
    const float m = fmaxf(carry + a, bb);
    float m_prev = __shfl_up_sync(0xffffffffu, m, 1);
    if (lane == 0) m_prev = carry;
    if (valid) {
      decay[(size_t)t * H + h] = expf(log_f + m_prev - m);
      kscale[(size_t)t * H + h] = expf(log_i - m);
      m_out[(size_t)t * H + h] = m;
    }
    carry = __shfl_sync(0xffffffffu, m, 31);  // lanes beyond the last token carry its m along unchanged
  }
  if (lane == 0) *mp = carry;
}

TS_EXPORT int ts_mlstm_gate_scan(const float* pre, const float* bias, float cap, float* m_state, long long slot_stride, const int* state_slots,
                                 const int* cu_seqlens, float* decay, float* kscale, float* m_out, int B, int H, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || !(cap > 0.f)) return TS_ERR_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)(((long long)B * H + 3) / 4);
  return ts_launch(mlstm_gate_scan_kernel, dim3(blocks), dim3(128), 0, (cudaStream_t)stream, pre, bias, cap, m_state, slot_stride, state_slots,
                   cu_seqlens, decay, kscale, m_out, B, H);
}

template <typename TA>
__global__ void mlstm_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ m, const TA* __restrict__ g, long long ld_g,
                                       const float* __restrict__ w, TA* __restrict__ out, int T, int H, int e, float eps) {
  ts_pdl_prologue();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const float* row = o + ((size_t)t * H + h) * (e + 1);
  const float inv = 1.f / (fmaxf(fabsf(row[e]), expf(-m[(size_t)t * H + h])) + 1e-6f);
  float ss = 0.f;
  for (int i = lane; i < e; i += 32) {
    const float v = row[i] * inv;
    ss += v * v;
  }
  ss = ts_warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / (float)e + eps);
  const TA* grow = g + (size_t)t * ld_g + (size_t)h * e;
  const float* wrow = w + (size_t)h * e;
  TA* orow = out + ((size_t)t * H + h) * e;
  for (int i = lane; i < e; i += 32)
    orow[i] = ts_from_float<TA>(row[i] * inv * rstd * wrow[i] * (1.f / (1.f + expf(-ts_to_float(grow[i])))));
}

TS_EXPORT int ts_mlstm_norm_gate(const float* o, const float* m, const void* g, long long ld_g, int act_dtype, const float* w, void* out, int T,
                                 int H, int e, float eps, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || e <= 0) return TS_ERR_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)(((long long)T * H + 3) / 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(mlstm_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, s, o, m, (const float*)g, ld_g, w, (float*)out, T, H, e, eps);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(mlstm_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, s, o, m, (const __nv_bfloat16*)g, ld_g, w,
                     (__nv_bfloat16*)out, T, H, e, eps);
  return TS_ERR_BAD_ARGUMENT;
}

// grid (columns in blocks of 128, tokens): columns 0..C-1 are channels of the convolution, columns C..C+H-1 the heads' step sizes
template <typename TA>
__global__ void ssm_conv_kernel(const TA* __restrict__ xin, long long ld, const float* __restrict__ taps_w, const float* __restrict__ bias,
                                int K, const float* __restrict__ conv_state, long long slot_stride, const int* __restrict__ state_slots,
                                const int* __restrict__ cu_seqlens, const int* __restrict__ seq_index, float* __restrict__ out, int T, int C,
                                const float* __restrict__ dt_raw, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                float* __restrict__ dt, float* __restrict__ decay, int H) {
  ts_pdl_prologue();
  const int col = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
  if (col >= C + H) return;
  if (col >= C) {
    const int h = col - C;
    const float step = rg_softplus(dt_raw[(size_t)t * H + h] + dt_bias[h]);
    dt[(size_t)t * H + h] = step;
    decay[(size_t)t * H + h] = expf(-expf(a_log[h]) * step);
    return;
  }
  const int b = seq_index[t];
  if (b < 0) {
    out[(size_t)t * C + col] = 0.f;
    return;
  }
  const int t_begin = cu_seqlens[b];
  const float* st = conv_state + (size_t)state_slots[b] * slot_stride;  // [K-1, C]: the inputs before the portion, oldest first
  float acc = bias[col];
  for (int j = 0; j < K; ++j) {
    const int p = t - (K - 1) + j;
    const float in = p >= t_begin ? ts_to_float(xin[(size_t)p * ld + col]) : st[(size_t)(K - 1 + p - t_begin) * C + col];
    acc = fmaf(taps_w[(size_t)col * K + j], in, acc);
  }
  out[(size_t)t * C + col] = rg_silu(acc);
}

TS_EXPORT int ts_ssm_conv(const void* xin, int act_dtype, long long ld, const float* taps_w, const float* bias, int K, const float* conv_state,
                          long long slot_stride, const int* state_slots, const int* cu_seqlens, const int* seq_index, float* out, int T, int C,
                          const float* dt_raw, const float* dt_bias, const float* a_log, float* dt, float* decay, int H, void* stream) {
  if (T <= 0) return 0;
  if (C <= 0 || K < 1 || H < 0) return TS_ERR_BAD_ARGUMENT;
  if (T > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  const dim3 grid((C + H + 127) / 128, T);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(ssm_conv_kernel<float>, grid, dim3(128), 0, s, (const float*)xin, ld, taps_w, bias, K, conv_state, slot_stride, state_slots,
                     cu_seqlens, seq_index, out, T, C, dt_raw, dt_bias, a_log, dt, decay, H);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(ssm_conv_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)xin, ld, taps_w, bias, K, conv_state,
                     slot_stride, state_slots, cu_seqlens, seq_index, out, T, C, dt_raw, dt_bias, a_log, dt, decay, H);
  return TS_ERR_BAD_ARGUMENT;
}

template <typename TA>
__global__ void ssm_conv_state_kernel(const TA* __restrict__ xin, long long ld, int K, float* __restrict__ conv_state, long long slot_stride,
                                      const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens, int C) {
  ts_pdl_prologue();
  const int col = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (col >= C) return;
  const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1], n = t_end - t_begin;
  if (n <= 0) return;
  float* st = conv_state + (size_t)state_slots[b] * slot_stride;
  for (int j = 0; j < K - 1; ++j) {  // entry j becomes the input at position t_end - (K-1) + j; upwards, so that a kept entry is read before it is overwritten
    const int p = t_end - (K - 1) + j;
    st[(size_t)j * C + col] = p >= t_begin ? ts_to_float(xin[(size_t)p * ld + col]) : st[(size_t)(j + n) * C + col];
  }
}

TS_EXPORT int ts_ssm_conv_state(const void* xin, int act_dtype, long long ld, int K, float* conv_state, long long slot_stride,
                                const int* state_slots, const int* cu_seqlens, int B, int C, void* stream) {
  if (B <= 0 || K <= 1) return 0;
  if (C <= 0 || B > 65535) return TS_ERR_BAD_ARGUMENT;
  const dim3 grid((C + 127) / 128, B);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(ssm_conv_state_kernel<float>, grid, dim3(128), 0, s, (const float*)xin, ld, K, conv_state, slot_stride, state_slots,
                     cu_seqlens, C);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(ssm_conv_state_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, (const __nv_bfloat16*)xin, ld, K, conv_state, slot_stride,
                     state_slots, cu_seqlens, C);
  return TS_ERR_BAD_ARGUMENT;
}

// one CTA per (token, part)
template <typename TA>
__global__ void __launch_bounds__(256) ssm_gate_norm_kernel(const float* __restrict__ o, const float* __restrict__ x, long long ld_x,
                                                            const float* __restrict__ D, const TA* __restrict__ z, long long ld_z,
                                                            const float* __restrict__ w, TA* __restrict__ out, int H, int e, int parts,
                                                            float eps) {
  ts_pdl_prologue();
  __shared__ float red[33];
  const int t = blockIdx.x / parts, part = blockIdx.x - t * parts;
  const int inner = H * e, n = inner / parts, c0 = part * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int c = c0 + i;
    const float y = (o[(size_t)t * inner + c] + D[c / e] * x[(size_t)t * ld_x + c]) * rg_silu(ts_to_float(z[(size_t)t * ld_z + c]));
    ss += y * y;
  }
  ss = ts_block_sum(ss, red);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int c = c0 + i;
    const float y = (o[(size_t)t * inner + c] + D[c / e] * x[(size_t)t * ld_x + c]) * rg_silu(ts_to_float(z[(size_t)t * ld_z + c]));
    out[(size_t)t * inner + c] = ts_from_float<TA>(y * rstd * w[c]);
  }
}

TS_EXPORT int ts_ssm_gate_norm(const float* o, const float* x, long long ld_x, const float* D, const void* z, long long ld_z, int act_dtype,
                               const float* w, void* out, int T, int H, int e, int parts, float eps, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || e <= 0 || parts <= 0 || (H * e) % parts) return TS_ERR_BAD_ARGUMENT;
  if ((long long)T * parts > 0x7fffffffLL) return TS_ERR_UNSUPPORTED_SIZE;
  const int n = H * e / parts;
  const int threads = n >= 256 ? 256 : ((n + 31) / 32) * 32;
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(ssm_gate_norm_kernel<float>, dim3(T * parts), dim3(threads), 0, s, o, x, ld_x, D, (const float*)z, ld_z, w, (float*)out, H, e,
                     parts, eps);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(ssm_gate_norm_kernel<__nv_bfloat16>, dim3(T * parts), dim3(threads), 0, s, o, x, ld_x, D, (const __nv_bfloat16*)z, ld_z, w,
                     (__nv_bfloat16*)out, H, e, parts, eps);
  return TS_ERR_BAD_ARGUMENT;
}

// x[i] *= factor, float32 (what an architecture multiplies its logits by)
__global__ void scale_rows_kernel(float* __restrict__ x, long long n, float factor) {
  ts_pdl_prologue();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= factor;
}

TS_EXPORT int ts_scale_rows(float* x, long long n, float factor, void* stream) {
  if (n <= 0) return 0;
  const unsigned blocks = (unsigned)min((n + 255) / 256, (long long)148 * 16);
  return ts_launch(scale_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, n, factor);
}

// x[i] = cap * tanh(x[i] / cap), float32 (logits bent through a soft cap)
__global__ void softcap_rows_kernel(float* __restrict__ x, long long n, float cap, float inv_cap) {
  ts_pdl_prologue();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv_cap);
}

TS_EXPORT int ts_softcap_rows(float* x, long long n, float cap, void* stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return TS_ERR_BAD_ARGUMENT;
  const unsigned blocks = (unsigned)min((n + 255) / 256, (long long)148 * 16);
  return ts_launch(softcap_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, n, cap, 1.f / cap);
}
