// A short causal convolution over time, per channel, on the rows of a step:
//
//   c[t, ch] = sum_j w[ch, j] * x[t - (K-1) + j, ch]            (the last tap weighs the current token)
//   out[t, ch] = act(c + bias[ch])            mode CONV_PLAIN
//   out[t, ch] = x[t, ch] + c                 mode CONV_ADD_INPUT (a sublayer that reads its input plus the convolution of it)
//
// with act = silu or nothing.  Inputs before a portion's first token come from the request's state
// slot: the last K - 1 inputs of the sequence, oldest first, float32 [K-1, C]; zeros for a new
// request (the runner zeroes a slot at admission).  `ts_ssm_conv_state` (recurrent_gates.cu)
// writes a portion's last K - 1 inputs back after this kernel has run.  Sums are float32 whatever
// the element types; input and output types are free of each other (float32 rows in, bfloat16
// rows out, for instance).  A token of a padded lane (seq_index < 0) gets zeros.
#include "common.cuh"

#define CONV_ACT_NONE 0
#define CONV_ACT_SILU 1

template <typename TI, typename TO>
__global__ void causal_conv_kernel(const TI* __restrict__ xin, long long ld, const float* __restrict__ taps_w, const float* __restrict__ bias,
                                   int K, const float* __restrict__ conv_state, long long slot_stride, const int* __restrict__ state_slots,
                                   const int* __restrict__ cu_seqlens, const int* __restrict__ seq_index, TO* __restrict__ out, long long ld_out,
                                   int T, int C, int act, int add_input) {
  ts_pdl_prologue();
  const long long total = (long long)T * C;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / C), col = (int)(idx - (long long)t * C);
    const int b = seq_index[t];
    if (b < 0) {
      out[(size_t)t * ld_out + col] = ts_from_float<TO>(0.f);
      continue;
    }
    const int t_begin = cu_seqlens[b];
    const float* st = conv_state + (size_t)state_slots[b] * slot_stride;  // [K-1, C]: the inputs before the portion, oldest first
    float acc = bias ? bias[col] : 0.f;
    float cur = 0.f;
    for (int j = 0; j < K; ++j) {
      const int p = t - (K - 1) + j;
      const float in = p >= t_begin ? ts_to_float(xin[(size_t)p * ld + col]) : st[(size_t)(K - 1 + p - t_begin) * C + col];
      acc = fmaf(taps_w[(size_t)col * K + j], in, acc);
      cur = in;
    }
    if (act == CONV_ACT_SILU) acc = acc / (1.f + expf(-acc));
    if (add_input) acc += cur;
    out[(size_t)t * ld_out + col] = ts_from_float<TO>(acc);
  }
}

template <typename TI, typename TO>
static int conv_launch(const void* xin, long long ld, const float* taps_w, const float* bias, int K, const float* conv_state,
                       long long slot_stride, const int* state_slots, const int* cu_seqlens, const int* seq_index, void* out, long long ld_out,
                       int T, int C, int act, int add_input, cudaStream_t s) {
  const long long total = (long long)T * C;
  const unsigned blocks = (unsigned)min((total + 255) / 256, (long long)148 * 32);
  return ts_launch(causal_conv_kernel<TI, TO>, dim3(blocks), dim3(256), 0, s, (const TI*)xin, ld, taps_w, bias, K, conv_state, slot_stride,
                   state_slots, cu_seqlens, seq_index, (TO*)out, ld_out, T, C, act, add_input);
}

TS_EXPORT int ts_causal_conv(const void* xin, int in_dtype, long long ld, const float* taps_w, const float* bias, int K, const float* conv_state,
                             long long slot_stride, const int* state_slots, const int* cu_seqlens, const int* seq_index, void* out,
                             int out_dtype, long long ld_out, int T, int C, int act, int add_input, void* stream) {
  if (T <= 0) return 0;
  if (C <= 0 || K < 1 || (act != CONV_ACT_NONE && act != CONV_ACT_SILU) || (K > 1 && conv_state == nullptr)) return TS_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
#define CONV_CASE(TI, TO) \
  return conv_launch<TI, TO>(xin, ld, taps_w, bias, K, conv_state, slot_stride, state_slots, cu_seqlens, seq_index, out, ld_out, T, C, act, add_input, s)
  if (in_dtype == TS_DTYPE_F32 && out_dtype == TS_DTYPE_F32) CONV_CASE(float, float);
  if (in_dtype == TS_DTYPE_F32 && out_dtype == TS_DTYPE_BF16) CONV_CASE(float, __nv_bfloat16);
  if (in_dtype == TS_DTYPE_BF16 && out_dtype == TS_DTYPE_F32) CONV_CASE(__nv_bfloat16, float);
  if (in_dtype == TS_DTYPE_BF16 && out_dtype == TS_DTYPE_BF16) CONV_CASE(__nv_bfloat16, __nv_bfloat16);
#undef CONV_CASE
  return TS_ERR_BAD_ARGUMENT;
}
