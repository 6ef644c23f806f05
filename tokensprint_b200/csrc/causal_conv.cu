// A short causal convolution over time, per channel, on the rows of a step:
//
//   c[t, ch] = sum_j w[ch, j] * x[t - (K-1) + j, ch]            (the last tap weighs the current token)
//   out[t, ch] = act(c + bias[ch])            mode CONV_PLAIN
//   out[t, ch] = x[t, ch] + c                 mode CONV_ADD_INPUT (a sublayer that reads its input plus the convolution of it)
//
// with act = silu or nothing.  The weights come tap by tap, [K, C] (what a checkpoint stores as [C, K] is
// transposed once when it is loaded): the threads of a warp then read one tap's weights of neighbouring
// channels from one line (channel by channel, every lane met a line of its own at every load, and the
// load pipe, not the memory, set the kernel's time: 147 us for 2,048 x 4,096 entries).  Inputs before a portion's first token come from the request's state
// slot: the last K - 1 inputs of the sequence, oldest first, float32 [K-1, C]; zeros for a new
// request (the runner zeroes a slot at admission).  The same launch brings the slot up to date: the
// thread of a portion's first token also works out the portion's next K - 2 tokens (the only ones that
// read the slot; their own threads leave at once) and then writes the portion's last K - 1 inputs
// there, oldest first and upwards, so that an entry that a short portion keeps is read before it is
// overwritten: nobody else touches that sequence's entries of these channels.  Sums are float32 whatever
// the element types; input and output types are free of each other (float32 rows in, bfloat16
// rows out, for instance).  A token of a padded lane (seq_index < 0) gets zeros.
#include "common.cuh"

#define CONV_ACT_NONE 0
#define CONV_ACT_SILU 1

template <typename TI, typename TO>
__global__ void causal_conv_kernel(const TI* __restrict__ xin, long long ld, const float* __restrict__ taps_w, const float* __restrict__ bias,
                                   int K, float* __restrict__ conv_state, long long slot_stride, const int* __restrict__ state_slots,
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
    const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1];
    const int first = t - t_begin, n = t_end - t_begin;
    if (first > 0 && first < K - 1) continue;  // worked out by the thread of the portion's first token
    float* st = conv_state + (size_t)state_slots[b] * slot_stride;  // [K-1, C]: the inputs before the portion, oldest first
    const int count = first == 0 ? max(1, min(K - 1, n)) : 1;
    for (int tt = t; tt < t + count; ++tt) {
      float acc = bias ? bias[col] : 0.f;
      float cur = 0.f;
      for (int j = 0; j < K; ++j) {
        const int p = tt - (K - 1) + j;
        const float in = p >= t_begin ? ts_to_float(xin[(size_t)p * ld + col]) : st[(size_t)(K - 1 + p - t_begin) * C + col];
        acc = fmaf(taps_w[(size_t)j * C + col], in, acc);
        cur = in;
      }
      if (act == CONV_ACT_SILU) acc = acc / (1.f + expf(-acc));
      if (add_input) acc += cur;
      out[(size_t)tt * ld_out + col] = ts_from_float<TO>(acc);
    }
    if (first == 0)
      for (int j = 0; j < K - 1; ++j) {  // entry j becomes the input at position t_end - (K-1) + j
        const int p = t_end - (K - 1) + j;
        st[(size_t)j * C + col] = p >= t_begin ? ts_to_float(xin[(size_t)p * ld + col]) : st[(size_t)(j + n) * C + col];
      }
  }
}

// Eight consecutive channels per thread, read and written as 16-byte pieces: for widths that are multiples of 8
// (rows and bases on 16-byte boundaries).  One block row per token, so no index is ever divided.
__device__ __forceinline__ void conv_load8(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void conv_load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void conv_store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void conv_store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(128) causal_conv_vec_kernel(const TI* __restrict__ xin, long long ld, const float* __restrict__ taps_w,
                                                              const float* __restrict__ bias, int K, float* __restrict__ conv_state,
                                                              long long slot_stride, const int* __restrict__ state_slots,
                                                              const int* __restrict__ cu_seqlens, const int* __restrict__ seq_index,
                                                              TO* __restrict__ out, long long ld_out, int C, int act, int add_input) {
  ts_pdl_prologue();
  const int t = blockIdx.x, col = (blockIdx.y * 128 + threadIdx.x) * 8;
  if (col >= C) return;
  const int b = seq_index[t];
  float acc[8], cur[8], w[8];
  if (b < 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    conv_store8(out + (size_t)t * ld_out + col, acc);
    return;
  }
  const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1];
  const int first = t - t_begin, n = t_end - t_begin;
  if (first > 0 && first < K - 1) return;  // worked out by the thread of the portion's first token
  float* st = conv_state + (size_t)state_slots[b] * slot_stride;
  const int count = first == 0 ? max(1, min(K - 1, n)) : 1;
  for (int tt = t; tt < t + count; ++tt) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = bias ? bias[col + i] : 0.f;
    for (int j = 0; j < K; ++j) {
      const int p = tt - (K - 1) + j;
      if (p >= t_begin) conv_load8(xin + (size_t)p * ld + col, cur);
      else conv_load8(st + (size_t)(K - 1 + p - t_begin) * C + col, cur);
      conv_load8(taps_w + (size_t)j * C + col, w);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[i], cur[i], acc[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (act == CONV_ACT_SILU) acc[i] = acc[i] / (1.f + expf(-acc[i]));
      if (add_input) acc[i] += cur[i];
    }
    conv_store8(out + (size_t)tt * ld_out + col, acc);
  }
  if (first == 0)
    for (int j = 0; j < K - 1; ++j) {  // entry j becomes the input at position t_end - (K-1) + j
      const int p = t_end - (K - 1) + j;
      if (p >= t_begin) conv_load8(xin + (size_t)p * ld + col, cur);
      else conv_load8(st + (size_t)(j + n) * C + col, cur);
      conv_store8(st + (size_t)j * C + col, cur);
    }
}

template <typename TI, typename TO>
static int conv_launch(const void* xin, long long ld, const float* taps_w, const float* bias, int K, float* conv_state,
                       long long slot_stride, const int* state_slots, const int* cu_seqlens, const int* seq_index, void* out, long long ld_out,
                       int T, int C, int act, int add_input, cudaStream_t s) {
  const bool aligned = C % 8 == 0 && ld % 8 == 0 && ld_out % 8 == 0 && slot_stride % 4 == 0 &&
                       (((uintptr_t)xin | (uintptr_t)out | (uintptr_t)conv_state | (uintptr_t)taps_w) & 15) == 0;
  if (aligned)
    return ts_launch(causal_conv_vec_kernel<TI, TO>, dim3(T, (C / 8 + 127) / 128), dim3(128), 0, s, (const TI*)xin, ld, taps_w, bias, K, conv_state,
                     slot_stride, state_slots, cu_seqlens, seq_index, (TO*)out, ld_out, C, act, add_input);
  const long long total = (long long)T * C;
  const unsigned blocks = (unsigned)min((total + 255) / 256, (long long)148 * 32);
  return ts_launch(causal_conv_kernel<TI, TO>, dim3(blocks), dim3(256), 0, s, (const TI*)xin, ld, taps_w, bias, K, conv_state, slot_stride,
                   state_slots, cu_seqlens, seq_index, (TO*)out, ld_out, T, C, act, add_input);
}

TS_EXPORT int ts_causal_conv(const void* xin, int in_dtype, long long ld, const float* taps_w, const float* bias, int K, float* conv_state,
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
