// The gated delta rule: per head a state S [d, e] in float32 that is decayed, corrected by what it
// already returns for the new key, and read out, token by token:
//
//   q^ = q / sqrt(sum q^2 + unit_eps) * q_scale,   k^ = k / sqrt(sum k^2 + unit_eps)       (per head)
//   beta = sigmoid(b),   g = exp(-exp(A_log_h) * softplus(a + dt_bias_h))                  (per token and head)
//   S <- g S;   u = beta (v - S^T k^);   S <- S + k^ u^T;   o = S^T q^
//
// Since o = (g S)^T q^ + u (k^ . q^), one walk over the decayed state gives both S^T k^ and the
// read-out's first term, and the update runs in a second walk: two passes over a thread's part of
// the state per token and one round of shuffles.
//
// delta_scan: one CTA per (sequence, head, block of value columns).  A thread owns one value
// column and 4 M key channels of it in registers, in fours that interleave with those of the other
// R - 1 lanes of its column (so that the lanes' 16-byte reads of the staged q^ and k^ rows fall on
// consecutive pieces of shared memory); the R lanes add their partial sums by shuffles.  The CTA
// walks its sequence's tokens of the step in order, DR_TB at a time: q, k (normed to unit length in
// the staging pass), v, beta, g and k^ . q^ of those tokens are staged in shared memory by all
// threads, then every thread runs the round's updates from there.  The state is read from the
// request's slot before the first token and written back after the last, so a sequence may be cut
// anywhere, and a token's result depends on nothing but its own sequence: the same sums in the same
// order whatever else is in the batch.  In the slot the state lies value column by value column
// ([H, e, d]: a thread's channels are then contiguous fours).  A sequence without tokens in this
// step (a padded lane of a fixed-size batch) touches nothing.  q and k heads may be shared by
// groups of value heads (head h reads q/k head h / (H / G)).  Everything is float32.
#include "common.cuh"

#define DR_TB 8          // tokens staged at a time
#define DR_THREADS 128
#define DR_MAX_KEY_DIM 1024

__device__ __forceinline__ float dr_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

template <int M>
__global__ void __launch_bounds__(DR_THREADS) delta_scan_kernel(
    const float* __restrict__ x, long long ld, int q_off, int k_off, int v_off, const float* __restrict__ ba, long long ld_ba,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ state, long long slot_stride,
    const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens, float* __restrict__ out, int H, int G, int d, int e, int R,
    float q_scale, float unit_eps) {
  ts_pdl_prologue();
  extern __shared__ __align__(16) float dr_smem[];
  const int b = blockIdx.x, h = blockIdx.y;
  const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1];
  if (t_end <= t_begin) return;
  const int cols = DR_THREADS / R;  // value columns of this CTA
  const int dpad = 4 * M * R;
  float* qs = dr_smem;                     // [DR_TB][dpad]
  float* ks = qs + DR_TB * dpad;           // [DR_TB][dpad]
  float* vs = ks + DR_TB * dpad;           // [DR_TB][cols]
  float* gs = vs + DR_TB * cols;           // [DR_TB] decay
  float* bs = gs + DR_TB;                  // [DR_TB] beta
  float* kqs = bs + DR_TB;                 // [DR_TB] k^ . q^
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = tid % R, cl = tid / R;
  const int col = blockIdx.z * cols + cl;
  const bool live = col < e;
  const int hk = h / (H / G);

  float S[4 * M];
  float* sp = state + (size_t)state_slots[b] * slot_stride + ((size_t)h * e + (live ? col : 0)) * d;
#pragma unroll
  for (int m = 0; m < M; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i = 4 * (r + R * m) + c;
      S[4 * m + c] = (live && i < d) ? sp[i] : 0.f;
    }
  const float decay_rate = expf(a_log[h]);
  const float bias_h = dt_bias[h];

  for (int t0 = t_begin; t0 < t_end; t0 += DR_TB) {
    const int nt = min(DR_TB, t_end - t0);
    __syncthreads();  // the round before is read out
    for (int i = tid; i < nt * dpad; i += DR_THREADS) {
      const int tt = i / dpad, c = i - tt * dpad;
      const float* row = x + (size_t)(t0 + tt) * ld;
      qs[i] = c < d ? row[q_off + hk * d + c] : 0.f;
      ks[i] = c < d ? row[k_off + hk * d + c] : 0.f;
    }
    for (int i = tid; i < nt * cols; i += DR_THREADS) {
      const int tt = i / cols, c = i - tt * cols;
      const int vc = blockIdx.z * cols + c;
      vs[i] = vc < e ? x[(size_t)(t0 + tt) * ld + v_off + h * e + vc] : 0.f;
    }
    if (tid < nt) {
      const float* g_row = ba + (size_t)(t0 + tid) * ld_ba;
      bs[tid] = 1.f / (1.f + expf(-g_row[h]));
      gs[tid] = expf(-decay_rate * dr_softplus(g_row[H + h] + bias_h));
    }
    __syncthreads();
    // unit length, the query's scale and k^ . q^: a warp per token
    for (int tt = warp; tt < nt; tt += DR_THREADS / 32) {
      float* qr = qs + tt * dpad;
      float* kr = ks + tt * dpad;
      float sq = 0.f, sk = 0.f, qk = 0.f;
      for (int c = lane; c < d; c += 32) {
        sq = fmaf(qr[c], qr[c], sq);
        sk = fmaf(kr[c], kr[c], sk);
        qk = fmaf(qr[c], kr[c], qk);
      }
      sq = ts_warp_sum(sq), sk = ts_warp_sum(sk), qk = ts_warp_sum(qk);
      const float mq = q_scale / sqrtf(sq + unit_eps), mk = 1.f / sqrtf(sk + unit_eps);
      for (int c = lane; c < d; c += 32) {
        qr[c] *= mq;
        kr[c] *= mk;
      }
      if (lane == 0) kqs[tt] = qk * mq * mk;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float g = gs[tt];
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * dpad);
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * dpad);
      float4 kv[M];
      float rk = 0.f, rq = 0.f;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        kv[m] = k4[r + R * m];
        const float4 qv = q4[r + R * m];
        S[4 * m + 0] *= g, S[4 * m + 1] *= g, S[4 * m + 2] *= g, S[4 * m + 3] *= g;
        rk = fmaf(S[4 * m + 0], kv[m].x, rk), rq = fmaf(S[4 * m + 0], qv.x, rq);
        rk = fmaf(S[4 * m + 1], kv[m].y, rk), rq = fmaf(S[4 * m + 1], qv.y, rq);
        rk = fmaf(S[4 * m + 2], kv[m].z, rk), rq = fmaf(S[4 * m + 2], qv.z, rq);
        rk = fmaf(S[4 * m + 3], kv[m].w, rk), rq = fmaf(S[4 * m + 3], qv.w, rq);
      }
      for (int o = R >> 1; o > 0; o >>= 1) {
        rk += __shfl_xor_sync(0xffffffffu, rk, o);
        rq += __shfl_xor_sync(0xffffffffu, rq, o);
      }
      const float u = bs[tt] * (vs[tt * cols + cl] - rk);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        S[4 * m + 0] = fmaf(kv[m].x, u, S[4 * m + 0]);
        S[4 * m + 1] = fmaf(kv[m].y, u, S[4 * m + 1]);
        S[4 * m + 2] = fmaf(kv[m].z, u, S[4 * m + 2]);
        S[4 * m + 3] = fmaf(kv[m].w, u, S[4 * m + 3]);
      }
      if (live && r == 0) out[(size_t)(t0 + tt) * H * e + (size_t)h * e + col] = fmaf(u, kqs[tt], rq);
    }
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int i = 4 * (r + R * m) + c;
        if (i < d) sp[i] = S[4 * m + c];
      }
  }
}

// How the state of one head is cut over threads for key width d: M fours of channels per thread and
// R lanes per value column (R a power of two up to 32, 4 M R >= d).  `ctas_wanted`: with fewer CTAs
// than this at M fours, a column is given to more lanes (so that more CTAs run).
static void dr_shape(int d, int e, int pairs, int ctas_wanted, int* M_out, int* R_out) {
  int M = 4, R = 1;
  while (4 * M * R < d && R < 32) R <<= 1;
  if (4 * M * R < d) M = 8;
  while (M > 1 && R < 32 && (long long)pairs * ((e + DR_THREADS / R - 1) / (DR_THREADS / R)) < ctas_wanted) {
    M >>= 1;
    R <<= 1;
  }
  while (M > 1 && 4 * (M >> 1) * R >= d) M >>= 1;  // no thread holds fours that lie beyond d altogether
  *M_out = M, *R_out = R;
}

TS_EXPORT int ts_delta_scan(const float* x, long long ld, int q_off, int k_off, int v_off, const float* ba, long long ld_ba, const float* a_log,
                            const float* dt_bias, float* state, long long slot_stride, const int* state_slots, const int* cu_seqlens,
                            float* out, int B, int H, int G, int d, int e, float q_scale, float unit_eps, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0) return TS_ERR_BAD_ARGUMENT;
  if (d > DR_MAX_KEY_DIM || B > 65535 * 16 || H > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  int M, R;
  dr_shape(d, e, B * H, 2 * 148, &M, &R);
  const int cols = DR_THREADS / R;
  const dim3 grid(B, H, (e + cols - 1) / cols);
  if (grid.z > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  const size_t smem = (size_t)(2 * DR_TB * 4 * M * R + DR_TB * cols + 3 * DR_TB) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
#define DR_CASE(MM)                                                                                                                   \
  case MM: {                                                                                                                          \
    static size_t set = 0;                                                                                                            \
    if (smem > 48 * 1024 && smem > set) {                                                                                             \
      cudaError_t err = cudaFuncSetAttribute(delta_scan_kernel<MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
      if (err != cudaSuccess) return (int)err;                                                                                        \
      set = smem;                                                                                                                     \
    }                                                                                                                                 \
    return ts_launch(delta_scan_kernel<MM>, grid, dim3(DR_THREADS), smem, s, x, ld, q_off, k_off, v_off, ba, ld_ba, a_log, dt_bias, \
                     state, slot_stride, state_slots, cu_seqlens, out, H, G, d, e, R, q_scale, unit_eps);                            \
  }
  switch (M) {
    DR_CASE(1)
    DR_CASE(2)
    DR_CASE(4)
    DR_CASE(8)
  }
#undef DR_CASE
  return TS_ERR_BAD_ARGUMENT;
}
