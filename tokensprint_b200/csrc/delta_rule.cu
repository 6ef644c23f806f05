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
// walks its sequence's tokens of the step in order, up to 16 at a time: q, k (normed to unit length in
// the staging pass), v, beta, g and k^ . q^ of those tokens are staged in shared memory by all
// threads (the next round's rows are asked for before the round's updates begin and wait in registers),
// then every thread runs the round's updates from there.  The state is read from the
// request's slot before the first token and written back after the last, so a sequence may be cut
// anywhere, and a token's result depends on nothing but its own sequence: the same sums in the same
// order whatever else is in the batch.  In the slot the state lies value column by value column
// ([H, e, d]: a thread's channels are then contiguous fours).  A sequence without tokens in this
// step (a padded lane of a fixed-size batch) touches nothing.  q and k heads may be shared by
// groups of value heads (head h reads q/k head h / (H / G)).  Everything is float32.
#include "common.cuh"

#define DR_THREADS 128
#define DR_MAX_KEY_DIM 1024
// Tokens staged at a time: 16, fewer where the padded key width exceeds 128 (a round's q and k rows are at most 2,048
// entries each, 16 per thread, which wait in registers while the round before is worked through).
__host__ __device__ constexpr int dr_round_tokens(int dpad) { return dpad <= 128 ? 16 : 2048 / dpad; }

__device__ __forceinline__ float dr_softplus(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// M fours of key channels per thread, R lanes per value column (4 M R >= d), PF staged entries per thread and round.
template <int M, int R, int PF>
__global__ void __launch_bounds__(DR_THREADS) delta_scan_kernel(
    const float* __restrict__ x, long long ld, int q_off, int k_off, int v_off, const float* __restrict__ ba, long long ld_ba,
    const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ state, long long slot_stride,
    const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens, float* __restrict__ out, int H, int G, int d, int e,
    float q_scale, float unit_eps) {
  ts_pdl_prologue();
  constexpr int COLS = DR_THREADS / R;  // value columns of this CTA
  constexpr int DPAD = 4 * M * R;
  constexpr int DR_TB = dr_round_tokens(DPAD);
  constexpr int DR_LPT = DR_THREADS / DR_TB < 32 ? DR_THREADS / DR_TB : 32;  // lanes that share a token in the staging pass
  constexpr int PFV = (DR_TB * COLS + DR_THREADS - 1) / DR_THREADS;
  __shared__ __align__(16) float qs[DR_TB * DPAD];
  __shared__ __align__(16) float ks[DR_TB * DPAD];
  __shared__ float vs[DR_TB * COLS];
  __shared__ float gs[DR_TB], bs[DR_TB], kqs[DR_TB];
  const int b = blockIdx.x, h = blockIdx.y;
  const int t_begin = cu_seqlens[b], t_end = cu_seqlens[b + 1];
  if (t_end <= t_begin) return;
  const int tid = threadIdx.x;
  const int r = tid % R, cl = tid / R;
  const int col = blockIdx.z * COLS + cl;
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

  // What a thread fetches of a round: entries tid, tid + 128, ... of the round's [tokens x DPAD] q and k rows and of its
  // [tokens x COLS] values, and (threads 0 .. tokens - 1) the two gate rows of one token.  The next round's values are asked
  // for before this round's updates begin and wait in registers until these are done.
  float pq[PF], pk[PF], pv[PFV], pb = 0.f, pa = 0.f;
  auto fetch = [&](int t0) {
    const int nt = min(DR_TB, t_end - t0);
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      const int i = tid + u * DR_THREADS, tt = i / DPAD, c = i - tt * DPAD;
      const bool ok = tt < nt && c < d;
      const float* row = x + (size_t)(t0 + (ok ? tt : 0)) * ld + hk * d + (ok ? c : 0);
      pq[u] = ok ? row[q_off] : 0.f;
      pk[u] = ok ? row[k_off] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < PFV; ++u) {
      const int i = tid + u * DR_THREADS, tt = i / COLS, c = i - tt * COLS;
      const int vc = blockIdx.z * COLS + c;
      const bool ok = tt < nt && vc < e;
      pv[u] = ok ? x[(size_t)(t0 + tt) * ld + v_off + h * e + vc] : 0.f;
    }
    if (tid < nt) {
      const float* g_row = ba + (size_t)(t0 + tid) * ld_ba;
      pb = g_row[h];
      pa = g_row[H + h];
    }
  };
  fetch(t_begin);

  for (int t0 = t_begin; t0 < t_end; t0 += DR_TB) {
    const int nt = min(DR_TB, t_end - t0);
    __syncthreads();  // the round before is read out
#pragma unroll
    for (int u = 0; u < PF; ++u) {
      const int i = tid + u * DR_THREADS;
      if (i < DR_TB * DPAD) qs[i] = pq[u], ks[i] = pk[u];
    }
#pragma unroll
    for (int u = 0; u < PFV; ++u) {
      const int i = tid + u * DR_THREADS;
      if (i < DR_TB * COLS) vs[i] = pv[u];
    }
    if (tid < nt) {
      bs[tid] = 1.f / (1.f + expf(-pb));
      gs[tid] = expf(-decay_rate * dr_softplus(pa + bias_h));
    }
    __syncthreads();
    if (t0 + DR_TB < t_end) fetch(t0 + DR_TB);
    // unit length, the query's scale and k^ . q^: DR_LPT lanes per token, the tokens of the round side by side
    for (int tt = tid / DR_LPT; tt < DR_TB; tt += DR_THREADS / DR_LPT) {
      const int l = tid % DR_LPT;
      float* qr = qs + tt * DPAD;
      float* kr = ks + tt * DPAD;
      float sq = 0.f, sk = 0.f, qk = 0.f;
      for (int c = l; c < d; c += DR_LPT) {
        sq = fmaf(qr[c], qr[c], sq);
        sk = fmaf(kr[c], kr[c], sk);
        qk = fmaf(qr[c], kr[c], qk);
      }
#pragma unroll
      for (int o = DR_LPT >> 1; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        qk += __shfl_xor_sync(0xffffffffu, qk, o);
      }
      const float mq = q_scale / sqrtf(sq + unit_eps), mk = 1.f / sqrtf(sk + unit_eps);
      for (int c = l; c < d; c += DR_LPT) {
        qr[c] *= mq;
        kr[c] *= mk;
      }
      if (l == 0) kqs[tt] = qk * mq * mk;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float g = gs[tt];
      const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DPAD);
      const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DPAD);
      float4 kv[M];
      float rk[2] = {0.f, 0.f}, rq[2] = {0.f, 0.f};  // two chains each, so that a thread's sums do not wait on one another
#pragma unroll
      for (int m = 0; m < M; ++m) {
        kv[m] = k4[r + R * m];
        const float4 qv = q4[r + R * m];
        rk[0] = fmaf(S[4 * m + 0], kv[m].x, rk[0]), rq[0] = fmaf(S[4 * m + 0], qv.x, rq[0]);
        rk[1] = fmaf(S[4 * m + 1], kv[m].y, rk[1]), rq[1] = fmaf(S[4 * m + 1], qv.y, rq[1]);
        rk[0] = fmaf(S[4 * m + 2], kv[m].z, rk[0]), rq[0] = fmaf(S[4 * m + 2], qv.z, rq[0]);
        rk[1] = fmaf(S[4 * m + 3], kv[m].w, rk[1]), rq[1] = fmaf(S[4 * m + 3], qv.w, rq[1]);
      }
      // the sums run over the state as it was; the decay is one factor on each of them (S^T k of the decayed state is g S^T k)
      float sk = rk[0] + rk[1], sq = rq[0] + rq[1];
#pragma unroll
      for (int o = R >> 1; o > 0; o >>= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
      }
      sk *= g, sq *= g;
      const float u = bs[tt] * (vs[tt * COLS + cl] - sk);
#pragma unroll
      for (int m = 0; m < M; ++m) {
        S[4 * m + 0] = fmaf(g, S[4 * m + 0], kv[m].x * u);
        S[4 * m + 1] = fmaf(g, S[4 * m + 1], kv[m].y * u);
        S[4 * m + 2] = fmaf(g, S[4 * m + 2], kv[m].z * u);
        S[4 * m + 3] = fmaf(g, S[4 * m + 3], kv[m].w * u);
      }
      if (live && r == 0) out[(size_t)(t0 + tt) * H * e + (size_t)h * e + col] = fmaf(u, kqs[tt], sq);
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

template <int M, int R>
static int dr_launch(const float* x, long long ld, int q_off, int k_off, int v_off, const float* ba, long long ld_ba, const float* a_log,
                     const float* dt_bias, float* state, long long slot_stride, const int* state_slots, const int* cu_seqlens, float* out, int B,
                     int H, int G, int d, int e, float q_scale, float unit_eps, cudaStream_t s) {
  constexpr int COLS = DR_THREADS / R;
  constexpr int PF = (dr_round_tokens(4 * M * R) * 4 * M * R + DR_THREADS - 1) / DR_THREADS;
  static_assert(PF <= 16, "too many staged entries per thread");
  const dim3 grid(B, H, (e + COLS - 1) / COLS);
  if (grid.z > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  return ts_launch(delta_scan_kernel<M, R, PF>, grid, dim3(DR_THREADS), 0, s, x, ld, q_off, k_off, v_off, ba, ld_ba, a_log, dt_bias, state,
                   slot_stride, state_slots, cu_seqlens, out, H, G, d, e, q_scale, unit_eps);
}

// How the state of one head is cut over threads for key width d: a thread holds 16 key channels of its value column
// (fewer where the key is narrower, 32 where 16 each would need more than a warp's lanes), and as many lanes share a
// column as that takes.  The scan waits on its own chain of updates, token after token, so a prompt's time hardly depends
// on the cut (measured at 16 heads of 64 x 128, 2,048 tokens: 4 lanes of 16 channels 0.66 to 0.72 ms, 8 of 8 0.68, 16 of 4
// 0.62 to 0.64, 32 of which half hold nothing 0.95); what brought it there from 1.40 ms were the rows fetched a round
// ahead, the staging pass over all of a round's tokens at once and lane counts known at compile time.  More lanes mean
// more and smaller CTAs, which costs where many run side by side: with 16 lanes of 4 channels 32 heads took 0.81 ms
// instead of 0.66, and a decode step of 64 sequences, which only reads and writes the states, 0.11 to 0.12 of the copy
// bandwidth instead of 0.17 to 0.26.
TS_EXPORT int ts_delta_scan(const float* x, long long ld, int q_off, int k_off, int v_off, const float* ba, long long ld_ba, const float* a_log,
                            const float* dt_bias, float* state, long long slot_stride, const int* state_slots, const int* cu_seqlens,
                            float* out, int B, int H, int G, int d, int e, float q_scale, float unit_eps, int lanes, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || d <= 0 || e <= 0) return TS_ERR_BAD_ARGUMENT;
  if (d > DR_MAX_KEY_DIM || B > 65535 * 16 || H > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
#define DR_GO(MM, RR) \
  return dr_launch<MM, RR>(x, ld, q_off, k_off, v_off, ba, ld_ba, a_log, dt_bias, state, slot_stride, state_slots, cu_seqlens, out, B, H, G, d, e, q_scale, unit_eps, s)
  if (lanes > 0) {  // a given number of lanes per column (a power of two up to 32), for measurements
    const int fours = (d + 4 * lanes - 1) / (4 * lanes);
#define DR_LANES(RR)                        \
  if (lanes == RR) {                        \
    if (fours <= 1) DR_GO(1, RR);           \
    if (fours <= 2) DR_GO(2, RR);           \
    if (fours <= 4) DR_GO(4, RR);           \
    return TS_ERR_UNSUPPORTED_SIZE;         \
  }
    DR_LANES(1) DR_LANES(2) DR_LANES(4) DR_LANES(8) DR_LANES(16) DR_LANES(32)
#undef DR_LANES
    return TS_ERR_BAD_ARGUMENT;
  }
  if (d <= 4) DR_GO(1, 1);
  if (d <= 8) DR_GO(2, 1);
  if (d <= 16) DR_GO(4, 1);
  if (d <= 32) DR_GO(4, 2);
  if (d <= 64) DR_GO(4, 4);
  if (d <= 128) DR_GO(4, 8);
  if (d <= 256) DR_GO(4, 16);
  if (d <= 512) DR_GO(4, 32);
  DR_GO(8, 32);
#undef DR_GO
}
