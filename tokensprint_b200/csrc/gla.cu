// Gated linear attention: a recurrence with one decay per key channel, its state per request in
// float32, for prompt portions and single decoded tokens alike.
//
// Per head, with q, k, decay of d entries and v of e entries per token, and a state S [d, e]:
//   decay_t = sigmoid(z_t + bias)^(1/tau) = exp(logsigmoid(z_t + bias) / tau)
//   S_t = diag(decay_t) S_(t-1) + k_t v_t^T          row c of S belongs to key channel c
//   o_t = S_t^T (q_t * q_scale)
// then  out_t = o_t * rsqrt(mean_e(o_t^2) + eps) * w_norm * silu(g_t)   per head (gla_norm_gate).
//
// gla_decay: the decays of all tokens and channels once, float32 (every CTA of the scan that shares a
// head reads them; worked out inside the scan they were computed once per block of value columns).
//
// gla_scan: one CTA per (sequence, head, block of value columns).  A thread owns one value column
// and d / R key channels of it in registers, in fours that interleave with those of the other lanes
// (R lanes of a warp share a column and add their partial outputs by shuffles).  The CTA walks its sequence's tokens of the step in order,
// up to GLA_TB at a time: q, k, the decay and v of those tokens are staged in shared memory by all
// threads, then every thread runs the round's updates from there.
// The state is read from the request's slot before the first token and written back after the
// last, so a sequence may be cut anywhere, and a token's result depends on nothing but its own
// sequence: run in one piece, the same sums in the same order whatever else is in the batch (run
// in segments, see below, the grouping of the sums follows the step's longest portion and the
// number of sequences: float32 rounding, nothing else).
// A sequence without tokens in this step (a padded lane of a fixed-size batch) touches nothing.
#include "common.cuh"

#define GLA_TB 16        // tokens staged at a time, at most
#define GLA_MAX_KP 32    // key channels per thread, at most
#define GLA_THREADS 128
#define GLA_PF 8         // staged q (k, z) entries a thread fetches ahead per round: tb * dp <= GLA_THREADS * GLA_PF
#define GLA_PFV 4        // likewise for v: tb * cols <= GLA_THREADS * GLA_PFV
#ifndef GLA_MIN_BLOCKS
#define GLA_MIN_BLOCKS 4 // CTAs per SM the compiler plans the registers for (the scan waits on its own chain of updates: only more
                         // warps hide it; measured 1 / 3 / 4: 1.26 / 1.14 / 1.19 ms in segments, 1.56 / 1.58 / 1.25 in one piece)
#endif
#ifndef GLA_UNROLL
#define GLA_UNROLL 4     // tokens of a round whose loads and shuffles are in flight together
#endif
constexpr int GLA_UNROLL_TOKENS = GLA_UNROLL;

__device__ __forceinline__ float gla_log_sigmoid(float z) {
  // log(1 / (1 + exp(-z))) without overflow on either side
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// Loads that stay where they are written: the compiler otherwise moves a load whose value is first
// used after the round's updates down to that use, and the round then waits for device memory once
// per entry instead of never.
__device__ __forceinline__ float gla_load(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ __nv_bfloat16 gla_load(const __nv_bfloat16* p) {
  unsigned short v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return __ushort_as_bfloat16(v);
}

// The rounds are pipelined: while the threads run the updates of one round from shared memory, the
// loads of the next round's q, k, z and v are in flight into registers (issued before the updates,
// used after them), so the recurrence never waits for device memory.
//
// Long portions are cut into `segs` segments of `seg_len` tokens that run side by side (the recurrence
// is linear in the state): MODE 1 runs every segment but a sequence's last from a zero state (the
// first from the request's state) and leaves the state it ends with and the product of its decays;
// MODE 2 starts every segment from what the segments before it left, folded in order
// (S <- product * S + state), writes the read-outs, and the last segment writes the request's slot.
// MODE 0 is the whole portion in one piece (decode steps, short portions: the same sums whatever the cut).
template <typename TA, int KP, int MODE>
__global__ void __launch_bounds__(GLA_THREADS, GLA_MIN_BLOCKS) gla_scan_kernel(
    const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, long long ld_qkv, const float* __restrict__ decay,
    float q_scale, float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens,
    float* __restrict__ o, int H, int d, int e, int R, int cols_per_cta, int tb, int segs, int seg_len, float* __restrict__ seg_state,
    float* __restrict__ seg_decay, float* __restrict__ seg_start, const float* __restrict__ kscale, int decay_scalar, int groups, int ev,
    long long slot_stride) {
  ts_pdl_prologue();
  extern __shared__ __align__(16) float sm[];
  // staged per token: q, k, decay [dp] each, v [cols]
  const int dp = R * KP;  // d padded to the channels the threads cover
  float* sq = sm;
  float* sk = sq + tb * dp;
  float* sa = sk + tb * dp;
  float* sv = sa + tb * dp;  // [tb][cols_per_cta]
  const int b = MODE == 0 ? blockIdx.x : blockIdx.x / segs, seg = MODE == 0 ? 0 : blockIdx.x - b * segs;
  const int h = blockIdx.y, col0 = blockIdx.z * cols_per_cta;
  const int t_begin = cu_seqlens[b] + seg * seg_len, t_end = MODE == 0 ? cu_seqlens[b + 1] : min(cu_seqlens[b + 1], t_begin + seg_len);
  if (t_end <= t_begin) return;
  const bool last = t_end == cu_seqlens[b + 1];
  if (MODE == 1 && last) return;  // nobody starts from what a sequence's last segment leaves
  const int r = threadIdx.x % R, cj = threadIdx.x / R;  // lanes of one column sit side by side
  const int col = col0 + cj;
  const bool has_col = col < e;
  // Register i of a thread holds key channel CH(i): its channels come in fours, and the fours of the R lanes of a column
  // are interleaved (lane r owns fours r, r + R, r + 2 R, ...), so that the 16-byte loads of a warp's lanes fall on
  // consecutive 16-byte pieces of the staged rows: no two of them meet in a bank of shared memory.
#define CH(i) (((((i) >> 2) * R + r) << 2) + ((i) & 3))
  float* S = state + (size_t)state_slots[b] * slot_stride + ((size_t)h * d) * e;
  const size_t state_elems = (size_t)d * e;
  float* seg_L = MODE == 0 ? nullptr : seg_state + (((size_t)b * segs + seg) * H + h) * state_elems;   // this segment's end state
  float* seg_P = MODE == 0 ? nullptr : seg_decay + (((size_t)b * segs + seg) * H + h) * d;             // this segment's decay product
  float* seg_S0 = MODE == 0 ? nullptr : seg_start + ((size_t)b * H + h) * state_elems;                 // the request's state as the step found it
  float s_reg[KP];
  float p_reg[MODE == 1 ? KP : 1];
  if (MODE == 0 || (seg == 0 && (MODE == 1 || last))) {
    // the request's state (MODE 2: only a sequence of one segment reads the slot, which it alone writes in this launch)
#pragma unroll
    for (int i = 0; i < KP; ++i) s_reg[i] = (has_col && CH(i) < d) ? S[(size_t)(CH(i)) * e + col] : 0.f;
    if (MODE == 1 && has_col) {
#pragma unroll
      for (int i = 0; i < KP; ++i)
        if (CH(i) < d) seg_S0[(size_t)(CH(i)) * e + col] = s_reg[i];
    }
  } else if (MODE == 1) {
#pragma unroll
    for (int i = 0; i < KP; ++i) s_reg[i] = 0.f;
  } else if (seg == 0) {
#pragma unroll
    for (int i = 0; i < KP; ++i) s_reg[i] = (has_col && CH(i) < d) ? seg_S0[(size_t)(CH(i)) * e + col] : 0.f;
  } else {
    // what the segments before left, folded in order (the first one's end state already holds the request's state)
    const float* L = seg_state + (((size_t)b * segs) * H + h) * state_elems;
#pragma unroll
    for (int i = 0; i < KP; ++i) s_reg[i] = (has_col && CH(i) < d) ? L[(size_t)(CH(i)) * e + col] : 0.f;
    for (int j = 1; j < seg; ++j) {
      L = seg_state + (((size_t)b * segs + j) * H + h) * state_elems;
      const float* P = seg_decay + (((size_t)b * segs + j) * H + h) * d;
#pragma unroll
      for (int i = 0; i < KP; ++i)
        if (has_col && CH(i) < d) s_reg[i] = fmaf(P[CH(i)], s_reg[i], L[(size_t)(CH(i)) * e + col]);
    }
  }
  if (MODE == 1) {
#pragma unroll
    for (int i = 0; i < KP; ++i) p_reg[i] = 1.f;
  }

  const size_t qk_off = (size_t)(h / (H / groups)) * d, a_off = (size_t)h * d, v_off = (size_t)h * ev + col0;
  // what this thread fetches for a round: entries threadIdx.x + j * GLA_THREADS of the round's [tokens][dp] and [tokens][cols]
  TA fq[GLA_PF], fk[GLA_PF], fv[GLA_PFV];
  float fa[GLA_PF], fb[GLA_PF];
  // Entry i of a round is channel i % dp of token i / dp (for v: column i % cols of token i / cols); a thread's
  // entries lie GLA_THREADS apart, so their places are found once, by steps, without a division per entry.
  const int Hd = H * d;
  const int step_t = GLA_THREADS / dp, step_c = GLA_THREADS % dp, first_t = (int)threadIdx.x / dp, first_c = (int)threadIdx.x % dp;
  const int vstep_t = GLA_THREADS / cols_per_cta, vstep_c = GLA_THREADS % cols_per_cta;
  const int vfirst_t = (int)threadIdx.x / cols_per_cta, vfirst_c = (int)threadIdx.x % cols_per_cta;
  auto fetch = [&](int t0) {
    const int nt = min(tb, t_end - t0);
    int tt = first_t, c = first_c;
#pragma unroll
    for (int j = 0; j < GLA_PF; ++j) {
      {  // an entry beyond the round's tokens or the head's channels reads a valid place and is not used
        const int tr = t0 + min(tt, nt - 1), cr = min(c, d - 1);
        const size_t at = (size_t)tr * ld_qkv + qk_off + cr;
        fq[j] = gla_load(q + at);
        fk[j] = gla_load(k + at);
        fa[j] = decay_scalar ? gla_load(decay + (size_t)tr * H + h) : gla_load(decay + (size_t)tr * Hd + a_off + cr);
        fb[j] = kscale ? gla_load(kscale + (size_t)tr * H + h) : 1.f;
      }
      tt += step_t, c += step_c;
      if (c >= dp) c -= dp, ++tt;
    }
    tt = vfirst_t, c = vfirst_c;
#pragma unroll
    for (int j = 0; j < GLA_PFV; ++j) {
      fv[j] = gla_load(v + (size_t)(t0 + min(tt, nt - 1)) * ld_qkv + v_off + min(c, ev - 1 - col0));
      tt += vstep_t, c += vstep_c;
      if (c >= cols_per_cta) c -= cols_per_cta, ++tt;
    }
  };
  auto stage = [&](int t0) {  // the fetched entries into shared memory as float32, q scaled
    const int nt = min(tb, t_end - t0);
    int tt = first_t, c = first_c;
#pragma unroll
    for (int j = 0; j < GLA_PF; ++j) {
      if (tt < nt) {
        const bool real = c < d;
        const int i = tt * dp + c;
        sq[i] = real ? ts_to_float(fq[j]) * q_scale : 0.f;
        sk[i] = real ? ts_to_float(fk[j]) * fb[j] : 0.f;
        sa[i] = real ? fa[j] : 1.f;
      }
      tt += step_t, c += step_c;
      if (c >= dp) c -= dp, ++tt;
    }
    tt = vfirst_t, c = vfirst_c;
#pragma unroll
    for (int j = 0; j < GLA_PFV; ++j) {
      if (tt < nt) sv[tt * cols_per_cta + c] = (col0 + c < ev) ? ts_to_float(fv[j]) : (col0 + c < e ? 1.f : 0.f);
      tt += vstep_t, c += vstep_c;
      if (c >= cols_per_cta) c -= cols_per_cta, ++tt;
    }
  };

  fetch(t_begin);
  for (int t0 = t_begin; t0 < t_end; t0 += tb) {
    const int nt = min(tb, t_end - t0);
    __syncthreads();  // the round before has been read
    stage(t0);
    __syncthreads();
    if (t0 + tb < t_end) fetch(t0 + tb);  // in flight while this round's updates run
#pragma unroll(KP > 16 ? 1 : GLA_UNROLL_TOKENS)  // several tokens' loads and shuffles in flight where the registers allow
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = sv[tt * cols_per_cta + cj];
      // a thread's channels come in fours that start on 16-byte boundaries: 16-byte loads
      const float4* pq = reinterpret_cast<const float4*>(sq + tt * dp) + r;
      const float4* pk = reinterpret_cast<const float4*>(sk + tt * dp) + r;
      const float4* pa = reinterpret_cast<const float4*>(sa + tt * dp) + r;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};  // four chains: the read-out is a sum of KP terms, its order is fixed by KP alone
#pragma unroll
      for (int i = 0; i < KP / 4; ++i) {
        const float4 a4 = pa[i * R], k4 = pk[i * R];
        s_reg[4 * i + 0] = fmaf(a4.x, s_reg[4 * i + 0], k4.x * vv);
        s_reg[4 * i + 1] = fmaf(a4.y, s_reg[4 * i + 1], k4.y * vv);
        s_reg[4 * i + 2] = fmaf(a4.z, s_reg[4 * i + 2], k4.z * vv);
        s_reg[4 * i + 3] = fmaf(a4.w, s_reg[4 * i + 3], k4.w * vv);
        if (MODE == 1) {  // no read-outs yet: the product of the segment's decays instead
          p_reg[(MODE == 1 ? 4 * i : 0) + 0] *= a4.x;
          p_reg[(MODE == 1 ? 4 * i + 1 : 0)] *= a4.y;
          p_reg[(MODE == 1 ? 4 * i + 2 : 0)] *= a4.z;
          p_reg[(MODE == 1 ? 4 * i + 3 : 0)] *= a4.w;
        } else {
          const float4 q4 = pq[i * R];
          acc[0] = fmaf(s_reg[4 * i + 0], q4.x, acc[0]);
          acc[1] = fmaf(s_reg[4 * i + 1], q4.y, acc[1]);
          acc[2] = fmaf(s_reg[4 * i + 2], q4.z, acc[2]);
          acc[3] = fmaf(s_reg[4 * i + 3], q4.w, acc[3]);
        }
      }
      if (MODE != 1) {
        float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        for (int w = 1; w < R; w <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, w);
        if (r == 0 && has_col) o[((size_t)(t0 + tt) * H + h) * e + col] = sum;
      }
    }
  }
  if (MODE == 1) {
    if (has_col) {
#pragma unroll
      for (int i = 0; i < KP; ++i)
        if (CH(i) < d) seg_L[(size_t)(CH(i)) * e + col] = s_reg[i];
    }
    if (blockIdx.z == 0 && cj == 0) {  // the decays do not depend on the column: one thread per group of channels writes them
#pragma unroll
      for (int i = 0; i < KP; ++i)
        if (CH(i) < d) seg_P[CH(i)] = p_reg[MODE == 1 ? i : 0];
    }
  } else if (has_col && (MODE == 0 || last)) {
#pragma unroll
    for (int i = 0; i < KP; ++i)
      if (CH(i) < d) S[(size_t)(CH(i)) * e + col] = s_reg[i];
  }
}


// A step in which every sequence brings one token at most (decode): nothing is staged, no barrier is met.  One CTA per
// (sequence, head, block of value columns) as above; a thread reads the token's q, k and decay entries of its own
// channels straight from device memory (the lanes of other columns read the same words), updates its part of the
// state's column once and adds the read-out over the column's lanes.  Few registers, so many CTAs an SM: a decode
// step is a chain of a few dependent loads per CTA and nothing else, and only CTAs in flight hide it.
template <typename TA, int KP>
__global__ void __launch_bounds__(GLA_THREADS) gla_step_kernel(
    const TA* __restrict__ q, const TA* __restrict__ k, const TA* __restrict__ v, long long ld_qkv, const float* __restrict__ decay,
    float q_scale, float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens,
    float* __restrict__ o, int H, int d, int e, int R, int cols_per_cta, const float* __restrict__ kscale, int decay_scalar, int groups,
    int ev, long long slot_stride) {
  ts_pdl_prologue();
  const int b = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * cols_per_cta;
  const int t = cu_seqlens[b];
  if (cu_seqlens[b + 1] <= t) return;  // a lane of a fixed-size batch without a request
  const int r = threadIdx.x % R, cj = threadIdx.x / R;
  const int col = col0 + cj;
  const bool has_col = col < e;
  float* S = state + (size_t)state_slots[b] * slot_stride + ((size_t)h * d) * e;
  float s_reg[KP];
#pragma unroll
  for (int i = 0; i < KP; ++i) s_reg[i] = (has_col && CH(i) < d) ? S[(size_t)(CH(i)) * e + col] : 0.f;
  const size_t row = (size_t)t * ld_qkv, qk_off = (size_t)(h / (H / groups)) * d;
  const float scale_k = kscale ? kscale[(size_t)t * H + h] : 1.f;
  const float a_all = decay_scalar ? decay[(size_t)t * H + h] : 1.f;
  const float* a_row = decay + (size_t)t * H * d + (size_t)h * d;
  const float vv = !has_col ? 0.f : (col < ev ? ts_to_float(v[row + (size_t)h * ev + col]) : 1.f);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < KP; ++i) {
    const int ch = CH(i);
    if (ch < d) {
      const float a = decay_scalar ? a_all : a_row[ch];
      s_reg[i] = fmaf(a, s_reg[i], ts_to_float(k[row + qk_off + ch]) * scale_k * vv);
      acc = fmaf(s_reg[i], ts_to_float(q[row + qk_off + ch]) * q_scale, acc);
    }
  }
  for (int w = 1; w < R; w <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
  if (has_col) {
    if (r == 0) o[((size_t)t * H + h) * e + col] = acc;
#pragma unroll
    for (int i = 0; i < KP; ++i)
      if (CH(i) < d) S[(size_t)(CH(i)) * e + col] = s_reg[i];
  }
}
#undef CH

// What the general form of the recurrence has beyond gated linear attention's (see ts_linear_scan).
struct GlaExtra {
  const float* kscale;    // [T, H] a factor on k per (token, head), or null
  int decay_scalar;       // 1: decay is [T, H], one number per (token, head) for all key channels
  int groups;             // q and k have `groups` heads; head h reads group h / (H / groups)
  int ev;                 // columns of v per head; the state has e >= ev columns, column ev (if any) sees the value 1
  long long slot_stride;  // floats from one request's state to the next
};

template <typename TA, int KP, int MODE>
static int launch_gla_scan(const void* q, const void* k, const void* v, long long ld_qkv, const float* decay, float q_scale, float* state,
                           const int* state_slots, const int* cu_seqlens, float* o, int B, int H, int d, int e, int R, int segs, int seg_len,
                           float* scratch, cudaStream_t s, const GlaExtra& x) {
  const int cols = GLA_THREADS / R, dp = R * KP;
  // tokens per round: what the threads' fetch registers hold, at most GLA_TB
  const int tb = min(GLA_TB, min(GLA_THREADS * GLA_PF / dp, GLA_THREADS * GLA_PFV / cols));
  if (tb < 1) return TS_ERR_UNSUPPORTED_SIZE;
  const size_t smem = (size_t)tb * (3 * dp + cols) * sizeof(float);  // at most 16 * (3 * 64 + 128) or 1 * (3 * 1024 + 4) floats: below 48 KB
  const dim3 grid(B * segs, H, (e + cols - 1) / cols);
  if (grid.y > 65535 || grid.z > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  // scratch of the segmented scan: end states [B, segs, H, d, e], decay products [B, segs, H, d], start states [B, H, d, e]
  float* seg_state = scratch;
  float* seg_decay = scratch ? seg_state + (size_t)B * segs * H * d * e : nullptr;
  float* seg_start = scratch ? seg_decay + (size_t)B * segs * H * d : nullptr;
  return ts_launch(gla_scan_kernel<TA, KP, MODE>, grid, dim3(GLA_THREADS), smem, s, (const TA*)q, (const TA*)k, (const TA*)v, ld_qkv, decay,
                   q_scale, state, state_slots, cu_seqlens, o, H, d, e, R, cols, tb, segs, seg_len, seg_state, seg_decay, seg_start, x.kscale,
                   x.decay_scalar, x.groups, x.ev, x.slot_stride);
}

template <typename TA, int KP>
static int launch_gla_scan_modes(const void* q, const void* k, const void* v, long long ld_qkv, const float* decay, float q_scale, float* state,
                                 const int* state_slots, const int* cu_seqlens, float* o, int B, int H, int d, int e, int R, int segs,
                                 int seg_len, float* scratch, cudaStream_t s, const GlaExtra& x) {
  if (segs <= 1)
    return launch_gla_scan<TA, KP, 0>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, R, 1, 0, nullptr, s, x);
  const int st = launch_gla_scan<TA, KP, 1>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, R, segs, seg_len,
                                            scratch, s, x);
  if (st != 0) return st;
  return launch_gla_scan<TA, KP, 2>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, R, segs, seg_len, scratch, s, x);
}

template <typename TA>
static int dispatch_gla_scan(const void* q, const void* k, const void* v, long long ld_qkv, const float* decay, float q_scale, float* state,
                             const int* state_slots, const int* cu_seqlens, float* o, int B, int H, int d, int e, int segs, int seg_len,
                             float* scratch, cudaStream_t s, const GlaExtra& x) {
  // R lanes per column, a power of two, so that a thread holds at most GLA_MAX_KP channels
  int R = 1;
  while (R < 32 && (d + R - 1) / R > GLA_MAX_KP) R <<= 1;
  if (segs == 1 && seg_len == 1) {
    // one token per sequence at most: the kernel without staging, as few lanes per column as the registers allow
    // (a warp then covers 32 / R consecutive columns of a state row), more while the grid would leave SMs idle
    while (R < 32 && (d + R - 1) / R > 4 && (long long)B * H * ((e + GLA_THREADS / R - 1) / (GLA_THREADS / R)) < 4 * 148) R <<= 1;
    const int kp1 = (d + R - 1) / R, cols = GLA_THREADS / R;
    const dim3 grid(B, H, (e + cols - 1) / cols);
    if (grid.y > 65535 || grid.z > 65535) return TS_ERR_UNSUPPORTED_SIZE;
#define GLA_STEP_CASE(KP) \
    if (kp1 <= KP) \
      return ts_launch(gla_step_kernel<TA, KP>, grid, dim3(GLA_THREADS), 0, s, (const TA*)q, (const TA*)k, (const TA*)v, ld_qkv, decay, q_scale, \
                       state, state_slots, cu_seqlens, o, H, d, e, R, cols, x.kscale, x.decay_scalar, x.groups, x.ev, x.slot_stride)
    GLA_STEP_CASE(4);
    GLA_STEP_CASE(8);
    GLA_STEP_CASE(12);
    GLA_STEP_CASE(16);
    GLA_STEP_CASE(24);
    GLA_STEP_CASE(32);
#undef GLA_STEP_CASE
    return TS_ERR_UNSUPPORTED_SIZE;
  }
  // more lanes per column (fewer channels per thread, more CTAs) while the grid would leave SMs idle
  // or a thread's chain of updates per token would be long; a function of the sizes and the batch alone
  while (R < 32 && (d + R - 1) / R > 4 &&
         ((d + R - 1) / R > 16 || (long long)B * max(segs, 1) * H * ((e + GLA_THREADS / R - 1) / (GLA_THREADS / R)) < 2 * 148))
    R <<= 1;
  if (const char* forced = getenv("TS_GLA_LANES")) {  // for measurements: a fixed number of lanes per column
    const int want = atoi(forced);
    if (want >= 1 && want <= 32 && (want & (want - 1)) == 0 && (d + want - 1) / want <= GLA_MAX_KP) R = want;
  }
  const int kp = (d + R - 1) / R;
  if (kp > GLA_MAX_KP) return TS_ERR_UNSUPPORTED_SIZE;  // d > 1024
  static_assert(GLA_MAX_KP % 4 == 0, "a thread's channels come in fours");
#define GLA_CASE(KP) \
  if (kp <= KP) \
    return launch_gla_scan_modes<TA, KP>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, R, segs, seg_len, scratch, s, x)
  GLA_CASE(4);
  GLA_CASE(8);
  GLA_CASE(12);
  GLA_CASE(16);
  GLA_CASE(24);
  GLA_CASE(32);
#undef GLA_CASE
  return TS_ERR_UNSUPPORTED_SIZE;
}

// decay[t, c] = sigmoid(z[t, c] + bias[c])^(1/tau) = exp(logsigmoid(z + bias) / tau), float32, for all H*d channels c.
template <typename TA>
__global__ void gla_decay_kernel(const TA* __restrict__ z, long long ld_z, const float* __restrict__ bias, float inv_tau,
                                 float* __restrict__ decay, int T, int n) {
  ts_pdl_prologue();
  const int t = blockIdx.y;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n; c += gridDim.x * blockDim.x) {
    const float zz = ts_to_float(z[(size_t)t * ld_z + c]) + (bias ? bias[c] : 0.f);
    decay[(size_t)t * n + c] = expf(gla_log_sigmoid(zz) * inv_tau);
  }
}

// z [T, H*d] with row stride ld_z; bias [H*d] float32 or null; decay [T, H*d] float32.
TS_EXPORT int ts_gla_decay(const void* z, long long ld_z, int act_dtype, const float* bias, float tau, float* decay, int T, int n,
                           void* stream) {
  if (T <= 0) return 0;
  if (n <= 0 || !(tau > 0.f)) return TS_ERR_BAD_ARGUMENT;
  if (T > 65535 * 64) return TS_ERR_UNSUPPORTED_SIZE;
  // rows in the grid's y; beyond 65,535 rows a block takes several (a row index is then folded into the channel index)
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((n + 255) / 256, T);
  if (grid.y > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(gla_decay_kernel<float>, grid, dim3(256), 0, s, (const float*)z, ld_z, bias, 1.f / tau, decay, T, n);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(gla_decay_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)z, ld_z, bias, 1.f / tau, decay, T, n);
  return TS_ERR_BAD_ARGUMENT;
}

// Floats of scratch that a scan of B sequences in `segs` segments each needs.
TS_EXPORT long long ts_gla_scan_scratch_floats(int B, int segs, int H, int d, int e) {
  if (segs <= 1) return 0;
  return (long long)B * segs * H * d * e + (long long)B * segs * H * d + (long long)B * H * d * e;
}

// q, k [T, H*d] and v [T, H*e] are views with the common row stride ld_qkv (columns of one product's
// result); decay [T, H*d] float32 (gla_decay); state [slots, H, d, e] float32; o [T, H*e] float32.
// segs > 1: every sequence's tokens of the step are cut into segments of seg_len tokens (segs * seg_len
// covers the longest) that run side by side, through `scratch` (ts_gla_scan_scratch_floats); two launches.
// segs == 1: seg_len is the longest portion of the step where the caller knows it, else 0; 1 (every sequence
// brings one token at most) runs the kernel that stages nothing.
TS_EXPORT int ts_gla_scan(const void* q, const void* k, const void* v, long long ld_qkv, int act_dtype, const float* decay, float q_scale,
                          float* state, const int* state_slots, const int* cu_seqlens, float* o, int B, int H, int d, int e, int segs,
                          int seg_len, float* scratch, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || d <= 0 || e <= 0 || segs < 1 || (segs > 1 && (seg_len < 1 || scratch == nullptr))) return TS_ERR_BAD_ARGUMENT;
  if ((long long)B * segs > 0x7fffffffLL) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const GlaExtra x = {nullptr, 0, H, e, (long long)H * d * e};
  if (act_dtype == TS_DTYPE_F32)
    return dispatch_gla_scan<float>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, segs, seg_len, scratch, s, x);
  if (act_dtype == TS_DTYPE_BF16)
    return dispatch_gla_scan<__nv_bfloat16>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, segs, seg_len,
                                            scratch, s, x);
  return TS_ERR_BAD_ARGUMENT;
}

// The same recurrence in its general form, for mixers whose decay is one number per (token, head):
//   S_t = a_t S_(t-1) + (b_t k_t) v_t^T,   o_t = S_t^T (q_t * q_scale)
// decay = a [T, H] float32 (`decay_scalar` = 1; 0: [T, H*d] as above); kscale = b [T, H] float32 or null;
// q, k [T, groups*d] (head h reads group h / (H / groups)) and v [T, H*ev], views with the common row
// stride ld_qkv; the state of a request starts `slot_stride` floats after the one before it and holds
// [H, d, e] with e = ev or ev + 1: a column beyond v's sees the value 1 in every token, so that it
// carries sum_t (products of decays) b_t k_t, the normaliser of a matrix memory, and its read-out
// n_t . q_t arrives as column ev of o [T, H*e].
TS_EXPORT int ts_linear_scan(const void* q, const void* k, const void* v, long long ld_qkv, int act_dtype, const float* decay,
                             int decay_scalar, const float* kscale, float q_scale, float* state, long long slot_stride, const int* state_slots,
                             const int* cu_seqlens, float* o, int B, int H, int groups, int d, int ev, int e, int segs, int seg_len,
                             float* scratch, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || d <= 0 || ev <= 0 || (e != ev && e != ev + 1) || groups <= 0 || H % groups || segs < 1 ||
      (segs > 1 && (seg_len < 1 || scratch == nullptr)) || slot_stride < (long long)H * d * e)
    return TS_ERR_BAD_ARGUMENT;
  if ((long long)B * segs > 0x7fffffffLL) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const GlaExtra x = {kscale, decay_scalar ? 1 : 0, groups, ev, slot_stride};
  if (act_dtype == TS_DTYPE_F32)
    return dispatch_gla_scan<float>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, segs, seg_len, scratch, s, x);
  if (act_dtype == TS_DTYPE_BF16)
    return dispatch_gla_scan<__nv_bfloat16>(q, k, v, ld_qkv, decay, q_scale, state, state_slots, cu_seqlens, o, B, H, d, e, segs, seg_len,
                                            scratch, s, x);
  return TS_ERR_BAD_ARGUMENT;
}

// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * w * silu(g[t, h, :]); one warp per (token, head).
template <typename TA>
__global__ void gla_norm_gate_kernel(const float* __restrict__ o, const TA* __restrict__ g, long long ld_g, const float* __restrict__ w,
                                     TA* __restrict__ out, int T, int H, int e, float eps) {
  ts_pdl_prologue();
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item - (long long)t * H);
  const float* row = o + ((size_t)t * H + h) * e;
  float ss = 0.f;
  for (int i = lane; i < e; i += 32) ss += row[i] * row[i];
  ss = ts_warp_sum(ss);
  const float rstd = 1.f / sqrtf(ss / (float)e + eps);
  const TA* grow = g + (size_t)t * ld_g + (size_t)h * e;
  TA* orow = out + ((size_t)t * H + h) * e;
  for (int i = lane; i < e; i += 32) {
    const float gate = ts_to_float(grow[i]);
    orow[i] = ts_from_float<TA>(row[i] * rstd * w[i] * (gate / (1.f + expf(-gate))));
  }
}

TS_EXPORT int ts_gla_norm_gate(const float* o, const void* g, long long ld_g, int act_dtype, const float* w, void* out, int T, int H, int e,
                               float eps, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || e <= 0) return TS_ERR_BAD_ARGUMENT;
  const long long items = (long long)T * H;
  const unsigned blocks = (unsigned)((items + 3) / 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(gla_norm_gate_kernel<float>, dim3(blocks), dim3(128), 0, s, o, (const float*)g, ld_g, w, (float*)out, T, H, e, eps);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(gla_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, s, o, (const __nv_bfloat16*)g, ld_g, w,
                     (__nv_bfloat16*)out, T, H, e, eps);
  return TS_ERR_BAD_ARGUMENT;
}
