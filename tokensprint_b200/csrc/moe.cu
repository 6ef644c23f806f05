// A feed-forward of routed experts, for any sizes and both element types, without a trip to the
// host: every grid is sized from the step's token count alone.
//
//   router_topk : per token, from float32 router logits (+ a bias per expert, if given): the `top`
//                 largest logits (the lower index wins a tie) with their experts; their weights are
//                 sigmoid(logit), handed on as they are or divided by their sum (`renormalize`), or
//                 the softmax over the chosen logits alone (`score_mode`); or, with the softmax over all
//                 logits as scores, the `top` largest of score + correction (a number per expert that
//                 steers the choice only) with the scores themselves as weights.
//   moe_plan    : the (token, choice) pairs sorted by expert: offsets[e] .. offsets[e+1] are expert
//                 e's places in `order` (pair indices), tile_offsets[e] its first row tile of
//                 `tile_rows` places (64 for the kernels here, more for the tensor-core ones).
//   moe_gate_up : for the pairs of each expert, rows x[token] * weight(pair) times the expert's gate
//                 and up matrices, then the gated activation (`act_mode`): with a = min(g, limit),
//                 b = clamp(u, -limit, limit), a * sigmoid(alpha a) * (b + 1); or silu(g) * u
//                                                                  -> act[place, I]
//   moe_down    : act[place] times the expert's down matrix       -> pair_out[pair, N]
//                 Experts without a gate matrix (`act_mode` gelu, gate null): gelu(u) alone.
//   moe_combine : out[t] = sum over the token's pairs (each times its weight, if weights are given)
//                 (+ shared[t]), summed in float32 in the order of the choices.  A chosen index at or
//                 beyond `E` (given with `ids`) is an identity expert: it has no matrices and no place
//                 in the plan, and its output is the token's input row x[t] itself.
//
// The two products are FFMA tiles of 64 x 64 with float32 sums over k in increasing order: a
// pair's result does not depend on its place inside its expert's rows, so the order in which the
// plan happens to list an expert's pairs changes nothing.
#include "common.cuh"
#include "moe_act.cuh"

#define MOE_BM 64
#define MOE_BN 64
#define MOE_BK 16
#define MOE_MAX_EXPERTS 4096


// The choice of one token by one warp: logits z [E] (shared or global memory), the bias already in.
__device__ __forceinline__ void router_choose(float* z, int E, int top, int renormalize, int score_mode, int* my_ids, float* my_w,
                                              int lane, const float* __restrict__ correction) {
  if (score_mode == ROUTER_SCORE_SOFTMAX_ALL) {
    // z becomes the softmax over all experts; the choice below then runs over z + correction
    float mx = -INFINITY, sum = 0.f;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = ts_warp_max(mx);
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - mx);
    sum = ts_warp_sum(sum);
    for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - mx) / sum;
    __syncwarp();
  }
  float total = 0.f, first = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= (my_ids[j] == e);
      const float v = z[e] + (correction ? correction[e] : 0.f);
      if (!taken && (v > best || (v == best && e < best_e))) {
        best = v;
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) {
        best = ov;
        best_e = oe;
      }
    }
    if (k == 0) first = best;  // the largest logit: the softmax's reference point
    const float score = score_mode == ROUTER_SCORE_SOFTMAX_ALL ? z[best_e < E ? best_e : 0]
                      : score_mode == ROUTER_SCORE_SOFTMAX_CHOSEN ? expf(best - first) : 1.f / (1.f + expf(-best));
    total += score;
    if (lane == 0) {
      my_ids[k] = best_e < E ? best_e : 0;
      my_w[k] = score;
    }
    __syncwarp();
  }
  if ((renormalize || score_mode == ROUTER_SCORE_SOFTMAX_CHOSEN) && lane == 0)
    for (int k = 0; k < top; ++k) my_w[k] /= total;
}

__global__ void router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int top, int renormalize,
                                   int score_mode, int* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ correction) {
  ts_pdl_prologue();
  extern __shared__ float zs[];  // [4][E]: a token's logits with the bias added
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp = blockIdx.x * (blockDim.x >> 5) + w;
  if (warp >= T) return;
  float* z = zs + (size_t)w * E;
  for (int e = lane; e < E; e += 32) z[e] = logits[(size_t)warp * E + e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  router_choose(z, E, top, renormalize, score_mode, ids + (size_t)warp * top, weights + (size_t)warp * top, lane, correction);
}

TS_EXPORT int ts_router_topk(const float* logits, const float* bias, int T, int E, int top, int renormalize, int score_mode, int* ids,
                             float* weights, const float* correction, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E) return TS_ERR_BAD_ARGUMENT;
  if ((size_t)4 * E * sizeof(float) > 48 * 1024) return TS_ERR_UNSUPPORTED_SIZE;
  return ts_launch(router_topk_kernel, dim3((T + 3) / 4), dim3(128), (size_t)4 * E * sizeof(float), (cudaStream_t)stream, logits, bias, T, E,
                   top, renormalize, score_mode, ids, weights, correction);
}

// One block: counts per expert, their prefix sums, then every pair takes the next place of its expert.
__global__ void moe_plan_kernel(const int* __restrict__ ids, int P, int E, int tile_rows, int* __restrict__ offsets,
                                int* __restrict__ tile_offsets, int* __restrict__ order) {
  ts_pdl_prologue();
  extern __shared__ int sm[];
  int* count = sm;           // [E]
  int* cursor = sm + E;      // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = rows;
      tile_offsets[e] = tiles;
      cursor[e] = rows;
      rows += count[e];
      tiles += (count[e] + tile_rows - 1) / tile_rows;
    }
    offsets[E] = rows;
    tile_offsets[E] = tiles;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) order[atomicAdd(&cursor[e], 1)] = i;
  }
}

TS_EXPORT int ts_moe_plan(const int* ids, int P, int E, int tile_rows, int* offsets, int* tile_offsets, int* order, void* stream) {
  if (P <= 0) return 0;
  if (tile_rows <= 0) return TS_ERR_BAD_ARGUMENT;
  if (E <= 0 || E > MOE_MAX_EXPERTS) return TS_ERR_UNSUPPORTED_SIZE;
  return ts_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), (cudaStream_t)stream, ids, P, E, tile_rows, offsets,
                   tile_offsets, order);
}

// Which expert a row tile belongs to: the last e with tile_offsets[e] <= tile.
__device__ __forceinline__ int moe_tile_expert(const int* __restrict__ tile_offsets, int E, int tile) {
  int lo = 0, hi = E;  // invariant: tile_offsets[lo] <= tile < tile_offsets[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_offsets[mid] <= tile) lo = mid; else hi = mid;
  }
  return lo;
}

template <typename TA>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const TA* __restrict__ x, const float* __restrict__ pair_weight,
                                                          const int* __restrict__ order, const int* __restrict__ offsets,
                                                          const int* __restrict__ tile_offsets, const TA* __restrict__ gate,
                                                          const TA* __restrict__ up, TA* __restrict__ act, int E, int K, int I, int top,
                                                          float limit, float alpha, int act_mode) {
  ts_pdl_prologue();
  __shared__ float As[MOE_BK][MOE_BM + 1];
  __shared__ float Gs[MOE_BK][MOE_BN + 1];
  __shared__ float Us[MOE_BK][MOE_BN + 1];
  __shared__ int src_row[MOE_BM];
  __shared__ float src_scale[MOE_BM];
  const int tile = blockIdx.y;
  if (tile >= tile_offsets[E]) return;
  const int e = moe_tile_expert(tile_offsets, E, tile);
  const int row0 = offsets[e] + (tile - tile_offsets[e]) * MOE_BM, row_end = offsets[e + 1];
  const int n0 = blockIdx.x * MOE_BN;
  for (int r = threadIdx.x; r < MOE_BM; r += 256) {
    const int place = row0 + r;
    const int pair = place < row_end ? order[place] : -1;
    src_row[r] = pair < 0 ? -1 : pair / top;
    src_scale[r] = pair < 0 ? 0.f : pair_weight[pair];
  }
  __syncthreads();
  const TA* G = gate + (size_t)e * I * K;
  const TA* U = up + (size_t)e * I * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float accg[4][4] = {}, accu[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += MOE_BK) {
    for (int i = threadIdx.x; i < MOE_BM * MOE_BK; i += 256) {
      const int r = i / MOE_BK, c = i % MOE_BK;
      const int gk = k0 + c, gn = n0 + r, sr = src_row[r];
      As[c][r] = (sr >= 0 && gk < K) ? ts_to_float(x[(size_t)sr * K + gk]) * src_scale[r] : 0.f;
      const bool w_ok = gn < I && gk < K;
      Gs[c][r] = (w_ok && gate != nullptr) ? ts_to_float(G[(size_t)gn * K + gk]) : 0.f;
      Us[c][r] = w_ok ? ts_to_float(U[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_BK; ++k) {
      float a[4], g[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        g[j] = Gs[k][tx * 4 + j];
        u[j] = Us[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          accg[i][j] = fmaf(a[i], g[j], accg[i][j]);
          accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int place = row0 + ty * 4 + i;
    if (place >= row_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= I) continue;
      // the sums are rounded to the element type first, as a product stored to memory would be
      const float gv = ts_to_float(ts_from_float<TA>(accg[i][j])), uv = ts_to_float(ts_from_float<TA>(accu[i][j]));
      act[(size_t)place * I + gn] = ts_from_float<TA>(moe_gated_activation(act_mode, gv, uv, limit, alpha));
    }
  }
}

template <typename TA>
__global__ void __launch_bounds__(256) moe_down_kernel(const TA* __restrict__ act, const int* __restrict__ order,
                                                       const int* __restrict__ offsets, const int* __restrict__ tile_offsets,
                                                       const TA* __restrict__ down, TA* __restrict__ pair_out, int E, int I, int N) {
  ts_pdl_prologue();
  __shared__ float As[MOE_BK][MOE_BM + 1];
  __shared__ float Ws[MOE_BK][MOE_BN + 1];
  const int tile = blockIdx.y;
  if (tile >= tile_offsets[E]) return;
  const int e = moe_tile_expert(tile_offsets, E, tile);
  const int row0 = offsets[e] + (tile - tile_offsets[e]) * MOE_BM, row_end = offsets[e + 1];
  const int n0 = blockIdx.x * MOE_BN;
  const TA* W = down + (size_t)e * N * I;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < I; k0 += MOE_BK) {
    for (int i = threadIdx.x; i < MOE_BM * MOE_BK; i += 256) {
      const int r = i / MOE_BK, c = i % MOE_BK;
      const int gk = k0 + c, gn = n0 + r, place = row0 + r;
      As[c][r] = (place < row_end && gk < I) ? ts_to_float(act[(size_t)place * I + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < I) ? ts_to_float(W[(size_t)gn * I + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MOE_BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int place = row0 + ty * 4 + i;
    if (place >= row_end) continue;
    const size_t pair = (size_t)order[place];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) pair_out[pair * N + gn] = ts_from_float<TA>(acc[i][j]);
    }
  }
}

TS_EXPORT int ts_moe_gate_up(const void* x, int act_dtype, const float* pair_weight, const int* order, const int* offsets,
                             const int* tile_offsets, const void* gate, const void* up, void* act, int P, int E, int K, int I, int top,
                             float limit, float alpha, int act_mode, void* stream) {
  if (P <= 0) return 0;
  if (E <= 0 || K <= 0 || I <= 0 || top <= 0 || ((gate == nullptr) != (act_mode == MOE_ACT_GELU))) return TS_ERR_BAD_ARGUMENT;
  const dim3 grid((I + MOE_BN - 1) / MOE_BN, (P + MOE_BM - 1) / MOE_BM + E);
  if (grid.y > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(moe_gate_up_kernel<float>, grid, dim3(256), 0, s, (const float*)x, pair_weight, order, offsets, tile_offsets,
                     (const float*)gate, (const float*)up, (float*)act, E, K, I, top, limit, alpha, act_mode);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(moe_gate_up_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x, pair_weight, order, offsets,
                     tile_offsets, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)act, E, K, I, top, limit, alpha, act_mode);
  return TS_ERR_BAD_ARGUMENT;
}

TS_EXPORT int ts_moe_down(const void* act, int act_dtype, const int* order, const int* offsets, const int* tile_offsets, const void* down,
                          void* pair_out, int P, int E, int I, int N, void* stream) {
  if (P <= 0) return 0;
  if (E <= 0 || I <= 0 || N <= 0) return TS_ERR_BAD_ARGUMENT;
  const dim3 grid((N + MOE_BN - 1) / MOE_BN, (P + MOE_BM - 1) / MOE_BM + E);
  if (grid.y > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(moe_down_kernel<float>, grid, dim3(256), 0, s, (const float*)act, order, offsets, tile_offsets, (const float*)down,
                     (float*)pair_out, E, I, N);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(moe_down_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)act, order, offsets, tile_offsets,
                     (const __nv_bfloat16*)down, (__nv_bfloat16*)pair_out, E, I, N);
  return TS_ERR_BAD_ARGUMENT;
}

template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ pair_out, const TA* __restrict__ shared, TA* __restrict__ out,
                                   const float* __restrict__ pair_weight, int N, int top, size_t total, const int* __restrict__ ids, int E,
                                   const TA* __restrict__ x) {
  ts_pdl_prologue();
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / N;
  const int n = (int)(idx - t * N);
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    const bool identity = ids != nullptr && ids[t * top + k] >= E;  // no expert ran for this pair: its output is the input row
    const float v = identity ? ts_to_float(x[idx]) : ts_to_float(pair_out[(t * top + k) * N + n]);
    sum += v * (pair_weight ? pair_weight[t * top + k] : 1.f);
  }
  if (shared) sum += ts_to_float(shared[idx]);
  out[idx] = ts_from_float<TA>(sum);
}

TS_EXPORT int ts_moe_combine(const void* pair_out, const void* shared, void* out, const float* pair_weight, int act_dtype, int T, int N,
                             int top, const int* ids, int E, const void* x, void* stream) {
  if (T <= 0) return 0;
  if (N <= 0 || top <= 0 || (ids != nullptr && x == nullptr)) return TS_ERR_BAD_ARGUMENT;
  const size_t total = (size_t)T * N;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(moe_combine_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)pair_out, (const float*)shared, (float*)out, pair_weight, N, top, total, ids, E, (const float*)x);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(moe_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, s, (const __nv_bfloat16*)pair_out,
                     (const __nv_bfloat16*)shared, (__nv_bfloat16*)out, pair_weight, N, top, total, ids, E, (const __nv_bfloat16*)x);
  return TS_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------
// The router in one kernel: float32 logits of RT tokens against every expert's row, then the
// choice.  A block keeps its tokens' rows in shared memory as float32 (they come as the float32
// residual rows or as their rounding in the compute type) and every warp walks expert rows with
// 16-byte loads, so a router row is read once per RT tokens.  A logit's sum runs over the width
// in a fixed order (lane-strided partial sums, then the warp's tree): it does not depend on the
// tokens beside it, nor on how many tokens a CTA takes.
#define ROUTER_MAX_TOKENS 4

template <typename TX>
__global__ void __launch_bounds__(256) router_kernel(const TX* __restrict__ x, const float* __restrict__ router,
                                                     const float* __restrict__ bias, int T, int W, int E, int top, int renormalize,
                                                     int score_mode, int rt, int* __restrict__ ids, float* __restrict__ weights,
                                                     const float* __restrict__ correction) {
  ts_pdl_prologue();
  extern __shared__ float rs[];
  float* xs = rs;                    // [rt][W]
  float* logits = rs + (size_t)rt * W;  // [rt][E]
  const int t0 = blockIdx.x * rt;
  const int nt = min(rt, T - t0);
  for (int i = threadIdx.x; i < nt * W; i += blockDim.x) xs[i] = ts_to_float(x[(size_t)t0 * W + i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    const float* row = router + (size_t)e * W;
    float acc[ROUTER_MAX_TOKENS] = {0.f, 0.f, 0.f, 0.f};
    if ((W & 3) == 0) {  // 16-byte loads, several in flight: a step of few tokens is a chain of such loads and little else
      const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 8
      for (int k = lane; k < (W >> 2); k += 32) {
        const float4 w = row4[k];
#pragma unroll
        for (int j = 0; j < ROUTER_MAX_TOKENS; ++j)
          if (j < nt) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)j * W + 4 * k);
            acc[j] = fmaf(xv.x, w.x, acc[j]);
            acc[j] = fmaf(xv.y, w.y, acc[j]);
            acc[j] = fmaf(xv.z, w.z, acc[j]);
            acc[j] = fmaf(xv.w, w.w, acc[j]);
          }
      }
    } else {
      for (int k = lane; k < W; k += 32) {
        const float w = row[k];
#pragma unroll
        for (int j = 0; j < ROUTER_MAX_TOKENS; ++j)
          if (j < nt) acc[j] = fmaf(xs[(size_t)j * W + k], w, acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_TOKENS; ++j) {
      const float v = ts_warp_sum(acc[j]);
      if (lane == 0 && j < nt) logits[(size_t)j * E + e] = v + (bias ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (warp >= nt) return;
  router_choose(logits + (size_t)warp * E, E, top, renormalize, score_mode, ids + (size_t)(t0 + warp) * top,
                weights + (size_t)(t0 + warp) * top, lane, correction);
}

TS_EXPORT int ts_router(const void* x, int x_dtype, const float* router, const float* bias, int T, int W, int E, int top, int renormalize,
                        int score_mode, int* ids, float* weights, const float* correction, void* stream) {
  if (T <= 0) return 0;
  if (W <= 0 || E <= 0 || top <= 0 || top > E) return TS_ERR_BAD_ARGUMENT;
  // tokens per CTA: four where there are CTAs enough for every SM several times over (a router row is
  // then read once per four tokens), fewer in steps of few tokens (more CTAs, shorter chains of loads)
  int rt = T >= 2048 ? ROUTER_MAX_TOKENS : (T >= 512 ? 2 : 1);
  while (rt > 1 && (size_t)rt * (W + E) * sizeof(float) > 200 * 1024) rt >>= 1;
  const size_t smem = (size_t)rt * (W + E) * sizeof(float);
  if (smem > 227 * 1024) return TS_ERR_UNSUPPORTED_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((T + rt - 1) / rt);
  if (x_dtype == TS_DTYPE_F32) {
    static size_t set32 = 0;
    if (smem > 48 * 1024 && smem > set32) {
      cudaError_t e = cudaFuncSetAttribute(router_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024));
      if (e != cudaSuccess) return (int)e;
      set32 = 227 * 1024;
    }
    return ts_launch(router_kernel<float>, grid, dim3(256), smem, s, (const float*)x, router, bias, T, W, E, top, renormalize, score_mode, rt, ids, weights, correction);
  }
  if (x_dtype == TS_DTYPE_BF16) {
    static size_t set16 = 0;
    if (smem > 48 * 1024 && smem > set16) {
      cudaError_t e = cudaFuncSetAttribute(router_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(227 * 1024));
      if (e != cudaSuccess) return (int)e;
      set16 = 227 * 1024;
    }
    return ts_launch(router_kernel<__nv_bfloat16>, grid, dim3(256), smem, s, (const __nv_bfloat16*)x, router, bias, T, W, E, top, renormalize,
                     score_mode, rt, ids, weights, correction);
  }
  return TS_ERR_BAD_ARGUMENT;
}
