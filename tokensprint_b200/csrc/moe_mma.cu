// The two products of a routed feed-forward on the tensor cores (bfloat16, mma.sync m16n8k16,
// float32 sums), over the plan that moe.cu makes: the (token, choice) pairs sorted by expert, in
// row tiles (of 128 places, or of 16 in steps of few tokens) that never straddle two experts.
//
// A CTA takes one row tile and 128 weight rows: for the first product the gate rows and
// the up rows of the same 64 outputs (so the activation is the epilogue), for the second 128 rows
// of the down matrix.  Both operands stream through shared memory in slices of 64 along k, three
// slices in flight (16-byte cp.async); a row of A is the token's row (first product: found through
// the pair's index) or the pair's activation row (second).  The pair's routing weight multiplies
// the float32 sums, not the rounded input: (w x) . g = w (x . g) without a second rounding of x.
// Every output element is one chain of sums over k in a fixed order, whatever rows share the tile.
#include "common.cuh"
#include "moe_act.cuh"

namespace {

constexpr int NB = 128, BK = 64, KS = BK + 8;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ int tile_expert(const int* __restrict__ tile_offsets, int E, int tile) {
  int lo = 0, hi = E;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_offsets[mid] <= tile) lo = mid; else hi = mid;
  }
  return lo;
}

// WM x WN warps: a warp owns MT tiles of 16 rows and NB / WN of the 128 weight rows in shared memory
// (the more of both, the fewer shared-memory loads per MMA: MT + NT / 2 loads feed MT * NT MMAs).
// MODE 1 (gate and up): the first half of a warp's weight rows are gate rows and the second half the up
// rows of the same outputs (so both operands of an activation sit in one thread); else 128 rows of one
// matrix: MODE 0 the down product (rows of A by place, results by pair), MODE 2 the first product of
// experts without a gate (rows of A by the pair's token, the activation of the weighted sums by place).
template <int MODE, int WM, int WN, int MT, int STAGES>
__global__ void __launch_bounds__(32 * WM * WN) moe_mma_kernel(const __nv_bfloat16* __restrict__ A, const float* __restrict__ pair_weight,
                                                               const int* __restrict__ order, const int* __restrict__ offsets,
                                                               const int* __restrict__ tile_offsets, const __nv_bfloat16* __restrict__ B0,
                                                               const __nv_bfloat16* __restrict__ B1, __nv_bfloat16* __restrict__ out, int E,
                                                               int K, int NOUT, int top, float limit, float alpha, int act_mode) {
  constexpr bool GATE_UP = MODE == 1, BY_TOKEN = MODE != 0;
  constexpr int BM = 16 * MT * WM, THREADS = 32 * WM * WN, CW = NB / WN, HALF = CW / 2, NT = CW / 8;
  constexpr size_t STAGE_ELEMS = (size_t)(BM + NB) * KS;
  ts_pdl_prologue();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __shared__ const __nv_bfloat16* a_src[BM];
  __shared__ int a_pair[BM];
  const int tile = blockIdx.y;
  if (tile >= tile_offsets[E]) return;
  const int e = tile_expert(tile_offsets, E, tile);
  const int row0 = offsets[e] + (tile - tile_offsets[e]) * BM, row_end = offsets[e + 1];
  const int n0 = blockIdx.x * (GATE_UP ? NB / 2 : NB);
  for (int r = threadIdx.x; r < BM; r += THREADS) {
    const int place = row0 + r;
    const int pair = place < row_end ? order[place] : -1;
    a_pair[r] = pair;
    a_src[r] = pair < 0 ? nullptr : (BY_TOKEN ? A + (size_t)(pair / top) * K : A + (size_t)place * K);
  }
  __syncthreads();
  const __nv_bfloat16* W0 = B0 + (size_t)e * NOUT * K;
  const __nv_bfloat16* W1 = GATE_UP ? B1 + (size_t)e * NOUT * K : nullptr;

  auto load_stage = [&](int kt, int stage) {
    __nv_bfloat16* As = smem + (size_t)stage * STAGE_ELEMS;
    __nv_bfloat16* Bs = As + (size_t)BM * KS;
    const int k0 = kt * BK;
    for (int c = threadIdx.x; c < BM * (BK / 8); c += THREADS) {
      const int r = c >> 3, part = c & 7, k = k0 + part * 8;
      __nv_bfloat16* d = As + (size_t)r * KS + part * 8;
      if (a_src[r] != nullptr && k < K) cp_async16(d, a_src[r] + k);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int c = threadIdx.x; c < NB * (BK / 8); c += THREADS) {
      const int r = c >> 3, part = c & 7, k = k0 + part * 8;
      __nv_bfloat16* d = Bs + (size_t)r * KS + part * 8;
      const __nv_bfloat16* src;
      int n;
      if (GATE_UP) {
        const int within = r % CW;
        n = n0 + (r / CW) * HALF + within % HALF;
        src = (within < HALF ? W0 : W1) + (size_t)n * K;
      } else {
        n = n0 + r;
        src = W0 + (size_t)n * K;
      }
      if (n < NOUT && k < K) cp_async16(d, src + k);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  const int nk = (K + BK - 1) / BK;
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < nk) load_stage(s, s);
    cp_async_commit();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, quad = lane >> 2, qi = lane & 3;
  const int wm = warp / WN, wn = warp % WN;
  float acc[MT][NT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[m][i][0] = acc[m][i][1] = acc[m][i][2] = acc[m][i][3] = 0.f;

  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    if (kt + STAGES - 1 < nk) load_stage(kt + STAGES - 1, (kt + STAGES - 1) % STAGES);
    cp_async_commit();
    const __nv_bfloat16* As = smem + (size_t)(kt % STAGES) * STAGE_ELEMS + (size_t)wm * 16 * MT * KS;
    const __nv_bfloat16* Bs = smem + (size_t)(kt % STAGES) * STAGE_ELEMS + (size_t)BM * KS + (size_t)wn * CW * KS;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      unsigned a[MT][4];
#pragma unroll
      for (int m = 0; m < MT; ++m) ldmatrix_x4(a[m], As + (size_t)(m * 16 + (lane & 15)) * KS + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nb = 0; nb < NT / 2; ++nb) {
        unsigned b[4];
        ldmatrix_x4(b, Bs + (size_t)(nb * 16 + (lane >> 4) * 8 + (lane & 7)) * KS + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          mma_bf16(acc[m][2 * nb], a[m], b[0], b[1]);
          mma_bf16(acc[m][2 * nb + 1], a[m], b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int rl = (wm * MT + m) * 16 + quad + 8 * r;
      const int pair = a_pair[rl];
      if (pair < 0) continue;
      if (GATE_UP) {
        const float w = pair_weight[pair];
        __nv_bfloat16* dst = out + (size_t)(row0 + rl) * NOUT;
#pragma unroll
        for (int nb = 0; nb < NT / 2; ++nb) {
          const int n = n0 + wn * HALF + nb * 8 + 2 * qi;
          float y[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            // the sums are rounded to bfloat16 first, as a product stored to memory would be
            const float gv = __bfloat162float(__float2bfloat16_rn(w * acc[m][nb][2 * r + c]));
            const float uv = __bfloat162float(__float2bfloat16_rn(w * acc[m][nb + NT / 2][2 * r + c]));
            y[c] = moe_gated_activation(act_mode, gv, uv, limit, alpha);
          }
          if (n + 1 < NOUT && (NOUT & 1) == 0) {
            *reinterpret_cast<__nv_bfloat162*>(dst + n) = __floats2bfloat162_rn(y[0], y[1]);
          } else {
            if (n < NOUT) dst[n] = __float2bfloat16_rn(y[0]);
            if (n + 1 < NOUT) dst[n + 1] = __float2bfloat16_rn(y[1]);
          }
        }
      } else if (MODE == 2) {
        const float w = pair_weight[pair];
        __nv_bfloat16* dst = out + (size_t)(row0 + rl) * NOUT;
#pragma unroll
        for (int nb = 0; nb < NT; ++nb) {
          const int n = n0 + wn * CW + nb * 8 + 2 * qi;
          float y[2];
#pragma unroll
          for (int c = 0; c < 2; ++c)  // the sums are rounded to bfloat16 first, as a product stored to memory would be
            y[c] = moe_gated_activation(act_mode, 0.f, __bfloat162float(__float2bfloat16_rn(w * acc[m][nb][2 * r + c])), limit, alpha);
          if (n + 1 < NOUT && (NOUT & 1) == 0) {
            *reinterpret_cast<__nv_bfloat162*>(dst + n) = __floats2bfloat162_rn(y[0], y[1]);
          } else {
            if (n < NOUT) dst[n] = __float2bfloat16_rn(y[0]);
            if (n + 1 < NOUT) dst[n + 1] = __float2bfloat16_rn(y[1]);
          }
        }
      } else {
        __nv_bfloat16* dst = out + (size_t)pair * NOUT;
#pragma unroll
        for (int nb = 0; nb < NT; ++nb) {
          const int n = n0 + wn * CW + nb * 8 + 2 * qi;
          if (n + 1 < NOUT && (NOUT & 1) == 0) {
            *reinterpret_cast<__nv_bfloat162*>(dst + n) = __floats2bfloat162_rn(acc[m][nb][2 * r], acc[m][nb][2 * r + 1]);
          } else {
            if (n < NOUT) dst[n] = __float2bfloat16_rn(acc[m][nb][2 * r]);
            if (n + 1 < NOUT) dst[n + 1] = __float2bfloat16_rn(acc[m][nb][2 * r + 1]);
          }
        }
      }
    }
}

// Two shapes: many rows per expert (tiles of 128 rows, 2 x 4 warps of 64 rows x 32 weight rows each,
// 3 slices in flight) and few (tiles of 16 rows, 4 warps side by side over the 128 weight rows, 3 slices in
// flight, three CTAs per SM: the step then streams the chosen experts' weights and little else).
constexpr int ROWS_MANY = 128, ROWS_FEW = 16;

template <int MODE, int WM, int WN, int MT, int STAGES>
int launch(const void* A, const float* pair_weight, const int* order, const int* offsets, const int* tile_offsets, const void* B0,
           const void* B1, void* out, int P, int E, int K, int NOUT, int top, float limit, float alpha, int act_mode, cudaStream_t s) {
  constexpr int BM = 16 * MT * WM;
  constexpr size_t SMEM_BYTES = (size_t)STAGES * (BM + NB) * KS * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_mma_kernel<MODE, WM, WN, MT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int cols = MODE == 1 ? NB / 2 : NB;
  const dim3 grid((NOUT + cols - 1) / cols, (P + BM - 1) / BM + E);
  if (grid.y > 65535) return TS_ERR_UNSUPPORTED_SIZE;
  return ts_launch(moe_mma_kernel<MODE, WM, WN, MT, STAGES>, grid, dim3(32 * WM * WN), SMEM_BYTES, s, (const __nv_bfloat16*)A, pair_weight,
                   order, offsets, tile_offsets, (const __nv_bfloat16*)B0, (const __nv_bfloat16*)B1, (__nv_bfloat16*)out, E, K, NOUT, top,
                   limit, alpha, act_mode);
}

}  // namespace

// Places per row tile of the two shapes: what the plan's tile_offsets must be made for.
TS_EXPORT int ts_moe_mma_row_tile(int few_rows) { return few_rows ? ROWS_FEW : ROWS_MANY; }

// bfloat16 only; K (the inner width) must be a multiple of 8 and every base address 16-byte aligned;
// tile_rows: the row tile the plan was made for (one of the two above).
TS_EXPORT int ts_moe_gate_up_mma(const void* x, const float* pair_weight, const int* order, const int* offsets, const int* tile_offsets,
                                 const void* gate, const void* up, void* act, int P, int E, int K, int I, int top, float limit, float alpha,
                                 int act_mode, int tile_rows, void* stream) {
  if (P <= 0) return 0;
  if (E <= 0 || K <= 0 || I <= 0 || top <= 0 || (tile_rows != ROWS_MANY && tile_rows != ROWS_FEW)) return TS_ERR_BAD_ARGUMENT;
  if ((gate == nullptr) != (act_mode == MOE_ACT_GELU)) return TS_ERR_BAD_ARGUMENT;
  if (K % 8 || (((uintptr_t)x | (uintptr_t)gate | (uintptr_t)up) & 15)) return TS_ERR_UNSUPPORTED_SIZE;
  if (gate == nullptr) {  // experts without a gate matrix: 128 rows of the up matrix per CTA
    if (tile_rows == ROWS_MANY)
      return launch<2, 2, 4, 4, 3>(x, pair_weight, order, offsets, tile_offsets, up, nullptr, act, P, E, K, I, top, limit, alpha, act_mode, (cudaStream_t)stream);
    return launch<2, 1, 4, 1, 3>(x, pair_weight, order, offsets, tile_offsets, up, nullptr, act, P, E, K, I, top, limit, alpha, act_mode, (cudaStream_t)stream);
  }
  if (tile_rows == ROWS_MANY)
    return launch<1, 2, 4, 4, 3>(x, pair_weight, order, offsets, tile_offsets, gate, up, act, P, E, K, I, top, limit, alpha, act_mode, (cudaStream_t)stream);
  return launch<1, 1, 4, 1, 3>(x, pair_weight, order, offsets, tile_offsets, gate, up, act, P, E, K, I, top, limit, alpha, act_mode, (cudaStream_t)stream);
}

TS_EXPORT int ts_moe_down_mma(const void* act, const int* order, const int* offsets, const int* tile_offsets, const void* down,
                              void* pair_out, int P, int E, int I, int N, int tile_rows, void* stream) {
  if (P <= 0) return 0;
  if (E <= 0 || I <= 0 || N <= 0 || (tile_rows != ROWS_MANY && tile_rows != ROWS_FEW)) return TS_ERR_BAD_ARGUMENT;
  if (I % 8 || (((uintptr_t)act | (uintptr_t)down) & 15)) return TS_ERR_UNSUPPORTED_SIZE;
  if (tile_rows == ROWS_MANY)
    return launch<0, 2, 4, 4, 3>(act, nullptr, order, offsets, tile_offsets, down, nullptr, pair_out, P, E, I, N, 1, 0.f, 0.f, 0, (cudaStream_t)stream);
  return launch<0, 1, 4, 1, 3>(act, nullptr, order, offsets, tile_offsets, down, nullptr, pair_out, P, E, I, N, 1, 0.f, 0.f, 0, (cudaStream_t)stream);
}
