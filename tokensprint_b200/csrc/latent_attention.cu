// Latent attention: what is cached per token is one row [c ; r], the normed low-rank latent c
// (`rank` entries) and one rotated key part r (`rot` entries) that all heads share.  Head a's key
// is [U_k,a c ; r] and its value U_v,a c, so with q'_a = U_k,a^T q_a (the "absorbed" query)
//
//   score_a(t, j) = (q'_a(t) . c(j) + q_rot,a(t) . r(j)) * scale,   o'_a(t) = sum_j p_a(t, j) c(j),
//
// and the head's output is U_v,a o'_a(t): every head reads the same cached rows, as keys over all
// rank + rot entries and as values over the first `rank`.
//
// Two kernels here, both for any sizes and both element types:
//   latent_prepare: per token, from the stacked projection [q heads | latent and key part | gate
//     logits]: RMS norm of the latent, rotation of the key part and of every head's rotated
//     query part (angles, sines and cosines in float32), store of [c ; r] into the cache by slot,
//     rotated query parts into the absorbed-query buffer, sigmoid of the gate logits.  Cosines and
//     sines may carry a `magnitude` (stretched frequencies come with one).  The queries may come
//     from a tensor of their own (`q_src`: a layer whose queries pass a latent first), and a layer
//     that reads another layer's cached rows has no latent of its own (`kv_off` < 0: queries only).
//   latent_attention_simple: CUDA cores, one warp per (token, head), scores, softmax and sums in
//     float32: the float32 path's attention and the yardstick of the tensor-core kernel.
#include "common.cuh"

#define LAT_PAIR_HALF 0         // entry j turns with entry j + dims/2
#define LAT_PAIR_NEIGHBOURS 1   // entry 2i turns with entry 2i + 1

#define LAT_MAX_PAIRS 512

// One entry of a rotated vector: x[j] after the turn by the token's angle of its pair, whose
// cosine and sine are cs[pair].
template <typename TA>
__device__ __forceinline__ float lat_rotated(const TA* __restrict__ x, int j, int dims, int pairing, const float2* __restrict__ cs) {
  const float v = ts_to_float(x[j]);
  if (j >= dims) return v;  // behind the rotated entries
  int pair, partner;
  bool first;
  if (pairing == LAT_PAIR_NEIGHBOURS) {
    pair = j >> 1;
    first = (j & 1) == 0;
    partner = j ^ 1;
  } else {
    const int half = dims >> 1;
    first = j < half;
    pair = first ? j : j - half;
    partner = first ? j + half : j - half;
  }
  const float w = ts_to_float(x[partner]);
  return first ? v * cs[pair].x - w * cs[pair].y : v * cs[pair].x + w * cs[pair].y;
}

template <typename TA>
__global__ void latent_prepare_kernel(const TA* __restrict__ proj, long long ld, int q_off, int kv_off, int gate_off,
                                      TA* __restrict__ q_abs, TA* __restrict__ cache, const int* __restrict__ slot_mapping,
                                      const int* __restrict__ positions, const float* __restrict__ latent_weight, float eps,
                                      const float* __restrict__ inv_freq, int rot_dims, int pairing, float* __restrict__ gates,
                                      int H, int nope, int rot, int rank, float magnitude, const TA* __restrict__ q_src, long long ld_q) {
  ts_pdl_prologue();
  __shared__ float scratch[33];
  __shared__ float2 cs[LAT_MAX_PAIRS];  // (cos, sin) of the token's angles, shared by the key part and every head
  const int t = blockIdx.x;
  const TA* row = proj + (size_t)t * ld;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < (rot_dims >> 1); i += blockDim.x) {
    float sn, c;
    sincosf(pos * inv_freq[i], &sn, &c);
    cs[i] = make_float2(c * magnitude, sn * magnitude);
  }  // the block-wide sum below has a barrier before anyone reads the table
  const int slot = (slot_mapping && kv_off >= 0) ? slot_mapping[t] : -1;
  const int key_dim = rank + rot;
  // the latent: RMS norm with a plain weight
  const TA* lat = row + (kv_off >= 0 ? kv_off : 0);
  float ss = 0.f;
  if (kv_off >= 0)
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
      const float v = ts_to_float(lat[i]);
      ss += v * v;
    }
  ss = ts_block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)rank + eps);
  if (slot >= 0) {
    TA* dst = cache + (size_t)slot * key_dim;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = ts_from_float<TA>(ts_to_float(lat[i]) * rstd * latent_weight[i]);
    for (int j = threadIdx.x; j < rot; j += blockDim.x)
      dst[rank + j] = ts_from_float<TA>(lat_rotated(lat + rank, j, rot_dims, pairing, cs));
  }
  // every head's rotated query part, behind the place of its absorbed part
  for (int i = threadIdx.x; i < H * rot; i += blockDim.x) {
    const int a = i / rot, j = i - a * rot;
    const TA* qr = (q_src ? q_src + (size_t)t * ld_q : row + q_off) + (size_t)a * (nope + rot) + nope;
    q_abs[((size_t)t * H + a) * key_dim + rank + j] = ts_from_float<TA>(lat_rotated(qr, j, rot_dims, pairing, cs));
  }
  if (gates)
    for (int a = threadIdx.x; a < H; a += blockDim.x) gates[(size_t)t * H + a] = 1.f / (1.f + expf(-ts_to_float(row[gate_off + a])));
}

TS_EXPORT int ts_latent_prepare(const void* proj, int act_dtype, long long ld, int q_off, int kv_off, int gate_off, void* q_abs,
                                void* cache, const int* slot_mapping, const int* positions, const float* latent_weight, float eps,
                                const float* inv_freq, int rot_dims, int pairing, float* gates, int T, int H, int nope, int rot,
                                int rank, float magnitude, const void* q_src, long long ld_q, void* stream) {
  if (T <= 0) return 0;
  if (rot_dims > 2 * LAT_MAX_PAIRS) return TS_ERR_UNSUPPORTED_SIZE;
  if (H <= 0 || nope < 0 || rot < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || (rot_dims > 0 && !inv_freq) ||
      (pairing != LAT_PAIR_HALF && pairing != LAT_PAIR_NEIGHBOURS) || (kv_off < 0 && cache != nullptr) || (proj == nullptr && (q_src == nullptr || kv_off >= 0 || gates)))
    return TS_ERR_BAD_ARGUMENT;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 128;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(latent_prepare_kernel<float>, dim3(T), dim3(threads), 0, s, (const float*)proj, ld, q_off, kv_off, gate_off,
                     (float*)q_abs, (float*)cache, slot_mapping, positions, latent_weight, eps, inv_freq, rot_dims, pairing, gates, H,
                     nope, rot, rank, magnitude, (const float*)q_src, ld_q);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, s, (const __nv_bfloat16*)proj, ld, q_off, kv_off,
                     gate_off, (__nv_bfloat16*)q_abs, (__nv_bfloat16*)cache, slot_mapping, positions, latent_weight, eps, inv_freq,
                     rot_dims, pairing, gates, H, nope, rot, rank, magnitude, (const __nv_bfloat16*)q_src, ld_q);
  return TS_ERR_BAD_ARGUMENT;
}

// ---------------------------------------------------------------------------------------------

#define LAS_MAX_KEY_DIM 1024
#define LAS_MAX_RANK 1024
#define LAS_WARPS 4

// One warp per (token, head).  Keys are taken 32 at a time: each lane scores one cached row
// against the absorbed query (all rank + rot entries), the warp agrees on the running max, then
// all lanes walk the 32 rows together as values, each owning latent entries lane, lane + 32, ...
// The order of a query's sums depends on its own keys only.  `gates` (one factor per token and
// head, or null) multiplies the finished row.
template <typename TA>
__global__ void latent_attention_simple_kernel(const TA* __restrict__ q_abs, const TA* __restrict__ cache, TA* __restrict__ out,
                                               const float* __restrict__ gates, const int* __restrict__ positions,
                                               const int* __restrict__ seq_index, const int* __restrict__ block_table,
                                               int max_blocks, int page, int T, int H, int rank, int rot, float scale, int window) {
  ts_pdl_prologue();
  __shared__ float qs[LAS_WARPS][LAS_MAX_KEY_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * LAS_WARPS + warp;
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H);
  const int a = (int)(item - (long long)t * H);
  const int key_dim = rank + rot;
  TA* orow = out + ((size_t)t * H + a) * rank;
  const int b = seq_index[t];
  if (b < 0) {  // a padded lane of a fixed-size batch
    for (int i = lane; i < rank; i += 32) orow[i] = ts_from_float<TA>(0.f);
    return;
  }
  const int p = positions[t];
  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int* table = block_table + (size_t)b * max_blocks;
  const TA* qrow = q_abs + ((size_t)t * H + a) * key_dim;
  for (int i = lane; i < key_dim; i += 32) qs[warp][i] = ts_to_float(qrow[i]);
  __syncwarp();

  constexpr int ACC = LAS_MAX_RANK / 32;
  float acc[ACC];
#pragma unroll
  for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int base = lo; base <= p; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    size_t slot = 0;
    if (j <= p) {
      slot = (size_t)table[j / page] * page + (j % page);
      const TA* krow = cache + slot * key_dim;
      float dot = 0.f;
      for (int i = 0; i < key_dim; ++i) dot += qs[warp][i] * ts_to_float(krow[i]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, ts_warp_max(s));
    const float corr = expf(m - m_new);
    const float pj = (j <= p) ? expf(s - m_new) : 0.f;
    l = l * corr + ts_warp_sum(pj);
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] *= corr;
    const int n = min(32, p - base + 1);
    for (int kk = 0; kk < n; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pj, kk);
      const size_t sk = __shfl_sync(0xffffffffu, (unsigned long long)slot, kk);
      const TA* vrow = cache + sk * key_dim;
#pragma unroll
      for (int i = 0; i < ACC; ++i) {
        const int dim = lane + 32 * i;
        if (dim < rank) acc[i] += pk * ts_to_float(vrow[dim]);
      }
    }
    m = m_new;
  }
  const float f = (gates ? gates[(size_t)t * H + a] : 1.f) / l;
#pragma unroll
  for (int i = 0; i < ACC; ++i) {
    const int dim = lane + 32 * i;
    if (dim < rank) orow[dim] = ts_from_float<TA>(acc[i] * f);
  }
}

TS_EXPORT int ts_latent_attention_simple(const void* q_abs, const void* cache, int act_dtype, void* out, const float* gates,
                                         const int* positions, const int* seq_index, const int* block_table, int max_blocks,
                                         int page, int T, int H, int rank, int rot, float scale, int window, void* stream) {
  if (T <= 0) return 0;
  if (H <= 0 || rank <= 0 || rot < 0 || page <= 0 || max_blocks <= 0) return TS_ERR_BAD_ARGUMENT;
  if (rank + rot > LAS_MAX_KEY_DIM || rank > LAS_MAX_RANK) return TS_ERR_UNSUPPORTED_SIZE;
  const long long items = (long long)T * H;
  const unsigned blocks = (unsigned)((items + LAS_WARPS - 1) / LAS_WARPS);
  cudaStream_t s = (cudaStream_t)stream;
  if (act_dtype == TS_DTYPE_F32)
    return ts_launch(latent_attention_simple_kernel<float>, dim3(blocks), dim3(LAS_WARPS * 32), 0, s, (const float*)q_abs,
                     (const float*)cache, (float*)out, gates, positions, seq_index, block_table, max_blocks, page, T, H, rank, rot,
                     scale, window);
  if (act_dtype == TS_DTYPE_BF16)
    return ts_launch(latent_attention_simple_kernel<__nv_bfloat16>, dim3(blocks), dim3(LAS_WARPS * 32), 0, s,
                     (const __nv_bfloat16*)q_abs, (const __nv_bfloat16*)cache, (__nv_bfloat16*)out, gates, positions, seq_index,
                     block_table, max_blocks, page, T, H, rank, rot, scale, window);
  return TS_ERR_BAD_ARGUMENT;
}
