// QJL sign-sketch key quantizer and its GQA score estimator (the reference's `qjl` baseline method).
//
// quantize: keys come in groups of G tokens; per group a set of outlier channels is given.  For every
// token the sign bits of  S k_inlier  and  S k_outlier  (S = sketch_dim x 128 projection, k split by
// the outlier mask) are packed LSB-first, 8 per byte, plus the norm of the outlier part.
// score:    for a query q and a key sketched that way
//     score = sqrt(pi/2)/s * |k_in| * sum_p sgn_p * (qS - q_out S)_p  +  sqrt(pi/2)/s_o * |k_out| * sum_{p<s_o} sgn'_p * (q_out S)_p
// with q_out = q restricted to the group's outlier channels and |k_in| = sqrt(|k|^2 - |k_out|^2).
//
// quant_kernel and score_kernel are CUDA-core kernels: one CTA per (group, chunk of 32 tokens); thread =
// (token, block of 32 projections); the sign sums run over "bit set" terms only:
// sum_p sgn_p x_p = 2 sum_{bit_p} x_p - sum_p x_p.  They serve unaligned buffers and sketch dims that are
// not multiples of 128; otherwise quant_mma_kernel (persistent, projection resident in shared memory) and
// score_mma_kernel (sign sums on the warp MMA, several groups per CTA) run.
#include "cq_common.cuh"
#include "cq_ptx.cuh"

namespace cq {
namespace qjl {

constexpr int WARPS = 8, THREADS = WARPS * 32;
constexpr int MAX_SKETCH = 256;       // projections per token handled by one CTA (32 per warp)
constexpr int D_CHUNK = 16;           // channels of the projection staged per step

template <typename TP> __device__ __forceinline__ float proj_f(TP v);
template <> __device__ __forceinline__ float proj_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float proj_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float proj_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// keys [groups][G][128], outlier_idx [groups][oc], proj [sketch][128] -> key_quant [groups][G][sketch/8],
// key_outlier_quant [groups][G][o_sketch/8], outlier_norm [groups][G]
template <typename T, typename TP>
__global__ void __launch_bounds__(THREADS)
quant_kernel(const T* __restrict__ keys, const uint8_t* __restrict__ outlier_idx, const TP* __restrict__ proj,
             uint8_t* __restrict__ key_quant, uint8_t* __restrict__ key_outlier_quant, T* __restrict__ outlier_norm,
             int G, int sketch, int o_sketch, int oc) {
  __shared__ float key_s[kHeadDim][33];            // [channel][token], padded
  __shared__ float proj_s[D_CHUNK][MAX_SKETCH];    // [channel in chunk][projection]
  __shared__ uint8_t mask_s[kHeadDim];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const int64_t grp = blockIdx.x;
  const int tok0 = blockIdx.y * 32;
  const int n_tok = min(32, G - tok0);
  if (tid < kHeadDim) mask_s[tid] = 0;
  __syncthreads();
  if (tid < oc) mask_s[outlier_idx[grp * oc + tid] & (kHeadDim - 1)] = 1;
  const T* kbase = keys + (grp * G + tok0) * kHeadDim;
  for (int i = tid; i < 32 * kHeadDim; i += THREADS) {
    const int t = i >> 7, d = i & (kHeadDim - 1);
    key_s[d][t] = t < n_tok ? Elem<T>::to_f(kbase[t * kHeadDim + d]) : 0.f;
  }
  float acc_in[32], acc_out[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) { acc_in[j] = 0.f; acc_out[j] = 0.f; }
  const int p0 = warp * 32;                         // this warp's projections
  for (int d0 = 0; d0 < kHeadDim; d0 += D_CHUNK) {
    __syncthreads();                                // previous chunk consumed (first pass: key_s, mask_s written)
    for (int i = tid; i < sketch * D_CHUNK; i += THREADS) {
      const int p = i / D_CHUNK, dd = i % D_CHUNK;
      proj_s[dd][p] = proj_f<TP>(proj[(int64_t)p * kHeadDim + d0 + dd]);
    }
    __syncthreads();
    if (p0 < sketch) {
#pragma unroll 4
      for (int dd = 0; dd < D_CHUNK; ++dd) {
        const float kv = key_s[d0 + dd][lane];
        const float4* pr = reinterpret_cast<const float4*>(&proj_s[dd][p0]);
        if (mask_s[d0 + dd]) {                      // uniform over the CTA
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = pr[j];
            acc_out[4 * j] = fmaf(v.x, kv, acc_out[4 * j]); acc_out[4 * j + 1] = fmaf(v.y, kv, acc_out[4 * j + 1]);
            acc_out[4 * j + 2] = fmaf(v.z, kv, acc_out[4 * j + 2]); acc_out[4 * j + 3] = fmaf(v.w, kv, acc_out[4 * j + 3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = pr[j];
            acc_in[4 * j] = fmaf(v.x, kv, acc_in[4 * j]); acc_in[4 * j + 1] = fmaf(v.y, kv, acc_in[4 * j + 1]);
            acc_in[4 * j + 2] = fmaf(v.z, kv, acc_in[4 * j + 2]); acc_in[4 * j + 3] = fmaf(v.w, kv, acc_in[4 * j + 3]);
          }
        }
      }
    }
  }
  if (lane < n_tok && p0 < sketch) {
    uint32_t w_in = 0, w_out = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      w_in |= (acc_in[j] > 0.f ? 1u : 0u) << j;
      w_out |= (acc_out[j] > 0.f ? 1u : 0u) << j;
    }
    const int64_t tok = grp * G + tok0 + lane;
    *reinterpret_cast<uint32_t*>(key_quant + tok * (sketch / 8) + p0 / 8) = w_in;
    if (p0 < o_sketch) *reinterpret_cast<uint32_t*>(key_outlier_quant + tok * (o_sketch / 8) + p0 / 8) = w_out;
  }
  if (warp == 0 && lane < n_tok) {
    float ss = 0.f;
    for (int d = 0; d < kHeadDim; ++d)
      if (mask_s[d]) ss = fmaf(key_s[d][lane], key_s[d][lane], ss);
    outlier_norm[grp * G + tok0 + lane] = Elem<T>::from_f(sqrtf(ss));
  }
}

// One CTA per (batch x KV head, group, chunk of 32 tokens).  R = query heads per KV head held per thread.
template <typename T, typename TP, int R>
__global__ void __launch_bounds__(THREADS)
score_kernel(const uint8_t* __restrict__ key_quant, const uint8_t* __restrict__ key_outlier_quant,
             const T* __restrict__ key_norm, const T* __restrict__ key_outlier_norm,
             const uint8_t* __restrict__ outlier_idx, const float* __restrict__ query_sketch,
             const T* __restrict__ query, const TP* __restrict__ proj_score, float* __restrict__ scores,
             int n_groups, int G, int n_rep, int sketch, int o_sketch, int oc) {
  __shared__ __align__(16) float qin_s[MAX_SKETCH][R];     // (q S - q_out S)_p per head
  __shared__ __align__(16) float qout_s[MAX_SKETCH][R];    // (q_out S)_p per head
  __shared__ float q_s[R][kHeadDim];
  __shared__ float part_s[WARPS][32][2 * R];
  __shared__ float tot_s[2][R];
  __shared__ uint8_t otl_s[kHeadDim];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const int64_t kbh = blockIdx.x;                           // batch * n_kv_heads + kv head
  const int n = blockIdx.y, tok0 = blockIdx.z * 32;
  const int n_tok = min(32, G - tok0);
  const int64_t qrow0 = kbh * n_rep;                        // first query head of this KV head
  const int64_t grp = kbh * n_groups + n;
  for (int i = tid; i < R * kHeadDim; i += THREADS) {
    const int r = i >> 7, d = i & (kHeadDim - 1);
    q_s[r][d] = r < n_rep ? Elem<T>::to_f(query[(qrow0 + r) * kHeadDim + d]) : 0.f;
  }
  if (tid < oc) otl_s[tid] = outlier_idx[grp * oc + tid] & (kHeadDim - 1);
  if (tid < 2 * R) tot_s[tid / R][tid % R] = 0.f;
  __syncthreads();
  // sketches of the query's outlier part and of the rest, per projection; their totals per head
  for (int p = tid; p < sketch; p += THREADS) {
    float o[R];
#pragma unroll
    for (int r = 0; r < R; ++r) o[r] = 0.f;
    for (int i = 0; i < oc; ++i) {
      const int d = otl_s[i];
      const float pv = proj_f<TP>(proj_score[(int64_t)d * sketch + p]);
#pragma unroll
      for (int r = 0; r < R; ++r) o[r] = fmaf(q_s[r][d], pv, o[r]);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float qs = r < n_rep ? query_sketch[(qrow0 + r) * sketch + p] : 0.f;
      qin_s[p][r] = qs - o[r];
      qout_s[p][r] = o[r];
    }
  }
  __syncthreads();
  // totals per head over the projections: (which, head) pairs dealt over the warps, lanes stride p
  for (int pr = warp; pr < 2 * R; pr += WARPS) {
    const int which = pr / R, r = pr % R;
    const int lim = which == 0 ? sketch : o_sketch;
    float t = 0.f;
    for (int p = lane; p < lim; p += 32) t += which == 0 ? qin_s[p][r] : qout_s[p][r];
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) tot_s[which][r] = t;
  }
  // set-bit sums of this warp's 32 projections for token `lane`
  float s_in[R], s_out[R];
#pragma unroll
  for (int r = 0; r < R; ++r) { s_in[r] = 0.f; s_out[r] = 0.f; }
  const int p0 = warp * 32;
  if (lane < n_tok && p0 < sketch) {
    const int64_t tok = grp * G + tok0 + lane;
    const uint32_t w_in = *reinterpret_cast<const uint32_t*>(key_quant + tok * (sketch / 8) + p0 / 8);
    const uint32_t w_out = p0 < o_sketch ? *reinterpret_cast<const uint32_t*>(key_outlier_quant + tok * (o_sketch / 8) + p0 / 8) : 0u;
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
      const bool b_in = (w_in >> k) & 1u, b_out = (w_out >> k) & 1u;
#pragma unroll
      for (int r4 = 0; r4 < R; r4 += 4) {
        const float4 a = *reinterpret_cast<const float4*>(&qin_s[p0 + k][r4]);
        const float4 b = *reinterpret_cast<const float4*>(&qout_s[p0 + k][r4]);
        if (b_in) { s_in[r4] += a.x; s_in[r4 + 1] += a.y; s_in[r4 + 2] += a.z; s_in[r4 + 3] += a.w; }
        if (b_out) { s_out[r4] += b.x; s_out[r4 + 1] += b.y; s_out[r4 + 2] += b.z; s_out[r4 + 3] += b.w; }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) { part_s[warp][lane][r] = s_in[r]; part_s[warp][lane][R + r] = s_out[r]; }
  __syncthreads();
  for (int i = tid; i < 32 * R; i += THREADS) {
    const int t = i / R, r = i % R;
    if (t >= n_tok || r >= n_rep) continue;
    float si = 0.f, so = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) { si += part_s[w][t][r]; so += part_s[w][t][R + r]; }
    const float inner = 2.f * si - tot_s[0][r], outer = 2.f * so - tot_s[1][r];
    const int64_t tok = grp * G + tok0 + t;
    const float norm_o = Elem<T>::to_f(key_outlier_norm[tok]);
    const float norm_k = Elem<T>::to_f(key_norm[tok]);
    // |k_in|: the two norms are rounded separately, so the difference can dip below zero
    const float norm_in = sqrtf(fmaxf(norm_k * norm_k - norm_o * norm_o, 0.f));
    const float scl = 1.2533141373155001f / (float)sketch, scl_o = 1.2533141373155001f / (float)o_sketch;
    scores[(qrow0 + r) * ((int64_t)n_groups * G) + (int64_t)n * G + tok0 + t] =
        scl * norm_in * inner + scl_o * norm_o * outer;
  }
}

// The same estimate on the warp MMA (sketch dims multiples of 128).
// One CTA walks GPC consecutive groups of one (batch, KV head); per group and chunk of 32 tokens:
//   1. thread = projection p: the query-side terms x_p = (q S - q_out S)_p and (q_out S)_p per head, stored as
//      fp16 pairs hi = fp16(x), lo = fp16(x - hi) in B-fragment order (the fp32 accumulator then holds the
//      fp32-rounded sum).  With at most four query heads per KV head hi and lo share the eight MMA columns,
//      otherwise two MMAs per step.
//   2. eight warp tasks = (16-token tile) x (inlier | outlier sketch) x (half of the projections):
//      A = the signs of 16 tokens x 16 projections as +-2^-24 (fp16 subnormal with the sign bit from the
//      packed bit), so the MMA sums  sgn_p x_p  directly.
//   3. thread = (token, head): norms, scale, store.
// The B fragments and the partial sums are double-buffered: two CTA barriers per group; the sketch words
// of the next group and the norms of this one are fetched before step 1.
constexpr int GPC = 8;                  // groups per CTA
constexpr int B_PITCH = 132;            // words per B-fragment column: lanes (g, c) of a fragment load hit 32 banks

template <typename T, typename TP, int R>
__global__ void __launch_bounds__(THREADS)
score_mma_kernel(const uint8_t* __restrict__ key_quant, const uint8_t* __restrict__ key_outlier_quant,
                 const T* __restrict__ key_norm, const T* __restrict__ key_outlier_norm,
                 const uint8_t* __restrict__ outlier_idx, const float* __restrict__ query_sketch,
                 const T* __restrict__ query, const TP* __restrict__ proj_score, float* __restrict__ scores,
                 int n_groups, int G, int n_rep, int sketch, int o_sketch, int oc) {
  constexpr int NV = R / 4;                                  // fragment arrays per sketch: hi|lo in one, or hi and lo
  __shared__ __align__(16) float qd_s[kHeadDim][R];          // query values [channel][head]
  __shared__ __align__(16) __half b_s[2][2][NV][8][B_PITCH * 2];           // [buffer][in|out][hi|lo][column][projection]
  __shared__ float part_s[2][2][32][2 * R + 1];              // [buffer][projection half][token][in heads | out heads]
  __shared__ uint8_t otl_s[GPC][kHeadDim];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const int64_t kbh = blockIdx.x;
  const int n0 = blockIdx.y * GPC, n_here = min(GPC, n_groups - n0);
  const int tok0 = blockIdx.z * 32;
  const int n_tok = min(32, G - tok0);
  const int64_t qrow0 = kbh * n_rep;
  for (int i = tid; i < R * kHeadDim; i += THREADS) {
    const int r = i >> 7, d = i & (kHeadDim - 1);
    qd_s[d][r] = r < n_rep ? Elem<T>::to_f(query[(qrow0 + r) * kHeadDim + d]) : 0.f;
  }
  for (int i = tid; i < n_here * oc; i += THREADS)
    otl_s[i / oc][i % oc] = outlier_idx[(kbh * n_groups + n0) * oc + i] & (kHeadDim - 1);
  // this thread's projection: the sketch of the whole query per head
  const int p = tid;
  float qs_reg[R];
#pragma unroll
  for (int r = 0; r < R; ++r) qs_reg[r] = (p < sketch && r < n_rep) ? query_sketch[(qrow0 + r) * sketch + p] : 0.f;
  // this warp's MMA task and its sketch words
  const int mt = warp & 1, io = (warp >> 1) & 1, kh = warp >> 2;
  const int g = lane >> 2, c = lane & 3;
  const int dim = io == 0 ? sketch : o_sketch;
  const int n_ks = min(8, dim / 16 - kh * 8);                // k-steps of 16 projections in this half
  const uint8_t* kbase = io == 0 ? key_quant : key_outlier_quant;
  const int row_bytes = dim / 8;
  const int t_lo = mt * 16 + g, t_hi = t_lo + 8;
  auto load_words = [&](int gl, uint4& w_lo, uint4& w_hi) {
    w_lo = make_uint4(0u, 0u, 0u, 0u); w_hi = make_uint4(0u, 0u, 0u, 0u);
    if (n_ks <= 0 || gl >= n_here) return;
    const int64_t tok = (kbh * n_groups + n0 + gl) * G + tok0;
    if (t_lo < n_tok) w_lo = *reinterpret_cast<const uint4*>(kbase + (tok + t_lo) * row_bytes + kh * 16);
    if (t_hi < n_tok) w_hi = *reinterpret_cast<const uint4*>(kbase + (tok + t_hi) * row_bytes + kh * 16);
  };
  uint4 cur_lo, cur_hi;
  load_words(0, cur_lo, cur_hi);
  // epilogue role: (token, head)
  const int et = tid / R, er = tid % R;
  const bool e_live = tid < 32 * R && et < n_tok && er < n_rep;
  __syncthreads();

  for (int gl = 0; gl < n_here; ++gl) {
    const int buf = gl & 1;
    const int64_t grp = kbh * n_groups + n0 + gl;
    uint4 nxt_lo, nxt_hi;
    load_words(gl + 1, nxt_lo, nxt_hi);
    float norm_k = 0.f, norm_o = 0.f;
    if (e_live) {
      norm_k = Elem<T>::to_f(key_norm[grp * G + tok0 + et]);
      norm_o = Elem<T>::to_f(key_outlier_norm[grp * G + tok0 + et]);
    }
    // ---- 1. query-side terms of projection p
    if (p < sketch) {
      float o[R];
#pragma unroll
      for (int r = 0; r < R; ++r) o[r] = 0.f;
      for (int i = 0; i < oc; ++i) {
        const int d = otl_s[gl][i];
        const float pv = proj_f<TP>(proj_score[(int64_t)d * sketch + p]);
#pragma unroll
        for (int r4 = 0; r4 < R; r4 += 4) {
          const float4 qv = *reinterpret_cast<const float4*>(&qd_s[d][r4]);
          o[r4] = fmaf(qv.x, pv, o[r4]); o[r4 + 1] = fmaf(qv.y, pv, o[r4 + 1]);
          o[r4 + 2] = fmaf(qv.z, pv, o[r4 + 2]); o[r4 + 3] = fmaf(qv.w, pv, o[r4 + 3]);
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          if (which == 1 && p >= o_sketch) continue;
          const float x = which == 0 ? qs_reg[r] - o[r] : o[r];
          const __half hi = __float2half_rn(x);
          const __half lo = __float2half_rn(x - __half2float(hi));
          if constexpr (R == 4) {
            b_s[buf][which][0][r][p] = hi;
            b_s[buf][which][0][r + 4][p] = lo;
          } else {
            b_s[buf][which][0][r][p] = hi;
            b_s[buf][which][NV - 1][r][p] = lo;
          }
        }
      }
    }
    __syncthreads();
    // ---- 2. sign sums on the MMA
    {
      float acc[NV][4];
#pragma unroll
      for (int v = 0; v < NV; ++v) { acc[v][0] = acc[v][1] = acc[v][2] = acc[v][3] = 0.f; }
      if (n_ks > 0) {
        const uint32_t wl[4] = {cur_lo.x, cur_lo.y, cur_lo.z, cur_lo.w}, wh[4] = {cur_hi.x, cur_hi.y, cur_hi.z, cur_hi.w};
        const uint32_t* bw[NV];
#pragma unroll
        for (int v = 0; v < NV; ++v) bw[v] = reinterpret_cast<const uint32_t*>(&b_s[buf][io][v][g][0]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (j < n_ks) {
            // inverted bits 2c, 2c+1 of the step's first byte and of its second byte give the sign bits of
            // columns (2c, 2c+1) and (2c+8, 2c+9); the magnitude is one unit in the last place
            const uint32_t zl = ~(wl[j >> 1] >> (16 * (j & 1) + 2 * c)) & 0x0303u;
            const uint32_t zh = ~(wh[j >> 1] >> (16 * (j & 1) + 2 * c)) & 0x0303u;
            const uint32_t a0 = (((zl << 15) | (zl << 30)) & 0x80008000u) | 0x00010001u;
            const uint32_t a1 = (((zh << 15) | (zh << 30)) & 0x80008000u) | 0x00010001u;
            const uint32_t a2 = (((zl << 7) | (zl << 22)) & 0x80008000u) | 0x00010001u;
            const uint32_t a3 = (((zh << 7) | (zh << 22)) & 0x80008000u) | 0x00010001u;
            const int pp = (kh * 8 + j) * 8 + c;                // pair of projections 2pp, 2pp+1
#pragma unroll
            for (int v = 0; v < NV; ++v) ptx::mma_f16(acc[v], a0, a1, a2, a3, bw[v][pp], bw[v][pp + 4]);
          }
        }
      }
      // acc[.][0..1] = (token g, columns 2c, 2c+1), acc[.][2..3] = (token g + 8, same columns)
      constexpr float UNSCALE = 16777216.f;                    // the signs were +-2^-24
      if constexpr (R == 4) {
        // columns 0-3 hold the hi sums of heads 0-3, columns 4-7 the lo sums: lanes c and c+2 pair up
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[0][e] += __shfl_xor_sync(0xffffffffu, acc[0][e], 2);
        if (c < 2) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            part_s[buf][kh][mt * 16 + g + 8 * (e >> 1)][io * R + 2 * c + (e & 1)] = acc[0][e] * UNSCALE;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          part_s[buf][kh][mt * 16 + g + 8 * (e >> 1)][io * R + 2 * c + (e & 1)] = (acc[0][e] + acc[NV - 1][e]) * UNSCALE;
      }
    }
    __syncthreads();
    // ---- 3. norms and scale
    if (e_live) {
      const float inner = part_s[buf][0][et][er] + part_s[buf][1][et][er];
      const float outer = part_s[buf][0][et][R + er] + part_s[buf][1][et][R + er];
      // |k_in|: the two norms are rounded separately, so the difference can dip below zero
      const float norm_in = sqrtf(fmaxf(norm_k * norm_k - norm_o * norm_o, 0.f));
      const float scl = 1.2533141373155001f / (float)sketch, scl_o = 1.2533141373155001f / (float)o_sketch;
      scores[(qrow0 + er) * ((int64_t)n_groups * G) + (int64_t)(n0 + gl) * G + tok0 + et] =
          scl * norm_in * inner + scl_o * norm_o * outer;
    }
    cur_lo = nxt_lo; cur_hi = nxt_hi;
  }
}

// ---- the quantizer on the warp MMA ---------------------------------------------------------------
// The sums of a chunk are a [32 tokens x 128] x [128 x sketch] product.  A persistent CTA (one per SM)
// keeps the whole projection in shared memory as fp16 hi/lo pairs in B-fragment order (hi = fp16(x),
// lo = fp16(x - hi): the fp32 accumulator then holds the fp32-rounded sum) and walks (group, chunk)
// items: keys staged as fp16 rows, A fragments by ldmatrix, once as they are (all channels) and once
// ANDed with the group's outlier mask; inlier sum = all - outlier.  Warp = 16 projections.
constexpr int QW = 16, QTHREADS = QW * 32;
constexpr int KPITCH = 136;                           // halves per staged key row: ldmatrix rows hit distinct banks
constexpr int Q_PF_BYTES = 2 * 32 * 8 * 32 * 8;       // [hi|lo][n-tile][k-step][lane] x (b0, b1)
constexpr int Q_KEY_BYTES = 2 * 32 * KPITCH * 2;      // two staged chunks
constexpr int Q_SMEM = Q_PF_BYTES + Q_KEY_BYTES + 32 + 128;

template <typename T> struct Half8;
template <> struct Half8<__half> {
  static __device__ __forceinline__ uint4 conv(uint4 v) { return v; }
};
template <> struct Half8<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t two(uint32_t w) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
    const __half2 h = __floats2half2_rn(f.x, f.y);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ uint4 conv(uint4 v) { return make_uint4(two(v.x), two(v.y), two(v.z), two(v.w)); }
};

template <typename T, typename TP>
__global__ void __launch_bounds__(QTHREADS, 1)
quant_mma_kernel(const T* __restrict__ keys, const uint8_t* __restrict__ outlier_idx, const TP* __restrict__ proj,
                 uint8_t* __restrict__ key_quant, uint8_t* __restrict__ key_outlier_quant,
                 T* __restrict__ outlier_norm, int64_t n_groups, int G, int sketch, int o_sketch, int oc) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint2* pf = reinterpret_cast<uint2*>(smem);
  __half* key_s = reinterpret_cast<__half*>(smem + Q_PF_BYTES);
  uint32_t* mask_s = reinterpret_cast<uint32_t*>(smem + Q_PF_BYTES + Q_KEY_BYTES);     // [2][4]
  uint8_t* byte_s = smem + Q_PF_BYTES + Q_KEY_BYTES + 32;                               // [128], warp 0 only
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  // projection fragments: b0 = (P[p][d], P[p][d+1]), b1 = (P[p][d+8], P[p][d+9]) with p = 8 nt + g, d = 16 ks + 2c
  for (int i = tid; i < 32 * 8 * 32; i += QTHREADS) {
    const int nt = i >> 8, ks = (i >> 5) & 7, l = i & 31;
    const int p = 8 * nt + (l >> 2), d = 16 * ks + 2 * (l & 3);
    uint32_t hi[2] = {0u, 0u}, lo[2] = {0u, 0u};
    if (p < sketch) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float x0 = proj_f<TP>(proj[(int64_t)p * kHeadDim + d + 8 * j]);
        const float x1 = proj_f<TP>(proj[(int64_t)p * kHeadDim + d + 8 * j + 1]);
        const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
        const __half l0 = __float2half_rn(x0 - __half2float(h0)), l1 = __float2half_rn(x1 - __half2float(h1));
        hi[j] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
        lo[j] = (uint32_t)__half_as_ushort(l0) | ((uint32_t)__half_as_ushort(l1) << 16);
      }
    }
    pf[((0 * 32 + nt) * 8 + ks) * 32 + l] = make_uint2(hi[0], hi[1]);
    pf[((1 * 32 + nt) * 8 + ks) * 32 + l] = make_uint2(lo[0], lo[1]);
  }
  const int n_chunks = (G + 31) / 32;
  const int64_t n_items = n_groups * n_chunks;
  // loader role: token row lt, eight channels from 8 * seg
  const int lt = tid >> 4, seg = tid & 15;
  auto fetch = [&](int64_t item) -> uint4 {
    const int64_t grp = item / n_chunks;
    const int tok0 = (int)(item % n_chunks) * 32;
    if (tok0 + lt >= G) return make_uint4(0u, 0u, 0u, 0u);
    return *reinterpret_cast<const uint4*>(keys + ((grp * G + tok0 + lt) * kHeadDim + 8 * seg));
  };
  int64_t item = blockIdx.x;
  uint4 cur = make_uint4(0u, 0u, 0u, 0u);
  if (item < n_items) cur = fetch(item);
  const int p0 = 16 * warp;
  for (int it = 0; item < n_items; item += gridDim.x, ++it) {
    const int buf = it & 1;
    const int64_t grp = item / n_chunks;
    const int tok0 = (int)(item % n_chunks) * 32;
    const int n_tok = min(32, G - tok0);
    *reinterpret_cast<uint4*>(key_s + (buf * 32 + lt) * KPITCH + 8 * seg) = Half8<T>::conv(cur);
    if (warp == 0) {                                  // the group's outlier channels as a 128-bit mask
      reinterpret_cast<uint32_t*>(byte_s)[lane] = 0u;
      __syncwarp();
      for (int i = lane; i < oc; i += 32) byte_s[outlier_idx[grp * oc + i] & (kHeadDim - 1)] = 1;
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t w = __ballot_sync(0xffffffffu, byte_s[32 * j + lane] != 0);
        if (lane == 0) mask_s[buf * 4 + j] = w;
      }
      __syncwarp();
    }
    __syncthreads();
    uint4 nxt = make_uint4(0u, 0u, 0u, 0u);
    if (item + gridDim.x < n_items) nxt = fetch(item + gridDim.x);
    const uint32_t mw[4] = {mask_s[buf * 4], mask_s[buf * 4 + 1], mask_s[buf * 4 + 2], mask_s[buf * 4 + 3]};
    {  // norm of the outlier part, from the values as loaded
      const uint32_t mbyte = (mw[seg >> 2] >> (8 * (seg & 3))) & 0xffu;
      const T* e = reinterpret_cast<const T*>(&cur);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float x = Elem<T>::to_f(e[j]);
        if ((mbyte >> j) & 1u) ss = fmaf(x, x, ss);
      }
#pragma unroll
      for (int o = 8; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (seg == 0 && lt < n_tok) outlier_norm[grp * G + tok0 + lt] = Elem<T>::from_f(sqrtf(ss));
    }
    if (p0 < sketch) {
      float acc_t[2][2][4], acc_o[2][2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) { acc_t[mt][nt][e] = 0.f; acc_o[mt][nt][e] = 0.f; }
      const uint32_t a_base = ptx::smem_u32(key_s + (buf * 32 + (lane & 7) + 8 * ((lane >> 3) & 1)) * KPITCH + 8 * (lane >> 4));
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        // channels 16ks + (2c, 2c+1) and + (2c+8, 2c+9): all-ones halves where the channel is an outlier
        const uint32_t m = mw[ks >> 1] >> (16 * (ks & 1) + 2 * c);
        const uint32_t m_lo = ((m & 1u) ? 0x0000ffffu : 0u) | ((m & 2u) ? 0xffff0000u : 0u);
        const uint32_t m_hi = ((m & 0x100u) ? 0x0000ffffu : 0u) | ((m & 0x200u) ? 0xffff0000u : 0u);
        uint2 b[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int v = 0; v < 2; ++v) b[nt][v] = pf[((v * 32 + 2 * warp + nt) * 8 + ks) * 32 + lane];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          uint32_t a0, a1, a2, a3;
          ptx::ldmatrix_x4(a_base + (uint32_t)((mt * 16 * KPITCH + ks * 16) * 2), a0, a1, a2, a3);
          const uint32_t o0 = a0 & m_lo, o1 = a1 & m_lo, o2 = a2 & m_hi, o3 = a3 & m_hi;
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int v = 0; v < 2; ++v) {
              ptx::mma_f16(acc_t[mt][nt], a0, a1, a2, a3, b[nt][v].x, b[nt][v].y);
              ptx::mma_f16(acc_o[mt][nt], o0, o1, o2, o3, b[nt][v].x, b[nt][v].y);
            }
        }
      }
      // acc[..][0..1] = (token g, projections 2c, 2c+1 of the n-tile), acc[..][2..3] = (token g + 8, same)
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t bits_in = 0u, bits_out = 0u;
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float out = acc_o[mt][nt][2 * hh + e], in = acc_t[mt][nt][2 * hh + e] - out;
              bits_in |= (in > 0.f ? 1u : 0u) << (8 * nt + 2 * c + e);
              bits_out |= (out > 0.f ? 1u : 0u) << (8 * nt + 2 * c + e);
            }
          bits_in |= __shfl_xor_sync(0xffffffffu, bits_in, 1); bits_in |= __shfl_xor_sync(0xffffffffu, bits_in, 2);
          bits_out |= __shfl_xor_sync(0xffffffffu, bits_out, 1); bits_out |= __shfl_xor_sync(0xffffffffu, bits_out, 2);
          const int t = 16 * mt + g + 8 * hh;
          if (c == 0 && t < n_tok) {
            const int64_t tok = grp * G + tok0 + t;
            *reinterpret_cast<uint16_t*>(key_quant + tok * (sketch / 8) + 2 * warp) = (uint16_t)bits_in;
            if (p0 < o_sketch)
              *reinterpret_cast<uint16_t*>(key_outlier_quant + tok * (o_sketch / 8) + 2 * warp) = (uint16_t)bits_out;
          }
        }
    }
    cur = nxt;
  }
}

static bool sizes_ok(int G, int sketch, int o_sketch, int oc) {
  return G > 0 && sketch > 0 && sketch <= MAX_SKETCH && sketch % 32 == 0 && o_sketch > 0 && o_sketch <= sketch &&
         o_sketch % 32 == 0 && oc >= 0 && oc <= kHeadDim;
}

static bool mma_ptrs_ok(const void* a, const void* b) { return aligned16(a) && aligned16(b); }

}  // namespace qjl
}  // namespace cq

using namespace cq;

extern "C" int cq_qjl_quant(const void* keys, const uint8_t* outlier_indices, const void* proj, int proj_dtype,
                            int64_t n_groups_total, int group_size, int head_dim, int sketch_dim,
                            int outlier_sketch_dim, int outlier_count, int dtype, uint8_t* key_quant,
                            uint8_t* key_outlier_quant, void* outlier_norms, void* stream) {
  if (n_groups_total == 0) return CQ_OK;
  if (!keys || !outlier_indices || !proj || !key_quant || !key_outlier_quant || !outlier_norms || n_groups_total < 0)
    return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (proj_dtype != CQ_DTYPE_F32 && proj_dtype != dtype) return CQ_ERR_BAD_ARG;
  if (head_dim != kHeadDim || !qjl::sizes_ok(group_size, sketch_dim, outlier_sketch_dim, outlier_count))
    return CQ_ERR_UNSUPPORTED;
  if (n_groups_total > 0x7fffffff) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // aligned rows: the persistent tensor-core kernel, one CTA per SM
  if (aligned16(keys) && (reinterpret_cast<uintptr_t>(key_quant) & 1u) == 0 &&
      (reinterpret_cast<uintptr_t>(key_outlier_quant) & 1u) == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return CQ_ERR_LAUNCH;
    const int64_t items = n_groups_total * ((group_size + 31) / 32);
    const unsigned grid_mma = (unsigned)(items < sms ? items : sms);
#define CQ_QJL_QUANT_MMA(T, TP)                                                                                 \
    do {                                                                                                        \
      auto kern = qjl::quant_mma_kernel<T, TP>;                                                                 \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, qjl::Q_SMEM) != cudaSuccess)  \
        return CQ_ERR_LAUNCH;                                                                                   \
      kern<<<grid_mma, qjl::QTHREADS, qjl::Q_SMEM, st>>>(static_cast<const T*>(keys), outlier_indices,          \
          static_cast<const TP*>(proj), key_quant, key_outlier_quant, static_cast<T*>(outlier_norms),           \
          n_groups_total, group_size, sketch_dim, outlier_sketch_dim, outlier_count);                           \
    } while (0)
    if (dtype == CQ_DTYPE_F16) {
      if (proj_dtype == CQ_DTYPE_F32) CQ_QJL_QUANT_MMA(__half, float); else CQ_QJL_QUANT_MMA(__half, __half);
    } else {
      if (proj_dtype == CQ_DTYPE_F32) CQ_QJL_QUANT_MMA(__nv_bfloat16, float); else CQ_QJL_QUANT_MMA(__nv_bfloat16, __nv_bfloat16);
    }
#undef CQ_QJL_QUANT_MMA
    return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
  }
  dim3 grid((unsigned)n_groups_total, (unsigned)((group_size + 31) / 32));
#define CQ_QJL_QUANT(T, TP)                                                                                   \
  qjl::quant_kernel<T, TP><<<grid, qjl::THREADS, 0, st>>>(static_cast<const T*>(keys), outlier_indices,       \
      static_cast<const TP*>(proj), key_quant, key_outlier_quant, static_cast<T*>(outlier_norms), group_size,  \
      sketch_dim, outlier_sketch_dim, outlier_count)
  if (dtype == CQ_DTYPE_F16) {
    if (proj_dtype == CQ_DTYPE_F32) CQ_QJL_QUANT(__half, float); else CQ_QJL_QUANT(__half, __half);
  } else {
    if (proj_dtype == CQ_DTYPE_F32) CQ_QJL_QUANT(__nv_bfloat16, float); else CQ_QJL_QUANT(__nv_bfloat16, __nv_bfloat16);
  }
#undef CQ_QJL_QUANT
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_qjl_gqa_score(const uint8_t* key_quant, const uint8_t* key_outlier_quant, const void* key_norm,
                                const void* key_outlier_norm, const uint8_t* outlier_indices,
                                const float* query_sketch, const void* query, const void* proj_score,
                                int proj_dtype, int batch, int n_kv_heads, int n_rep, int n_groups, int group_size,
                                int head_dim, int sketch_dim, int outlier_sketch_dim, int outlier_count, int dtype,
                                float* scores, void* stream) {
  if (batch == 0 || n_groups == 0) return CQ_OK;
  if (!key_quant || !key_outlier_quant || !key_norm || !key_outlier_norm || !outlier_indices || !query_sketch ||
      !query || !proj_score || !scores)
    return CQ_ERR_BAD_ARG;
  if (batch < 0 || n_kv_heads <= 0 || n_rep <= 0 || n_groups < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (proj_dtype != CQ_DTYPE_F32 && proj_dtype != dtype) return CQ_ERR_BAD_ARG;
  if (head_dim != kHeadDim || n_rep > kMaxRep || !qjl::sizes_ok(group_size, sketch_dim, outlier_sketch_dim, outlier_count))
    return CQ_ERR_UNSUPPORTED;
  if (n_groups > 65535) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)(batch * n_kv_heads), (unsigned)n_groups, (unsigned)((group_size + 31) / 32));
  // sketch rows that are whole 16-byte words: the tensor-core variant, several groups per CTA
  const bool use_mma = sketch_dim % 128 == 0 && outlier_sketch_dim % 128 == 0 && qjl::mma_ptrs_ok(key_quant, key_outlier_quant);
  if (use_mma) grid.y = (unsigned)((n_groups + qjl::GPC - 1) / qjl::GPC);
#define CQ_QJL_SCORE(T, TP, R)                                                                                 \
  do { (use_mma ? qjl::score_mma_kernel<T, TP, R> : qjl::score_kernel<T, TP, R>)<<<grid, qjl::THREADS, 0, st>>>(key_quant, key_outlier_quant, \
      static_cast<const T*>(key_norm), static_cast<const T*>(key_outlier_norm), outlier_indices, query_sketch,  \
      static_cast<const T*>(query), static_cast<const TP*>(proj_score), scores, n_groups, group_size, n_rep,    \
      sketch_dim, outlier_sketch_dim, outlier_count); } while (0)
#define CQ_QJL_SCORE_R(T, TP) do { if (n_rep <= 4) CQ_QJL_SCORE(T, TP, 4); else CQ_QJL_SCORE(T, TP, 8); } while (0)
  if (dtype == CQ_DTYPE_F16) {
    if (proj_dtype == CQ_DTYPE_F32) CQ_QJL_SCORE_R(__half, float); else CQ_QJL_SCORE_R(__half, __half);
  } else {
    if (proj_dtype == CQ_DTYPE_F32) CQ_QJL_SCORE_R(__nv_bfloat16, float); else CQ_QJL_SCORE_R(__nv_bfloat16, __nv_bfloat16);
  }
#undef CQ_QJL_SCORE_R
#undef CQ_QJL_SCORE
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}
