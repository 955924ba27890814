// Decode-step attention over [system | visual (group-format quantized) | text] keys.
//
// Math (decode step of the reference, patch_internvl.py:556-592, calibration :376-385):
//   s_vis[t] = rnd(rnd(sum_d q[d]*(ks[d,G]*code[d,t] + kmn[d,G])) / sqrt(D))      G = t/32
//   s_fp[t]  = rnd(rnd(q . K_fp[t]) / sqrt(D))
//   if calibrate: s_vis <- affine remap of [min,max] onto [min,max-3], op by op in the dtype
//   p = softmax_fp32([s_sys | s_vis | s_txt] + mask), rounded to the dtype
//   o = sum_t p_vis[t]*(vs[t,g]*code[t,d] + vmn[t,g]) + sum_t p_fp[t]*V_fp[t]
// "Post-scaling": K is never dequantised.  Per 32-token group the query is pre-multiplied by
// the group's channel scales, q'[d] = q[d]*ks[d,G], and the minimum folds into one scalar
// bias = sum_d q[d]*kmn[d,G]; the inner loop is then a select-and-add over code bits.
// K/V bytes are read once per KV head and shared by its n_rep query heads (no repeat_kv).
//
// Four launches on the caller's stream, exchanging through the caller's workspace:
//   1 scores  : all logits -> workspace (dtype), visual and fp tiles in one grid
//   2 stats   : per (batch, q head): calibration constants, running max, 1/sum(exp)
//   3 attn.V  : split over tokens, fp32 partial outputs -> workspace
//   4 combine : add the splits, round to the dtype
#include <mutex>

#include "cq_common.cuh"
#include "cq_decode_shared.cuh"

namespace cq {

constexpr int SC_TOK = 512;     // visual tokens per CTA in the score kernel (16 groups)
constexpr int SC_GROUPS = SC_TOK / kGroup;
constexpr int SC_FP_TOK = 64;   // fp tokens per CTA in the score kernel
constexpr int SC_THREADS = 256;
constexpr int AV_TOK = 512;     // visual tokens per split in the attn.V kernel
constexpr int AV_SUB = 128;     // staged at a time
constexpr int AV_FP_TOK = 128;  // fp tokens per split
constexpr int AV_THREADS = 128;
constexpr int STATS_FLOATS = 8;

struct DecodeDims {
  int batch, hq, hkv, n_rep, t_vis, t_fp, t_sys, t_all, calibrate;
  int n_vis_tiles, n_fp_tiles, n_vis_splits, n_fp_splits;
  int64_t fp_stride_b, fp_stride_h, mask_stride_b;
};

struct Calib {
  float mn, denom, range;
};

template <typename T>
__device__ __forceinline__ float calibrate_one(float s, const Calib& c) {
  float n = rnd<T>(__fdiv_rn(rnd<T>(s - c.mn), c.denom));
  return rnd<T>(rnd<T>(n * c.range) + c.mn);
}

// Position of key j of the workspace order [visual | fp] inside the mask order [sys|visual|text].
__device__ __forceinline__ int mask_pos(int j, int t_vis, int t_sys) {
  if (j < t_vis) return t_sys + j;
  const int f = j - t_vis;
  return f < t_sys ? f : t_vis + f;
}

template <typename T>
__device__ __forceinline__ float final_logit(const T* row, const T* mask_row, int j,
                                             const DecodeDims& dm, const Calib& c) {
  float s = Elem<T>::to_f(row[j]);
  if (dm.calibrate && j < dm.t_vis) s = calibrate_one<T>(s, c);
  if (mask_row) s = rnd<T>(s + Elem<T>::to_f(mask_row[mask_pos(j, dm.t_vis, dm.t_sys)]));
  return s;
}

// ------------------------------------------------------------------------------------------
// 1. scores
// ------------------------------------------------------------------------------------------
template <typename T, int BITS>
__global__ void __launch_bounds__(SC_THREADS)
scores_kernel(DecodeDims dm, const T* __restrict__ q, const int32_t* __restrict__ k_code,
              const T* __restrict__ k_scale, const T* __restrict__ k_mn,
              const T* __restrict__ k_fp, T* __restrict__ scores) {
  constexpr int FPI = 32 / BITS;
  constexpr int WPT = SC_GROUPS * BITS;          // words per channel row per tile
  constexpr unsigned CMASK = (1u << BITS) - 1u;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* q_s = reinterpret_cast<float*>(smem_raw);                       // [kMaxRep][128]
  float* qp_s = q_s + kMaxRep * kHeadDim;                                // [8 warps][128][kMaxRep]
  unsigned* code_s = reinterpret_cast<unsigned*>(qp_s + 8 * kHeadDim * kMaxRep);  // [128][WPT]
  T* ks_s = reinterpret_cast<T*>(code_s + kHeadDim * WPT);               // [128][SC_GROUPS]
  T* kmn_s = ks_s + kHeadDim * SC_GROUPS;

  const int bhk = blockIdx.y;
  const int b = bhk / dm.hkv, hk = bhk % dm.hkv;
  const int n_rep = dm.n_rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float sqrt_d = 11.313708498984761f;   // sqrt(128)

  for (int i = threadIdx.x; i < n_rep * kHeadDim; i += SC_THREADS)
    q_s[i] = Elem<T>::to_f(q[((int64_t)b * dm.hq + (int64_t)hk * n_rep) * kHeadDim + i]);

  if ((int)blockIdx.x < dm.n_vis_tiles) {
    const int g0 = blockIdx.x * SC_GROUPS;
    const int n_groups = dm.t_vis / kGroup;
    const int live_groups = min(SC_GROUPS, n_groups - g0);
    const int64_t words_per_row = (int64_t)n_groups * BITS;
    const int32_t* code_g = k_code + (int64_t)bhk * kHeadDim * words_per_row + (int64_t)g0 * BITS;
    const T* ks_g = k_scale + (int64_t)bhk * kHeadDim * n_groups + g0;
    const T* kmn_g = k_mn + (int64_t)bhk * kHeadDim * n_groups + g0;
    for (int i = threadIdx.x; i < kHeadDim * WPT; i += SC_THREADS) {
      const int d = i / WPT, w = i % WPT;
      code_s[i] = w < live_groups * BITS ? (unsigned)__ldg(code_g + d * words_per_row + w) : 0u;
    }
    for (int i = threadIdx.x; i < kHeadDim * SC_GROUPS; i += SC_THREADS) {
      const int d = i / SC_GROUPS, g = i % SC_GROUPS;
      const bool ok = g < live_groups;
      ks_s[i] = ok ? __ldg(ks_g + (int64_t)d * n_groups + g) : Elem<T>::from_f(0.f);
      kmn_s[i] = ok ? __ldg(kmn_g + (int64_t)d * n_groups + g) : Elem<T>::from_f(0.f);
    }
    __syncthreads();

    float* qp_w = qp_s + warp * kHeadDim * kMaxRep;
    for (int g = warp; g < live_groups; g += SC_THREADS / 32) {
      // q'[d][h] = q[h][d]*ks[d,G];  bias[h] = sum_d q[h][d]*kmn[d,G]
      float bias[kMaxRep];
#pragma unroll
      for (int h = 0; h < kMaxRep; ++h) bias[h] = 0.f;
      for (int d = lane; d < kHeadDim; d += 32) {
        const float s = Elem<T>::to_f(ks_s[d * SC_GROUPS + g]);
        const float z = Elem<T>::to_f(kmn_s[d * SC_GROUPS + g]);
#pragma unroll
        for (int h = 0; h < kMaxRep; ++h) {
          if (h < n_rep) {
            const float qv = q_s[h * kHeadDim + d];
            qp_w[d * kMaxRep + h] = qv * s;
            bias[h] = fmaf(qv, z, bias[h]);
          }
        }
      }
#pragma unroll
      for (int h = 0; h < kMaxRep; ++h) bias[h] = warp_sum(bias[h]);
      __syncwarp();

      // lane = token of the group
      const int tok = lane;
      const int widx = g * BITS + tok / FPI;
      const int shift = (tok % FPI) * BITS;
      float acc[kMaxRep];
#pragma unroll
      for (int h = 0; h < kMaxRep; ++h) acc[h] = 0.f;
#pragma unroll 4
      for (int d = 0; d < kHeadDim; ++d) {
        const unsigned c = (code_s[d * WPT + widx] >> shift) & CMASK;
        const float4 qa = *reinterpret_cast<const float4*>(&qp_w[d * kMaxRep]);
        if (BITS == 1) {
          if (c) { acc[0] += qa.x; acc[1] += qa.y; acc[2] += qa.z; acc[3] += qa.w; }
        } else {
          const float cf = (float)c;
          acc[0] = fmaf(cf, qa.x, acc[0]); acc[1] = fmaf(cf, qa.y, acc[1]);
          acc[2] = fmaf(cf, qa.z, acc[2]); acc[3] = fmaf(cf, qa.w, acc[3]);
        }
        if (n_rep > 4) {
          const float4 qb = *reinterpret_cast<const float4*>(&qp_w[d * kMaxRep + 4]);
          const float cf = (float)c;
          acc[4] = fmaf(cf, qb.x, acc[4]); acc[5] = fmaf(cf, qb.y, acc[5]);
          acc[6] = fmaf(cf, qb.z, acc[6]); acc[7] = fmaf(cf, qb.w, acc[7]);
        }
      }
      const int t = (g0 + g) * kGroup + tok;
#pragma unroll
      for (int h = 0; h < kMaxRep; ++h) {
        if (h < n_rep) {
          const float raw = rnd<T>(acc[h] + bias[h]);
          const float sc = __fdiv_rn(raw, sqrt_d);
          scores[((int64_t)b * dm.hq + hk * n_rep + h) * dm.t_all + t] = Elem<T>::from_f(sc);
        }
      }
      __syncwarp();
    }
  } else {
    __syncthreads();
    // full-precision tokens: one warp per token, lane owns 4 channels
    const int tile = blockIdx.x - dm.n_vis_tiles;
    const T* kf = k_fp + (int64_t)b * dm.fp_stride_b + (int64_t)hk * dm.fp_stride_h;
    for (int i = warp; i < SC_FP_TOK; i += SC_THREADS / 32) {
      const int t = tile * SC_FP_TOK + i;
      if (t >= dm.t_fp) break;
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(kf + (int64_t)t * kHeadDim) + lane);
      const typename Elem<T>::T2* p2 = reinterpret_cast<const typename Elem<T>::T2*>(&raw);
      const float2 k01 = Elem<T>::to_f2(p2[0]), k23 = Elem<T>::to_f2(p2[1]);
      for (int h = 0; h < n_rep; ++h) {
        const float4 qv = *reinterpret_cast<const float4*>(&q_s[h * kHeadDim + lane * 4]);
        float dot = qv.x * k01.x + qv.y * k01.y + qv.z * k23.x + qv.w * k23.y;
        dot = warp_sum(dot);
        if (lane == 0) {
          const float sc = __fdiv_rn(rnd<T>(dot), sqrt_d);
          scores[((int64_t)b * dm.hq + hk * n_rep + h) * dm.t_all + dm.t_vis + t] = Elem<T>::from_f(sc);
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// 2. stats: per (batch, q head) calibration constants, max logit, 1/sum(exp)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_reduce(float v, float* red, int op) {
  // op: 0 sum, 1 max, 2 min.  blockDim.x == 256.
  v = op == 0 ? warp_sum(v) : (op == 1 ? warp_max(v) : warp_min(v));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
  for (int i = 1; i < 8; ++i) r = op == 0 ? r + red[i] : (op == 1 ? fmaxf(r, red[i]) : fminf(r, red[i]));
  return r;
}

template <typename T>
__global__ void __launch_bounds__(256)
stats_kernel(DecodeDims dm, const T* __restrict__ scores, const T* __restrict__ mask,
             float* __restrict__ stats) {
  __shared__ float red[8];
  const int row = blockIdx.x;   // b*hq + h
  const T* s = scores + (int64_t)row * dm.t_all;
  const T* mrow = mask ? mask + (int64_t)(row / dm.hq) * dm.mask_stride_b : nullptr;
  Calib c{0.f, 1.f, 0.f};
  if (dm.calibrate && dm.t_vis > 0) {
    float mn = INFINITY, mx = -INFINITY;
    for (int j = threadIdx.x; j < dm.t_vis; j += 256) {
      const float v = Elem<T>::to_f(s[j]);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
    mn = block_reduce(mn, red, 2);
    mx = block_reduce(mx, red, 1);
    c.mn = mn;
    c.denom = rnd<T>(rnd<T>(mx - mn) + 1e-8f);
    c.range = rnd<T>(rnd<T>(mx + (-3.f)) - mn);
  }
  float m = -INFINITY;
  for (int j = threadIdx.x; j < dm.t_all; j += 256) m = fmaxf(m, final_logit<T>(s, mrow, j, dm, c));
  m = block_reduce(m, red, 1);
  float l = 0.f;
  for (int j = threadIdx.x; j < dm.t_all; j += 256) l += __expf(final_logit<T>(s, mrow, j, dm, c) - m);
  l = block_reduce(l, red, 0);
  if (threadIdx.x == 0) {
    float* o = stats + (int64_t)row * STATS_FLOATS;
    o[0] = c.mn; o[1] = c.denom; o[2] = c.range; o[3] = m; o[4] = 1.f / l;
  }
}

// ------------------------------------------------------------------------------------------
// 3. attn.V partials
// ------------------------------------------------------------------------------------------
template <typename T, int BITS>
__global__ void __launch_bounds__(AV_THREADS)
av_kernel(DecodeDims dm, const T* __restrict__ scores, const T* __restrict__ mask,
          const float* __restrict__ stats, const int32_t* __restrict__ v_code,
          const T* __restrict__ v_scale, const T* __restrict__ v_mn, const T* __restrict__ v_fp,
          float* __restrict__ partial) {
  constexpr int FPI = 32 / BITS;
  constexpr int WPT = kHeadDim / FPI;             // words per token
  constexpr unsigned CMASK = (1u << BITS) - 1u;
  __shared__ unsigned code_s[AV_SUB * WPT];
  __shared__ T vs_s[AV_SUB * 4];
  __shared__ T vmn_s[AV_SUB * 4];
  __shared__ float p_s[kMaxRep][AV_SUB];

  const int bhk = blockIdx.y;
  const int b = bhk / dm.hkv, hk = bhk % dm.hkv;
  const int n_rep = dm.n_rep;
  const int d = threadIdx.x;
  const int n_splits = dm.n_vis_splits + dm.n_fp_splits;
  const int64_t row0 = (int64_t)b * dm.hq + hk * n_rep;
  const T* mrow = mask ? mask + (int64_t)b * dm.mask_stride_b : nullptr;

  float acc[kMaxRep];
#pragma unroll
  for (int h = 0; h < kMaxRep; ++h) acc[h] = 0.f;

  const bool vis = (int)blockIdx.x < dm.n_vis_splits;
  const int split_tok0 = vis ? blockIdx.x * AV_TOK : (blockIdx.x - dm.n_vis_splits) * AV_FP_TOK;
  const int split_end = vis ? min(dm.t_vis, split_tok0 + AV_TOK) : min(dm.t_fp, split_tok0 + AV_FP_TOK);

  for (int t0 = split_tok0; t0 < split_end; t0 += AV_SUB) {
    const int nt = min(AV_SUB, split_end - t0);
    __syncthreads();
    // probabilities for this sub-tile, rounded to the dtype as the reference does
    for (int i = threadIdx.x; i < n_rep * AV_SUB; i += AV_THREADS) {
      const int h = i / AV_SUB, tt = i % AV_SUB;
      float p = 0.f;
      if (tt < nt) {
        const float* st = stats + (row0 + h) * STATS_FLOATS;
        const Calib c{st[0], st[1], st[2]};
        const int j = (vis ? 0 : dm.t_vis) + t0 + tt;
        const float x = final_logit<T>(scores + (row0 + h) * dm.t_all, mrow, j, dm, c);
        p = rnd<T>(__expf(x - st[3]) * st[4]);
      }
      p_s[h][tt] = p;
    }
    if (vis) {
      const int32_t* cg = v_code + ((int64_t)bhk * dm.t_vis + t0) * WPT;
      for (int i = threadIdx.x; i < nt * WPT; i += AV_THREADS) code_s[i] = (unsigned)__ldg(cg + i);
      const T* sg = v_scale + ((int64_t)bhk * dm.t_vis + t0) * 4;
      const T* zg = v_mn + ((int64_t)bhk * dm.t_vis + t0) * 4;
      for (int i = threadIdx.x; i < nt * 4; i += AV_THREADS) {
        vs_s[i] = __ldg(sg + i);
        vmn_s[i] = __ldg(zg + i);
      }
      __syncthreads();
      const int widx = d / FPI, shift = (d % FPI) * BITS, g = d / kGroup;
      for (int tt = 0; tt < nt; ++tt) {
        const float c = (float)((code_s[tt * WPT + widx] >> shift) & CMASK);
        const float v = fmaf(Elem<T>::to_f(vs_s[tt * 4 + g]), c, Elem<T>::to_f(vmn_s[tt * 4 + g]));
#pragma unroll
        for (int h = 0; h < kMaxRep; ++h)
          if (h < n_rep) acc[h] = fmaf(p_s[h][tt], v, acc[h]);
      }
    } else {
      __syncthreads();
      const T* vf = v_fp + (int64_t)b * dm.fp_stride_b + (int64_t)hk * dm.fp_stride_h +
                    (int64_t)t0 * kHeadDim + d;
      for (int tt = 0; tt < nt; ++tt) {
        const float v = Elem<T>::to_f(__ldg(vf + (int64_t)tt * kHeadDim));
#pragma unroll
        for (int h = 0; h < kMaxRep; ++h)
          if (h < n_rep) acc[h] = fmaf(p_s[h][tt], v, acc[h]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < kMaxRep; ++h)
    if (h < n_rep) partial[((row0 + h) * n_splits + blockIdx.x) * kHeadDim + d] = acc[h];
}

// ------------------------------------------------------------------------------------------
// 4. combine
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
combine_kernel(const float* __restrict__ partial, int n_splits, T* __restrict__ out) {
  const int64_t row = blockIdx.x;
  const float* p = partial + row * n_splits * kHeadDim + threadIdx.x;
  float s = 0.f;
  for (int i = 0; i < n_splits; ++i) s += p[(int64_t)i * kHeadDim];
  out[row * kHeadDim + threadIdx.x] = Elem<T>::from_f(s);
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
struct WsLayout {
  size_t scores_off, stats_off, partial_off, total;
};

static DecodeDims make_dims(const cq_decode_args* a) {
  DecodeDims dm;
  dm.batch = a->batch; dm.hq = a->n_q_heads; dm.hkv = a->n_kv_heads;
  dm.n_rep = a->n_q_heads / a->n_kv_heads;
  dm.t_vis = a->t_vis; dm.t_fp = a->t_fp; dm.t_sys = a->t_sys;
  dm.t_all = a->t_vis + a->t_fp;
  dm.calibrate = a->calibrate ? 1 : 0;
  dm.n_vis_tiles = (a->t_vis + SC_TOK - 1) / SC_TOK;
  dm.n_fp_tiles = (a->t_fp + SC_FP_TOK - 1) / SC_FP_TOK;
  dm.n_vis_splits = (a->t_vis + AV_TOK - 1) / AV_TOK;
  dm.n_fp_splits = (a->t_fp + AV_FP_TOK - 1) / AV_FP_TOK;
  dm.fp_stride_b = a->fp_stride_b; dm.fp_stride_h = a->fp_stride_h;
  dm.mask_stride_b = a->mask_stride_b;
  return dm;
}

static WsLayout make_layout(const DecodeDims& dm) {
  WsLayout w;
  const size_t rows = (size_t)dm.batch * dm.hq;
  w.scores_off = 256;   // the first 256 bytes are the sticky device status word of the workspace
  w.stats_off = w.scores_off + align_up(rows * (size_t)dm.t_all * 2, 256);
  w.partial_off = w.stats_off + align_up(rows * STATS_FLOATS * sizeof(float), 256);
  w.total = w.partial_off + rows * (size_t)(dm.n_vis_splits + dm.n_fp_splits) * kHeadDim * sizeof(float);
  return w;
}

static int validate(const cq_decode_args* a) {
  if (!a) return CQ_ERR_BAD_ARG;
  if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0) return CQ_ERR_BAD_ARG;
  if (a->n_q_heads % a->n_kv_heads) return CQ_ERR_BAD_ARG;
  if (a->t_vis < 0 || a->t_fp < 0 || a->t_vis + a->t_fp <= 0) return CQ_ERR_BAD_ARG;
  if (a->t_sys < 0 || a->t_sys > a->t_fp) return CQ_ERR_BAD_ARG;
  if (a->dtype != CQ_DTYPE_F16 && a->dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (!a->q || !a->out) return CQ_ERR_BAD_ARG;
  if (a->t_vis > 0 && (!a->k_code || !a->k_scale || !a->k_mn || !a->v_code || !a->v_scale || !a->v_mn))
    return CQ_ERR_BAD_ARG;
  if (a->t_fp > 0 && (!a->k_fp || !a->v_fp)) return CQ_ERR_BAD_ARG;
  if (a->head_dim != kHeadDim || a->group_size != kGroup) return CQ_ERR_UNSUPPORTED;
  if (a->bits != 1 && a->bits != 2 && a->bits != 4) return CQ_ERR_UNSUPPORTED;
  if (a->t_vis % kGroup) return CQ_ERR_UNSUPPORTED;
  if (a->n_q_heads / a->n_kv_heads > kMaxRep) return CQ_ERR_UNSUPPORTED;
  if (a->t_fp > 0 && (!aligned16(a->k_fp) || a->fp_stride_b % 8 || a->fp_stride_h % 8)) return CQ_ERR_BAD_ARG;
  return CQ_OK;
}

template <typename T, int BITS>
static int run_decode(const cq_decode_args* a, const DecodeDims& dm, const WsLayout& w,
                      unsigned char* ws, cudaStream_t st) {
  T* scores = reinterpret_cast<T*>(ws + w.scores_off);
  float* stats = reinterpret_cast<float*>(ws + w.stats_off);
  float* partial = reinterpret_cast<float*>(ws + w.partial_off);
  const T* mask = static_cast<const T*>(a->mask);
  const size_t smem = (size_t)kMaxRep * kHeadDim * 4 + 8 * kHeadDim * kMaxRep * 4 +
                      (size_t)kHeadDim * SC_GROUPS * BITS * 4 + 2 * (size_t)kHeadDim * SC_GROUPS * sizeof(T);
  auto kern = scores_kernel<T, BITS>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return CQ_ERR_LAUNCH;
  dim3 g1((unsigned)(dm.n_vis_tiles + dm.n_fp_tiles), (unsigned)(dm.batch * dm.hkv));
  kern<<<g1, SC_THREADS, smem, st>>>(dm, static_cast<const T*>(a->q), a->k_code,
                                     static_cast<const T*>(a->k_scale), static_cast<const T*>(a->k_mn),
                                     static_cast<const T*>(a->k_fp), scores);
  int rc = check_launch();
  if (rc != CQ_OK) return rc;
  stats_kernel<T><<<(unsigned)(dm.batch * dm.hq), 256, 0, st>>>(dm, scores, mask, stats);
  rc = check_launch();
  if (rc != CQ_OK) return rc;
  dim3 g3((unsigned)(dm.n_vis_splits + dm.n_fp_splits), (unsigned)(dm.batch * dm.hkv));
  av_kernel<T, BITS><<<g3, AV_THREADS, 0, st>>>(dm, scores, mask, stats, a->v_code,
                                                static_cast<const T*>(a->v_scale),
                                                static_cast<const T*>(a->v_mn),
                                                static_cast<const T*>(a->v_fp), partial);
  rc = check_launch();
  if (rc != CQ_OK) return rc;
  combine_kernel<T><<<(unsigned)(dm.batch * dm.hq), kHeadDim, 0, st>>>(
      partial, dm.n_vis_splits + dm.n_fp_splits, static_cast<T*>(a->out));
  return check_launch();
}

template <typename T>
static int run_decode_bits(const cq_decode_args* a, const DecodeDims& dm, const WsLayout& w,
                           unsigned char* ws, cudaStream_t st) {
  switch (a->bits) {
    case 1: return run_decode<T, 1>(a, dm, w, ws, st);
    case 2: return run_decode<T, 2>(a, dm, w, ws, st);
    default: return run_decode<T, 4>(a, dm, w, ws, st);
  }
}

}  // namespace cq

extern "C" size_t cq_decode_attn_workspace_bytes(const cq_decode_args* args) {
  if (cq::validate(args) != CQ_OK) return 0;
  if (cq::mma_path_eligible(args)) return cq::mma_path_workspace_bytes(args);
  return cq::make_layout(cq::make_dims(args)).total;
}

static int decode_attn_impl(const cq_decode_args* args, void* workspace, size_t workspace_bytes, void* stream,
                            int* status_word) {
  int rc = cq::validate(args);
  if (rc != CQ_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cq::mma_path_eligible(args)) {
    if (!workspace || workspace_bytes < cq::mma_path_workspace_bytes(args) || !cq::aligned16(workspace))
      return CQ_ERR_WORKSPACE;
    return cq::mma_path_run(args, workspace, st, nullptr, status_word);
  }
  if (args->t_fp_dev) return CQ_ERR_UNSUPPORTED;   // device-side token count: tensor-core path only
  if ((int64_t)args->batch * args->n_kv_heads > 65535) return CQ_ERR_UNSUPPORTED;   // grid.y of the general kernels
  const cq::DecodeDims dm = cq::make_dims(args);
  const cq::WsLayout w = cq::make_layout(dm);
  if (!workspace || workspace_bytes < w.total || !cq::aligned16(workspace)) return CQ_ERR_WORKSPACE;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  if (args->dtype == CQ_DTYPE_F16) return cq::run_decode_bits<__half>(args, dm, w, ws, st);
  return cq::run_decode_bits<__nv_bfloat16>(args, dm, w, ws, st);
}

extern "C" int cq_decode_attn(const cq_decode_args* args, void* workspace, size_t workspace_bytes,
                              void* stream) {
  return decode_attn_impl(args, workspace, workspace_bytes, stream, nullptr);
}

// ---- per-launch timing of one step (tensor-core path) ------------------------------------------------
extern "C" int cq_decode_attn_profile(const cq_decode_args* args, void* workspace, size_t workspace_bytes,
                                      void* stream, float* launch_ms) {
  if (!launch_ms) return CQ_ERR_BAD_ARG;
  int rc = cq::validate(args);
  if (rc != CQ_OK) return rc;
  if (!cq::mma_path_eligible(args)) return CQ_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < cq::mma_path_workspace_bytes(args) || !cq::aligned16(workspace))
    return CQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaEvent_t ev[5] = {};
  for (int i = 0; i < 5; ++i)
    if (cudaEventCreate(&ev[i]) != cudaSuccess) rc = CQ_ERR_LAUNCH;
  if (rc == CQ_OK) rc = cq::mma_path_run(args, workspace, st, ev);
  if (rc == CQ_OK && cudaEventSynchronize(ev[4]) != cudaSuccess) rc = CQ_ERR_LAUNCH;
  for (int i = 0; i < 4 && rc == CQ_OK; ++i)
    if (cudaEventElapsedTime(&launch_ms[i], ev[i], ev[i + 1]) != cudaSuccess) rc = CQ_ERR_LAUNCH;
  for (int i = 0; i < 5; ++i)
    if (ev[i]) cudaEventDestroy(ev[i]);
  return rc;
}

// ---- sticky device status of a workspace --------------------------------------------------------------
extern "C" int cq_workspace_status(const void* workspace, void* stream) {
  if (!workspace) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int word = 0;
  if (cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return CQ_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return CQ_ERR_LAUNCH;
  return word == 0 ? CQ_OK : (word == CQ_ERR_TIMEOUT ? CQ_ERR_TIMEOUT : CQ_ERR_LAUNCH);
}

// ---- the same step for callers whose query and result live in host memory -------------------------
namespace cq {
static size_t host_stage_bytes(const cq_decode_args* a) {
  return align_up((size_t)a->batch * a->n_q_heads * kHeadDim * 2, 256);
}
// Page-locked query rows -> their device staging rows, 16 bytes per thread, read over the host link by the kernel
// itself.  The score launch that follows is a programmatic dependent launch: it sets up its barriers and streams its
// first key tiles while this copy runs, and touches the query only after it (griddepcontrol.wait); behind a
// copy-engine transfer it could not start early.
__global__ void stage_query_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int n) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i];
}
// device-visible address of a page-locked host buffer, or nullptr for pageable memory (asked on every
// call: an address can change from page-locked to pageable between calls)
static void* mapped_host_ptr(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) == cudaSuccess && attr.type == cudaMemoryTypeHost) return attr.devicePointer;
  (void)cudaGetLastError();
  return nullptr;
}
// One page-locked, device-mapped status word per device for the host-buffer entry point: a kernel whose
// bounded wait runs out stores into it directly, and the host reads it after the stream has drained, without
// a copy of its own.  Made on the first call on a device (the one allocation of this entry point) and kept.
struct HostStatus { volatile int* host; int* dev; };
static int host_status_word(HostStatus* out) {
  static std::mutex mu;
  static HostStatus words[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CQ_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev].host) {
    void* h = nullptr; void* d = nullptr;
    if (cudaHostAlloc(&h, 64, cudaHostAllocMapped) != cudaSuccess) return CQ_ERR_LAUNCH;
    if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) { cudaFreeHost(h); return CQ_ERR_LAUNCH; }
    *static_cast<int*>(h) = 0;
    words[dev].host = static_cast<volatile int*>(h);
    words[dev].dev = static_cast<int*>(d);
  }
  *out = words[dev];
  return CQ_OK;
}
}  // namespace cq

extern "C" int* cq_host_status_word(void) {
  cq::HostStatus hs;
  return cq::host_status_word(&hs) == CQ_OK ? const_cast<int*>(hs.host) : nullptr;
}

extern "C" size_t cq_decode_attn_host_workspace_bytes(const cq_decode_args* args) {
  if (!args) return 0;
  cq_decode_args a = *args;                       // q / out are not device operands here
  a.q = reinterpret_cast<const void*>(uintptr_t(256));
  a.out = reinterpret_cast<void*>(uintptr_t(256));
  const size_t base = cq_decode_attn_workspace_bytes(&a);
  if (base == 0) return 0;
  return cq::align_up(base, 256) + 2 * cq::host_stage_bytes(&a);
}

extern "C" int cq_decode_attn_host(const cq_decode_args* args, const void* q_host, void* out_host,
                                   void* workspace, size_t workspace_bytes, void* stream) {
  if (!args || !q_host || !out_host) return CQ_ERR_BAD_ARG;
  if (!workspace) return CQ_ERR_WORKSPACE;
  cq_decode_args a = *args;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  a.q = ws; a.out = ws;                           // placeholders for the argument check
  const int ok = cq::validate(&a);
  if (ok != CQ_OK) return ok;
  const size_t stage = cq::host_stage_bytes(&a);
  const size_t base = cq_decode_attn_workspace_bytes(&a);
  const size_t base_al = cq::align_up(base, 256);
  if (!workspace || workspace_bytes < base_al + 2 * stage || !cq::aligned16(workspace)) return CQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  void* q_dev = ws + base_al;
  void* out_stage = ws + base_al + stage;
  const size_t bytes = (size_t)a.batch * a.n_q_heads * cq::kHeadDim * 2;
  const void* q_map = cq::aligned16(q_host) ? cq::mapped_host_ptr(q_host) : nullptr;
  if (q_map) {
    const int n16 = (int)(bytes / 16);
    cq::stage_query_kernel<<<(n16 + 255) / 256, 256, 0, st>>>(static_cast<const uint4*>(q_map), static_cast<uint4*>(q_dev), n16);
    if (cudaGetLastError() != cudaSuccess) return CQ_ERR_LAUNCH;
  } else if (cudaMemcpyAsync(q_dev, q_host, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) {
    return CQ_ERR_LAUNCH;
  }
  // page-locked result buffer: the last launch stores straight into it; pageable: staged copy
  void* out_map = cq::aligned16(out_host) ? cq::mapped_host_ptr(out_host) : nullptr;
  a.q = q_dev;
  a.out = out_map ? out_map : out_stage;
  // a bounded device-side wait that runs out leaves out_host unwritten or stale: the kernels report it in a
  // host-visible word that is read once the stream has drained (sticky, like the word of a workspace)
  cq::HostStatus hs;
  int rc = cq::host_status_word(&hs);
  if (rc != CQ_OK) return rc;
  rc = decode_attn_impl(&a, workspace, base, st, hs.dev);
  if (rc != CQ_OK) return rc;
  if (!out_map && cudaMemcpyAsync(out_host, out_stage, bytes, cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return CQ_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return CQ_ERR_LAUNCH;
  return *hs.host == 0 ? CQ_OK : CQ_ERR_TIMEOUT;
}
