// CalibQuant uint8 format: whole-span per-channel min-max quantizer with a clip factor, MSB-first
// byte packing, and the two look-up-table vector-matrix products of the decode step.
//
// Reference semantics (every torch op rounds to the tensor dtype):
//   quant   calibquant.py:24-42   x_min = rnd(amin_t(x)*clip), x_max = rnd(amax_t(x)*clip)
//                                 s  = rnd(rnd(x_max - x_min)/(2^b-1)),  zp = rnd(-x_min / s)
//                                 x_q = round_half_even(clamp(rnd(rnd(x/s) + zp), 0, 2^b-1))
//   encode  calibquant.py:114-137 byte j of a token holds channels j*dpe .. j*dpe+dpe-1, channel i
//                                 at bit offset b*(dpe-1-i)              (dpe = 8/b)
//   fused_kernel    calibquant.py:54-111   s[t] = sum_d w[d]*LUT[code[t,d]]   fp32 acc, fp16 out
//   fused_kernel_wv calibquant.py:192-276  o[d] = sum_t w[t]*LUT[code[t,d]]   fp32 acc, fp16 out
// Layouts: x [B,T,H,D] (strided), codes/enc [B,H,T,*], scale/zp [B,H,D] (the reference keeps them
// as [B,1,H,D]; same memory).  D == 128.
#include <type_traits>

#include "cq_common.cuh"
#include "cq_ptx.cuh"

namespace cq {
namespace calib {

template <typename T> struct Pk2;
template <> struct Pk2<__half> { static __device__ __forceinline__ __half2 magic() { return __float2half2_rn(1024.f); } };
template <> struct Pk2<__nv_bfloat16> { static __device__ __forceinline__ __nv_bfloat162 magic() { return __float2bfloat162_rn(128.f); } };

constexpr int MM_SLICES = 8;   // token slices per (b,h) in the min/max kernel

// ---- per-channel min/max over tokens -> scale, zero point -----------------------------------------
template <typename T>
__global__ void __launch_bounds__(kHeadDim * MM_SLICES)
minmax_kernel(const T* __restrict__ x, int heads, int t_len, int64_t sb, int64_t st, int64_t sh,
              float clip, int levels, T* __restrict__ scale, T* __restrict__ zp) {
  __shared__ float mn_s[MM_SLICES][kHeadDim], mx_s[MM_SLICES][kHeadDim];
  const int bh = blockIdx.x, b = bh / heads, h = bh % heads;
  const int d = threadIdx.x % kHeadDim, sl = threadIdx.x / kHeadDim;
  const T* p = x + b * sb + h * sh + d;
  float mn = INFINITY, mx = -INFINITY;
  for (int t = sl; t < t_len; t += MM_SLICES) {
    const float v = Elem<T>::to_f(p[(int64_t)t * st]);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  mn_s[sl][d] = mn;
  mx_s[sl][d] = mx;
  __syncthreads();
  if (sl == 0) {
    for (int i = 1; i < MM_SLICES; ++i) {
      mn = fminf(mn, mn_s[i][d]);
      mx = fmaxf(mx, mx_s[i][d]);
    }
    const float x_min = rnd<T>(mn * clip), x_max = rnd<T>(mx * clip);
    const float s = rnd<T>(__fdiv_rn(rnd<T>(x_max - x_min), (float)levels));
    const float z = rnd<T>(__fdiv_rn(-x_min, s));
    scale[(int64_t)bh * kHeadDim + d] = Elem<T>::from_f(s);
    zp[(int64_t)bh * kHeadDim + d] = Elem<T>::from_f(z);
  }
}

// ---- the same reduction spread over the whole GPU ---------------------------------------------------
// One (batch, head) per CTA leaves most SMs idle when there are few heads, so the token axis is cut into
// slices: CTA = (slice, batch x head), thread = 8 channels (one 128-bit load) of every 16th token, packed
// 16-bit min/max (exact).  The slices meet in the output arrays themselves, which hold the running
// minimum (scale array) and maximum (zero-point array) as order-preserving 16-bit keys updated by
// compare-and-swap; a last launch turns them into scale and zero point with the arithmetic of minmax_kernel.
__device__ __forceinline__ unsigned short key16(unsigned short b) {
  return (b & 0x8000u) ? (unsigned short)~b : (unsigned short)(b | 0x8000u);
}
__device__ __forceinline__ unsigned short unkey16(unsigned short k) {
  return (k & 0x8000u) ? (unsigned short)(k & 0x7fffu) : (unsigned short)~k;
}
__global__ void minmax_init_kernel(unsigned short* __restrict__ mn_key, unsigned short* __restrict__ mx_key, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) { mn_key[i] = 0xffffu; mx_key[i] = 0u; }
}

template <typename T>
__global__ void __launch_bounds__(256)
minmax_slice_kernel(const T* __restrict__ x, int heads, int t_len, int64_t sb, int64_t st, int64_t sh,
                    unsigned short* __restrict__ mn_key, unsigned short* __restrict__ mx_key) {
  using T2 = typename Elem<T>::T2;
  __shared__ uint32_t red_s[8][16][8];
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int tid = threadIdx.x, col = tid & 15, tl = tid >> 4;
  const int per = (t_len + gridDim.x - 1) / gridDim.x;
  const int t_begin = blockIdx.x * per, t_end = min(t_len, t_begin + per);
  if (t_begin >= t_end) return;                       // uniform over the CTA
  const T* base = x + b * sb + h * sh + col * 8;
  // every thread starts from a row of its slice, so no neutral element is needed
  uint4 first = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)min(t_begin + tl, t_end - 1) * st));
  T2 mn[4], mx[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) mn[i] = mx[i] = reinterpret_cast<const T2*>(&first)[i];
  for (int t = t_begin + tl; t < t_end; t += 64) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int tt = t + 16 * u < t_end ? t + 16 * u : t;
      v[u] = __ldg(reinterpret_cast<const uint4*>(base + (int64_t)tt * st));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        mn[i] = __hmin2(mn[i], reinterpret_cast<const T2*>(&v[u])[i]);
        mx[i] = __hmax2(mx[i], reinterpret_cast<const T2*>(&v[u])[i]);
      }
  }
  // the two token lanes of a warp, then the eight warps
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t a = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&mn[i]), 16);
    uint32_t c = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<uint32_t*>(&mx[i]), 16);
    mn[i] = __hmin2(mn[i], *reinterpret_cast<T2*>(&a));
    mx[i] = __hmax2(mx[i], *reinterpret_cast<T2*>(&c));
  }
  if ((tid & 31) < 16) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      red_s[tid >> 5][col][i] = *reinterpret_cast<uint32_t*>(&mn[i]);
      red_s[tid >> 5][col][4 + i] = *reinterpret_cast<uint32_t*>(&mx[i]);
    }
  }
  __syncthreads();
  if (tid < kHeadDim) {
    const int c8 = tid >> 3, e = tid & 7;
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float2 a = Elem<T>::to_f2(*reinterpret_cast<const T2*>(&red_s[w][c8][e >> 1]));
      const float2 c = Elem<T>::to_f2(*reinterpret_cast<const T2*>(&red_s[w][c8][4 + (e >> 1)]));
      lo = fminf(lo, (e & 1) ? a.y : a.x);
      hi = fmaxf(hi, (e & 1) ? c.y : c.x);
    }
    const T lo_t = Elem<T>::from_f(lo), hi_t = Elem<T>::from_f(hi);      // exact: they are elements of x
    const unsigned short klo = key16(*reinterpret_cast<const unsigned short*>(&lo_t));
    const unsigned short khi = key16(*reinterpret_cast<const unsigned short*>(&hi_t));
    unsigned short* pmn = mn_key + (int64_t)bh * kHeadDim + tid;
    unsigned short* pmx = mx_key + (int64_t)bh * kHeadDim + tid;
    unsigned short old = *pmn;
    while (klo < old) {
      const unsigned short seen = atomicCAS(pmn, old, klo);
      if (seen == old) break;
      old = seen;
    }
    old = *pmx;
    while (khi > old) {
      const unsigned short seen = atomicCAS(pmx, old, khi);
      if (seen == old) break;
      old = seen;
    }
  }
}

template <typename T>
__global__ void minmax_finish_kernel(T* __restrict__ scale, T* __restrict__ zp, int n, float clip, int levels) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const unsigned short bl = unkey16(reinterpret_cast<const unsigned short*>(scale)[i]);
  const unsigned short bh = unkey16(reinterpret_cast<const unsigned short*>(zp)[i]);
  const float mn = Elem<T>::to_f(*reinterpret_cast<const T*>(&bl)), mx = Elem<T>::to_f(*reinterpret_cast<const T*>(&bh));
  const float x_min = rnd<T>(mn * clip), x_max = rnd<T>(mx * clip);
  const float s = rnd<T>(__fdiv_rn(rnd<T>(x_max - x_min), (float)levels));
  const float z = rnd<T>(__fdiv_rn(-x_min, s));
  scale[i] = Elem<T>::from_f(s);
  zp[i] = Elem<T>::from_f(z);
}

// ---- quantize (+ optional dequantize) and/or encode ---------------------------------------------
// thread = 8 consecutive channels of one token.  xq_out (optional, layout of x, contiguous
// [B,T,H,D]) receives the codes as numbers of the data dtype (post_scale) or the dequantized values;
// enc_out (optional) receives the packed bytes [B,H,T,D*bits/8].
template <typename T, int BITS>
__global__ void __launch_bounds__(256)
quantize_kernel(const T* __restrict__ x, int heads, int t_len, int64_t sb, int64_t st, int64_t sh,
                const T* __restrict__ scale, const T* __restrict__ zp, int dequantize,
                T* __restrict__ xq_out, uint8_t* __restrict__ enc_out, int64_t n_chunks) {
  constexpr int LEVELS = (1 << BITS) - 1;
  const int64_t chunk = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (chunk >= n_chunks) return;
  const int c8 = (int)(chunk % 16);                 // which 8-channel chunk of the 128
  const int64_t bth = chunk / 16;
  const int h = (int)(bth % heads);
  const int64_t bt = bth / heads;
  const int t = (int)(bt % t_len), b = (int)(bt / t_len);
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + b * sb + (int64_t)t * st + h * sh) + c8);
  const uint4 sraw = __ldg(reinterpret_cast<const uint4*>(scale + ((int64_t)b * heads + h) * kHeadDim) + c8);
  const uint4 zraw = __ldg(reinterpret_cast<const uint4*>(zp + ((int64_t)b * heads + h) * kHeadDim) + c8);
  const T* xv = reinterpret_cast<const T*>(&raw);
  const T* sv = reinterpret_cast<const T*>(&sraw);
  const T* zv = reinterpret_cast<const T*>(&zraw);
  unsigned codes[8];
  uint4 outw;
  T* ov = reinterpret_cast<T*>(&outw);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float s = Elem<T>::to_f(sv[i]), z = Elem<T>::to_f(zv[i]);
    float y = rnd<T>(rnd<T>(__fdiv_rn(Elem<T>::to_f(xv[i]), s)) + z);
    y = rintf(fminf(fmaxf(y, 0.f), (float)LEVELS));
    codes[i] = (unsigned)y;
    ov[i] = Elem<T>::from_f(dequantize ? rnd<T>(s * rnd<T>(y - z)) : y);
  }
  if (xq_out) reinterpret_cast<uint4*>(xq_out)[chunk] = outw;
  if (enc_out) {
    // MSB-first: channel i of a byte at bit BITS*(dpe-1-i)
    uint8_t* dst = enc_out + ((((int64_t)b * heads + h) * t_len + t) * (kHeadDim * BITS / 8)) + c8 * BITS;
    if (BITS == 1) {
      unsigned v = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) v |= codes[i] << (7 - i);
      dst[0] = (uint8_t)v;
    } else if (BITS == 2) {
      const unsigned v0 = (codes[0] << 6) | (codes[1] << 4) | (codes[2] << 2) | codes[3];
      const unsigned v1 = (codes[4] << 6) | (codes[5] << 4) | (codes[6] << 2) | codes[7];
      *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(v0 | (v1 << 8));
    } else {
      unsigned v = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) v |= ((codes[2 * j] << 4) | codes[2 * j + 1]) << (8 * j);
      *reinterpret_cast<uint32_t*>(dst) = v;
    }
  }
}

// ---- 1- and 2-bit codes without a division per element ----------------------------------------------
// With scale > 0 the reference's code  rint(clamp(rnd(rnd(x / s) + z)))  is a non-decreasing step function
// of x, and s, z are fixed per channel for the whole span.  So per channel and level k there is a largest
// number theta_k of the data type whose code is <= k, found once per CTA by bisection over the ordered
// 16-bit patterns with the reference arithmetic itself (IEEE division), and  code(x) = sum_k [x > theta_k]
// holds exactly for every x.  CTA = (token range, batch x head); thread = the same 8 channels of every
// 16th token, thresholds in registers; channels with a degenerate scale make the CTA fall back to the
// per-element arithmetic.
constexpr int QT_TOKENS = 2048;        // tokens per CTA

template <typename T>
__device__ __forceinline__ float ref_code(float x, float s, float z, int levels) {
  const float y = rnd<T>(rnd<T>(__fdiv_rn(x, s)) + z);
  return rintf(fminf(fmaxf(y, 0.f), (float)levels));
}
template <typename T> struct Finite16;
template <> struct Finite16<__half> { static constexpr unsigned short MAXPOS = 0x7bffu; };
template <> struct Finite16<__nv_bfloat16> { static constexpr unsigned short MAXPOS = 0x7f7fu; };

template <typename T, int BITS>
__global__ void __launch_bounds__(256)
quantize_thr_kernel(const T* __restrict__ x, int heads, int t_len, int64_t sb, int64_t st, int64_t sh,
                    const T* __restrict__ scale, const T* __restrict__ zp,
                    T* __restrict__ xq_out, uint8_t* __restrict__ enc_out) {
  using T2 = typename Elem<T>::T2;
  constexpr int LEVELS = (1 << BITS) - 1;
  __shared__ __align__(16) T thr_s[LEVELS][kHeadDim];
  const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
  const int tid = threadIdx.x;
  const int t0 = blockIdx.x * QT_TOKENS, n_tok = min(QT_TOKENS, t_len - t0);
  int bad = 0;
  if (tid < kHeadDim) {
    const float s = Elem<T>::to_f(scale[(int64_t)bh * kHeadDim + tid]);
    const float z = Elem<T>::to_f(zp[(int64_t)bh * kHeadDim + tid]);
    bad = !(s > 0.f) || isinf(s) || isnan(z) || isinf(z);
    if (!bad) {
      const unsigned short k_min = key16((unsigned short)(Finite16<T>::MAXPOS | 0x8000u)), k_max = key16(Finite16<T>::MAXPOS);
#pragma unroll
      for (int k = 0; k < LEVELS; ++k) {
        unsigned lo = k_min, hi = k_max;
        unsigned short theta;
        const unsigned short b_lo = unkey16((unsigned short)lo), b_hi = unkey16((unsigned short)hi);
        if (ref_code<T>(Elem<T>::to_f(*reinterpret_cast<const T*>(&b_lo)), s, z, LEVELS) > (float)k) {
          theta = 0xfc00u;                              // every finite number exceeds level k: -inf
          if (sizeof(T) == 2 && Finite16<T>::MAXPOS == 0x7f7fu) theta = 0xff80u;
        } else if (ref_code<T>(Elem<T>::to_f(*reinterpret_cast<const T*>(&b_hi)), s, z, LEVELS) <= (float)k) {
          theta = b_hi;                                 // only +inf exceeds the largest finite number
        } else {
          while (hi - lo > 1) {
            const unsigned mid = (lo + hi) >> 1;
            const unsigned short bm = unkey16((unsigned short)mid);
            if (ref_code<T>(Elem<T>::to_f(*reinterpret_cast<const T*>(&bm)), s, z, LEVELS) <= (float)k) lo = mid; else hi = mid;
          }
          theta = unkey16((unsigned short)lo);
        }
        thr_s[k][tid] = *reinterpret_cast<const T*>(&theta);
      }
    }
  }
  const int any_bad = __syncthreads_or(bad);
  const int c8 = tid & 15, tl = tid >> 4;
  const T* src = x + b * sb + h * sh + c8 * 8;
  if (any_bad) {                                       // uniform: the reference arithmetic per element
    const uint4 sraw = *reinterpret_cast<const uint4*>(scale + (int64_t)bh * kHeadDim + c8 * 8);
    const uint4 zraw = *reinterpret_cast<const uint4*>(zp + (int64_t)bh * kHeadDim + c8 * 8);
    const T* sv = reinterpret_cast<const T*>(&sraw);
    const T* zv = reinterpret_cast<const T*>(&zraw);
    for (int t = tl; t < n_tok; t += 16) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)(t0 + t) * st));
      const T* xv = reinterpret_cast<const T*>(&raw);
      unsigned codes[8];
      uint4 outw;
      T* ov = reinterpret_cast<T*>(&outw);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float y = ref_code<T>(Elem<T>::to_f(xv[i]), Elem<T>::to_f(sv[i]), Elem<T>::to_f(zv[i]), LEVELS);
        codes[i] = (unsigned)y;
        ov[i] = Elem<T>::from_f(y);
      }
      const int64_t chunk = (((int64_t)b * t_len + t0 + t) * heads + h) * 16 + c8;
      if (xq_out) reinterpret_cast<uint4*>(xq_out)[chunk] = outw;
      if (enc_out) {
        uint8_t* dst = enc_out + (((int64_t)bh * t_len + t0 + t) * (kHeadDim * BITS / 8)) + c8 * BITS;
        if (BITS == 1) {
          unsigned v = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) v |= codes[i] << (7 - i);
          dst[0] = (uint8_t)v;
        } else {
          const unsigned v0 = (codes[0] << 6) | (codes[1] << 4) | (codes[2] << 2) | codes[3];
          const unsigned v1 = (codes[4] << 6) | (codes[5] << 4) | (codes[6] << 2) | codes[7];
          *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(v0 | (v1 << 8));
        }
      }
    }
    return;
  }
  T2 thr[LEVELS][4];
#pragma unroll
  for (int k = 0; k < LEVELS; ++k) {
    const uint4 w = *reinterpret_cast<const uint4*>(&thr_s[k][c8 * 8]);
#pragma unroll
    for (int i = 0; i < 4; ++i) thr[k][i] = reinterpret_cast<const T2*>(&w)[i];
  }
  for (int t = tl; t < n_tok; t += 16) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)(t0 + t) * st));
    const T2* xv = reinterpret_cast<const T2*>(&raw);
    T2 cnt[4];                                         // codes as numbers of the data type
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      cnt[i] = __hgt2(xv[i], thr[0][i]);
#pragma unroll
      for (int k = 1; k < LEVELS; ++k) cnt[i] = __hadd2(cnt[i], __hgt2(xv[i], thr[k][i]));
    }
    if (xq_out) {
      const int64_t chunk = (((int64_t)b * t_len + t0 + t) * heads + h) * 16 + c8;
      reinterpret_cast<uint4*>(xq_out)[chunk] = *reinterpret_cast<const uint4*>(cnt);
    }
    if (enc_out) {
      uint8_t* dst = enc_out + (((int64_t)bh * t_len + t0 + t) * (kHeadDim * BITS / 8)) + c8 * BITS;
      if (BITS == 1) {
        // MSB-first: channel i at bit 7 - i; pair p = channels (2p, 2p+1) -> bits 7-2p (low half), 22-2p (high half)
        unsigned r = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          r |= __hgt2_mask(xv[i], thr[0][i]) & ((0x80u >> (2 * i)) | (0x400000u >> (2 * i)));
        dst[0] = (uint8_t)((r | (r >> 16)) & 0xffu);
      } else {
        unsigned c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const T2 m = __hadd2(cnt[i], Pk2<T>::magic());          // 0..3 in the low mantissa bits
          const unsigned u = *reinterpret_cast<const unsigned*>(&m) & 0x00030003u;
          c[i] = ((u & 0xffffu) << 2) | (u >> 16);                // (code 2i, code 2i+1) as four bits
        }
        *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(((c[0] << 4) | c[1]) | (((c[2] << 4) | c[3]) << 8));
      }
    }
  }
}

// ---- encode integer codes [rows, D] (int64) -> bytes ---------------------------------------------
template <int BITS>
__global__ void encode_i64_kernel(const int64_t* __restrict__ codes, uint8_t* __restrict__ out, int64_t n_bytes) {
  constexpr int DPE = 8 / BITS;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_bytes) return;
  unsigned v = 0;
#pragma unroll
  for (int j = 0; j < DPE; ++j) v += (unsigned)codes[i * DPE + j] << (BITS * (DPE - 1 - j));
  out[i] = (uint8_t)v;
}

__device__ __forceinline__ unsigned code_at(const uint8_t* row, int d, int bits) {
  const int dpe = 8 / bits;
  return (row[d / dpe] >> (bits * (dpe - 1 - d % dpe))) & ((1u << bits) - 1u);
}

// ---- s[b,h,t] = sum_d w[b,h,d]*LUT[code[b,hk,t,d]] : warp per token, lane owns 4 channels ------------
template <typename T>
__global__ void __launch_bounds__(256)
lut_scores_kernel(const T* __restrict__ lut, const T* __restrict__ w, const uint8_t* __restrict__ enc,
                  int hq, int hkv_enc, int t_len, int bits, __half* __restrict__ out) {
  __shared__ float w_s[kMaxRep][kHeadDim];
  __shared__ float lut_s[16];
  const int bhk = blockIdx.y, b = bhk / hkv_enc, hk = bhk % hkv_enc;
  const int n_rep = hq / hkv_enc;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < n_rep * kHeadDim; i += blockDim.x)
    w_s[i / kHeadDim][i % kHeadDim] = Elem<T>::to_f(w[((int64_t)b * hq + (int64_t)hk * n_rep) * kHeadDim + i]);
  if (threadIdx.x < (1 << bits)) lut_s[threadIdx.x] = Elem<T>::to_f(lut[threadIdx.x]);
  __syncthreads();
  const int row_bytes = kHeadDim * bits / 8;
  for (int t = blockIdx.x * 8 + warp; t < t_len; t += gridDim.x * 8) {
    const uint8_t* row = enc + ((int64_t)bhk * t_len + t) * row_bytes;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = lut_s[code_at(row, lane * 4 + i, bits)];
    for (int r = 0; r < n_rep; ++r) {
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) dot = fmaf(w_s[r][lane * 4 + i], v[i], dot);
      dot = warp_sum(dot);
      if (lane == 0) out[((int64_t)b * hq + (int64_t)hk * n_rep + r) * t_len + t] = __float2half_rn(dot);
    }
  }
}

// ---- o[b,h,d] = sum_t w[b,h,t]*LUT[code[b,hk,t,d]] : thread = channel, split over tokens ------------
constexpr int WV_TCHUNK = 256;
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
lut_out_partial_kernel(const T* __restrict__ lut, const T* __restrict__ w, const uint8_t* __restrict__ enc,
                       int hq, int hkv_enc, int t_len, int bits, float* __restrict__ partial, int n_rows) {
  __shared__ float w_s[kMaxRep][WV_TCHUNK];
  __shared__ float lut_s[16];
  const int bhk = blockIdx.y, b = bhk / hkv_enc, hk = bhk % hkv_enc;
  const int n_rep = hq / hkv_enc;
  const int t0 = blockIdx.x * WV_TCHUNK, nt = min(WV_TCHUNK, t_len - t0);
  const int d = threadIdx.x;
  for (int i = threadIdx.x; i < n_rep * WV_TCHUNK; i += blockDim.x) {
    const int r = i / WV_TCHUNK, tt = i % WV_TCHUNK;
    w_s[r][tt] = tt < nt ? Elem<T>::to_f(w[((int64_t)b * hq + (int64_t)hk * n_rep + r) * t_len + t0 + tt]) : 0.f;
  }
  if (threadIdx.x < (1 << bits)) lut_s[threadIdx.x] = Elem<T>::to_f(lut[threadIdx.x]);
  __syncthreads();
  const int row_bytes = kHeadDim * bits / 8;
  const uint8_t* base = enc + ((int64_t)bhk * t_len + t0) * row_bytes;
  float acc[kMaxRep];
#pragma unroll
  for (int r = 0; r < kMaxRep; ++r) acc[r] = 0.f;
  for (int tt = 0; tt < nt; ++tt) {
    const float v = lut_s[code_at(base + (int64_t)tt * row_bytes, d, bits)];
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r)
      if (r < n_rep) acc[r] = fmaf(w_s[r][tt], v, acc[r]);
  }
#pragma unroll
  for (int r = 0; r < kMaxRep; ++r)
    if (r < n_rep)
      partial[((int64_t)blockIdx.x * n_rows + (int64_t)b * hq + (int64_t)hk * n_rep + r) * kHeadDim + d] = acc[r];
}

__global__ void lut_out_finalize_kernel(const float* __restrict__ partial, __half* __restrict__ out, int chunks,
                                        int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int c = 0; c < chunks; ++c) s += partial[(int64_t)c * total + i];
  out[i] = __float2half_rn(s);
}

using namespace ptx;

// ---- s[b,h,t] = sum_d w[b,h,d] * LUT[code[b,hk,t,d]] on the warp MMA -------------------------------------
// Valid when the LUT is affine in the code (LUT[c] = l0 + c*step, which the identity LUT is): then
//   s = l0 * sum_d w[d] + step * sum_d w[d]*code[t,d]
// and the second sum is an MMA with A = codes (rows = tokens, k = channels) and B = w.  The packed
// dimension is the contracted one here, so an A register (two k values of one token) is one AND of
// the token's code word: its low half takes a field of byte 0 (or 1), its high half the same field of
// byte 2 (or 3); the channel each k index stands for follows from that, and B is gathered to match.
// A field at bit p of a half is the fp16 subnormal code * 2^(p-24); B carries 2^(4-p), so every
// product weighs 2^-20.
template <int BITS>
struct LutMap {
  // channel that k-block kb, lane column c, slot (0: a0.lo, 1: a0.hi, 2: a2.lo, 3: a2.hi) reads, and the
  // bit position of its field inside the 16-bit half
  static __device__ __forceinline__ void get(int kb, int c, int slot, int& chan, int& pos) {
    if (BITS == 1) {             // word j = kb/2 (32 channels), bytes s, s+2 with s = kb%2
      const int j = kb >> 1, s = kb & 1;
      const int byte = s + 2 * (slot & 1);
      pos = 2 * c + (slot >> 1);
      chan = 32 * j + 8 * byte + (7 - pos);
    } else if (BITS == 2) {      // word kb (16 channels): a0 from bytes 0,2, a2 from bytes 1,3; field c
      const int byte = (slot >> 1) + 2 * (slot & 1);
      pos = 2 * c;
      chan = 16 * kb + 4 * byte + (3 - c);
    } else {                     // words 2kb (a0) and 2kb+1 (a2), 8 channels each; nibble (c&1) of byte c>>1 (+2)
      const int word = 2 * kb + (slot >> 1);
      const int byte = (c >> 1) + 2 * (slot & 1);
      pos = 0;                   // shifted down to bit 0 before masking
      chan = 8 * word + 2 * byte + (1 - (c & 1));
    }
  }
};

constexpr int LS_TOK = 64;       // tokens per warp iteration (4 m-tiles)

// Score type of the fused decode step: `fused_kernel(...) / sd - bias_k` is an fp16 tensor minus a tensor of
// the data dtype, so torch keeps fp16 for fp16 data and promotes to fp32 for bf16 data.
template <typename T> struct StepScore;
template <> struct StepScore<__half> {
  using type = __half;
  static __device__ __forceinline__ float r(float v) { return rnd<__half>(v); }
  static __device__ __forceinline__ __half make(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float load(__half v) { return __half2float(v); }
};
template <> struct StepScore<__nv_bfloat16> {
  using type = float;
  static __device__ __forceinline__ float r(float v) { return v; }
  static __device__ __forceinline__ float make(float v) { return v; }
  static __device__ __forceinline__ float load(float v) { return v; }
};

__device__ __forceinline__ void put_score(__half& dst, float v) { dst = __float2half_rn(v); }
__device__ __forceinline__ void put_score(float& dst, float v) { dst = v; }
__device__ __forceinline__ void put_half(__half& dst, __half v) { dst = v; }
__device__ __forceinline__ void put_half(float& dst, __half v) { dst = __half2float(v); }

// With STEP set this is the visual-score launch of the fused decode step (patch_internvl.py:366-372):
// `w` is the query, the weights become rnd(q * scale_key), the table is the identity and the epilogue
// applies `/ sqrt(D) - bias_k` with bias_k = sum_d(scale_key*zero_point_key*q) / sqrt(D).
struct StepScoreArgs {
  const void* scale;      // [B, scale_heads, D]
  const void* zero_point;
  int scale_heads;        // the query-head count (as the reference keeps them) or the code-head count
  void* out;              // [B,Hq,T] of StepScore<T>::type
  uint16_t* lut_out;      // receives the fp16 identity table 0..15 for the later attn.V launch
};

template <typename T, int BITS, bool STEP = false>
__global__ void __launch_bounds__(128)
lut_scores_mma_kernel(const T* __restrict__ lut, const T* __restrict__ w, const uint8_t* __restrict__ enc,
                      int hq, int hkv_enc, int t_len, __half* __restrict__ out, StepScoreArgs sa = StepScoreArgs{}) {
  using SOut = typename std::conditional<STEP, typename StepScore<T>::type, __half>::type;
  constexpr int ROW_BYTES = kHeadDim * BITS / 8;          // 16 / 32 / 64
  constexpr int WORDS = ROW_BYTES / 4;
  __shared__ float w_s[kMaxRep][kHeadDim];
  __shared__ float wsum_s[kMaxRep];
  __shared__ float lut_s[16];
  __shared__ __align__(16) SOut out_s[4][kMaxRep][LS_TOK + 8];
  __shared__ float bias_s[STEP ? kMaxRep : 1][STEP ? kHeadDim : 1];
  const int bhk = blockIdx.y, b = bhk / hkv_enc, hk = bhk % hkv_enc;
  const int n_rep = hq / hkv_enc;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int64_t row0 = (int64_t)b * hq + (int64_t)hk * n_rep;
  const float sd = sqrtf((float)kHeadDim), inv_sd = 1.f / sd;
  (void)inv_sd;
  for (int i = tid; i < kMaxRep * kHeadDim; i += 128) {
    const int r = i >> 7, d = i & (kHeadDim - 1);
    float wv = r < n_rep ? Elem<T>::to_f(w[(row0 + r) * kHeadDim + d]) : 0.f;
    if (STEP) {
      float bp = 0.f;
      if (r < n_rep) {
        const int64_t srow = sa.scale_heads == hq ? row0 + r : (int64_t)b * sa.scale_heads + hk;
        const float sk = Elem<T>::to_f(static_cast<const T*>(sa.scale)[srow * kHeadDim + d]);
        const float zk = Elem<T>::to_f(static_cast<const T*>(sa.zero_point)[srow * kHeadDim + d]);
        bp = rnd<T>(rnd<T>(sk * zk) * wv);
        wv = rnd<T>(wv * sk);
      }
      bias_s[STEP ? r : 0][STEP ? d : 0] = bp;
    }
    w_s[r][d] = wv;
  }
  if (STEP) {
    if (tid < 16) lut_s[tid] = (float)tid;
    if (blockIdx.x == 0 && blockIdx.y == 0 && tid < 16) sa.lut_out[tid] = __half_as_ushort(__float2half_rn((float)tid));
  } else if (tid < (1 << BITS)) lut_s[tid] = Elem<T>::to_f(lut[tid]);
  __syncthreads();
  for (int r = warp; r < kMaxRep; r += 4) {               // sum_d w[r][d], a warp per head
    float s = warp_sum(w_s[r][lane] + w_s[r][lane + 32] + w_s[r][lane + 64] + w_s[r][lane + 96]);
    if (STEP) {       // bias_k: the sum rounds to the data dtype, so does the division
      const int rr = STEP ? r : 0;
      const float bsum = warp_sum(bias_s[rr][STEP ? lane : 0] + bias_s[rr][STEP ? lane + 32 : 0] +
                                  bias_s[rr][STEP ? lane + 64 : 0] + bias_s[rr][STEP ? lane + 96 : 0]);
      s = rnd<T>(__fdiv_rn(rnd<T>(bsum), sd));
    }
    if (lane == 0) wsum_s[r] = s;                          // STEP: bias_k of the head
  }
  const float l0 = lut_s[0], step = lut_s[1] - lut_s[0];
  bool affine = true;
#pragma unroll
  for (int i = 2; i < (1 << BITS); ++i) affine = affine && (lut_s[i] == l0 + (float)i * step);
  __syncthreads();
  const uint8_t* base = enc + (int64_t)bhk * t_len * ROW_BYTES;

  if (!affine) {
    // arbitrary LUT: one token per warp iteration, a lane owns 4 channels
    for (int t = blockIdx.x * 4 + warp; t < t_len; t += gridDim.x * 4) {
      const uint8_t* row = base + (int64_t)t * ROW_BYTES;
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = lane * 4 + i;
        constexpr int DPE = 8 / BITS;
        v[i] = lut_s[(row[d / DPE] >> (BITS * (DPE - 1 - d % DPE))) & ((1u << BITS) - 1u)];
      }
      for (int r = 0; r < n_rep; ++r) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) dot = fmaf(w_s[r][lane * 4 + i], v[i], dot);
        dot = warp_sum(dot);
        if (lane == 0) out[(row0 + r) * t_len + t] = __float2half_rn(dot);
      }
    }
    return;
  }

  // B fragments of this lane: head n = g, eight k-blocks
  uint32_t b0[8], b1[8];
#pragma unroll
  for (int kb = 0; kb < 8; ++kb) {
    float v[4];
#pragma unroll
    for (int slot = 0; slot < 4; ++slot) {
      int chan, pos;
      LutMap<BITS>::get(kb, c, slot, chan, pos);
      v[slot] = g < n_rep ? w_s[g][chan] * exp2f((float)(4 - pos)) : 0.f;
    }
    const __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
    b0[kb] = *reinterpret_cast<const uint32_t*>(&lo);
    b1[kb] = *reinterpret_cast<const uint32_t*>(&hi);
  }
  // masks of the lane's fields: low half and high half of the register take the same field
  constexpr uint32_t FIELD = (1u << BITS) - 1u;
  const uint32_t m_a0 = BITS == 4 ? 0x000f000fu : (FIELD << (BITS == 1 ? 2 * c : 2 * c)) * 0x00010001u;
  const uint32_t m_a2 = BITS == 1 ? (1u << (2 * c + 1)) * 0x00010001u : m_a0;
  const int sh4 = 4 * (c & 1) + 8 * (c >> 1);             // 4 bits: shift that brings the lane's nibble to bit 0

  const bool vec_ok = (t_len % 8) == 0;
  for (int t0 = (blockIdx.x * 4 + warp) * LS_TOK; t0 < t_len; t0 += gridDim.x * 4 * LS_TOK) {
    // m-tile mt: rows g and g+8 of tokens t0 + 16 mt ...; at 1 and 2 bits the loads of all four m-tiles
    // are issued before the first product
#pragma unroll(BITS == 4 ? 1 : 4)
    for (int mt = 0; mt < 4; ++mt) {
      uint32_t W[2][WORDS];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int t = min(t0 + 16 * mt + g + 8 * hf, t_len - 1);
        const uint4* rp = reinterpret_cast<const uint4*>(base + (int64_t)t * ROW_BYTES);
#pragma unroll
        for (int q4 = 0; q4 < WORDS / 4; ++q4) {
          const uint4 v = __ldg(rp + q4);
          W[hf][4 * q4] = v.x; W[hf][4 * q4 + 1] = v.y; W[hf][4 * q4 + 2] = v.z; W[hf][4 * q4 + 3] = v.w;
        }
      }
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kb = 0; kb < 8; ++kb) {
        uint32_t a0, a1, a2, a3;
        if (BITS == 1) {
          const uint32_t x0 = W[0][kb >> 1] >> (8 * (kb & 1)), x1 = W[1][kb >> 1] >> (8 * (kb & 1));
          a0 = x0 & m_a0; a1 = x1 & m_a0; a2 = x0 & m_a2; a3 = x1 & m_a2;
        } else if (BITS == 2) {
          const uint32_t x0 = W[0][kb], x1 = W[1][kb];
          a0 = x0 & m_a0; a1 = x1 & m_a0; a2 = (x0 >> 8) & m_a0; a3 = (x1 >> 8) & m_a0;
        } else {
          a0 = (W[0][2 * kb] >> sh4) & m_a0; a1 = (W[1][2 * kb] >> sh4) & m_a0;
          a2 = (W[0][2 * kb + 1] >> sh4) & m_a0; a3 = (W[1][2 * kb + 1] >> sh4) & m_a0;
        }
        mma_f16(acc, a0, a1, a2, a3, b0[kb], b1[kb]);
      }
      // acc[0..1] = (token 16mt+g, heads 2c, 2c+1), acc[2..3] = (token 16mt+g+8, same heads)
      if (STEP && std::is_same<T, __half>::value) {
        // fp16 data: the three roundings of `fused_kernel(...) / sqrt(D) - bias_k` on packed pairs of heads.
        // raw / sqrt(D) is a product with the fp32 reciprocal: at most one fp32 ulp from the IEEE quotient,
        // i.e. after the rounding to fp16 one score in about 4 000 differs, by one fp16 ulp.
        const __half2 bias2 = __floats2half2_rn(wsum_s[2 * c], wsum_s[2 * c + 1]);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const float2 raw = __half22float2(__floats2half2_rn(acc[2 * hf] * 1048576.f, acc[2 * hf + 1] * 1048576.f));
          const __half2 sc = __hsub2(__floats2half2_rn(raw.x * inv_sd, raw.y * inv_sd), bias2);
          const int tt = 16 * mt + g + 8 * hf;
          if (2 * c < n_rep) put_half(out_s[warp][2 * c][tt], __low2half(sc));
          if (2 * c + 1 < n_rep) put_half(out_s[warp][2 * c + 1][tt], __high2half(sc));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int r = 2 * c + (e & 1), tt = 16 * mt + g + 8 * (e >> 1);
          if (r < n_rep) {
            if (STEP) {
              const float raw = rnd<__half>(acc[e] * 1048576.f);                      // fused_kernel's fp16 output
              put_score(out_s[warp][r][tt], StepScore<T>::r(rnd<__half>(raw * inv_sd) - wsum_s[r]));
            } else {
              put_score(out_s[warp][r][tt], fmaf(step * 1048576.f, acc[e], l0 * wsum_s[r]));
            }
          }
        }
      }
    }
    __syncwarp();
    SOut* outp = STEP ? static_cast<SOut*>(sa.out) : reinterpret_cast<SOut*>(out);
    constexpr int PER16 = 16 / (int)sizeof(SOut);          // scores per 16-byte store
    if (vec_ok && t0 + LS_TOK <= t_len) {
      for (int i = lane; i < n_rep * (LS_TOK / PER16); i += 32) {
        const int r = i / (LS_TOK / PER16), ch = i % (LS_TOK / PER16);
        *reinterpret_cast<uint4*>(outp + (row0 + r) * t_len + t0 + PER16 * ch) =
            *reinterpret_cast<const uint4*>(&out_s[warp][r][PER16 * ch]);
      }
    } else {
      for (int i = lane; i < n_rep * LS_TOK; i += 32) {
        const int r = i / LS_TOK, tt = i % LS_TOK;
        if (t0 + tt < t_len) outp[(row0 + r) * t_len + t0 + tt] = out_s[warp][r][tt];
      }
    }
    __syncwarp();
  }
}


// ---- o[b,h,d] = sum_t w[b,h,t] * LUT[code[b,hk,t,d]] on the warp MMA (affine LUT, 1 or 2 bits) ----------
// A = codes with rows = channels and k = tokens: the two tokens of an A register come from two token
// rows, merged by one byte permute; rows g and g+8 of two m-tiles share that byte (1 bit: bits
// 4(g&1)+2i+{0,1} of byte g>>1 of a 32-channel word; 2 bits: the two fields 2(g&1)+{0,1}... of byte g>>1 of a
// 16-channel word), so the permute is shared.  B = w (k = tokens, n = heads).  Each CTA takes WO_TOK
// tokens of one (batch, code head): its four warps take a quarter each, then reduce in shared memory
// and write one fp32 partial per (row, channel); a second launch sums the partials.
constexpr int WO_TOK = 1024;

template <typename T, int BITS>
__global__ void __launch_bounds__(128)
lut_out_mma_kernel(const T* __restrict__ lut, const T* __restrict__ w, const uint8_t* __restrict__ enc,
                   int hq, int hkv_enc, int t_len, float* __restrict__ partial, int n_rows) {
  constexpr int ROW_BYTES = kHeadDim * BITS / 8;          // 16 / 32 / 64
  constexpr int WORDS = ROW_BYTES / 4;                    // 4 / 8 / 16
  // m-tiles (16 channels) per code word: 2 / 1; at 4 bits an m-tile spans two words and takes its own code path
  constexpr int MT_PER_WORD = BITS == 4 ? 1 : 2 / BITS;
  __shared__ __align__(16) __half w_s[kMaxRep][WO_TOK + 8];
  __shared__ float red_s[4][kMaxRep][kHeadDim + 4];
  __shared__ float wsum_s[kMaxRep];
  __shared__ float lut_s[4];
  const int bhk = blockIdx.y, b = bhk / hkv_enc, hk = bhk % hkv_enc;
  const int n_rep = hq / hkv_enc;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int64_t row0 = (int64_t)b * hq + (int64_t)hk * n_rep;
  const int t0 = blockIdx.x * WO_TOK, nt = min(WO_TOK, t_len - t0);
  for (int i = tid; i < n_rep * WO_TOK; i += 128) {        // rows past n_rep are never read
    const int r = i / WO_TOK, tt = i % WO_TOK;
    w_s[r][tt] = __float2half_rn(tt < nt ? Elem<T>::to_f(w[(row0 + r) * t_len + t0 + tt]) : 0.f);
  }
  if (tid < (1 << BITS)) lut_s[tid] = Elem<T>::to_f(lut[tid]);
  __syncthreads();
  for (int r = warp; r < n_rep; r += 4) {                 // sum_t w[r][t] over the CTA's tokens, a warp per head
    float s = 0.f;
    for (int tt = lane; tt < WO_TOK; tt += 32) s += __half2float(w_s[r][tt]);     // zero past nt
    s = warp_sum(s);
    if (lane == 0) wsum_s[r] = s;
  }
  const float l0 = lut_s[0], step = lut_s[1] - lut_s[0];
  bool affine = true;
#pragma unroll
  for (int i = 2; i < (1 << BITS); ++i) affine = affine && (lut_s[i] == l0 + (float)i * step);
  if (!affine) {
    // arbitrary LUT: thread = channel, serial over the CTA's tokens
    float a[kMaxRep];
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r) a[r] = 0.f;
    const uint8_t* rows = enc + ((int64_t)bhk * t_len + t0) * ROW_BYTES;
    for (int tt = 0; tt < nt; ++tt) {
      const float v = lut_s[code_at(rows + (int64_t)tt * ROW_BYTES, tid, BITS)];
#pragma unroll
      for (int r = 0; r < kMaxRep; ++r)
        if (r < n_rep) a[r] = fmaf(__half2float(w_s[r][tt]), v, a[r]);
    }
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r)
      if (r < n_rep) partial[((int64_t)blockIdx.x * n_rows + row0 + r) * kHeadDim + tid] = a[r];
    return;
  }
  __syncthreads();       // wsum_s

  // lane constants: byte of the word, masks of rows g / g+8 for the m-tile(s) of a word, accumulator scales
  constexpr uint32_t FIELD = (1u << BITS) - 1u;
  const uint32_t sel = (uint32_t)((g >> 1) | ((g >> 1) << 4) | ((4 + (g >> 1)) << 8) | ((4 + (g >> 1)) << 12));
  uint32_t m0[MT_PER_WORD], m1[MT_PER_WORD];
  float sc0[MT_PER_WORD], sc1[MT_PER_WORD];
  int ch0[MT_PER_WORD], ch1[MT_PER_WORD];                 // channel inside the word's span of rows g / g+8
#pragma unroll
  for (int i = 0; i < MT_PER_WORD; ++i) {
    // bit offset inside the byte of the field row g stands for; row g+8 takes the next field
    const int p0 = BITS == 1 ? 4 * (g & 1) + 2 * i : 4 * (g & 1), p1 = p0 + BITS;
    m0[i] = (FIELD << p0) * 0x00010001u;
    m1[i] = (FIELD << p1) * 0x00010001u;
    sc0[i] = exp2f((float)(24 - p0));
    sc1[i] = exp2f((float)(24 - p1));
    // MSB-first: the field at bit offset p of byte y is channel (8/BITS)*y + (8/BITS - 1 - p/BITS)
    ch0[i] = (8 / BITS) * (g >> 1) + (8 / BITS - 1 - p0 / BITS);
    ch1[i] = (8 / BITS) * (g >> 1) + (8 / BITS - 1 - p1 / BITS);
  }
  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const uint8_t* base = enc + ((int64_t)bhk * t_len + t0) * ROW_BYTES;
  const int tw0 = warp * (WO_TOK / 4);
#pragma unroll 4
  for (int ks = 0; ks < WO_TOK / 4 / 16; ++ks) {
    const int tk = tw0 + ks * 16;                          // first token of the k-step inside the CTA's span
    if (tk >= nt) break;
    const __half* wr = &w_s[g < n_rep ? g : 0][tk + 2 * c];
    uint32_t bq0 = *reinterpret_cast<const uint32_t*>(wr), bq1 = *reinterpret_cast<const uint32_t*>(wr + 8);
    if (g >= n_rep) { bq0 = 0u; bq1 = 0u; }
    if constexpr (BITS == 4) {
      // A byte is two channels (first one in the high nibble).  Lane g takes byte g%4 of the words 4q + 2(g/4) and
      // 4q + 2(g/4) + 1 of every 32-channel quarter q (one 8-byte load per token row): rows g / g+8 of the m-tiles
      // 2q and 2q+1 are the low / high nibble of that byte, i.e. channels 8W + 2(g%4) + 1 and 8W + 2(g%4).
      const int last = nt - 1;
      const uint8_t* pa = base + (int64_t)min(tk + 2 * c, last) * ROW_BYTES + 8 * (g >> 2);
      const uint8_t* pb = base + (int64_t)min(tk + 2 * c + 1, last) * ROW_BYTES + 8 * (g >> 2);
      const uint8_t* pc = base + (int64_t)min(tk + 2 * c + 8, last) * ROW_BYTES + 8 * (g >> 2);
      const uint8_t* pd = base + (int64_t)min(tk + 2 * c + 9, last) * ROW_BYTES + 8 * (g >> 2);
      const uint32_t sel4 = (uint32_t)((g & 3) | ((g & 3) << 4) | ((4 + (g & 3)) << 8) | ((4 + (g & 3)) << 12));
      uint2 va[4], vb[4], vc[4], vd[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        va[q] = __ldg(reinterpret_cast<const uint2*>(pa + 16 * q)); vb[q] = __ldg(reinterpret_cast<const uint2*>(pb + 16 * q));
        vc[q] = __ldg(reinterpret_cast<const uint2*>(pc + 16 * q)); vd[q] = __ldg(reinterpret_cast<const uint2*>(pd + 16 * q));
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t x01a = prmt(va[q].x, vb[q].x, sel4), x89a = prmt(vc[q].x, vd[q].x, sel4);
        mma_f16(acc[2 * q], x01a & 0x000f000fu, x01a & 0x00f000f0u, x89a & 0x000f000fu, x89a & 0x00f000f0u, bq0, bq1);
        const uint32_t x01b = prmt(va[q].y, vb[q].y, sel4), x89b = prmt(vc[q].y, vd[q].y, sel4);
        mma_f16(acc[2 * q + 1], x01b & 0x000f000fu, x01b & 0x00f000f0u, x89b & 0x000f000fu, x89b & 0x00f000f0u, bq0, bq1);
      }
      continue;
    }
    // token rows 2c, 2c+1, 2c+8, 2c+9 of the k-step (clamped: tokens past the end have w = 0)
    uint32_t Wa[WORDS], Wb[WORDS], Wc[WORDS], Wd[WORDS];
    {
      const int last = nt - 1;
      const uint4* ra = reinterpret_cast<const uint4*>(base + (int64_t)min(tk + 2 * c, last) * ROW_BYTES);
      const uint4* rb = reinterpret_cast<const uint4*>(base + (int64_t)min(tk + 2 * c + 1, last) * ROW_BYTES);
      const uint4* rc = reinterpret_cast<const uint4*>(base + (int64_t)min(tk + 2 * c + 8, last) * ROW_BYTES);
      const uint4* rd = reinterpret_cast<const uint4*>(base + (int64_t)min(tk + 2 * c + 9, last) * ROW_BYTES);
#pragma unroll
      for (int q4 = 0; q4 < WORDS / 4; ++q4) {
        const uint4 va = __ldg(ra + q4), vb = __ldg(rb + q4), vc = __ldg(rc + q4), vd = __ldg(rd + q4);
        Wa[4 * q4] = va.x; Wa[4 * q4 + 1] = va.y; Wa[4 * q4 + 2] = va.z; Wa[4 * q4 + 3] = va.w;
        Wb[4 * q4] = vb.x; Wb[4 * q4 + 1] = vb.y; Wb[4 * q4 + 2] = vb.z; Wb[4 * q4 + 3] = vb.w;
        Wc[4 * q4] = vc.x; Wc[4 * q4 + 1] = vc.y; Wc[4 * q4 + 2] = vc.z; Wc[4 * q4 + 3] = vc.w;
        Wd[4 * q4] = vd.x; Wd[4 * q4 + 1] = vd.y; Wd[4 * q4 + 2] = vd.z; Wd[4 * q4 + 3] = vd.w;
      }
    }
#pragma unroll
    for (int wd = 0; wd < WORDS; ++wd) {
      const uint32_t x01 = prmt(Wa[wd], Wb[wd], sel), x89 = prmt(Wc[wd], Wd[wd], sel);
#pragma unroll
      for (int i = 0; i < MT_PER_WORD; ++i)
        mma_f16(acc[wd * MT_PER_WORD + i], x01 & m0[i], x01 & m1[i], x89 & m0[i], x89 & m1[i], bq0, bq1);
    }
  }
  // ---- reduce the four warps: acc[j][0..1] = (row g, heads 2c, 2c+1), acc[j][2..3] = (row g+8, ...)
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = j % MT_PER_WORD, span = (j / MT_PER_WORD) * (32 / BITS);   // channels covered by the word
    int d0 = span + ch0[i], d1 = span + ch1[i];
    float s0 = sc0[i], s1 = sc1[i];
    if (BITS == 4) {                     // rows g / g+8 = low / high nibble of byte g%4 of word W
      const int W = 4 * (j >> 1) + 2 * (g >> 2) + (j & 1);
      d0 = 8 * W + 2 * (g & 3) + 1; d1 = 8 * W + 2 * (g & 3);
      s0 = 16777216.f; s1 = 1048576.f;   // 2^24 for a field at bit 0, 2^20 at bit 4
    }
    if (2 * c < n_rep) { red_s[warp][2 * c][d0] = acc[j][0] * s0; red_s[warp][2 * c][d1] = acc[j][2] * s1; }
    if (2 * c + 1 < n_rep) { red_s[warp][2 * c + 1][d0] = acc[j][1] * s0; red_s[warp][2 * c + 1][d1] = acc[j][3] * s1; }
  }
  __syncthreads();
  for (int r = 0; r < n_rep; ++r) {
    const float s = red_s[0][r][tid] + red_s[1][r][tid] + red_s[2][r][tid] + red_s[3][r][tid];
    partial[((int64_t)blockIdx.x * n_rows + row0 + r) * kHeadDim + tid] = fmaf(step, s, l0 * wsum_s[r]);
  }
}



// ---- fused decode step, launch 2: full-precision scores, calibration, softmax -------------------------------
// One CTA per (batch, query head).  The whole row [sys | visual | text] lives in shared memory as fp32:
//   s_fp[t]  = rnd(rnd(q . k_fp[t]) / sqrt(D))                               patch_internvl.py:362-365
//   s_vis    = calibrated visual scores (every op rounded to the score dtype)                 :376-385
//   att      = rnd(softmax_fp32(row))                                                        :388-390
// Outputs: att over the visual span as fp16 (the weights of fused_kernel_wv, :396), att over the fp tokens in
// the data dtype, and rnd(sum of the visual att) for the zero-point term (:399).
constexpr int SM_THREADS = 1024;

__device__ __forceinline__ float block_reduce(float v, float* red, int op) {   // op 0: sum, 1: max, 2: min
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = op == 0 ? warp_sum(v) : op == 1 ? warp_max(v) : warp_min(v);
  __syncthreads();                       // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int n = (blockDim.x + 31) >> 5;
  float r = red[0];
  for (int i = 1; i < n; ++i) r = op == 0 ? r + red[i] : op == 1 ? fmaxf(r, red[i]) : fminf(r, red[i]);
  return r;
}

template <typename T>
__global__ void __launch_bounds__(SM_THREADS)
step_softmax_kernel(const T* __restrict__ q, const T* __restrict__ k_fp, int64_t fp_stride_b, int64_t fp_stride_h,
                    int hq, int hkv, int t_vis, int t_fp, int t_sys, int calibrate,
                    const typename StepScore<T>::type* __restrict__ s_vis, const T* __restrict__ mask,
                    int64_t mask_stride_b, __half* __restrict__ a_vis, T* __restrict__ a_fp,
                    float* __restrict__ a_sum, const int32_t* __restrict__ t_fp_dev, int t_fp_cap) {
  if (t_fp_dev) t_fp = min(*t_fp_dev, t_fp_cap);      // live count kept on the device; rows of a_fp stay t_fp_cap apart
  extern __shared__ float row[];         // [t_vis + t_fp], visual scores first
  __shared__ float red[32];
  __shared__ float q_s[kHeadDim];
  using SS = StepScore<T>;
  const int bh = blockIdx.x, b = bh / hq, h = bh % hq, hk = h / (hq / hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float sd = sqrtf((float)kHeadDim);
  if (tid < kHeadDim) q_s[tid] = Elem<T>::to_f(q[(int64_t)bh * kHeadDim + tid]);
  __syncthreads();
  const T* kb = k_fp + b * fp_stride_b + hk * fp_stride_h;
  for (int t = warp; t < t_fp; t += SM_THREADS / 32) {
    const T* kr = kb + (int64_t)t * kHeadDim + lane * 4;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) dot = fmaf(q_s[lane * 4 + i], Elem<T>::to_f(kr[i]), dot);
    dot = warp_sum(dot);
    if (lane == 0) row[t_vis + t] = rnd<T>(__fdiv_rn(rnd<T>(dot), sd));
  }
  const typename SS::type* sv = s_vis + (int64_t)bh * t_vis;
  float mx = -INFINITY, mn = INFINITY;
  for (int t = tid; t < t_vis; t += SM_THREADS) {
    const float v = SS::load(sv[t]);
    row[t] = v;
    mx = fmaxf(mx, v);
    mn = fminf(mn, v);
  }
  if (calibrate && t_vis > 0) {
    mx = block_reduce(mx, red, 1);
    mn = block_reduce(mn, red, 2);
    const float span = SS::r(SS::r(mx + -3.f) - mn);              // tgt_max - tgt_min
    const float denom = SS::r(SS::r(mx - mn) + 1e-8f);
    for (int t = tid; t < t_vis; t += SM_THREADS) {
      const float n = SS::r(__fdiv_rn(SS::r(row[t] - mn), denom));
      row[t] = SS::r(SS::r(n * span) + mn);
    }
  }
  __syncthreads();
  if (mask) {                            // additive mask in the original key order [sys | visual | text] (:404-410)
    const T* mr = mask + b * mask_stride_b;
    for (int t = tid; t < t_vis; t += SM_THREADS) row[t] = SS::r(row[t] + Elem<T>::to_f(mr[t_sys + t]));
    for (int t = tid; t < t_fp; t += SM_THREADS)
      row[t_vis + t] = SS::r(row[t_vis + t] + Elem<T>::to_f(mr[t < t_sys ? t : t_vis + t]));
    __syncthreads();
  }
  const int total = t_vis + t_fp;
  float m = -INFINITY;
  for (int t = tid; t < total; t += SM_THREADS) m = fmaxf(m, row[t]);
  m = block_reduce(m, red, 1);
  float sum = 0.f;
  for (int t = tid; t < total; t += SM_THREADS) {
    const float e = __expf(row[t] - m);
    row[t] = e;
    sum += e;
  }
  sum = block_reduce(sum, red, 0);
  const float inv = 1.f / sum;
  float vs = 0.f;
  for (int t = tid; t < t_vis; t += SM_THREADS) {
    const float a = rnd<T>(row[t] * inv);
    a_vis[(int64_t)bh * t_vis + t] = __float2half_rn(a);
    vs += a;
  }
  for (int t = tid; t < t_fp; t += SM_THREADS) a_fp[(int64_t)bh * t_fp_cap + t] = Elem<T>::from_f(row[t_vis + t] * inv);
  vs = block_reduce(vs, red, 0);
  if (tid == 0) a_sum[bh] = rnd<T>(vs);
}

// The same launch for fp16 data without a mask and with t_vis % 8 == 0: the visual scores are fp16 numbers and stay
// fp16 through the calibration (every op of it rounds to fp16), so the row is kept as packed halves (half the
// shared memory: two CTAs per SM, one wave for 256 heads), the calibration runs on packed fp16 arithmetic, whose
// single rounding per op is the reference's, and the exponentials are recomputed in the last pass instead of stored.
constexpr int SMH_THREADS = 512;

__device__ __forceinline__ float ex2_fast(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__global__ void __launch_bounds__(SMH_THREADS, 2)
step_softmax_h_kernel(const __half* __restrict__ q, const __half* __restrict__ k_fp, int64_t fp_stride_b,
                      int64_t fp_stride_h, int hq, int hkv, int t_vis, int t_fp, int calibrate,
                      const __half* __restrict__ s_vis, __half* __restrict__ a_vis, __half* __restrict__ a_fp,
                      float* __restrict__ a_sum, const int32_t* __restrict__ t_fp_dev, int t_fp_cap) {
  if (t_fp_dev) t_fp = min(*t_fp_dev, t_fp_cap);
  extern __shared__ __align__(16) unsigned char sm_raw[];
  uint4* rv = reinterpret_cast<uint4*>(sm_raw);                          // t_vis halves
  float* fprow = reinterpret_cast<float*>(sm_raw + (size_t)t_vis * 2);   // t_fp floats
  __shared__ float red[32];
  __shared__ float q_s[kHeadDim];
  const int bh = blockIdx.x, b = bh / hq, h = bh % hq, hk = h / (hq / hkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float sd = sqrtf((float)kHeadDim);
  if (tid < kHeadDim) q_s[tid] = __half2float(q[(int64_t)bh * kHeadDim + tid]);
  __syncthreads();
  const __half* kb = k_fp + b * fp_stride_b + hk * fp_stride_h;
  float fmx = -INFINITY;
  for (int t = warp; t < t_fp; t += SMH_THREADS / 32) {
    const __half* kr = kb + (int64_t)t * kHeadDim + lane * 4;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) dot = fmaf(q_s[lane * 4 + i], __half2float(kr[i]), dot);
    dot = warp_sum(dot);
    const float sc = rnd<__half>(__fdiv_rn(rnd<__half>(dot), sd));
    if (lane == 0) fprow[t] = sc;
    fmx = fmaxf(fmx, sc);
  }
  const int nvec = t_vis >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(s_vis + (int64_t)bh * t_vis);
  __half2 mx2 = __float2half2_rn(-INFINITY), mn2 = __float2half2_rn(INFINITY);
  for (int i = tid; i < nvec; i += SMH_THREADS) {
    const uint4 v = src[i];
    rv[i] = v;
    const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) { mx2 = __hmax2(mx2, h2[j]); mn2 = __hmin2(mn2, h2[j]); }
  }
  float mx = fmaxf(__low2float(mx2), __high2float(mx2));
  if (calibrate && t_vis > 0) {
    const float mn = block_reduce(fminf(__low2float(mn2), __high2float(mn2)), red, 2);
    mx = block_reduce(mx, red, 1);
    const __half2 span2 = __float2half2_rn(rnd<__half>(rnd<__half>(mx + -3.f) - mn));      // tgt_max - tgt_min
    const float rden = 1.f / rnd<__half>(rnd<__half>(mx - mn) + 1e-8f);
    const __half2 mnh = __float2half2_rn(mn);
    mx2 = __float2half2_rn(-INFINITY);
    for (int i = tid; i < nvec; i += SMH_THREADS) {
      uint4 v = rv[i];
      __half2* h2 = reinterpret_cast<__half2*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 d = __half22float2(__hsub2(h2[j], mnh));
        const __half2 n = __floats2half2_rn(d.x * rden, d.y * rden);
        h2[j] = __hadd2(__hmul2(n, span2), mnh);
        mx2 = __hmax2(mx2, h2[j]);
      }
      rv[i] = v;
    }
    mx = fmaxf(__low2float(mx2), __high2float(mx2));
  }
  const float m = block_reduce(fmaxf(mx, fmx), red, 1);      // also orders the row writes before the reads below
  constexpr float L2E = 1.4426950408889634f;
  const float ml = m * L2E;
  float sum = 0.f;
  for (int i = tid; i < nvec; i += SMH_THREADS) {
    const uint4 v = rv[i];
    const __half2* h2 = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __half22float2(h2[j]);
      sum += ex2_fast(fmaf(x.x, L2E, -ml)) + ex2_fast(fmaf(x.y, L2E, -ml));
    }
  }
  for (int t = tid; t < t_fp; t += SMH_THREADS) sum += ex2_fast(fmaf(fprow[t], L2E, -ml));
  sum = block_reduce(sum, red, 0);
  const float inv = 1.f / sum;
  float vs = 0.f;
  uint4* dst = reinterpret_cast<uint4*>(a_vis + (int64_t)bh * t_vis);
  for (int i = tid; i < nvec; i += SMH_THREADS) {
    uint4 v = rv[i];
    __half2* h2 = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __half22float2(h2[j]);
      h2[j] = __floats2half2_rn(ex2_fast(fmaf(x.x, L2E, -ml)) * inv, ex2_fast(fmaf(x.y, L2E, -ml)) * inv);
      const float2 a = __half22float2(h2[j]);
      vs += a.x + a.y;
    }
    dst[i] = v;
  }
  for (int t = tid; t < t_fp; t += SMH_THREADS)
    a_fp[(int64_t)bh * t_fp_cap + t] = __float2half_rn(ex2_fast(fmaf(fprow[t], L2E, -ml)) * inv);
  vs = block_reduce(vs, red, 0);
  if (tid == 0) a_sum[bh] = rnd<__half>(vs);
}

// ---- fused decode step, launch 4: scale / zero point of V, full-precision tokens, bf16 output -------------
// o = fused_kernel_wv(...) * scale_v - scale_v*zero_point_v*sum(att_vis) + att_sys @ V_sys + att_txt @ V_txt
// (patch_internvl.py:396-436), thread = channel.  Products of an fp16 tensor with a bf16 one promote to fp32.
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
step_finish_kernel(const float* __restrict__ partial, int chunks, int n_rows, const T* __restrict__ scale_v,
                   const T* __restrict__ zp_v, int scale_heads, const T* __restrict__ a_fp,
                   const float* __restrict__ a_sum, const T* __restrict__ v_fp, int64_t fp_stride_b,
                   int64_t fp_stride_h, int hq, int hkv, int t_fp, int t_sys, __nv_bfloat16* __restrict__ out,
                   const int32_t* __restrict__ t_fp_dev) {
  using SS = StepScore<T>;
  const int t_fp_cap = t_fp;
  if (t_fp_dev) t_fp = min(*t_fp_dev, t_fp_cap);
  extern __shared__ float att_s[];       // [t_fp]
  const int bh = blockIdx.x, b = bh / hq, h = bh % hq, hk = h / (hq / hkv), d = threadIdx.x;
  for (int t = d; t < t_fp; t += kHeadDim) att_s[t] = Elem<T>::to_f(a_fp[(int64_t)bh * t_fp_cap + t]);
  float acc = 0.f;
  for (int c = 0; c < chunks; ++c) acc += partial[((int64_t)c * n_rows + bh) * kHeadDim + d];
  const int64_t srow = scale_heads == hq ? bh : (int64_t)b * scale_heads + hk;
  float o = 0.f;
  if (chunks) {                          // no visual span: nothing quantized to add
    const float sv = Elem<T>::to_f(scale_v[srow * kHeadDim + d]), zv = Elem<T>::to_f(zp_v[srow * kHeadDim + d]);
    o = SS::r(rnd<__half>(acc) * sv);
    o = SS::r(o - rnd<T>(rnd<T>(sv * zv) * a_sum[bh]));
  }
  __syncthreads();
  const T* vb = v_fp + b * fp_stride_b + hk * fp_stride_h + d;
  float seg = 0.f;
  const int ts = min(t_sys, t_fp);
  for (int t = 0; t < ts; ++t) seg = fmaf(att_s[t], Elem<T>::to_f(vb[(int64_t)t * kHeadDim]), seg);
  o = SS::r(o + rnd<T>(seg));
  seg = 0.f;
  for (int t = ts; t < t_fp; ++t) seg = fmaf(att_s[t], Elem<T>::to_f(vb[(int64_t)t * kHeadDim]), seg);
  o = SS::r(o + rnd<T>(seg));
  out[(int64_t)bh * kHeadDim + d] = __float2bfloat16_rn(o);
}

}  // namespace calib
}  // namespace cq

using namespace cq;

static bool dtype_ok(int dt) { return dt == CQ_DTYPE_F16 || dt == CQ_DTYPE_BF16; }
static bool bits_ok(int b) { return b == 1 || b == 2 || b == 4; }

extern "C" int cq_calib_minmax(const void* x, int batch, int t_len, int heads, int head_dim, const int64_t* strides,
                               int bits, float clip, int dtype, void* scale, void* zero_point, void* stream) {
  if (!x || !strides || !scale || !zero_point || batch <= 0 || t_len <= 0 || heads <= 0) return CQ_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return CQ_ERR_BAD_ARG;
  if (!bits_ok(bits) || head_dim != kHeadDim) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int levels = (1 << bits) - 1;
  const unsigned grid = (unsigned)(batch * heads);
  // rows of eight channels that can be read as 16-byte words: the sliced reduction over the whole GPU
  if (aligned16(x) && strides[0] % 8 == 0 && strides[1] % 8 == 0 && strides[2] % 8 == 0 && t_len >= 256 &&
      grid <= 65535u && (int64_t)grid * kHeadDim <= 0x7fffffff) {
    const int n = (int)(grid * kHeadDim);
    int slices = (int)((4 * 148 + grid - 1) / grid);
    slices = max(1, min(slices, (t_len + 63) / 64));
    unsigned short* kmn = static_cast<unsigned short*>(scale);
    unsigned short* kmx = static_cast<unsigned short*>(zero_point);
    calib::minmax_init_kernel<<<(n + 255) / 256, 256, 0, st>>>(kmn, kmx, n);
    const dim3 g2((unsigned)slices, grid);
    if (dtype == CQ_DTYPE_F16) {
      calib::minmax_slice_kernel<__half><<<g2, 256, 0, st>>>(static_cast<const __half*>(x), heads, t_len, strides[0],
                                                            strides[1], strides[2], kmn, kmx);
      calib::minmax_finish_kernel<__half><<<(n + 255) / 256, 256, 0, st>>>(static_cast<__half*>(scale),
                                                                          static_cast<__half*>(zero_point), n, clip, levels);
    } else {
      calib::minmax_slice_kernel<__nv_bfloat16><<<g2, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), heads, t_len,
                                                                   strides[0], strides[1], strides[2], kmn, kmx);
      calib::minmax_finish_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, st>>>(
          static_cast<__nv_bfloat16*>(scale), static_cast<__nv_bfloat16*>(zero_point), n, clip, levels);
    }
    return check_launch();
  }
  if (dtype == CQ_DTYPE_F16)
    calib::minmax_kernel<__half><<<grid, kHeadDim * calib::MM_SLICES, 0, st>>>(
        static_cast<const __half*>(x), heads, t_len, strides[0], strides[1], strides[2], clip, levels,
        static_cast<__half*>(scale), static_cast<__half*>(zero_point));
  else
    calib::minmax_kernel<__nv_bfloat16><<<grid, kHeadDim * calib::MM_SLICES, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), heads, t_len, strides[0], strides[1], strides[2], clip, levels,
        static_cast<__nv_bfloat16*>(scale), static_cast<__nv_bfloat16*>(zero_point));
  return check_launch();
}

template <typename T>
static int launch_quantize(const void* x, int batch, int t_len, int heads, const int64_t* s, int bits,
                           const void* scale, const void* zp, int dequantize, void* xq, uint8_t* enc,
                           cudaStream_t st) {
  const int64_t n_chunks = (int64_t)batch * t_len * heads * 16;
  const unsigned grid = (unsigned)((n_chunks + 255) / 256);
  const T* xp = static_cast<const T*>(x);
  const T* sp = static_cast<const T*>(scale);
  const T* zpp = static_cast<const T*>(zp);
  T* xo = static_cast<T*>(xq);
  // codes only (no dequantized output) at 1 or 2 bits: per-channel thresholds instead of divisions
  if (!dequantize && bits <= 2 && (int64_t)batch * heads <= 65535) {
    const dim3 g2((unsigned)((t_len + calib::QT_TOKENS - 1) / calib::QT_TOKENS), (unsigned)(batch * heads));
    if (bits == 1) calib::quantize_thr_kernel<T, 1><<<g2, 256, 0, st>>>(xp, heads, t_len, s[0], s[1], s[2], sp, zpp, xo, enc);
    else calib::quantize_thr_kernel<T, 2><<<g2, 256, 0, st>>>(xp, heads, t_len, s[0], s[1], s[2], sp, zpp, xo, enc);
    return check_launch();
  }
  switch (bits) {
    case 1: calib::quantize_kernel<T, 1><<<grid, 256, 0, st>>>(xp, heads, t_len, s[0], s[1], s[2], sp, zpp, dequantize, xo, enc, n_chunks); break;
    case 2: calib::quantize_kernel<T, 2><<<grid, 256, 0, st>>>(xp, heads, t_len, s[0], s[1], s[2], sp, zpp, dequantize, xo, enc, n_chunks); break;
    default: calib::quantize_kernel<T, 4><<<grid, 256, 0, st>>>(xp, heads, t_len, s[0], s[1], s[2], sp, zpp, dequantize, xo, enc, n_chunks); break;
  }
  return check_launch();
}

extern "C" int cq_calib_quantize(const void* x, int batch, int t_len, int heads, int head_dim, const int64_t* strides,
                                 int bits, int dtype, const void* scale, const void* zero_point, int dequantize,
                                 void* xq_out, uint8_t* enc_out, void* stream) {
  if (!x || !strides || !scale || !zero_point || batch <= 0 || t_len <= 0 || heads <= 0) return CQ_ERR_BAD_ARG;
  if (!xq_out && !enc_out) return CQ_ERR_BAD_ARG;
  if (!dtype_ok(dtype)) return CQ_ERR_BAD_ARG;
  if (!bits_ok(bits) || head_dim != kHeadDim) return CQ_ERR_UNSUPPORTED;
  if (!aligned16(x) || strides[0] % 8 || strides[1] % 8 || strides[2] % 8) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    return launch_quantize<__half>(x, batch, t_len, heads, strides, bits, scale, zero_point, dequantize, xq_out, enc_out, st);
  return launch_quantize<__nv_bfloat16>(x, batch, t_len, heads, strides, bits, scale, zero_point, dequantize, xq_out, enc_out, st);
}

extern "C" int cq_calib_encode_i64(const int64_t* codes, int64_t n_codes, int bits, uint8_t* out, void* stream) {
  if (!codes || !out || n_codes < 0) return CQ_ERR_BAD_ARG;
  if (!bits_ok(bits) || n_codes % (8 / bits)) return CQ_ERR_UNSUPPORTED;
  if (n_codes == 0) return CQ_OK;
  const int64_t n_bytes = n_codes * bits / 8;
  const unsigned grid = (unsigned)((n_bytes + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (bits) {
    case 1: calib::encode_i64_kernel<1><<<grid, 256, 0, st>>>(codes, out, n_bytes); break;
    case 2: calib::encode_i64_kernel<2><<<grid, 256, 0, st>>>(codes, out, n_bytes); break;
    default: calib::encode_i64_kernel<4><<<grid, 256, 0, st>>>(codes, out, n_bytes); break;
  }
  return check_launch();
}

extern "C" int cq_lut_scores(const void* lut, const void* weights, const uint8_t* enc, void* out, int batch,
                             int n_q_heads, int n_enc_heads, int t_len, int head_dim, int bits, int dtype,
                             void* stream) {
  if (!lut || !weights || !enc || !out || batch <= 0 || n_q_heads <= 0 || n_enc_heads <= 0 || t_len <= 0) return CQ_ERR_BAD_ARG;
  if (!dtype_ok(dtype) || n_q_heads % n_enc_heads) return CQ_ERR_BAD_ARG;
  if (!bits_ok(bits) || head_dim != kHeadDim || n_q_heads / n_enc_heads > kMaxRep) return CQ_ERR_UNSUPPORTED;
  if ((int64_t)batch * n_enc_heads > 65535) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (aligned16(enc)) {     // tensor-core kernel: 128-bit loads of the code rows
    // a CTA sets up the B fragments of its heads once, so it should stream a few thousand tokens; still at
    // least ~8 CTAs per SM over the whole grid
    const int per_cta = 4 * calib::LS_TOK;
    const int by_work = (t_len + 8 * per_cta - 1) / (8 * per_cta);
    const int by_fill = (148 * 8 + batch * n_enc_heads - 1) / (batch * n_enc_heads);
    const int max_x = (t_len + per_cta - 1) / per_cta;
    dim3 grid((unsigned)max(1, min(max_x, max(by_work, by_fill))), (unsigned)(batch * n_enc_heads));
    __half* o = static_cast<__half*>(out);
#define CQ_LUT_SCORES(T, B)                                                                                   \
  calib::lut_scores_mma_kernel<T, B><<<grid, 128, 0, st>>>(static_cast<const T*>(lut), static_cast<const T*>(weights), \
                                                          enc, n_q_heads, n_enc_heads, t_len, o)
#define CQ_LUT_SCORES_B(T) do { if (bits == 1) CQ_LUT_SCORES(T, 1); else if (bits == 2) CQ_LUT_SCORES(T, 2); else CQ_LUT_SCORES(T, 4); } while (0)
    if (dtype == CQ_DTYPE_F16) CQ_LUT_SCORES_B(__half); else CQ_LUT_SCORES_B(__nv_bfloat16);
#undef CQ_LUT_SCORES_B
#undef CQ_LUT_SCORES
    return check_launch();
  }
  dim3 grid((unsigned)min(1024, (t_len + 7) / 8), (unsigned)(batch * n_enc_heads));
  if (dtype == CQ_DTYPE_F16)
    calib::lut_scores_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(lut), static_cast<const __half*>(weights), enc,
                                                           n_q_heads, n_enc_heads, t_len, bits, static_cast<__half*>(out));
  else
    calib::lut_scores_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(lut), static_cast<const __nv_bfloat16*>(weights), enc,
                                                                  n_q_heads, n_enc_heads, t_len, bits, static_cast<__half*>(out));
  return check_launch();
}

extern "C" size_t cq_lut_out_workspace_bytes(int batch, int n_q_heads, int t_len) {
  if (batch <= 0 || n_q_heads <= 0 || t_len <= 0) return 0;
  const size_t chunks = (size_t)((t_len + calib::WV_TCHUNK - 1) / calib::WV_TCHUNK);
  return chunks * (size_t)batch * n_q_heads * kHeadDim * sizeof(float);
}

extern "C" int cq_lut_out(const void* lut, const void* weights, const uint8_t* enc, void* out, int batch,
                          int n_q_heads, int n_enc_heads, int t_len, int head_dim, int bits, int dtype,
                          void* workspace, size_t workspace_bytes, void* stream) {
  if (!lut || !weights || !enc || !out || batch <= 0 || n_q_heads <= 0 || n_enc_heads <= 0 || t_len <= 0) return CQ_ERR_BAD_ARG;
  if (!dtype_ok(dtype) || n_q_heads % n_enc_heads) return CQ_ERR_BAD_ARG;
  if (!bits_ok(bits) || head_dim != kHeadDim || n_q_heads / n_enc_heads > kMaxRep) return CQ_ERR_UNSUPPORTED;
  if ((int64_t)batch * n_enc_heads > 65535) return CQ_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < cq_lut_out_workspace_bytes(batch, n_q_heads, t_len)) return CQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const int rows = batch * n_q_heads;
  if (aligned16(enc)) {     // tensor-core kernel: WO_TOK tokens per CTA (fewer partials than the scalar one)
    const int chunks = (t_len + calib::WO_TOK - 1) / calib::WO_TOK;
    dim3 grid((unsigned)chunks, (unsigned)(batch * n_enc_heads));
#define CQ_LUT_OUT(T, B)                                                                                      \
  calib::lut_out_mma_kernel<T, B><<<grid, 128, 0, st>>>(static_cast<const T*>(lut), static_cast<const T*>(weights), enc, \
                                                       n_q_heads, n_enc_heads, t_len, ws, rows)
    if (dtype == CQ_DTYPE_F16) { if (bits == 1) CQ_LUT_OUT(__half, 1); else if (bits == 2) CQ_LUT_OUT(__half, 2); else CQ_LUT_OUT(__half, 4); }
    else { if (bits == 1) CQ_LUT_OUT(__nv_bfloat16, 1); else if (bits == 2) CQ_LUT_OUT(__nv_bfloat16, 2); else CQ_LUT_OUT(__nv_bfloat16, 4); }
#undef CQ_LUT_OUT
    int rc = check_launch();
    if (rc != CQ_OK) return rc;
    const int64_t total = (int64_t)rows * kHeadDim;
    calib::lut_out_finalize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(ws, static_cast<__half*>(out), chunks, total);
    return check_launch();
  }
  const int chunks = (t_len + calib::WV_TCHUNK - 1) / calib::WV_TCHUNK;
  dim3 grid((unsigned)chunks, (unsigned)(batch * n_enc_heads));
  if (dtype == CQ_DTYPE_F16)
    calib::lut_out_partial_kernel<__half><<<grid, kHeadDim, 0, st>>>(static_cast<const __half*>(lut), static_cast<const __half*>(weights), enc,
                                                                     n_q_heads, n_enc_heads, t_len, bits, ws, rows);
  else
    calib::lut_out_partial_kernel<__nv_bfloat16><<<grid, kHeadDim, 0, st>>>(static_cast<const __nv_bfloat16*>(lut), static_cast<const __nv_bfloat16*>(weights), enc,
                                                                            n_q_heads, n_enc_heads, t_len, bits, ws, rows);
  int rc = check_launch();
  if (rc != CQ_OK) return rc;
  const int64_t total = (int64_t)rows * kHeadDim;
  calib::lut_out_finalize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(ws, static_cast<__half*>(out), chunks, total);
  return check_launch();
}

// ---- fused decode step on the uint8 format: four launches -------------------------------------------------
namespace {
struct StepLayout {
  size_t scores, a_vis, a_fp, a_sum, lut, partial, total;
  int chunks;
};
StepLayout step_layout(const cq_u8_decode_args* a) {
  StepLayout l{};
  const size_t rows = (size_t)a->batch * a->n_q_heads;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  size_t off = 0;
  l.scores = off; off = up(off + rows * (size_t)a->t_vis * 4);
  l.a_vis = off;  off = up(off + rows * (size_t)a->t_vis * 2);
  l.a_fp = off;   off = up(off + rows * (size_t)a->t_fp * 2);
  l.a_sum = off;  off = up(off + rows * 4);
  l.lut = off;    off = up(off + 32);
  l.chunks = (a->t_vis + calib::WO_TOK - 1) / calib::WO_TOK;
  l.partial = off; off = up(off + (size_t)l.chunks * rows * kHeadDim * 4);
  l.total = off;
  return l;
}
int step_check(const cq_u8_decode_args* a) {
  if (!a) return CQ_ERR_BAD_ARG;
  if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->t_vis < 0 || a->t_fp < 0) return CQ_ERR_BAD_ARG;
  if (a->t_vis + a->t_fp == 0 || a->t_sys < 0 || a->t_sys > a->t_fp || a->reserved != 0) return CQ_ERR_BAD_ARG;
  if (a->n_q_heads % a->n_kv_heads || !dtype_ok(a->dtype)) return CQ_ERR_BAD_ARG;
  if (a->n_scale_heads != a->n_q_heads && a->n_scale_heads != a->n_kv_heads) return CQ_ERR_BAD_ARG;
  if (!bits_ok(a->bits) || a->head_dim != kHeadDim || a->n_q_heads / a->n_kv_heads > kMaxRep) return CQ_ERR_UNSUPPORTED;
  if ((int64_t)a->batch * a->n_kv_heads > 65535) return CQ_ERR_UNSUPPORTED;
  if ((size_t)(a->t_vis + a->t_fp) * 4 > 200 * 1024) return CQ_ERR_UNSUPPORTED;   // the score row must fit shared memory
  if ((size_t)a->t_fp * 4 > 160 * 1024) return CQ_ERR_UNSUPPORTED;
  if (!a->q || !a->out) return CQ_ERR_BAD_ARG;
  if (a->t_vis && (!a->enc_k || !a->enc_v || !a->scale_key || !a->zero_point_key || !a->scale_value || !a->zero_point_value))
    return CQ_ERR_BAD_ARG;
  if (a->t_vis && (!aligned16(a->enc_k) || !aligned16(a->enc_v))) return CQ_ERR_BAD_ARG;
  if (a->t_fp && (!a->k_fp || !a->v_fp)) return CQ_ERR_BAD_ARG;
  return CQ_OK;
}
}  // namespace

extern "C" size_t cq_u8_decode_attn_workspace_bytes(const cq_u8_decode_args* a) {
  if (step_check(a) != CQ_OK) return 0;
  return step_layout(a).total;
}

template <typename T>
static int launch_step(const cq_u8_decode_args* a, char* ws, cudaStream_t st) {
  using S = typename calib::StepScore<T>::type;
  const StepLayout l = step_layout(a);
  const int B = a->batch, hq = a->n_q_heads, hkv = a->n_kv_heads, rows = B * hq;
  S* scores = reinterpret_cast<S*>(ws + l.scores);
  __half* a_vis = reinterpret_cast<__half*>(ws + l.a_vis);
  T* a_fp = reinterpret_cast<T*>(ws + l.a_fp);
  float* a_sum = reinterpret_cast<float*>(ws + l.a_sum);
  uint16_t* lut = reinterpret_cast<uint16_t*>(ws + l.lut);
  float* partial = reinterpret_cast<float*>(ws + l.partial);
  const T* q = static_cast<const T*>(a->q);
  if (a->t_vis) {
    const int per_cta = 4 * calib::LS_TOK;
    const int by_work = (a->t_vis + 8 * per_cta - 1) / (8 * per_cta);
    const int by_fill = (148 * 8 + B * hkv - 1) / (B * hkv);
    const int max_x = (a->t_vis + per_cta - 1) / per_cta;
    dim3 grid((unsigned)max(1, min(max_x, max(by_work, by_fill))), (unsigned)(B * hkv));
    calib::StepScoreArgs sa{a->scale_key, a->zero_point_key, a->n_scale_heads, scores, lut};
    switch (a->bits) {
      case 1: calib::lut_scores_mma_kernel<T, 1, true><<<grid, 128, 0, st>>>(nullptr, q, a->enc_k, hq, hkv, a->t_vis, nullptr, sa); break;
      case 2: calib::lut_scores_mma_kernel<T, 2, true><<<grid, 128, 0, st>>>(nullptr, q, a->enc_k, hq, hkv, a->t_vis, nullptr, sa); break;
      default: calib::lut_scores_mma_kernel<T, 4, true><<<grid, 128, 0, st>>>(nullptr, q, a->enc_k, hq, hkv, a->t_vis, nullptr, sa); break;
    }
  }
  const size_t row_bytes = (size_t)(a->t_vis + a->t_fp) * 4;
  const size_t row_bytes_h = (size_t)a->t_vis * 2 + (size_t)a->t_fp * 4;
  if (std::is_same<T, __half>::value && !a->mask && a->t_vis > 0 && a->t_vis % 8 == 0 && row_bytes_h <= 100 * 1024) {
    if (cudaFuncSetAttribute(calib::step_softmax_h_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    calib::step_softmax_h_kernel<<<rows, calib::SMH_THREADS, row_bytes_h, st>>>(
        static_cast<const __half*>(a->q), static_cast<const __half*>(a->k_fp), a->fp_stride_b, a->fp_stride_h, hq, hkv,
        a->t_vis, a->t_fp, a->calibrate, reinterpret_cast<const __half*>(scores), a_vis, reinterpret_cast<__half*>(a_fp),
        a_sum, a->t_fp_dev, a->t_fp);
  } else {
    if (cudaFuncSetAttribute(calib::step_softmax_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    calib::step_softmax_kernel<T><<<rows, calib::SM_THREADS, row_bytes, st>>>(
        q, static_cast<const T*>(a->k_fp), a->fp_stride_b, a->fp_stride_h, hq, hkv, a->t_vis, a->t_fp, a->t_sys,
        a->calibrate, scores, static_cast<const T*>(a->mask), a->mask_stride_b, a_vis, a_fp, a_sum, a->t_fp_dev, a->t_fp);
  }
  if (a->t_vis) {
    dim3 grid((unsigned)l.chunks, (unsigned)(B * hkv));
    const __half* lut_h = reinterpret_cast<const __half*>(lut);
    if (a->bits == 1)
      calib::lut_out_mma_kernel<__half, 1><<<grid, 128, 0, st>>>(lut_h, a_vis, a->enc_v, hq, hkv, a->t_vis, partial, rows);
    else if (a->bits == 2)
      calib::lut_out_mma_kernel<__half, 2><<<grid, 128, 0, st>>>(lut_h, a_vis, a->enc_v, hq, hkv, a->t_vis, partial, rows);
    else
      calib::lut_out_mma_kernel<__half, 4><<<grid, 128, 0, st>>>(lut_h, a_vis, a->enc_v, hq, hkv, a->t_vis, partial, rows);
  }
  if (cudaFuncSetAttribute(calib::step_finish_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
    return CQ_ERR_LAUNCH;
  calib::step_finish_kernel<T><<<rows, kHeadDim, (size_t)a->t_fp * 4, st>>>(
      partial, a->t_vis ? l.chunks : 0, rows, static_cast<const T*>(a->scale_value), static_cast<const T*>(a->zero_point_value),
      a->n_scale_heads, a_fp, a_sum, static_cast<const T*>(a->v_fp), a->fp_stride_b, a->fp_stride_h, hq, hkv, a->t_fp,
      a->t_sys, static_cast<__nv_bfloat16*>(a->out), a->t_fp_dev);
  return check_launch();
}

extern "C" int cq_u8_decode_attn(const cq_u8_decode_args* a, void* workspace, size_t workspace_bytes, void* stream) {
  const int rc = step_check(a);
  if (rc != CQ_OK) return rc;
  if (!workspace || workspace_bytes < step_layout(a).total) return CQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->dtype == CQ_DTYPE_F16) return launch_step<__half>(a, static_cast<char*>(workspace), st);
  return launch_step<__nv_bfloat16>(a, static_cast<char*>(workspace), st);
}
