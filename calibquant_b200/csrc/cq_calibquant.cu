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
#include "cq_common.cuh"

namespace cq {
namespace calib {

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
  dim3 grid((unsigned)min(1024, (t_len + 7) / 8), (unsigned)(batch * n_enc_heads));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
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
  const int chunks = (t_len + calib::WV_TCHUNK - 1) / calib::WV_TCHUNK;
  dim3 grid((unsigned)chunks, (unsigned)(batch * n_enc_heads));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* ws = static_cast<float*>(workspace);
  const int rows = batch * n_q_heads;
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
