// Small fused kernels around the attention call of one decode step: the QKV split + rotary
// embedding + cache append that precedes it, and the two elementwise blocks of the decoder layer
// (residual add + RMSNorm, SwiGLU gate).  Each replaces a chain of 4-10 elementwise torch kernels
// whose launch gaps dominate a batch-16 decode step; all are memory-trivial (KBs per launch).
// Every value torch would round to the tensor dtype between two ops is rounded here as well.
#include "cq_common.cuh"

namespace cq {
namespace step {

constexpr int NORM_THREADS = 256;
constexpr int NORM_VEC = 8;          // elements per 16-byte access
constexpr int NORM_MAXV = 8;         // vectors per thread held in registers -> hidden <= 16384

template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_kernel(const T* __restrict__ delta, T* __restrict__ residual, const T* __restrict__ weight,
                   T* __restrict__ out, int hidden, float eps) {
  const int64_t row = blockIdx.x;
  const int tid = threadIdx.x;
  const int n_vec = hidden / NORM_VEC;
  T* res = residual + row * hidden;
  const T* dl = delta ? delta + row * hidden : nullptr;
  float v[NORM_MAXV][NORM_VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int iv = tid + k * NORM_THREADS;
    if (iv < n_vec) {
      uint4 raw = *reinterpret_cast<const uint4*>(res + iv * NORM_VEC);
      const T* r = reinterpret_cast<const T*>(&raw);
      if (dl) {
        const uint4 draw = *reinterpret_cast<const uint4*>(dl + iv * NORM_VEC);
        const T* d = reinterpret_cast<const T*>(&draw);
        uint4 sum;
        T* s = reinterpret_cast<T*>(&sum);
#pragma unroll
        for (int e = 0; e < NORM_VEC; ++e) {
          s[e] = Elem<T>::from_f(Elem<T>::to_f(r[e]) + Elem<T>::to_f(d[e]));   // hidden = hidden + delta
          v[k][e] = Elem<T>::to_f(s[e]);
        }
        *reinterpret_cast<uint4*>(res + iv * NORM_VEC) = sum;
      } else {
#pragma unroll
        for (int e = 0; e < NORM_VEC; ++e) v[k][e] = Elem<T>::to_f(r[e]);
      }
#pragma unroll
      for (int e = 0; e < NORM_VEC; ++e) ss = fmaf(v[k][e], v[k][e], ss);
    }
  }
  __shared__ float part[NORM_THREADS / 32];
  ss = warp_sum(ss);
  if ((tid & 31) == 0) part[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NORM_THREADS / 32; ++w) tot += part[w];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  if (!out) return;
  T* o = out + row * hidden;
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int iv = tid + k * NORM_THREADS;
    if (iv < n_vec) {
      const uint4 wraw = *reinterpret_cast<const uint4*>(weight + iv * NORM_VEC);
      const T* w = reinterpret_cast<const T*>(&wraw);
      uint4 res4;
      T* r = reinterpret_cast<T*>(&res4);
#pragma unroll
      for (int e = 0; e < NORM_VEC; ++e)   // weight * (x_fp32 * rsqrt(var + eps)).to(dtype)
        r[e] = Elem<T>::from_f(Elem<T>::to_f(w[e]) * rnd<T>(v[k][e] * inv));
      *reinterpret_cast<uint4*>(o + iv * NORM_VEC) = res4;
    }
  }
}

// One block of 64 threads per (batch row, head of the projection output); thread d owns the
// rotary pair (d, d + 64).
template <typename T>
__global__ void __launch_bounds__(64)
rope_split_append_kernel(const T* __restrict__ qkv, int64_t qkv_stride_b, const T* __restrict__ cos_t,
                         const T* __restrict__ sin_t, const int64_t* __restrict__ position_ids, int n_kv_heads,
                         int n_rep, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                         int64_t cache_stride_b, int64_t cache_stride_h, int capacity, int append_index,
                         const int32_t* __restrict__ t_fp_dev, int rope_len) {
  const int per_kv = n_rep + 2;
  const int b = blockIdx.x / (n_kv_heads * per_kv);
  const int rem = blockIdx.x % (n_kv_heads * per_kv);
  const int hk = rem / per_kv, slot = rem % per_kv;     // slot < n_rep: query head; n_rep: key; n_rep+1: value
  const int d = threadIdx.x;
  const T* src = qkv + b * qkv_stride_b + (int64_t)(hk * per_kv + slot) * kHeadDim;
  const int idx = t_fp_dev ? __ldg(t_fp_dev) - 1 : append_index;   // the live count includes this token
  T* dst;
  if (slot < n_rep) {
    dst = q_out + ((int64_t)b * n_kv_heads * n_rep + (int64_t)hk * n_rep + slot) * kHeadDim;
  } else {
    if (idx < 0 || idx >= capacity) return;             // a full cache drops the token instead of writing outside
    dst = (slot == n_rep ? k_cache : v_cache) + b * cache_stride_b + hk * cache_stride_h + (int64_t)idx * kHeadDim;
  }
  const float x0 = Elem<T>::to_f(src[d]), x1 = Elem<T>::to_f(src[d + 64]);
  if (slot == n_rep + 1) {                               // values are not rotated
    dst[d] = src[d];
    dst[d + 64] = src[d + 64];
    return;
  }
  int64_t pos = position_ids[b];
  pos = pos < 0 ? 0 : (pos >= rope_len ? rope_len - 1 : pos);
  const T* cr = cos_t + pos * kHeadDim;
  const T* sr = sin_t + pos * kHeadDim;
  // x*cos rounded, then + rotate_half(x)*sin with one more rounding (the product of two 16-bit
  // floats is exact in fp32)
  const float a0 = rnd<T>(x0 * Elem<T>::to_f(cr[d])), a1 = rnd<T>(x1 * Elem<T>::to_f(cr[d + 64]));
  dst[d] = Elem<T>::from_f(__fadd_rn(a0, __fmul_rn(-x1, Elem<T>::to_f(sr[d]))));
  dst[d + 64] = Elem<T>::from_f(__fadd_rn(a1, __fmul_rn(x0, Elem<T>::to_f(sr[d + 64]))));
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t n_vec) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_vec; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 graw = reinterpret_cast<const uint4*>(gate)[i], uraw = reinterpret_cast<const uint4*>(up)[i];
    const T* g = reinterpret_cast<const T*>(&graw);
    const T* u = reinterpret_cast<const T*>(&uraw);
    uint4 res;
    T* r = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = Elem<T>::to_f(g[e]);
      const float s = rnd<T>(x / (1.f + expf(-x)));      // silu(gate) as its own rounded tensor
      r[e] = Elem<T>::from_f(s * Elem<T>::to_f(u[e]));
    }
    reinterpret_cast<uint4*>(out)[i] = res;
  }
}

// the same gate on one matrix [rows, 2n] that holds the gate columns first and the up columns after them
// (the output of one GEMM against the stacked w1 / w3 weights): out [rows, n]
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_packed_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t rows, int64_t n_vec_row) {
  const int64_t total = rows * n_vec_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / n_vec_row, j = i % n_vec_row;
    const uint4 graw = reinterpret_cast<const uint4*>(gate_up)[r * 2 * n_vec_row + j];
    const uint4 uraw = reinterpret_cast<const uint4*>(gate_up)[r * 2 * n_vec_row + n_vec_row + j];
    const T* g = reinterpret_cast<const T*>(&graw);
    const T* u = reinterpret_cast<const T*>(&uraw);
    uint4 res;
    T* o = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = Elem<T>::to_f(g[e]);
      const float s = rnd<T>(x / (1.f + expf(-x)));
      o[e] = Elem<T>::from_f(s * Elem<T>::to_f(u[e]));
    }
    reinterpret_cast<uint4*>(out)[i] = res;
  }
}

// ---- prefill: split + rotary embedding of the whole prompt in one pass over the wqkv output ----------------
// One thread owns the channel chunks [8c, 8c+8) and [64+8c, 64+8c+8) of one 128-channel row (a query head, the
// key or the value of one KV head of one token): two 16-byte loads, the rotation of both chunks (they are each
// other's rotate_half partners), 16-byte stores.  Queries go to q_out, keys to k_out (both [B,T,H,128], what
// the prefill attention reads) and, for tokens outside the quantized span, to the full-precision cache together
// with the values.  Values inside the span are not copied at all (the pack kernel reads them in place).
template <typename T>
__global__ void __launch_bounds__(256)
prefill_rope_split_kernel(const T* __restrict__ qkv, int64_t stride_b, int64_t stride_t, const T* __restrict__ cos_t,
                          const T* __restrict__ sin_t, int rope_len, const int64_t* __restrict__ position_ids,
                          int t_len, int n_kv_heads, int n_rep, T* __restrict__ q_out, T* __restrict__ k_out,
                          T* __restrict__ k_cache, T* __restrict__ v_cache, int64_t cache_stride_b,
                          int64_t cache_stride_h, int capacity, int vis_start, int vis_len, int64_t total) {
  const int slots = n_kv_heads * (n_rep + 2);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i & 7);
    const int64_t row = i >> 3;                       // (b, t, slot)
    const int slot_all = (int)(row % slots);
    const int64_t bt = row / slots;
    const int t = (int)(bt % t_len);
    const int64_t b = bt / t_len;
    const int hk = slot_all / (n_rep + 2), slot = slot_all % (n_rep + 2);
    const T* src = qkv + b * stride_b + (int64_t)t * stride_t + (int64_t)slot_all * kHeadDim;
    const int fp_idx = t < vis_start ? t : (t >= vis_start + vis_len ? t - vis_len : -1);   // row in the fp cache
    const bool to_cache = fp_idx >= 0 && fp_idx < capacity && k_cache != nullptr;
    const uint4 lo = *reinterpret_cast<const uint4*>(src + 8 * c), hi = *reinterpret_cast<const uint4*>(src + 64 + 8 * c);
    if (slot == n_rep + 1) {                          // value: only the full-precision tokens are copied
      if (to_cache) {
        T* dst = v_cache + b * cache_stride_b + hk * cache_stride_h + (int64_t)fp_idx * kHeadDim;
        *reinterpret_cast<uint4*>(dst + 8 * c) = lo;
        *reinterpret_cast<uint4*>(dst + 64 + 8 * c) = hi;
      }
      continue;
    }
    int64_t pos = position_ids ? position_ids[b * t_len + t] : t;
    pos = pos < 0 ? 0 : (pos >= rope_len ? rope_len - 1 : pos);
    const T* cr = cos_t + pos * kHeadDim;
    const T* sr = sin_t + pos * kHeadDim;
    const uint4 c_lo = *reinterpret_cast<const uint4*>(cr + 8 * c), c_hi = *reinterpret_cast<const uint4*>(cr + 64 + 8 * c);
    const uint4 s_lo = *reinterpret_cast<const uint4*>(sr + 8 * c), s_hi = *reinterpret_cast<const uint4*>(sr + 64 + 8 * c);
    const T* x0 = reinterpret_cast<const T*>(&lo);  const T* x1 = reinterpret_cast<const T*>(&hi);
    const T* cl = reinterpret_cast<const T*>(&c_lo); const T* chh = reinterpret_cast<const T*>(&c_hi);
    const T* sl = reinterpret_cast<const T*>(&s_lo); const T* sh = reinterpret_cast<const T*>(&s_hi);
    uint4 o_lo, o_hi;
    T* ol = reinterpret_cast<T*>(&o_lo); T* oh = reinterpret_cast<T*>(&o_hi);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      // x*cos rounded, then + rotate_half(x)*sin with one more rounding (torch.addcmul on the rounded product)
      const float a = Elem<T>::to_f(x0[e]), bb = Elem<T>::to_f(x1[e]);
      const float p0 = rnd<T>(a * Elem<T>::to_f(cl[e])), p1 = rnd<T>(bb * Elem<T>::to_f(chh[e]));
      ol[e] = Elem<T>::from_f(__fadd_rn(p0, __fmul_rn(-bb, Elem<T>::to_f(sl[e]))));
      oh[e] = Elem<T>::from_f(__fadd_rn(p1, __fmul_rn(a, Elem<T>::to_f(sh[e]))));
    }
    T* dst;
    if (slot < n_rep) dst = q_out + ((b * t_len + t) * (int64_t)(n_kv_heads * n_rep) + (int64_t)hk * n_rep + slot) * kHeadDim;
    else dst = k_out + ((b * t_len + t) * (int64_t)n_kv_heads + hk) * kHeadDim;
    *reinterpret_cast<uint4*>(dst + 8 * c) = o_lo;
    *reinterpret_cast<uint4*>(dst + 64 + 8 * c) = o_hi;
    if (slot == n_rep && to_cache) {
      T* kc = k_cache + b * cache_stride_b + hk * cache_stride_h + (int64_t)fp_idx * kHeadDim;
      *reinterpret_cast<uint4*>(kc + 8 * c) = o_lo;
      *reinterpret_cast<uint4*>(kc + 64 + 8 * c) = o_hi;
    }
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace step
}  // namespace cq

using namespace cq;

extern "C" int cq_add_rmsnorm(const void* delta, void* residual, const void* weight, void* out, int64_t rows,
                              int hidden, float eps, int dtype, void* stream) {
  if (rows == 0) return CQ_OK;
  if (!residual || rows < 0 || hidden <= 0 || (out && !weight)) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (hidden % step::NORM_VEC || hidden > step::NORM_THREADS * step::NORM_VEC * step::NORM_MAXV) return CQ_ERR_UNSUPPORTED;
  if (!step::aligned16(residual) || !step::aligned16(delta) || !step::aligned16(weight) || !step::aligned16(out))
    return CQ_ERR_BAD_ARG;
  if (rows > 0x7fffffff) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    step::add_rmsnorm_kernel<__half><<<(unsigned)rows, step::NORM_THREADS, 0, st>>>(
        static_cast<const __half*>(delta), static_cast<__half*>(residual), static_cast<const __half*>(weight),
        static_cast<__half*>(out), hidden, eps);
  else
    step::add_rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, step::NORM_THREADS, 0, st>>>(
        static_cast<const __nv_bfloat16*>(delta), static_cast<__nv_bfloat16*>(residual),
        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), hidden, eps);
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_rope_split_append(const void* qkv, int64_t qkv_stride_b, const void* cos_table,
                                    const void* sin_table, int rope_len, const int64_t* position_ids, int batch,
                                    int n_kv_heads, int n_rep, int head_dim, void* q_out, void* k_cache,
                                    void* v_cache, int64_t cache_stride_b, int64_t cache_stride_h, int capacity,
                                    int append_index, const int32_t* t_fp_dev, int dtype, void* stream) {
  if (batch == 0) return CQ_OK;
  if (!qkv || !cos_table || !sin_table || !position_ids || !q_out || !k_cache || !v_cache) return CQ_ERR_BAD_ARG;
  if (batch < 0 || n_kv_heads <= 0 || n_rep <= 0 || rope_len <= 0 || capacity <= 0) return CQ_ERR_BAD_ARG;
  if (!t_fp_dev && (append_index < 0 || append_index >= capacity)) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (head_dim != kHeadDim) return CQ_ERR_UNSUPPORTED;
  const int64_t blocks = (int64_t)batch * n_kv_heads * (n_rep + 2);
  if (blocks > 0x7fffffff) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    step::rope_split_append_kernel<__half><<<(unsigned)blocks, 64, 0, st>>>(
        static_cast<const __half*>(qkv), qkv_stride_b, static_cast<const __half*>(cos_table),
        static_cast<const __half*>(sin_table), position_ids, n_kv_heads, n_rep, static_cast<__half*>(q_out),
        static_cast<__half*>(k_cache), static_cast<__half*>(v_cache), cache_stride_b, cache_stride_h, capacity,
        append_index, t_fp_dev, rope_len);
  else
    step::rope_split_append_kernel<__nv_bfloat16><<<(unsigned)blocks, 64, 0, st>>>(
        static_cast<const __nv_bfloat16*>(qkv), qkv_stride_b, static_cast<const __nv_bfloat16*>(cos_table),
        static_cast<const __nv_bfloat16*>(sin_table), position_ids, n_kv_heads, n_rep,
        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
        static_cast<__nv_bfloat16*>(v_cache), cache_stride_b, cache_stride_h, capacity, append_index, t_fp_dev,
        rope_len);
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_swiglu(const void* gate, const void* up, void* out, int64_t n, int dtype, void* stream) {
  if (n == 0) return CQ_OK;
  if (!gate || !up || !out || n < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (n % 8) return CQ_ERR_UNSUPPORTED;
  if (!step::aligned16(gate) || !step::aligned16(up) || !step::aligned16(out)) return CQ_ERR_BAD_ARG;
  const int64_t n_vec = n / 8;
  const unsigned grid = (unsigned)((n_vec + 255) / 256 < 148 * 8 ? (n_vec + 255) / 256 : 148 * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    step::swiglu_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(gate),
                                                      static_cast<const __half*>(up), static_cast<__half*>(out), n_vec);
  else
    step::swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gate),
                                                             static_cast<const __nv_bfloat16*>(up),
                                                             static_cast<__nv_bfloat16*>(out), n_vec);
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_swiglu_packed(const void* gate_up, void* out, int64_t rows, int64_t n, int dtype, void* stream) {
  if (rows == 0 || n == 0) return CQ_OK;
  if (!gate_up || !out || rows < 0 || n < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (n % 8) return CQ_ERR_UNSUPPORTED;
  if (!step::aligned16(gate_up) || !step::aligned16(out)) return CQ_ERR_BAD_ARG;
  const int64_t n_vec = n / 8, total = rows * n_vec;
  const unsigned grid = (unsigned)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    step::swiglu_packed_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(gate_up),
                                                             static_cast<__half*>(out), rows, n_vec);
  else
    step::swiglu_packed_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(gate_up),
                                                                    static_cast<__nv_bfloat16*>(out), rows, n_vec);
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_prefill_rope_split(const void* qkv, int64_t qkv_stride_b, int64_t qkv_stride_t, const void* cos_table,
                                     const void* sin_table, int rope_len, const int64_t* position_ids, int batch,
                                     int t_len, int n_kv_heads, int n_rep, int head_dim, void* q_out, void* k_out,
                                     void* k_cache, void* v_cache, int64_t cache_stride_b, int64_t cache_stride_h,
                                     int capacity, int vis_start, int vis_len, int dtype, void* stream) {
  if (batch == 0 || t_len == 0) return CQ_OK;
  if (!qkv || !cos_table || !sin_table || !q_out || !k_out) return CQ_ERR_BAD_ARG;
  if (batch < 0 || t_len < 0 || n_kv_heads <= 0 || n_rep <= 0 || rope_len <= 0) return CQ_ERR_BAD_ARG;
  if (vis_start < 0 || vis_len < 0 || vis_start + vis_len > t_len) return CQ_ERR_BAD_ARG;
  if ((k_cache == nullptr) != (v_cache == nullptr) || (k_cache && capacity <= 0)) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (head_dim != kHeadDim) return CQ_ERR_UNSUPPORTED;
  if (qkv_stride_b % 8 || qkv_stride_t % 8 || cache_stride_b % 8 || cache_stride_h % 8) return CQ_ERR_BAD_ARG;
  if (!step::aligned16(qkv) || !step::aligned16(cos_table) || !step::aligned16(sin_table) || !step::aligned16(q_out) ||
      !step::aligned16(k_out) || !step::aligned16(k_cache) || !step::aligned16(v_cache))
    return CQ_ERR_BAD_ARG;
  const int64_t total = (int64_t)batch * t_len * n_kv_heads * (n_rep + 2) * 8;
  const int64_t blocks = (total + 255) / 256;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    step::prefill_rope_split_kernel<__half><<<grid, 256, 0, st>>>(
        static_cast<const __half*>(qkv), qkv_stride_b, qkv_stride_t, static_cast<const __half*>(cos_table),
        static_cast<const __half*>(sin_table), rope_len, position_ids, t_len, n_kv_heads, n_rep,
        static_cast<__half*>(q_out), static_cast<__half*>(k_out), static_cast<__half*>(k_cache),
        static_cast<__half*>(v_cache), cache_stride_b, cache_stride_h, capacity, vis_start, vis_len, total);
  else
    step::prefill_rope_split_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(qkv), qkv_stride_b, qkv_stride_t, static_cast<const __nv_bfloat16*>(cos_table),
        static_cast<const __nv_bfloat16*>(sin_table), rope_len, position_ids, t_len, n_kv_heads, n_rep,
        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_out), static_cast<__nv_bfloat16*>(k_cache),
        static_cast<__nv_bfloat16*>(v_cache), cache_stride_b, cache_stride_h, capacity, vis_start, vis_len, total);
  return cudaGetLastError() == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}
