// Group-wise min-max quantize + bit-pack (group format), one pass over the data.
//
// Arithmetic contract (what makes the result bit-identical to qjl/new_pack.py:53-82 of the
// reference, whose torch ops each compute in fp32 and round to the tensor dtype):
//   r     = rnd(mx - mn)                  scale = rnd(r / (2^b - 1))
//   d     = rnd(x - mn)                   y     = rnd(d / scale)      (IEEE division)
//   code  = rint_half_even(clamp(y, 0, 2^b - 1))
// word w of a row holds elements w*fpi .. w*fpi+fpi-1, element i in bits [i*b, (i+1)*b).
#include "cq_common.cuh"
#include <cstdlib>

namespace cq {

template <typename T>
__device__ __forceinline__ void group_params(float mn, float mx, int levels, float& scale) {
  float r = rnd<T>(mx - mn);
  scale = rnd<T>(__fdiv_rn(r, (float)levels));
}

// Quotient d/scale for the code decision.  `rcp` is the correctly rounded 1/scale (computed once
// per group); one residual correction makes q faithful to well under one fp32 ulp.  That is
// enough for bit-exact codes: d and scale carry at most 11 significant bits, so the exact
// quotient is never closer than two fp32 ulps to any value at which rint(clamp(fp16(q))) changes
// (those break points are odd 12-bit multiples of a half fp16 ulp), hence q, the IEEE quotient and
// the exact quotient always fall on the same side of every break point.
__device__ __forceinline__ float quotient(float d, float scale, float rcp) {
  const float q = d * rcp;
  return fmaf(fmaf(-scale, q, d), rcp, q);
}

// quotient() of two elements at once on fp32 register pairs (same operations, same roundings)
__device__ __forceinline__ void quotient_pair(float d0, float d1, float s0, float s1, float r0, float r1,
                                              float& q0, float& q1) {
  asm("{\n\t.reg .b64 rd, rs, rr, rq, re;\n\t"
      "mov.b64 rd, {%2, %3};\n\tmov.b64 rs, {%4, %5};\n\tmov.b64 rr, {%6, %7};\n\t"
      "mul.rn.f32x2 rq, rd, rr;\n\t"
      "fma.rn.f32x2 re, rs, rq, rd;\n\t"
      "fma.rn.f32x2 rq, re, rr, rq;\n\t"
      "mov.b64 {%0, %1}, rq;\n\t}"
      : "=f"(q0), "=f"(q1) : "f"(d0), "f"(d1), "f"(-s0), "f"(-s1), "f"(r0), "f"(r1));
}

template <typename T>
__device__ __forceinline__ unsigned quantize_one(float x, float mn, float scale, float rcp, int levels) {
  float d = rnd<T>(x - mn);
  float y = rnd<T>(quotient(d, scale, rcp));
  y = fminf(fmaxf(y, 0.f), (float)levels);   // fmaxf drops the NaN of inf*0 (infinite scale) to 0
  return (unsigned)__float2int_rn(y);
}

// ---- 1- and 2-bit codes without a division ------------------------------------------------------
// rint(clamp(rnd(d/scale))) >= k+1 exactly when the real quotient d/scale lies above the break
// point c_k (see quotient()): c_0 = 1/2 + u/4, c_1 = 3/2 - u/2, c_2 = 5/2 + u, u = 2^-p the unit
// of the data type in [1,2) (p = 10 for fp16, 7 for bf16).  c_k has at most p+3 significant bits and
// scale at most p+1, so c_k*scale is exact in fp32 (2p+4 <= 24 bits), and d, being a number of the
// data type, exceeds it exactly when it exceeds the largest data-type number below it.  So
//     code = sum_k [ d > floor_T(c_k * scale) ]
// with one packed 16-bit compare per threshold and two elements.
template <typename T> struct Pk;
template <> struct Pk<__half> {
  using T2 = __half2;
  static constexpr float U = 0.0009765625f;    // 2^-10
  static __device__ __forceinline__ T2 floor2(float v) { const __half h = __float2half_rz(v); return __halves2half2(h, h); }
  static __device__ __forceinline__ T2 pair(float a, float b) { return __halves2half2(__float2half_rz(a), __float2half_rz(b)); }
  static __device__ __forceinline__ T2 bcast(float v) { return __float2half2_rn(v); }
  static __device__ __forceinline__ T2 pair_rn(float a, float b) { return __floats2half2_rn(a, b); }
  static __device__ __forceinline__ T2 magic() { return __float2half2_rn(1024.f); }
};
template <> struct Pk<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static constexpr float U = 0.0078125f;       // 2^-7
  static __device__ __forceinline__ T2 floor2(float v) { const __nv_bfloat16 h = __float2bfloat16_rz(v); return __halves2bfloat162(h, h); }
  static __device__ __forceinline__ T2 pair(float a, float b) { return __halves2bfloat162(__float2bfloat16_rz(a), __float2bfloat16_rz(b)); }
  static __device__ __forceinline__ T2 bcast(float v) { return __float2bfloat162_rn(v); }
  static __device__ __forceinline__ T2 pair_rn(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ T2 magic() { return __float2bfloat162_rn(128.f); }
};

template <typename T> __device__ __forceinline__ float break_point(int k) {
  return k == 0 ? 0.5f + 0.25f * Pk<T>::U : (k == 1 ? 1.5f - 0.5f * Pk<T>::U : 2.5f + Pk<T>::U);
}

// codes of two elements (low half -> bits [0,BITS), high half -> bits [16,16+BITS)) of d2 = x - mn
template <typename T, int BITS>
__device__ __forceinline__ unsigned codes2(typename Pk<T>::T2 d2, const typename Pk<T>::T2 (&thr)[3]) {
  if (BITS == 1) return __hgt2_mask(d2, thr[0]) & 0x00010001u;
  typename Pk<T>::T2 c = __hadd2(__hadd2(__hgt2(d2, thr[0]), __hgt2(d2, thr[1])), __hgt2(d2, thr[2]));
  c = __hadd2(c, Pk<T>::magic());          // 0..3 as integers in the low mantissa bits
  return *reinterpret_cast<unsigned*>(&c) & 0x00030003u;
}

// 4-bit codes of two elements (low half -> bits [0,4), high half -> bits [16,20)) with the reference's rounding
// points kept: d = x - mn rounded once to the data type, the quotient rounded to the data type, clamp and
// round-half-even there; only the quotient itself runs in fp32 (see quotient()).
template <typename T, bool PAIRED>
__device__ __forceinline__ unsigned codes4_pair(typename Pk<T>::T2 x2, typename Pk<T>::T2 mn2, float s0, float r0,
                                                float s1, float r1) {
  using T2 = typename Pk<T>::T2;
  const float2 d = Elem<T>::to_f2(__hsub2(x2, mn2));
  float q0, q1;
  if (PAIRED) {          // measured: a gain where both elements share the scale, a loss where they do not
    quotient_pair(d.x, d.y, s0, s1, r0, r1, q0, q1);
  } else {
    q0 = quotient(d.x, s0, r0);
    q1 = quotient(d.y, s1, r1);
  }
  T2 y = Pk<T>::pair_rn(q0, q1);
  y = __hmin2(__hmax2(y, Pk<T>::bcast(0.f)), Pk<T>::bcast(15.f));   // the maximum drops the NaN of inf * 0 to 0
  y = __hadd2(h2rint(y), Pk<T>::magic());                          // 0..15 in the low mantissa bits
  return *reinterpret_cast<unsigned*>(&y) & 0x000f000fu;
}

// ---- rows of L contiguous elements; a thread owns 8 consecutive elements (one 128-bit load),
// ---- four neighbouring lanes own one group of 32.
constexpr int PACK_CHUNKS_PER_THREAD = 4;   // independent 128-bit loads in flight per thread

template <typename T, int BITS>
__device__ __forceinline__ void pack_chunk(const uint4& raw, int64_t chunk, bool live,
                                           int32_t* __restrict__ code, T* __restrict__ scale_out,
                                           T* __restrict__ mn_out);

template <typename T, int BITS>
__global__ void __launch_bounds__(256)
pack_last_dim_kernel(const T* __restrict__ data, int64_t n_chunks, int32_t* __restrict__ code,
                     T* __restrict__ scale_out, T* __restrict__ mn_out) {
  uint4 raw[PACK_CHUNKS_PER_THREAD];
  int64_t chunk[PACK_CHUNKS_PER_THREAD];
#pragma unroll
  for (int k = 0; k < PACK_CHUNKS_PER_THREAD; ++k) {
    chunk[k] = ((int64_t)blockIdx.x * PACK_CHUNKS_PER_THREAD + k) * blockDim.x + threadIdx.x;
    raw[k] = make_uint4(0, 0, 0, 0);
    if (chunk[k] < n_chunks) raw[k] = __ldg(reinterpret_cast<const uint4*>(data) + chunk[k]);
  }
#pragma unroll
  for (int k = 0; k < PACK_CHUNKS_PER_THREAD; ++k)
    pack_chunk<T, BITS>(raw[k], chunk[k], chunk[k] < n_chunks, code, scale_out, mn_out);
}

template <typename T, int BITS>
__device__ __forceinline__ void pack_chunk(const uint4& raw, int64_t chunk, bool live,
                                           int32_t* __restrict__ code, T* __restrict__ scale_out,
                                           T* __restrict__ mn_out) {
  // n_chunks is a multiple of 4, so the four lanes of a group are live or dead together
  using T2 = typename Pk<T>::T2;
  constexpr int LEVELS = (1 << BITS) - 1;
  const T2* xv = reinterpret_cast<const T2*>(&raw);
  // min / max of the 8 elements in packed 16-bit arithmetic (exact), then across the quad
  T2 mn2 = __hmin2(__hmin2(xv[0], xv[1]), __hmin2(xv[2], xv[3]));
  T2 mx2 = __hmax2(__hmax2(xv[0], xv[1]), __hmax2(xv[2], xv[3]));
  const float2 fmn = Elem<T>::to_f2(mn2), fmx = Elem<T>::to_f2(mx2);
  float mn = fminf(fmn.x, fmn.y), mx = fmaxf(fmx.x, fmx.y);
  mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 2));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  float scale;
  group_params<T>(mn, mx, LEVELS, scale);
  unsigned local = 0;
  if (mx != mn) {
    if (BITS <= 2) {
      T2 thr[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) thr[k] = Pk<T>::floor2(break_point<T>(k) * scale);
      const T2 mnb = Pk<T>::bcast(mn);
      if (BITS == 1) {
        // all-ones compare masks, element 2i -> bit 2i, element 2i+1 -> bit 17+2i, folded at the end
        unsigned r = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) r |= __hgt2_mask(__hsub2(xv[i], mnb), thr[0]) & (0x00020001u << (2 * i));
        local = (r | (r >> 16)) & 0xffu;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned c = codes2<T, BITS>(__hsub2(xv[i], mnb), thr);   // x - mn: one rounding, as the reference
          local |= ((c & 0xffffu) | (c >> (16 - BITS))) << (2 * i * BITS);
        }
      }
    } else {
      const float rcp = __frcp_rn(scale);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = Elem<T>::to_f2(xv[i]);
        local |= quantize_one<T>(f.x, mn, scale, rcp, LEVELS) << (2 * i * BITS);
        local |= quantize_one<T>(f.y, mn, scale, rcp, LEVELS) << ((2 * i + 1) * BITS);
      }
    }
  }
  // BITS*8 bits per thread; 32/(BITS*8) threads make one word.
  constexpr int THREADS_PER_WORD = 4 / BITS;   // 4, 2, 1
  const int lane = threadIdx.x & 31;
  if (THREADS_PER_WORD > 1) {
    const int pos = lane % THREADS_PER_WORD;
    local <<= pos * 8 * BITS;
#pragma unroll
    for (int o = 1; o < THREADS_PER_WORD; o <<= 1) local |= __shfl_xor_sync(0xffffffffu, local, o);
  }
  if (!live) return;
  if (lane % THREADS_PER_WORD == 0) code[chunk / THREADS_PER_WORD] = (int32_t)local;
  if ((lane & 3) == 0) {
    scale_out[chunk >> 2] = Elem<T>::from_f(scale);
    mn_out[chunk >> 2] = Elem<T>::from_f(mn);
  }
}

// Rows of a [B,H,T,128] tensor given by element strides (t_len == 0: the rows are contiguous).
struct RowView { int64_t t_len = 0; int heads = 1; int64_t stride_b = 0, stride_h = 0, stride_t = 0; };

// ---- the same rows with a whole group of 32 per thread (four 128-bit loads): no exchange between lanes,
// ---- the group's scale and break points computed once instead of once per lane of a quad.  A warp's four
// ---- load instructions together cover 2 KB of consecutive bytes.
template <typename T, int BITS>
__global__ void __launch_bounds__(256)
pack_last_dim_group_kernel(const T* __restrict__ data, int64_t n_groups, int32_t* __restrict__ code,
                           T* __restrict__ scale_out, T* __restrict__ mn_out, RowView view = RowView{}) {
  using T2 = typename Pk<T>::T2;
  constexpr int LEVELS = (1 << BITS) - 1;
  const int64_t grp = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (grp >= n_groups) return;
  uint4 raw[4];
  const uint4* src = reinterpret_cast<const uint4*>(data) + grp * 4;
  if (view.t_len) {            // [B,H,T,128] rows addressed through element strides; outputs stay contiguous
    const int64_t row = grp >> 2, t = row % view.t_len, bh = row / view.t_len;
    src = reinterpret_cast<const uint4*>(data + (bh / view.heads) * view.stride_b + (bh % view.heads) * view.stride_h +
                                         t * view.stride_t + (grp & 3) * 32);
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) raw[k] = __ldg(src + k);
  const T2* xv = reinterpret_cast<const T2*>(raw);              // 16 pairs
  T2 mn2 = xv[0], mx2 = xv[0];
#pragma unroll
  for (int i = 1; i < 16; ++i) { mn2 = __hmin2(mn2, xv[i]); mx2 = __hmax2(mx2, xv[i]); }
  const float2 fmn = Elem<T>::to_f2(mn2), fmx = Elem<T>::to_f2(mx2);
  const float mn = fminf(fmn.x, fmn.y), mx = fmaxf(fmx.x, fmx.y);
  float scale;
  group_params<T>(mn, mx, LEVELS, scale);
  unsigned words[BITS];
#pragma unroll
  for (int w = 0; w < BITS; ++w) words[w] = 0u;
  if (mx != mn) {
    if (BITS <= 2) {
      T2 thr[3];
#pragma unroll
      for (int k = 0; k < 3; ++k) thr[k] = Pk<T>::floor2(break_point<T>(k) * scale);
      const T2 mnb = Pk<T>::bcast(mn);
      if (BITS == 1) {
        // all-ones compare masks: pair i of a half gives bit 2i (low element) and bit 17+2i (high element)
        unsigned r0 = 0, r1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          r0 |= __hgt2_mask(__hsub2(xv[i], mnb), thr[0]) & (0x00020001u << (2 * i));
          r1 |= __hgt2_mask(__hsub2(xv[8 + i], mnb), thr[0]) & (0x00020001u << (2 * i));
        }
        words[0] = ((r0 | (r0 >> 16)) & 0xffffu) | ((r1 | (r1 >> 16)) << 16);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const unsigned c = codes2<T, BITS>(__hsub2(xv[i], mnb), thr);   // x - mn: one rounding, as the reference
          words[(2 * i * BITS) >> 5] |= ((c & 0xffffu) | (c >> (16 - BITS))) << ((2 * i * BITS) & 31);
        }
      }
    } else {
      const float rcp = __frcp_rn(scale);
      const T2 mnb = Pk<T>::bcast(mn);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const unsigned c = codes4_pair<T, true>(xv[i], mnb, scale, rcp, scale, rcp);
        words[(2 * i * BITS) >> 5] |= ((c & 0xfu) | (c >> 12)) << ((2 * i * BITS) & 31);
      }
    }
  }
  if (BITS == 4) {
    *reinterpret_cast<uint4*>(code + grp * 4) = make_uint4(words[0], words[1 % BITS], words[2 % BITS], words[3 % BITS]);
  } else if (BITS == 2) {
    *reinterpret_cast<uint2*>(code + grp * 2) = make_uint2(words[0], words[1 % BITS]);
  } else {
    code[grp] = (int32_t)words[0];
  }
  scale_out[grp] = Elem<T>::from_f(scale);
  mn_out[grp] = Elem<T>::from_f(mn);
}

// ---- K per channel, transpose fused.  A CTA walks a span of 512 tokens (256 at 4 bits) of one
// ---- (batch, head) in sub-tiles of 128 tokens x 128 channels: coalesced 128-bit loads into shared
// ---- memory, then each thread reduces 32 tokens of two adjacent channels (one packed 16-bit pair
// ---- per token).  Words, scales and minima of the span collect in shared memory and leave with
// ---- the lanes running along each channel's row, so a store instruction covers whole sectors.
constexpr int KT_TOKENS = 128;
// 16-byte asynchronous copy into shared memory; !valid writes zeros and reads nothing
__device__ __forceinline__ void pack_cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void pack_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pack_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__host__ __device__ constexpr int kt_span(int bits) { return bits == 4 ? 256 : 512; }

template <typename T, int BITS>
__global__ void __launch_bounds__(256)
pack_k_per_channel_kernel(const T* __restrict__ k, int heads, int64_t T_len,
                          int64_t stride_b, int64_t stride_h, int64_t stride_t,
                          int32_t* __restrict__ code, T* __restrict__ scale_out,
                          T* __restrict__ mn_out) {
  using T2 = typename Pk<T>::T2;
  constexpr int LEVELS = (1 << BITS) - 1;
  constexpr int FPI = 32 / BITS;
  constexpr int WORDS_PER_GROUP = BITS;      // 32 tokens * BITS / 32
  constexpr int SPAN = kt_span(BITS);
  constexpr int SPAN_GROUPS = SPAN / 32;
  constexpr int WPR = SPAN_GROUPS * BITS;    // code words per channel row per span
  constexpr int CP = WPR + 1, SP = SPAN_GROUPS + 2;    // padded row pitches: rows on different banks
  extern __shared__ __align__(16) unsigned char pack_smem[];
  constexpr int TILES_BYTES = 2 * KT_TOKENS * kHeadDim * sizeof(T);      // two sub-tiles: one lands while one is read
  T (*tiles)[kHeadDim] = reinterpret_cast<T (*)[kHeadDim]>(pack_smem);  // [2 * KT_TOKENS][kHeadDim]
  unsigned (*code_s)[CP] = reinterpret_cast<unsigned (*)[CP]>(pack_smem + TILES_BYTES);
  T (*scale_s)[SP] = reinterpret_cast<T (*)[SP]>(pack_smem + TILES_BYTES + kHeadDim * CP * 4);
  T (*mn_s)[SP] = scale_s + kHeadDim;

  const int bh = blockIdx.y;
  const int b = bh / heads, h = bh % heads;
  const int64_t span0 = (int64_t)blockIdx.x * SPAN;
  const T* src = k + b * stride_b + h * stride_h;
  const int span_tok = (int)min((int64_t)SPAN, T_len - span0);   // multiple of 32
  const int gq = threadIdx.x / 64;        // group (of 32 tokens) inside the sub-tile
  const int cp = threadIdx.x % 64;        // channel pair

  // 2048 16-byte pieces per sub-tile, 8 per thread, copied asynchronously: sub-tile s+1 lands while s is read
  auto issue = [&](int sub) {
    const int64_t t0 = span0 + sub * KT_TOKENS;
    const int n_tok = min(KT_TOKENS, span_tok - sub * KT_TOKENS);
    T (*dst)[kHeadDim] = tiles + (sub & 1) * KT_TOKENS;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = threadIdx.x + j * 256;
      const int row = i / (kHeadDim / 8), col = i % (kHeadDim / 8);
      const bool valid = row < n_tok;
      pack_cp_async16(&dst[row][col * 8], src + (t0 + (valid ? row : 0)) * stride_t + col * 8, valid);
    }
    pack_cp_async_commit();
  };
  issue(0);
  for (int sub = 0; sub * KT_TOKENS < span_tok; ++sub) {
    const int n_tok = min(KT_TOKENS, span_tok - sub * KT_TOKENS);
    T (*tile)[kHeadDim] = tiles + (sub & 1) * KT_TOKENS;
    __syncthreads();                       // sub-tile sub-1 fully consumed: its buffer may be refilled
    if ((sub + 1) * KT_TOKENS < span_tok) {
      issue(sub + 1);
      pack_cp_async_wait<1>();
    } else {
      pack_cp_async_wait<0>();
    }
    __syncthreads();                       // every thread's pieces of this sub-tile have landed
    if (gq * 32 >= n_tok) continue;

    T2 xv[32];
#pragma unroll
    for (int t = 0; t < 32; ++t) xv[t] = *reinterpret_cast<const T2*>(&tile[gq * 32 + t][cp * 2]);
    T2 mn2 = xv[0], mx2 = xv[0];
#pragma unroll
    for (int t = 1; t < 32; ++t) {
      mn2 = __hmin2(mn2, xv[t]);
      mx2 = __hmax2(mx2, xv[t]);
    }
    const float2 fmn = Elem<T>::to_f2(mn2), fmx = Elem<T>::to_f2(mx2);
    float scale[2];
    group_params<T>(fmn.x, fmx.x, LEVELS, scale[0]);
    group_params<T>(fmn.y, fmx.y, LEVELS, scale[1]);
    const bool constant[2] = {fmx.x == fmn.x, fmx.y == fmn.y};
    unsigned words[2][WORDS_PER_GROUP];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
      for (int w = 0; w < WORDS_PER_GROUP; ++w) words[c][w] = 0u;

    if (BITS <= 2) {
      T2 thr[3];
#pragma unroll
      for (int kk = 0; kk < 3; ++kk)
        thr[kk] = Pk<T>::pair(break_point<T>(kk) * scale[0], break_point<T>(kk) * scale[1]);
      if (BITS == 1) {
        // all-ones compare masks: token t of a half gives bit t (first channel) and bit 16 + t (second channel)
        unsigned ra = 0, rb = 0;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          ra |= __hgt2_mask(__hsub2(xv[t], mn2), thr[0]) & (0x00010001u << t);
          rb |= __hgt2_mask(__hsub2(xv[16 + t], mn2), thr[0]) & (0x00010001u << t);
        }
        words[0][0] = (ra & 0xffffu) | (rb << 16);
        words[1][0] = (ra >> 16) | (rb & 0xffff0000u);
      } else {
        // codes of 16/BITS tokens collect in one register (first channel in the low half, second in the high
        // half: one multiply-add per token), then the halves go to the two channels' words
        constexpr int TPA = 16 / BITS;
#pragma unroll
        for (int t0 = 0; t0 < 32; t0 += TPA) {
          unsigned acc = 0;
#pragma unroll
          for (int j = 0; j < TPA; ++j) acc += codes2<T, BITS>(__hsub2(xv[t0 + j], mn2), thr) << (j * BITS);
          words[0][t0 / FPI] |= (acc & 0xffffu) << ((t0 % FPI) * BITS);
          words[1][t0 / FPI] |= (acc >> 16) << ((t0 % FPI) * BITS);
        }
      }
    } else {
      const float rcp[2] = {__frcp_rn(scale[0]), __frcp_rn(scale[1])};
#pragma unroll
      for (int t0 = 0; t0 < 32; t0 += 4) {               // four tokens per register, as above
        unsigned acc = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc += codes4_pair<T, false>(xv[t0 + j], mn2, scale[0], rcp[0], scale[1], rcp[1]) << (j * BITS);
        words[0][t0 / FPI] |= (acc & 0xffffu) << ((t0 % FPI) * BITS);
        words[1][t0 / FPI] |= (acc >> 16) << ((t0 % FPI) * BITS);
      }
    }
    const int gs = sub * (KT_TOKENS / 32) + gq;            // group inside the span
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int w = 0; w < WORDS_PER_GROUP; ++w)
        code_s[cp * 2 + c][gs * WORDS_PER_GROUP + w] = constant[c] ? 0u : words[c][w];
      scale_s[cp * 2 + c][gs] = Elem<T>::from_f(scale[c]);
      mn_s[cp * 2 + c][gs] = Elem<T>::from_f(c == 0 ? fmn.x : fmn.y);
    }
  }
  __syncthreads();

  // ---- flush the span: lanes run along a channel's row
  const int64_t n_groups = T_len / 32;
  const int64_t g0 = span0 / 32;
  const int live_groups = span_tok / 32, live_words = live_groups * WORDS_PER_GROUP;
  const int64_t row0 = (int64_t)bh * kHeadDim;
  for (int i = threadIdx.x; i < kHeadDim * WPR; i += 256) {
    const int ch = i / WPR, w = i % WPR;
    if (w < live_words) code[(row0 + ch) * (n_groups * WORDS_PER_GROUP) + g0 * WORDS_PER_GROUP + w] = (int32_t)code_s[ch][w];
  }
  for (int i = threadIdx.x; i < kHeadDim * SPAN_GROUPS; i += 256) {
    const int ch = i / SPAN_GROUPS, gg = i % SPAN_GROUPS;
    if (gg < live_groups) {
      scale_out[(row0 + ch) * n_groups + g0 + gg] = scale_s[ch][gg];
      mn_out[(row0 + ch) * n_groups + g0 + gg] = mn_s[ch][gg];
    }
  }
}

template <typename T>
int launch_pack_last_dim(const void* data, int64_t rows, int64_t L, int bits, int32_t* code,
                         void* scale, void* mn, cudaStream_t st) {
  const int64_t n_chunks = rows * L / 8;
  const int64_t per_block = 256 * PACK_CHUNKS_PER_THREAD;
  const int64_t blocks = (n_chunks + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) return CQ_ERR_UNSUPPORTED;
  const T* d = static_cast<const T*>(data);
  T* s = static_cast<T*>(scale);
  T* m = static_cast<T*>(mn);
  // aligned outputs: one group per thread; otherwise the lane-quad kernel with scalar stores
  if (aligned16(code) && aligned16(data)) {
    const int64_t n_groups = n_chunks / 4;
    const int64_t gblocks = (n_groups + 255) / 256;
    if (gblocks > 0x7fffffffLL) return CQ_ERR_UNSUPPORTED;
    switch (bits) {
      case 1: pack_last_dim_group_kernel<T, 1><<<(unsigned)gblocks, 256, 0, st>>>(d, n_groups, code, s, m); break;
      case 2: pack_last_dim_group_kernel<T, 2><<<(unsigned)gblocks, 256, 0, st>>>(d, n_groups, code, s, m); break;
      default: pack_last_dim_group_kernel<T, 4><<<(unsigned)gblocks, 256, 0, st>>>(d, n_groups, code, s, m); break;
    }
    return check_launch();
  }
  switch (bits) {
    case 1: pack_last_dim_kernel<T, 1><<<(unsigned)blocks, 256, 0, st>>>(d, n_chunks, code, s, m); break;
    case 2: pack_last_dim_kernel<T, 2><<<(unsigned)blocks, 256, 0, st>>>(d, n_chunks, code, s, m); break;
    default: pack_last_dim_kernel<T, 4><<<(unsigned)blocks, 256, 0, st>>>(d, n_chunks, code, s, m); break;
  }
  return check_launch();
}

template <typename T>
int launch_pack_k(const void* k, int batch, int heads, int64_t T_len, int64_t sb, int64_t sh,
                  int64_t st_, int bits, int32_t* code, void* scale, void* mn, cudaStream_t st) {
  const int span = kt_span(bits);
  dim3 grid((unsigned)((T_len + span - 1) / span), (unsigned)(batch * heads));
  const int wpr = span / 32 * bits;
  const size_t smem = 2 * (size_t)KT_TOKENS * kHeadDim * 2 + (size_t)kHeadDim * (wpr + 1) * 4 +
                      2 * (size_t)kHeadDim * (span / 32 + 2) * 2;
  cudaError_t e;
  switch (bits) {
    case 1: e = cudaFuncSetAttribute(pack_k_per_channel_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); break;
    case 2: e = cudaFuncSetAttribute(pack_k_per_channel_kernel<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); break;
    default: e = cudaFuncSetAttribute(pack_k_per_channel_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); break;
  }
  if (e != cudaSuccess) return CQ_ERR_LAUNCH;
  const T* d = static_cast<const T*>(k);
  T* s = static_cast<T*>(scale);
  T* m = static_cast<T*>(mn);
  switch (bits) {
    case 1: pack_k_per_channel_kernel<T, 1><<<grid, 256, smem, st>>>(d, heads, T_len, sb, sh, st_, code, s, m); break;
    case 2: pack_k_per_channel_kernel<T, 2><<<grid, 256, smem, st>>>(d, heads, T_len, sb, sh, st_, code, s, m); break;
    default: pack_k_per_channel_kernel<T, 4><<<grid, 256, smem, st>>>(d, heads, T_len, sb, sh, st_, code, s, m); break;
  }
  return check_launch();
}

}  // namespace cq

extern "C" int cq_pack_last_dim(const void* data, int64_t rows, int64_t L, int group_size,
                                int bits, int dtype, int32_t* code, void* scale, void* mn,
                                void* stream) {
  if (rows < 0 || L < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (bits != 1 && bits != 2 && bits != 4) return CQ_ERR_UNSUPPORTED;
  if (group_size != cq::kGroup || L % 32 != 0) return CQ_ERR_UNSUPPORTED;
  if (rows == 0 || L == 0) return CQ_OK;   // empty input: nothing to read or write
  if (!data || !code || !scale || !mn) return CQ_ERR_BAD_ARG;
  if (!cq::aligned16(data)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    return cq::launch_pack_last_dim<__half>(data, rows, L, bits, code, scale, mn, st);
  return cq::launch_pack_last_dim<__nv_bfloat16>(data, rows, L, bits, code, scale, mn, st);
}

extern "C" int cq_pack_v_per_token(const void* v, int batch, int heads, int64_t T, int D, int64_t stride_b,
                                   int64_t stride_h, int64_t stride_t, int group_size, int bits, int dtype,
                                   int32_t* code, void* scale, void* mn, void* stream) {
  if (batch < 0 || heads < 0 || T < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (bits != 1 && bits != 2 && bits != 4) return CQ_ERR_UNSUPPORTED;
  if (group_size != cq::kGroup || D != cq::kHeadDim) return CQ_ERR_UNSUPPORTED;
  if (batch == 0 || heads == 0 || T == 0) return CQ_OK;   // empty input
  if (!v || !code || !scale || !mn) return CQ_ERR_BAD_ARG;
  if (!cq::aligned16(v) || stride_b % 8 || stride_h % 8 || stride_t % 8) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cq::RowView view;
  view.t_len = T; view.heads = heads; view.stride_b = stride_b; view.stride_h = stride_h; view.stride_t = stride_t;
  const int64_t n_groups = (int64_t)batch * heads * T * 4;
  const int64_t gblocks = (n_groups + 255) / 256;
  if (gblocks > 0x7fffffffLL) return CQ_ERR_UNSUPPORTED;
#define CQ_LAUNCH_V(TYPE, B)                                                                              \
  cq::pack_last_dim_group_kernel<TYPE, B><<<(unsigned)gblocks, 256, 0, st>>>(                              \
      static_cast<const TYPE*>(v), n_groups, code, static_cast<TYPE*>(scale), static_cast<TYPE*>(mn), view)
  if (dtype == CQ_DTYPE_F16) {
    if (bits == 1) CQ_LAUNCH_V(__half, 1); else if (bits == 2) CQ_LAUNCH_V(__half, 2); else CQ_LAUNCH_V(__half, 4);
  } else {
    if (bits == 1) CQ_LAUNCH_V(__nv_bfloat16, 1); else if (bits == 2) CQ_LAUNCH_V(__nv_bfloat16, 2);
    else CQ_LAUNCH_V(__nv_bfloat16, 4);
  }
#undef CQ_LAUNCH_V
  return cq::check_launch();
}

extern "C" int cq_pack_k_per_channel(const void* k, int batch, int heads, int64_t T, int D,
                                     int64_t stride_b, int64_t stride_h, int64_t stride_t,
                                     int group_size, int bits, int dtype, int32_t* code,
                                     void* scale, void* mn, void* stream) {
  if (batch < 0 || heads < 0 || T < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (bits != 1 && bits != 2 && bits != 4) return CQ_ERR_UNSUPPORTED;
  if (group_size != cq::kGroup || T % 32 != 0 || D != cq::kHeadDim) return CQ_ERR_UNSUPPORTED;
  if (batch == 0 || heads == 0 || T == 0) return CQ_OK;   // empty input
  if (!k || !code || !scale || !mn) return CQ_ERR_BAD_ARG;
  if (!cq::aligned16(k) || stride_b % 8 || stride_h % 8 || stride_t % 8) return CQ_ERR_BAD_ARG;
  if ((int64_t)batch * heads > 65535) return CQ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    return cq::launch_pack_k<__half>(k, batch, heads, T, stride_b, stride_h, stride_t, bits, code, scale, mn, st);
  return cq::launch_pack_k<__nv_bfloat16>(k, batch, heads, T, stride_b, stride_h, stride_t, bits, code, scale, mn, st);
}
