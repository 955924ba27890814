// Decode-step attention, fast path: persistent CTAs, TMA-staged K/V tiles, packed-code dot
// products on the warp-level fp16 tensor-core MMA.
//
// Why a tensor-core instruction on an HBM-bound path: with GQA every packed K/V bit is used by
// n_rep (4..8) query heads, i.e. 16 multiply-adds per byte at 1 bit.  At HBM speed that is
// ~100 T multiply-adds/s, three times the fp32 FMA rate of the SMs, so a CUDA-core inner loop is
// instruction-issue bound at a fraction of the memory roofline.  The packed codes are therefore
// expanded *in registers* into fp16 MMA operands and contracted with m16n8k16:
//   * a byte permute (PRMT) drops one byte of two code words (two adjacent contraction indices)
//     into the low bytes of the two fp16 halves of a register, and one AND keeps the b-bit field of
//     the row this lane owns.  The surviving pattern c << s (c the code, s < 8) read as fp16 is the
//     subnormal c * 2^(s-24): exact, and linear in c.  The 2^(24-s) factor is applied to the fp32
//     accumulator of that row afterwards.  Two rows of a lane (adjacent tokens / channels) share
//     the PRMT (at 1 bit the rows of two m-tiles do), so an A operand register costs 1.25-1.5 integer
//     instructions.
//   * "post-scaling": the other operand carries the scales, never the codes:
//       scores : B[d][h] = q[h][d] * ks[d,G]          (per 32-token group G)
//       attn.V : B[t][h] = p[h][t] * vs[t,g]          (per 32-channel group g)
//     and the minima fold into one extra small MMA per tile (sum_d q*kmn, sum_t p*vmn), whose spare
//     column also yields sum_t p (the softmax denominator).
//
// Three launches per decode step (four with full-precision tokens) on the caller's stream; the
// streaming ones are persistent (grid = resident CTAs):
//   K1 scores   : logits (fp16-rounded exactly where the reference rounds) -> workspace, plus
//                 per-tile min/max of the visual logits for the calibration
//   K2 attn.V   : per chunk of visual tokens: calibrate, exp relative to the chunk max, accumulate,
//                 write (max, sum, acc[128]) partials
//   K2 fp       : (only with full-precision tokens) the same partials for chunks of 128 fp tokens
//   K3 combine  : merge the chunk partials (online-softmax rescale), round to the output dtype
//
// Eligibility (otherwise cq_decode_attn uses the general kernels): t_vis % 256 == 0,
// 16-byte aligned operands.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <utility>
#include <type_traits>

#include "cq_common.cuh"
#include "cq_ptx.cuh"
#include "cq_decode_shared.cuh"

namespace cq {
namespace mma {

using namespace ptx;

constexpr int THREADS = 128;
constexpr int K1_WARPS = 4;            // computing warps of a score CTA; each owns tile_g / K1_WARPS groups of a K tile
constexpr int K1_THREADS = (K1_WARPS + 1) * 32;   // + the TMA producer warp
// 32-token groups per K tile: 32, but 16 at 4 bits, where a ring of 32-group tiles (80 KB each) leaves room for
// one CTA per SM only and the kernel then runs with 1.2 warps per scheduler
__host__ __device__ constexpr int tile_g(int bits) { return bits == 4 ? 16 : 32; }
// attn.V work items: CT tokens per item, streamed as tiles of VT tokens.  Two shapes are compiled: the
// large one for long contexts, the small one when the large one would leave CTAs without work.
constexpr int VT_LARGE = 512, VT_SMALL = 256;
constexpr int K2_WARPS = 4;            // computing warps of an attn.V CTA
constexpr int K2_THREADS = (K2_WARPS + 1) * 32;   // + the producer warp
constexpr int K2_RESIDENT = 296;       // attn.V CTAs resident on the device (2 per SM), for the choice below
constexpr uint32_t WAIT_TRIES = 1u << 22;
constexpr float LOG2E = 1.4426950408889634f;

__host__ __device__ constexpr int k1_stage_bytes(int bits) { return tile_g(bits) * (bits * 512 + 512); }
__host__ __device__ constexpr int k1_stages(int bits) { return 3 * k1_stage_bytes(bits) <= 100 * 1024 ? 3 : 2; }
__host__ __device__ constexpr int k1_min_ctas(int bits) {
  return (220 * 1024) / (k1_stages(bits) * k1_stage_bytes(bits) + 2048) > 4 ? 4 : (220 * 1024) / (k1_stages(bits) * k1_stage_bytes(bits) + 2048);
}
__host__ __device__ constexpr int k1_code_row_bytes(int bits) { return tile_g(bits) * bits * 4 < 128 ? tile_g(bits) * bits * 4 : 128; }
// an attn.V stage: codes, scales, minima, and the logits of kMaxRep heads for the tile's tokens
// (logit rows are 16 bytes longer than a tile so that the heads fall on different banks)
// At 2 and 4 bits the codes arrive as swizzled TMA boxes, whose pattern is a function of the shared-memory
// address: stages then start on 1 KB boundaries.
__host__ __device__ constexpr int k2_stage_bytes(int bits, int vt) {
  return bits == 1 ? vt * (16 * bits + 16) + kMaxRep * (2 * vt + 16)
                   : (vt * (16 * bits + 16) + kMaxRep * (2 * vt + 16) + 1023) / 1024 * 1024;
}
__host__ __device__ constexpr int k2_stages(int bits, int vt) { return 3 * k2_stage_bytes(bits, vt) <= 76 * 1024 ? 3 : 2; }
__host__ __device__ constexpr int k2_smem_bytes(int bits, int vt) {
  return k2_stages(bits, vt) * k2_stage_bytes(bits, vt) + K2_WARPS * kMaxRep * 136 * 4 + 1024;
}

struct Dims {
  int batch, hq, hkv, n_rep, t_vis, t_fp, calibrate;
  int n_groups;        // t_vis / 32
  int n_ktiles;        // ceil(n_groups / tile_g(bits))
  int chunk_tok;       // tokens per attn.V tile: VT_LARGE or VT_SMALL
  int n_chunks;        // tiles per KV head: ceil(t_vis / chunk_tok); one partial slot each
  int n_fp_chunks;     // ceil(t_fp / 128)
  int n_slots;         // n_chunks + n_fp_chunks
  int pitch;           // score row pitch in elements (multiple of 8)
  int n_mm;            // min/max entries per row: n_ktiles * K1_WARPS
  int64_t fp_stride_b, fp_stride_h;
  const int32_t* t_fp_dev;   // optional: live number of fp tokens on the device (t_fp is then the capacity)
  int raw;                   // 1: plain quantized product (cq_qbmm): no 1/sqrt(D), no softmax, no normalisation
  const void* mask;          // optional additive mask [batch][t_sys | t_vis | text] in the data dtype
  int64_t mask_stride_b;
  int t_sys;                 // fp tokens that precede the visual span in the mask's key order
};

// Number of full-precision tokens this launch works on: the by-value extent, or, when the caller keeps
// the count on the device (a decode step replayed from a CUDA graph), that count clamped to it.
__device__ __forceinline__ int live_t_fp(const Dims& dm) {
  return dm.t_fp_dev ? min(__ldg(dm.t_fp_dev), dm.t_fp) : dm.t_fp;
}

// ---- per-lane constants for expanding packed codes into MMA A operands -------------------------
// A lane (g = lane/4) owns rows g and g+8 of a 16-row m-tile; they are mapped to two adjacent
// packed elements e, e+1 of the 32-element group the m-tile belongs to (m-tile i = 0, 1 of the group).
// Which element a row stands for is free, as long as the epilogue agrees:
//   2 bits: e = 16 i + 2g, so m-tile i is one word of the group;
//   4 bits: e = 16 (g/4) + 8 i + 2 (g%4): the lane's two m-tiles are the adjacent words 2(g/4), 2(g/4)+1 of the
//           group's four, fetched by one 8-byte load;
//   1 bit:  e = 4g + 2i, so both m-tiles take their bits from the same byte of the same word
//           and share one byte permute.
template <int BITS>
struct Expand {
  static __device__ __forceinline__ int elem(int i, int g) {
    return BITS == 1 ? 4 * g + 2 * i : BITS == 4 ? 16 * (g >> 2) + 8 * i + 2 * (g & 3) : 16 * i + 2 * g;
  }
  static __device__ __forceinline__ int bit_off(int i, int g) { return elem(i, g) * BITS; }
};

__device__ __forceinline__ uint32_t prmt_sel(int byte) {
  return (uint32_t)(byte | (byte << 4) | ((4 + byte) << 8) | ((4 + byte) << 12));
}

// barrier among a subset of the CTA's warps (the producer warp takes no part)
__device__ __forceinline__ void named_barrier_sync(int id, int n_threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

// ---- data-dtype helpers.  The MMA operands are always fp16: bf16 scales, minima and queries fit
// ---- fp16 exactly (8 significant bits) within its range, so they are converted on the way in,
// ---- while every value the reference rounds to the data dtype is rounded to T here too.
template <typename T> struct D16;
template <> struct D16<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ uint32_t to_h2(uint32_t v) { return v; }
  static __device__ __forceinline__ T2 round2(float a, float b) { return __floats2half2_rn(a, b); }
  static __device__ __forceinline__ T2 bcast(float a) { return __float2half2_rn(a); }
  static __device__ __forceinline__ T2 pair2(__half a, __half b) { return __halves2half2(a, b); }
  static __device__ __forceinline__ float2 to_f2(T2 v) { return __half22float2(v); }
  static __device__ __forceinline__ float big() { return 65504.f; }
  // two probabilities rounded to the data dtype, as an fp16 pair
  static __device__ __forceinline__ uint32_t prob_pair(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  // rnd(x / sqrt(128)) as the reference's division gives it: 1/sqrt(128) as two fp16 terms (the
  // second one carries the 1e-4 relative error of the first), product formed by one FMA, one rounding.
  // A plain multiply by fp16(1/sqrt(128)) lands on the neighbouring fp16 value for one logit in ten.
  static __device__ __forceinline__ T2 inv_sqrt_d(T2 x) {
    const __half2 c_hi = __float2half2_rn(0.08837890625f);                       // fp16(1/sqrt(128))
    const __half2 c_lo = __float2half2_rn(0.08838834764831845f - 0.08837890625f);
    return __hfma2(x, c_hi, __hmul2(x, c_lo));
  }
};
template <> struct D16<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ uint32_t to_h2(uint32_t v) {
    const __half2 h = __floats2half2_rn(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ T2 round2(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ T2 bcast(float a) { return __float2bfloat162_rn(a); }
  static __device__ __forceinline__ T2 pair2(__nv_bfloat16 a, __nv_bfloat16 b) { return __halves2bfloat162(a, b); }
  static __device__ __forceinline__ float2 to_f2(T2 v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ float big() { return 3.0e38f; }
  static __device__ __forceinline__ uint32_t prob_pair(float a, float b) {
    const __nv_bfloat162 r = __floats2bfloat162_rn(a, b);
    return to_h2(*reinterpret_cast<const uint32_t*>(&r));
  }
  // bf16(1/sqrt(128)) would be off by up to 2^-9 (a systematic error on every logit): multiply in fp32
  static __device__ __forceinline__ T2 inv_sqrt_d(T2 x) {
    const float2 f = __bfloat1622float2(x);
    return __floats2bfloat162_rn(f.x * 0.08838834764831845f, f.y * 0.08838834764831845f);
  }
};

// =================================================================================================
// K1: scores
// =================================================================================================
// Rows g / g+8 of m-tile i of a group are the adjacent tokens Expand::elem(i, g), +1.  The B operand
// carries q * ks (post-scaling).  With at most four query heads per KV head (SPLIT) the product is
// carried as two fp16 terms in neighbouring MMA columns, hi = rnd(q*ks) in column 2h and the exact
// remainder lo = q*ks - hi in column 2h+1 (lanes with odd g build the remainder), and the two columns
// are added in the epilogue: a single fp16 rounding of q*ks (2^-12 relative) moves one raw score in eight
// across an fp16 rounding boundary of the reference, 2% of a probability each.  With five to eight heads
// all eight columns carry heads and q*ks is rounded once.
//
// Warps 0-3 compute, warp 4 is the TMA producer: stages are handed over through a full barrier (bytes
// landed) and an empty barrier (one arrival per computing warp), so no warp waits for another warp's
// arithmetic, only for data.
// LDG: the variant for token counts that are not a multiple of 256.  The row pitches of the packed keys
// (T*bits/8 bytes) and of their scales and minima (T/16 bytes) are then no multiples of 16 bytes, which a tensor
// map cannot describe: the producer warp copies the code words with 4-byte cp.async into the same swizzled layout
// (words past the last group are zero-filled), the computing warps read their scale and minimum fragments straight
// from global memory, and groups past the end are neither stored nor counted in the min/max.
template <typename T, int BITS, bool SPLIT, bool LDG = false>
__global__ void __launch_bounds__(K1_THREADS, k1_min_ctas(BITS))
k1_scores(const __grid_constant__ CUtensorMap tm_code, const __grid_constant__ CUtensorMap tm_ks,
          const __grid_constant__ CUtensorMap tm_kmn, Dims dm, const T* __restrict__ q,
          T* __restrict__ scores, float2* __restrict__ tile_mm, int* __restrict__ status,
          const int32_t* __restrict__ code_g = nullptr, const T* __restrict__ ks_g = nullptr,
          const T* __restrict__ kmn_g = nullptr) {
  using T2 = typename D16<T>::T2;
  constexpr int STAGES = k1_stages(BITS);
  constexpr int STAGE_BYTES = k1_stage_bytes(BITS);
  constexpr int TILE_G = tile_g(BITS);
  constexpr int K1_GPW = TILE_G / K1_WARPS;
  constexpr int CODE_BYTES = TILE_G * BITS * 512;
  constexpr int KS_BYTES = TILE_G * 256;
  constexpr int ROW_BYTES = k1_code_row_bytes(BITS);   // bytes of a channel row inside one TMA box
  constexpr int N_BOXES = TILE_G * BITS * 4 / ROW_BYTES;
  constexpr int KS_ROW = TILE_G * 2;                   // bytes of a scale row
  constexpr int GU = 4 / BITS;             // groups per 16-byte chunk of a channel row
  constexpr int UNITS = K1_GPW / GU;       // chunks per warp
  constexpr uint32_t FIELD = (1u << BITS) - 1u;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int n_pairs = dm.batch * dm.hkv;
  const int n_items = n_pairs * dm.n_ktiles;

  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], LDG ? 32 : 1); mbar_init(&empty_bar[s], K1_WARPS); }
    mbar_fence_init();
  }
  __syncthreads();

  // every CTA takes a contiguous range of (KV head, tile) items: the query fragments are reloaded
  // only when the KV head changes, and neighbouring CTAs stream neighbouring tiles
  const int it_first = (int)(((int64_t)blockIdx.x * n_items) / gridDim.x);
  const int it_end = (int)(((int64_t)(blockIdx.x + 1) * n_items) / gridDim.x);

  if (LDG && warp == K1_WARPS) {
    // ---- producer, all 32 lanes: 4-byte asynchronous copies of the tile's code words into the swizzled boxes
    constexpr int WPR = TILE_G * BITS;                 // words of a channel row inside a tile
    const int64_t row_words = (int64_t)dm.n_groups * BITS;
    for (int k = 0; it_first + k < it_end; ++k) {
      const int it = it_first + k, s = k % STAGES;
      if (k >= STAGES && !mbar_wait_bounded(&empty_bar[s], (uint32_t)((k / STAGES - 1) & 1), WAIT_TRIES)) {
        if (lane == 0) atomicExch(status, CQ_ERR_TIMEOUT);
        break;
      }
      const int pair = it / dm.n_ktiles, tile = it % dm.n_ktiles;
      const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
      const int valid = min(TILE_G, dm.n_groups - tile * TILE_G) * BITS;     // live words of a row
      const int32_t* src0 = code_g + (int64_t)pair * kHeadDim * row_words + (int64_t)tile * WPR;
      for (int i = lane; i < kHeadDim * WPR; i += 32) {
        const int d = i / WPR, w = i % WPR;
        const int cb = (w * 4) % ROW_BYTES, box = (w * 4) / ROW_BYTES;
        const int sw = ROW_BYTES == 64 ? ((d >> 1) & 3) : (d & 7);
        const uint32_t dst = base + (uint32_t)(box * (128 * ROW_BYTES) + d * ROW_BYTES + (((cb >> 4) ^ sw) << 4) + (cb & 15));
        const bool live = w < valid;
        cp_async4_zfill(dst, src0 + (int64_t)d * row_words + (live ? w : 0), live ? 4u : 0u);
      }
      cp_async_mbar_arrive_noinc(&full_bar[s]);
    }
    return;
  }
  if (warp == K1_WARPS) {
    // ---- producer: one thread streams the CTA's tiles through the ring
    if (lane == 0) {
      fence_proxy_async_smem();
      for (int k = 0; it_first + k < it_end; ++k) {
        const int it = it_first + k, s = k % STAGES;
        if (k >= STAGES && !mbar_wait_bounded(&empty_bar[s], (uint32_t)((k / STAGES - 1) & 1), WAIT_TRIES)) {
          atomicExch(status, CQ_ERR_TIMEOUT);
          break;
        }
        const int pair = it / dm.n_ktiles, tile = it % dm.n_ktiles;
        unsigned char* base = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
#pragma unroll
        for (int bx = 0; bx < N_BOXES; ++bx)
          tma_load_2d(base + bx * (128 * ROW_BYTES), &tm_code, tile * TILE_G * BITS + bx * (ROW_BYTES / 4), pair * kHeadDim,
                      &full_bar[s]);
        tma_load_2d(base + CODE_BYTES, &tm_ks, tile * TILE_G, pair * kHeadDim, &full_bar[s]);
        tma_load_2d(base + CODE_BYTES + KS_BYTES, &tm_kmn, tile * TILE_G, pair * kHeadDim, &full_bar[s]);
      }
    }
    return;
  }

  // lane constants: selectors / masks / accumulator scales for the two m-tiles of a group
  uint32_t sel[2], m0[2], m1[2];
  int word_in_group[2];
  float sc0[2], sc1[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int off = Expand<BITS>::bit_off(i, g);
    word_in_group[i] = off / 32;
    const int byte = (off % 32) / 8, sh = off % 8;
    sel[i] = prmt_sel(byte);
    m0[i] = (FIELD << sh) * 0x00010001u;
    m1[i] = (FIELD << (sh + BITS)) * 0x00010001u;
    sc0[i] = exp2f((float)(24 - sh));
    sc1[i] = exp2f((float)(24 - sh - BITS));
  }
  (void)word_in_group;

  // The producer above streams only the packed keys, which no launch of a decode step writes, so it may run
  // ahead of the kernel before this one in the stream; the query and the score buffer
  // (still read by the previous step) are touched only after that kernel has completed.
  pdl_wait();
  int cur_pair = -1;
  uint32_t qA[8], qB[8];
  bool failed = false;
  const int q_head = SPLIT ? (g >> 1) : g;        // the head whose query this lane's B column carries
  const bool lo_lane = SPLIT && (g & 1);
  // heads this lane's accumulator columns stand for: SPLIT: head c (columns 2c = hi, 2c+1 = lo); else heads 2c, 2c+1
  const int out_head = SPLIT ? c : 2 * c;

  for (int k = 0;; ++k) {
    const int it = it_first + k;
    if (it >= it_end) break;
    const int s = k % STAGES;
    const int pair = it / dm.n_ktiles, tile = it % dm.n_ktiles;
    if (pair != cur_pair) {   // query fragments of this KV head's query heads (B operand, n = g)
      cur_pair = pair;
      const int b = pair / dm.hkv, hk = pair % dm.hkv;
      const T* qrow = q + ((int64_t)b * dm.hq + (int64_t)hk * dm.n_rep + q_head) * kHeadDim;
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        qA[kt] = q_head < dm.n_rep ? D16<T>::to_h2(*reinterpret_cast<const uint32_t*>(qrow + kt * 16 + 2 * c)) : 0u;
        qB[kt] = q_head < dm.n_rep ? D16<T>::to_h2(*reinterpret_cast<const uint32_t*>(qrow + kt * 16 + 2 * c + 8)) : 0u;
      }
    }
    if (!mbar_wait_bounded(&full_bar[s], (uint32_t)((k / STAGES) & 1), WAIT_TRIES)) {
      atomicExch(status, CQ_ERR_TIMEOUT);
      failed = true;
      break;
    }
    const uint32_t code_base = smem_u32(smem + s * STAGE_BYTES);
    const uint32_t ks_base = code_base + CODE_BYTES, kmn_base = ks_base + KS_BYTES;
    const int live_groups = min(TILE_G, dm.n_groups - tile * TILE_G);
    const int b = pair / dm.hkv, hk = pair % dm.hkv;

    if (warp * K1_GPW < live_groups) {
      // ---- scale fragments: ksA/ksB[kt] = (ks[16kt+2c][G], ks[16kt+2c+1][G]) / (+8), G = 8*col8+g.
      // Scale rows carry the TMA swizzle of their width (64 bytes: 16-byte chunk ^= bits 1-2 of the row;
      // 32 bytes: chunk ^= bit 2 of the row).
      const int col8 = (warp * K1_GPW) >> 3, g_in_col = (warp * K1_GPW) & 7;
      uint32_t ksA[8], ksB[8];
      float cb[4] = {0.f, 0.f, 0.f, 0.f};   // bias[G = 8*col8+g][columns 2c, 2c+1]
      if (LDG) {
        // fragments straight from global memory: lane (g, c) holds, for k-tile kt, the pairs of channels
        // 16kt + 2c (+1) and 16kt + 8 + 2c (+1) of group G = first group of the warp's eight + g
        const int G = tile * TILE_G + col8 * 8 + g;
        const bool live = G < dm.n_groups;
        const T* ksr = ks_g + (int64_t)pair * kHeadDim * dm.n_groups + (live ? G : 0);
        const T* mnr = kmn_g + (int64_t)pair * kHeadDim * dm.n_groups + (live ? G : 0);
        uint32_t zA[8], zB[8];
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
          const int64_t d0 = (int64_t)(16 * kt + 2 * c) * dm.n_groups, d1 = (int64_t)(16 * kt + 8 + 2 * c) * dm.n_groups;
          const T2 a = D16<T>::pair2(ksr[d0], ksr[d0 + dm.n_groups]), b2 = D16<T>::pair2(ksr[d1], ksr[d1 + dm.n_groups]);
          const T2 za = D16<T>::pair2(mnr[d0], mnr[d0 + dm.n_groups]), zb = D16<T>::pair2(mnr[d1], mnr[d1 + dm.n_groups]);
          ksA[kt] = live ? D16<T>::to_h2(*reinterpret_cast<const uint32_t*>(&a)) : 0u;
          ksB[kt] = live ? D16<T>::to_h2(*reinterpret_cast<const uint32_t*>(&b2)) : 0u;
          zA[kt] = live ? D16<T>::to_h2(*reinterpret_cast<const uint32_t*>(&za)) : 0u;
          zB[kt] = live ? D16<T>::to_h2(*reinterpret_cast<const uint32_t*>(&zb)) : 0u;
        }
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) mma_f16(cb, zA[kt], 0u, zB[kt], 0u, qA[kt], qB[kt]);
      } else {
        const int mat = lane >> 3, r = lane & 7;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {
          const int d = 16 * (2 * kp + (mat >> 1)) + 8 * (mat & 1) + r;
          const int sw = KS_ROW == 64 ? ((d >> 1) & 3) : ((d >> 2) & 1);
          const uint32_t off = (uint32_t)(d * KS_ROW + ((col8 ^ sw) << 4));
          ldmatrix_x4_trans(ks_base + off, ksA[2 * kp], ksB[2 * kp], ksA[2 * kp + 1], ksB[2 * kp + 1]);
          uint32_t z0, z1, z2, z3;
          ldmatrix_x4_trans(kmn_base + off, z0, z1, z2, z3);
          ksA[2 * kp] = D16<T>::to_h2(ksA[2 * kp]); ksB[2 * kp] = D16<T>::to_h2(ksB[2 * kp]);
          ksA[2 * kp + 1] = D16<T>::to_h2(ksA[2 * kp + 1]); ksB[2 * kp + 1] = D16<T>::to_h2(ksB[2 * kp + 1]);
          z0 = D16<T>::to_h2(z0); z1 = D16<T>::to_h2(z1); z2 = D16<T>::to_h2(z2); z3 = D16<T>::to_h2(z3);
          mma_f16(cb, z0, 0u, z1, 0u, qA[2 * kp], qB[2 * kp]);
          mma_f16(cb, z2, 0u, z3, 0u, qA[2 * kp + 1], qB[2 * kp + 1]);
        }
      }
      const int64_t row_a = ((int64_t)b * dm.hq + (int64_t)hk * dm.n_rep + out_head) * dm.pitch;
      const int64_t row_b = row_a + dm.pitch;
      T2 mnA = D16<T>::bcast(D16<T>::big()), mxA = D16<T>::bcast(-D16<T>::big()), mnB = mnA, mxB = mxA;

#pragma unroll 1
      for (int u = 0; u < UNITS; ++u) {
        const int cidx = warp * UNITS + u;                    // 16-byte chunk of the channel row
        const uint32_t box_off = (uint32_t)(cidx / (ROW_BYTES / 16)) * (uint32_t)(128 * ROW_BYTES);
        const int ch = cidx % (ROW_BYTES / 16);
        float acc[GU][2][4];
#pragma unroll
        for (int a = 0; a < GU; ++a)
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[a][i][e] = 0.f;
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
          uint32_t W[4][4];
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int d = 16 * kt + 2 * c + (rr & 1) + 8 * (rr >> 1);
            const int sw = ROW_BYTES == 64 ? ((d >> 1) & 3) : (d & 7);
            const uint32_t waddr = code_base + box_off + (uint32_t)(d * ROW_BYTES + ((ch ^ sw) << 4));
            if (BITS == 4) {     // the lane's word pair of the group (see Expand)
              const uint2 v = lds64(waddr + (uint32_t)(g >> 2) * 8u);
              W[rr][0] = v.x; W[rr][1] = v.y; W[rr][2] = 0u; W[rr][3] = 0u;
            } else {
              const uint4 v = lds128(waddr);
              W[rr][0] = v.x; W[rr][1] = v.y; W[rr][2] = v.z; W[rr][3] = v.w;
            }
          }
#pragma unroll
          for (int a = 0; a < GU; ++a) {
            const int gi = g_in_col + u * GU + a;             // group within the 8 of the scale fragment
            const uint32_t ksa = __shfl_sync(0xffffffffu, ksA[kt], 4 * gi + c);
            const uint32_t ksb = __shfl_sync(0xffffffffu, ksB[kt], 4 * gi + c);
            uint32_t b0 = hmul2_u32(qA[kt], ksa), b1 = hmul2_u32(qB[kt], ksb);
            if (lo_lane) {   // remainder term: the FMA forms q*ks exactly before subtracting the rounded product
              b0 = hfma2_neg_u32(qA[kt], ksa, b0);
              b1 = hfma2_neg_u32(qB[kt], ksb, b1);
            }
            if (BITS == 1) {   // one byte of the group's word feeds both m-tiles
              const uint32_t x01 = prmt(W[0][a], W[1][a], sel[0]), x89 = prmt(W[2][a], W[3][a], sel[0]);
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const uint32_t a0 = x01 & m0[i], a1 = x01 & m1[i], a2 = x89 & m0[i], a3 = x89 & m1[i];
                mma_f16(acc[a][i], a0, a1, a2, a3, b0, b1);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                uint32_t w0, w1, w8, w9;
                if (BITS == 4) {   // word i of the pair that was loaded
                  w0 = W[0][i]; w1 = W[1][i]; w8 = W[2][i]; w9 = W[3][i];
                } else {
                  const int wi = a * BITS + i;
                  w0 = W[0][wi]; w1 = W[1][wi]; w8 = W[2][wi]; w9 = W[3][wi];
                }
                const uint32_t x01 = prmt(w0, w1, sel[i]), x89 = prmt(w8, w9, sel[i]);
                const uint32_t a0 = x01 & m0[i], a1 = x01 & m1[i], a2 = x89 & m0[i], a3 = x89 & m1[i];
                mma_f16(acc[a][i], a0, a1, a2, a3, b0, b1);
              }
            }
          }
        }
        // ---- epilogue
#pragma unroll
        for (int a = 0; a < GU; ++a) {
          const int gi = g_in_col + u * GU + a;
          const float bias0 = __shfl_sync(0xffffffffu, cb[0], 4 * gi + c);
          const float bias1 = SPLIT ? 0.f : __shfl_sync(0xffffffffu, cb[1], 4 * gi + c);
          const int tokg = (tile * TILE_G + col8 * 8 + gi) * 32;
          if (LDG && tokg >= dm.t_vis) continue;      // a group past the end of a ragged last tile
          if (SPLIT) {      // one head per lane: columns 2c, 2c+1 are its two terms
            T2 sa[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const T2 ra = D16<T>::round2(fmaf(acc[a][i][0] + acc[a][i][1], sc0[i], bias0),
                                           fmaf(acc[a][i][2] + acc[a][i][3], sc1[i], bias0));
              sa[i] = dm.raw ? ra : D16<T>::inv_sqrt_d(ra);
            }
            if (c < dm.n_rep) {
              if (BITS == 1) {   // the lane's four tokens 4g .. 4g+3 are adjacent: one 8-byte store
                uint2 v;
                v.x = *reinterpret_cast<const uint32_t*>(&sa[0]); v.y = *reinterpret_cast<const uint32_t*>(&sa[1]);
                *reinterpret_cast<uint2*>(scores + row_a + tokg + 4 * g) = v;
              } else {
#pragma unroll
                for (int i = 0; i < 2; ++i)
                  *reinterpret_cast<T2*>(scores + row_a + tokg + Expand<BITS>::elem(i, g)) = sa[i];
              }
              mnA = __hmin2(mnA, __hmin2(sa[0], sa[1])); mxA = __hmax2(mxA, __hmax2(sa[0], sa[1]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int tok = tokg + Expand<BITS>::elem(i, g);      // rows g, g+8 = tokens tok, tok+1
              const T2 ra = D16<T>::round2(fmaf(acc[a][i][0], sc0[i], bias0), fmaf(acc[a][i][2], sc1[i], bias0));
              const T2 rb = D16<T>::round2(fmaf(acc[a][i][1], sc0[i], bias1), fmaf(acc[a][i][3], sc1[i], bias1));
              // the attention logits are the rounded product times 1/sqrt(D); the plain product stops at the rounding
              const T2 sva = dm.raw ? ra : D16<T>::inv_sqrt_d(ra), svb = dm.raw ? rb : D16<T>::inv_sqrt_d(rb);
              if (2 * c < dm.n_rep) {
                *reinterpret_cast<T2*>(scores + row_a + tok) = sva;
                mnA = __hmin2(mnA, sva); mxA = __hmax2(mxA, sva);
              }
              if (2 * c + 1 < dm.n_rep) {
                *reinterpret_cast<T2*>(scores + row_b + tok) = svb;
                mnB = __hmin2(mnB, svb); mxB = __hmax2(mxB, svb);
              }
            }
          }
        }
      }
      // the stage has been read: hand it back to the producer
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
      // ---- per-warp min/max of this tile, per head
      const float2 fmnA = D16<T>::to_f2(mnA), fmxA = D16<T>::to_f2(mxA), fmnB = D16<T>::to_f2(mnB), fmxB = D16<T>::to_f2(mxB);
      float lo_a = fminf(fmnA.x, fmnA.y), hi_a = fmaxf(fmxA.x, fmxA.y);
      float lo_b = fminf(fmnB.x, fmnB.y), hi_b = fmaxf(fmxB.x, fmxB.y);
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        lo_a = fminf(lo_a, __shfl_xor_sync(0xffffffffu, lo_a, o));
        hi_a = fmaxf(hi_a, __shfl_xor_sync(0xffffffffu, hi_a, o));
        if (!SPLIT) {
          lo_b = fminf(lo_b, __shfl_xor_sync(0xffffffffu, lo_b, o));
          hi_b = fmaxf(hi_b, __shfl_xor_sync(0xffffffffu, hi_b, o));
        }
      }
      if (g == 0 && !dm.raw) {
        const int64_t r0 = (int64_t)b * dm.hq + (int64_t)hk * dm.n_rep + out_head;
        if (out_head < dm.n_rep) tile_mm[r0 * dm.n_mm + tile * K1_WARPS + warp] = make_float2(lo_a, hi_a);
        if (!SPLIT && out_head + 1 < dm.n_rep) tile_mm[(r0 + 1) * dm.n_mm + tile * K1_WARPS + warp] = make_float2(lo_b, hi_b);
      }
    } else {
      if (lane == 0) mbar_arrive(&empty_bar[s]);
      if (lane < dm.n_rep && !dm.raw)      // dead part of a ragged last tile: neutral min/max entries
        tile_mm[((int64_t)b * dm.hq + (int64_t)hk * dm.n_rep + lane) * dm.n_mm + tile * K1_WARPS + warp] =
            make_float2(INFINITY, -INFINITY);
    }
  }
}

// =================================================================================================
// K2: attn.V partials
// =================================================================================================
template <typename T>
struct CalibH {   // per head: 16-bit pairs for packed arithmetic in the data dtype
  typename D16<T>::T2 mn, range, rdenom, rdenom_lo;
};

// rnd(rnd(rnd(s - mn) / denom) * range) + mn with the reference's rounding after every operation.  The
// quotient is a product with the reciprocal carried as two 16-bit terms, formed by one FMA: it differs from
// the rounded quotient in one case in 2^11 (fp16).
template <typename T>
__device__ __forceinline__ typename D16<T>::T2 calibrate2(typename D16<T>::T2 v, const CalibH<T>& cal) {
  v = __hsub2(v, cal.mn);
  v = __hfma2(v, cal.rdenom, __hmul2(v, cal.rdenom_lo));
  return __hadd2(__hmul2(v, cal.range), cal.mn);
}

template <typename T>
__device__ __forceinline__ void set_calib(CalibH<T>& cal, float lo, float hi) {
  const float denom = rnd<T>(rnd<T>(hi - lo) + 1e-8f);
  const float range = rnd<T>(rnd<T>(hi + (-3.f)) - lo);
  cal.mn = D16<T>::bcast(lo);
  cal.rdenom = D16<T>::bcast(1.f / denom);
  cal.rdenom_lo = D16<T>::bcast(1.f / denom - rnd<T>(1.f / denom));
  cal.range = D16<T>::bcast(range);
}

// 2^x by the hardware approximation (relative error 2^-22, far below the 16-bit rounding that follows)
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Full-precision tokens (system + text), chunks of 128, as a launch of its own that depends on nothing the other
// launches of a step write: it computes its own scores, so it can run beside k1_scores and k2_attn_v.
//   scores: s[h][t] = rnd(rnd(q_h . k_t) / sqrt(D)), 16-token MMA tiles with the K rows as A fragments straight
//           from global memory and the query heads as B, in the data dtype;
//   softmax partial of the chunk and out[h][d] = sum_t p[h][t] V[t][d] on the warp MMA: A = probabilities (rows =
//           heads, from shared memory), B = V rows staged in shared memory and read through ldmatrix.trans; warp w
//           owns channels 32w .. 32w+31.
// Writes the (max, sum, acc[128]) partials of the fp slots that k3 merges.
template <typename T>
__global__ void __launch_bounds__(THREADS)
k2_fp_tokens(Dims dm, const T* __restrict__ q, const T* __restrict__ k_fp, const T* __restrict__ v_fp,
             float* __restrict__ partial, float2* __restrict__ ml) {
  constexpr int PF_PITCH = 128 + 8;         // probability row pitch (elements): rows land on different banks
  constexpr int VROW = kHeadDim * 2 + 16;   // staged V row pitch in bytes, for conflict-free ldmatrix
  constexpr int FP_SUB = 128;               // tokens staged at a time
  __shared__ __align__(16) unsigned char smem[FP_SUB * VROW];
  __shared__ __align__(16) T pf_s[kMaxRep * PF_PITCH];    // scores, then probabilities, exact in the data dtype
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int n_pairs = dm.batch * dm.hkv;
  pdl_launch_dependents();
  pdl_wait();
  const int t_fp = live_t_fp(dm);
  const int n_fp_chunks = (t_fp + 127) / 128;
  for (int it = blockIdx.x; it < n_pairs * n_fp_chunks; it += gridDim.x) {
    const int pair = it / n_fp_chunks, fc = it % n_fp_chunks;
    const int b = pair / dm.hkv, hk = pair % dm.hkv;
    const int64_t row0 = (int64_t)b * dm.hq + (int64_t)hk * dm.n_rep;
    const int t0 = fc * 128, nt = min(128, t_fp - t0);
    __syncthreads();                        // the previous item's probabilities have been consumed
    // ---- scores of the chunk: warp w takes the 16-token tiles w and w + 4
    {
      const T* qrow = q + (row0 + (g < dm.n_rep ? g : 0)) * kHeadDim + 2 * c;
      const T* kf = k_fp + (int64_t)b * dm.fp_stride_b + (int64_t)hk * dm.fp_stride_h + 2 * c;
      uint32_t bq[8][2];
#pragma unroll
      for (int kt = 0; kt < 8; ++kt) {
        bq[kt][0] = g < dm.n_rep ? __ldg(reinterpret_cast<const uint32_t*>(qrow + kt * 16)) : 0u;
        bq[kt][1] = g < dm.n_rep ? __ldg(reinterpret_cast<const uint32_t*>(qrow + kt * 16 + 8)) : 0u;
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int tt = (warp + 4 * mt) * 16;             // first token of the tile inside the chunk
        if (tt >= nt) break;
        const T* k_lo = kf + (int64_t)(t0 + min(tt + g, nt - 1)) * kHeadDim;       // rows past the end repeat the last
        const T* k_hi = kf + (int64_t)(t0 + min(tt + g + 8, nt - 1)) * kHeadDim;   // token; their scores are not kept
        uint32_t a[8][4];
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
          a[kt][0] = __ldg(reinterpret_cast<const uint32_t*>(k_lo + kt * 16));
          a[kt][1] = __ldg(reinterpret_cast<const uint32_t*>(k_hi + kt * 16));
          a[kt][2] = __ldg(reinterpret_cast<const uint32_t*>(k_lo + kt * 16 + 8));
          a[kt][3] = __ldg(reinterpret_cast<const uint32_t*>(k_hi + kt * 16 + 8));
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
          if constexpr (std::is_same<T, __nv_bfloat16>::value)
            mma_bf16(acc, a[kt][0], a[kt][1], a[kt][2], a[kt][3], bq[kt][0], bq[kt][1]);
          else
            mma_f16(acc, a[kt][0], a[kt][1], a[kt][2], a[kt][3], bq[kt][0], bq[kt][1]);
        }
        // acc[0..1] = (token tt+g, heads 2c, 2c+1), acc[2..3] = (token tt+g+8, same heads)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = 2 * c + (e & 1), t = tt + g + 8 * (e >> 1);
          if (h < dm.n_rep && t < nt)
            pf_s[h * PF_PITCH + t] = Elem<T>::from_f(__fdiv_rn(rnd<T>(acc[e]), 11.313708498984761f));
        }
      }
    }
    __syncthreads();
    for (int h = warp; h < dm.n_rep; h += 4) {
      const T* srow = pf_s + h * PF_PITCH;               // overwritten in place by the probabilities (same lanes)
      const T* mrow = dm.mask ? static_cast<const T*>(dm.mask) + (int64_t)b * dm.mask_stride_b : nullptr;
      float xv[4], m_true = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = j * 32 + lane;
        xv[j] = t < nt ? Elem<T>::to_f(srow[t]) : -INFINITY;
        if (mrow && t < nt) {      // fp token f sits before (system) or after (text) the visual span
          const int f = t0 + t;
          xv[j] = rnd<T>(xv[j] + Elem<T>::to_f(mrow[f < dm.t_sys ? f : dm.t_vis + f]));
        }
        m_true = fmaxf(m_true, xv[j]);
      }
      m_true = warp_max(m_true);
      const float m = m_true == -INFINITY ? 0.f : m_true;
      float l = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = j * 32 + lane;
        const float p = t < nt ? rnd<T>(exp2f((xv[j] - m) * LOG2E)) : 0.f;
        pf_s[h * PF_PITCH + t] = Elem<T>::from_f(p);
        l += p;
      }
      l = warp_sum(l);
      if (lane == 0) ml[(row0 + h) * dm.n_slots + dm.n_chunks + fc] = make_float2(m_true, l);
    }
    __syncthreads();
    float accf[4][4];                        // [n-tile of 8 channels][C fragment]
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) accf[j][e] = 0.f;
    const T* vf = v_fp + (int64_t)b * dm.fp_stride_b + (int64_t)hk * dm.fp_stride_h + (int64_t)t0 * kHeadDim;
    const uint32_t vs_base = smem_u32(smem);
    for (int ts = 0; ts < nt; ts += FP_SUB) {
      if (ts > 0) __syncthreads();          // the previous sub-block has been multiplied
      // stage FP_SUB rows (zeros past the last token: their probabilities are 0, but 0 * junk is not)
      for (int i = tid; i < FP_SUB * 16; i += THREADS) {
        const int t = i >> 4, cidx = i & 15;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (ts + t < nt) v = __ldg(reinterpret_cast<const uint4*>(vf + (int64_t)(ts + t) * kHeadDim) + cidx);
        *reinterpret_cast<uint4*>(smem + t * VROW + cidx * 16) = v;
      }
      __syncthreads();
#pragma unroll 2
      for (int ks = 0; ks < FP_SUB / 16; ++ks) {
        if (ts + ks * 16 >= nt) break;
        const T* prow = pf_s + (g < dm.n_rep ? g : 0) * PF_PITCH + ts + ks * 16 + 2 * c;
        uint32_t a0 = *reinterpret_cast<const uint32_t*>(prow), a2 = *reinterpret_cast<const uint32_t*>(prow + 8);
        if (g >= dm.n_rep) { a0 = 0u; a2 = 0u; }
        // matrix (lane >> 3): tokens +0/+8 x channels +0/+8 of this warp's 16-channel half
        const uint32_t row_addr = vs_base + (uint32_t)(ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * VROW +
                                  (uint32_t)(warp * 32 + 8 * (lane >> 4)) * 2u;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t b00, b01, b10, b11;
          ldmatrix_x4_trans(row_addr + half * 32, b00, b01, b10, b11);
          if constexpr (std::is_same<T, __nv_bfloat16>::value) {
            mma_bf16(accf[2 * half], a0, 0u, a2, 0u, b00, b01);
            mma_bf16(accf[2 * half + 1], a0, 0u, a2, 0u, b10, b11);
          } else {
            mma_f16(accf[2 * half], a0, 0u, a2, 0u, b00, b01);
            mma_f16(accf[2 * half + 1], a0, 0u, a2, 0u, b10, b11);
          }
        }
      }
    }
    if (g < dm.n_rep) {
      float* dst = partial + ((row0 + g) * dm.n_slots + dm.n_chunks + fc) * kHeadDim + warp * 32 + 2 * c;
#pragma unroll
      for (int j = 0; j < 4; ++j) *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(accf[j][0], accf[j][1]);
    }
  }
}

// Warps 0-3 compute, warp 4 streams the tiles (V codes, scales, minima and the logits of the tile's tokens
// for every query head of the KV head) through a ring of shared-memory stages.  Every computing warp owns a
// quarter of a tile's tokens: it turns its logits into probabilities in registers, directly in the MMA
// fragment order, and accumulates P.(codes) for all 128 channels.  The accumulators live across all the
// tiles of a KV head that the CTA walks (the softmax reference is the calibrated maximum of the whole
// visual span, known before the first tile, so no rescaling is needed); the four warps are summed and one
// partial (max, sum, acc[128]) is written per head when the KV head changes or the CTA's range ends, into
// the slot of the range's first tile; the other tile slots of the range are marked empty (max = -inf).
template <typename T, int BITS, int VT>
__global__ void __launch_bounds__(K2_THREADS, 2)
k2_attn_v(const __grid_constant__ CUtensorMap tm_v,   // 2 and 4 bits: the value codes as [tokens][row words], swizzled boxes
          Dims dm, const T* scores, const float2* tile_mm,   // written by the launch before: no read-only loads
          const int32_t* __restrict__ v_code, const T* __restrict__ v_scale,
          const T* __restrict__ v_mn,
          float* __restrict__ partial, float2* __restrict__ ml, int* __restrict__ status) {
  using T2 = typename D16<T>::T2;
  constexpr int STAGES = k2_stages(BITS, VT);
  constexpr int STAGE_BYTES = k2_stage_bytes(BITS, VT);
  constexpr int CODE_BYTES = VT * 16 * BITS;
  constexpr int LOGIT_OFF = CODE_BYTES + VT * 16;      // after the scales and the minima
  constexpr int LROW = VT * 2 + 16;                    // bytes between the logit rows of two heads
  constexpr int TOK_BYTES = 16 * BITS;      // code bytes per token
  constexpr int WPT = 4 * BITS;             // code words per token
  constexpr int QTOK = VT / K2_WARPS;       // tokens of a tile each warp owns
  constexpr uint32_t FIELD = (1u << BITS) - 1u;
  constexpr int RED_STRIDE = 136;           // 128 channels + 4 group biases + 1 sum + pad
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* red_s = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES);   // [4 warps][kMaxRep][RED_STRIDE]
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ float m_s[kMaxRep];
  // per computing warp and head: {mn, range, 1/denom (two terms)} as 16-bit pairs, then -max*log2(e) in fp32
  __shared__ __align__(16) uint32_t cal_w[K2_WARPS][kMaxRep][8];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int n_pairs = dm.batch * dm.hkv;
  const int n_vt = dm.n_chunks;             // tiles per KV head
  const int n_items = n_pairs * n_vt;

  pdl_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], K2_WARPS); }
    mbar_fence_init();
  }
  __syncthreads();

  // every CTA takes a contiguous range of (KV head, tile) items
  const int it_first = (int)(((int64_t)blockIdx.x * n_items) / gridDim.x);
  const int it_end = (int)(((int64_t)(blockIdx.x + 1) * n_items) / gridDim.x);

  if (warp == K2_WARPS) {
    if (lane == 0) {
      fence_proxy_async_smem();
      // the packed values do not depend on the score launch: the first ring of tiles is requested before
      // waiting for it, the logit rows of those tiles after
      auto load_values = [&](int k) {
        const int it = it_first + k, s = k % STAGES;
        const int pair = it / n_vt, vt = it % n_vt;
        unsigned char* base = smem + s * STAGE_BYTES;
        const int64_t tok = (int64_t)pair * dm.t_vis + (int64_t)vt * VT;
        const int nt = min(VT, dm.t_vis - vt * VT);
        // a tiled load always delivers whole boxes of 256 rows (rows past the last token of the KV head are the
        // next head's, or zero past the end of the array; nobody reads them)
        const int code_rows = BITS == 1 ? nt : (nt + 255) / 256 * 256;
        mbar_expect_tx(&full_bar[s], (uint32_t)(code_rows * TOK_BYTES + nt * 16 + dm.n_rep * nt * 2));
        if (BITS == 1) {
          bulk_load_1d(base, v_code + tok * WPT, (uint32_t)(nt * TOK_BYTES), &full_bar[s]);
        } else {
          // token rows of 32 / 64 bytes: a plain copy would put the rows of a quarter warp's four tokens on the
          // same banks; the tiled load XORs the 16-byte chunk index with bits of the row number (nt % 256 == 0)
          for (int r0 = 0; r0 < nt; r0 += 256)
            tma_load_2d(base + r0 * TOK_BYTES, &tm_v, 0, (int)(tok + r0), &full_bar[s]);
        }
        bulk_load_1d(base + CODE_BYTES, v_scale + tok * 4, (uint32_t)(nt * 8), &full_bar[s]);
        bulk_load_1d(base + CODE_BYTES + VT * 8, v_mn + tok * 4, (uint32_t)(nt * 8), &full_bar[s]);
      };
      auto load_logits = [&](int k) {
        const int it = it_first + k, s = k % STAGES;
        const int pair = it / n_vt, vt = it % n_vt;
        unsigned char* base = smem + s * STAGE_BYTES;
        const int nt = min(VT, dm.t_vis - vt * VT);
        const T* srow = scores + (int64_t)pair * dm.n_rep * dm.pitch + (int64_t)vt * VT;
        for (int h = 0; h < dm.n_rep; ++h)
          bulk_load_1d(base + LOGIT_OFF + h * LROW, srow + (int64_t)h * dm.pitch, (uint32_t)(nt * 2), &full_bar[s]);
      };
      const int n_pre = min(STAGES, it_end - it_first);
      for (int k = 0; k < n_pre; ++k) load_values(k);
      pdl_wait();
      for (int k = 0; k < n_pre; ++k) load_logits(k);
      for (int k = n_pre; it_first + k < it_end; ++k) {
        if (!mbar_wait_bounded(&empty_bar[k % STAGES], (uint32_t)((k / STAGES - 1) & 1), WAIT_TRIES)) {
          atomicExch(status, CQ_ERR_TIMEOUT);
          break;
        }
        load_values(k);
        load_logits(k);
      }
    }
    return;
  }

  // lane constants for expanding the channel pair that rows g, g+8 of m-tile j stand for
  // (Expand::elem): at 1 bit two m-tiles share a word and the pattern repeats with j % 2, otherwise
  // it does not depend on j.
  uint32_t sel[2], m0[2], m1[2];
  float sc0[2], sc1[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int off = Expand<BITS>::bit_off(i, g);
    const int byte = (off % 32) / 8, sh = off % 8;
    sel[i] = prmt_sel(byte);
    m0[i] = (FIELD << sh) * 0x00010001u;
    m1[i] = (FIELD << (sh + BITS)) * 0x00010001u;
    sc0[i] = exp2f((float)(24 - sh));
    sc1[i] = exp2f((float)(24 - sh - BITS));
  }

  pdl_wait();          // the tile minima / maxima and (through the producer) the logits come from the score launch
  float acc[8][4];
  float cb[4] = {0.f, 0.f, 0.f, 0.f};
  int seg_pair = -1, seg_first = 0, seg_end = 0;     // the run of tiles of one KV head accumulated so far
  bool failed = false;
  // calibration constants and softmax reference of the head this lane's probabilities belong to (head g)
  CalibH<T> cal;
  cal.mn = cal.range = cal.rdenom = cal.rdenom_lo = D16<T>::bcast(0.f);
  float m_ref = 0.f;

  // sum the four warps' accumulators of the finished run and write its partial
  auto flush = [&]() {
    const int64_t row0 = (int64_t)seg_pair * dm.n_rep;
    float* mine = red_s + warp * kMaxRep * RED_STRIDE;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = (BITS == 1) ? (j & 1) : 0;
      // 4 bits: the two m-tiles of a 32-channel group take words {2hi, 2hi+1} of the group's four (hi = g / 4)
      const int ch = BITS == 1 ? 32 * (j >> 1) + Expand<1>::elem(i, g)
                   : BITS == 4 ? 32 * (j >> 1) + 16 * (g >> 2) + 8 * (j & 1) + 2 * (g & 3) : 16 * j + 2 * g;
      if (2 * c < dm.n_rep) {
        mine[(2 * c) * RED_STRIDE + ch] = acc[j][0] * sc0[i];
        mine[(2 * c) * RED_STRIDE + ch + 1] = acc[j][2] * sc1[i];
      }
      if (2 * c + 1 < dm.n_rep) {
        mine[(2 * c + 1) * RED_STRIDE + ch] = acc[j][1] * sc0[i];
        mine[(2 * c + 1) * RED_STRIDE + ch + 1] = acc[j][3] * sc1[i];
      }
    }
    if (g < dm.n_rep && c < 3) {      // bias columns 0..3 (c = 0,1) and the row sum (c = 2, col 4)
      mine[g * RED_STRIDE + 128 + 2 * c] = cb[0];
      if (c < 2) mine[g * RED_STRIDE + 128 + 2 * c + 1] = cb[1];
    }
    named_barrier_sync(1, K2_WARPS * 32);
    for (int h = 0; h < dm.n_rep; ++h) {
      float o = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < K2_WARPS; ++w) {
        const float* r = red_s + (w * kMaxRep + h) * RED_STRIDE;
        o += r[tid] + r[128 + (tid >> 5)];
        l += r[132];
      }
      partial[((row0 + h) * dm.n_slots + seg_first) * kHeadDim + tid] = o;
      if (tid == 0) ml[(row0 + h) * dm.n_slots + seg_first] = make_float2(m_s[h], l);
    }
    // the other tile slots of the run hold nothing
    for (int i = tid; i < dm.n_rep * (seg_end - seg_first - 1); i += K2_WARPS * 32) {
      const int h = i / (seg_end - seg_first - 1), sl = seg_first + 1 + i % (seg_end - seg_first - 1);
      ml[(row0 + h) * dm.n_slots + sl] = make_float2(-INFINITY, 0.f);
    }
    named_barrier_sync(1, K2_WARPS * 32);
  };

  for (int k = 0;; ++k) {
    const int it = it_first + k;
    if (it >= it_end) break;
    const int s = k % STAGES;
    const int pair = it / n_vt, vt = it % n_vt;
    if (pair != seg_pair) {
      if (seg_pair >= 0) flush();
      seg_pair = pair; seg_first = vt;
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
      cb[0] = cb[1] = cb[2] = cb[3] = 0.f;
      // calibration constants of head g: the four lanes of a head share the per-tile min/max entries
      float lo = INFINITY, hi = -INFINITY;
      if (g < dm.n_rep && !dm.raw) {
        const float2* mm = tile_mm + ((int64_t)pair * dm.n_rep + g) * dm.n_mm;
        // eight entries in flight per lane: the loads are L2 round trips, one after the other they cost the
        // CTA several thousand cycles at every change of KV head
        int i = c;
        for (; i + 28 < dm.n_mm; i += 32) {
          float2 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = mm[i + 4 * u];
#pragma unroll
          for (int u = 0; u < 8; ++u) { lo = fminf(lo, v[u].x); hi = fmaxf(hi, v[u].y); }
        }
        for (; i < dm.n_mm; i += 4) {
          const float2 v = mm[i];
          lo = fminf(lo, v.x);
          hi = fmaxf(hi, v.y);
        }
      }
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 1)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 1));
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 2)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, 2));
      m_ref = dm.raw ? 0.f : hi;
      if (dm.calibrate && g < dm.n_rep && !dm.raw) {
        set_calib<T>(cal, lo, hi);
        m_ref = D16<T>::to_f2(calibrate2<T>(D16<T>::bcast(hi), cal)).x;     // the maximum, calibrated like any logit
      }
      if (warp == 0 && c == 0 && g < dm.n_rep) m_s[g] = m_ref;              // read back by thread 0 in flush()
      // the lanes of the warp share out the (head, token pair) logits of a tile: the constants of every
      // head go to this warp's table
      __syncwarp();
      if (c == 0 && g < dm.n_rep) {
        uint32_t* e = cal_w[warp][g];
        e[0] = *reinterpret_cast<const uint32_t*>(&cal.mn); e[1] = *reinterpret_cast<const uint32_t*>(&cal.range);
        e[2] = *reinterpret_cast<const uint32_t*>(&cal.rdenom); e[3] = *reinterpret_cast<const uint32_t*>(&cal.rdenom_lo);
        e[4] = __float_as_uint(-m_ref * LOG2E);
      }
      __syncwarp();
    }
    seg_end = vt + 1;
    // additive mask of this batch row, at the tile's first visual key (added after calibration, rounded
    // to the data dtype as the tensor addition of the reference is)
    const T* mvis = dm.mask ? static_cast<const T*>(dm.mask) + (int64_t)(pair / dm.hkv) * dm.mask_stride_b +
                              dm.t_sys + vt * VT : nullptr;
    if (!mbar_wait_bounded(&full_bar[s], (uint32_t)((k / STAGES) & 1), WAIT_TRIES)) {
      atomicExch(status, CQ_ERR_TIMEOUT);
      failed = true;
      break;
    }
    const uint32_t code_b = smem_u32(smem + s * STAGE_BYTES);
    const uint32_t vs_b = code_b + CODE_BYTES, vmn_b = vs_b + VT * 8;
    const uint32_t lg_b = code_b + LOGIT_OFF + (uint32_t)((g < dm.n_rep ? g : 0) * LROW);
    const int nt_tile = min(VT, dm.t_vis - vt * VT);
    {
      // Scales and minima of this warp's quarter of the tile, re-laid out in place: each 16-byte
      // unit holds two tokens x four channel groups; it becomes four (token, token+1) pairs, one
      // per group, which is the MMA B-fragment order, so the main loop needs no permutes.  bf16
      // values are converted to fp16 on the way.
#pragma unroll
      for (int arr = 0; arr < 2; ++arr) {
        const uint32_t base = (arr == 0 ? vs_b : vmn_b) + (uint32_t)(warp * QTOK) * 8u;
#pragma unroll
        for (int i = 0; i < QTOK / 64; ++i) {
          const uint32_t addr = base + (uint32_t)(i * 32 + lane) * 16u;
          uint4 v = lds128(addr);
          v.x = D16<T>::to_h2(v.x); v.y = D16<T>::to_h2(v.y); v.z = D16<T>::to_h2(v.z); v.w = D16<T>::to_h2(v.w);
          const uint32_t o0 = prmt(v.x, v.z, 0x5410), o1 = prmt(v.x, v.z, 0x7632);
          const uint32_t o2 = prmt(v.y, v.w, 0x5410), o3 = prmt(v.y, v.w, 0x7632);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
        }
      }
      __syncwarp();
    }
    // ---- probabilities of this warp's quarter, all heads, in place over the logits: the lanes share out
    // the (head, token pair) elements; the head is uniform over the warp in every pass.  The reference rounds
    // the probabilities to the data dtype; they are then exact in fp16, the type the MMA takes.
    if (!(dm.raw && std::is_same<T, __half>::value)) {
      const uint32_t q_b = code_b + LOGIT_OFF + (uint32_t)(warp * QTOK) * 2u;
      const uint32_t cal_b = smem_u32(&cal_w[warp][0][0]);
      // Four heads at a time, in three sweeps: all loads, all arithmetic, all stores.  The shared-memory accesses are
      // volatile asm statements, which the compiler keeps in program order: written as load-compute-store per
      // element, the eight chains of a lane (4 heads x 2 token pairs) ran one after the other, ~1950 cycles per tile
      // (cycle counters); as sweeps they overlap.
      constexpr int NJ = QTOK / 64;
      for (int h0 = 0; h0 < dm.n_rep; h0 += 4) {
        uint4 cw[4];
        float mneg[4];
        uint32_t xin[4][NJ];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          const int h = min(h0 + hh, dm.n_rep - 1);            // heads past the last repeat it; their results are dropped
          cw[hh] = lds128(cal_b + (uint32_t)h * 32u);
          mneg[hh] = __uint_as_float(lds32(cal_b + (uint32_t)h * 32u + 16u));
#pragma unroll
          for (int j = 0; j < NJ; ++j) {
            const int tp = (j * 32 + lane) * 2;                 // first token of the pair, within the quarter
            xin[hh][j] = lds32(q_b + (uint32_t)(h * LROW + tp * 2));
          }
        }
        uint32_t pp[4][NJ];
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          CalibH<T> ch;
          ch.mn = *reinterpret_cast<const T2*>(&cw[hh].x); ch.range = *reinterpret_cast<const T2*>(&cw[hh].y);
          ch.rdenom = *reinterpret_cast<const T2*>(&cw[hh].z); ch.rdenom_lo = *reinterpret_cast<const T2*>(&cw[hh].w);
#pragma unroll
          for (int j = 0; j < NJ; ++j) {
            const int tp = (j * 32 + lane) * 2;
            if (dm.raw) {                                       // plain product: the row holds the weights themselves
              pp[hh][j] = D16<T>::to_h2(xin[hh][j]);
            } else {
              T2 v = *reinterpret_cast<const T2*>(&xin[hh][j]);
              if (dm.calibrate) v = calibrate2<T>(v, ch);
              if (mvis && warp * QTOK + tp < nt_tile)
                v = __hadd2(v, D16<T>::pair2(mvis[warp * QTOK + tp], mvis[warp * QTOK + tp + 1]));
              const float2 f = D16<T>::to_f2(v);
              pp[hh][j] = D16<T>::prob_pair(ex2_approx(fmaf(f.x, LOG2E, mneg[hh])), ex2_approx(fmaf(f.y, LOG2E, mneg[hh])));
            }
          }
        }
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
          const int h = h0 + hh;
#pragma unroll
          for (int j = 0; j < NJ; ++j) {
            const int tp = (j * 32 + lane) * 2;
            if (h < dm.n_rep && warp * QTOK + tp < nt_tile) {
              const uint32_t addr = q_b + (uint32_t)(h * LROW + tp * 2);
              asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(pp[hh][j]) : "memory");
            }
          }
        }
      }
      __syncwarp();
    }
    const uint32_t zoff = (uint32_t)(g < 4 ? g : 0) * 4u;   // this lane's column of the minima MMA
    const uint32_t z_and = g < 4 ? 0xffffffffu : 0u, z_or = g == 4 ? 0x3c003c00u : 0u;   // column 4 = ones
    // One k-step = 16 tokens.  Its shared-memory operands are fetched one k-step ahead of their use (the loads are
    // volatile asm statements and stay where they are written): probabilities, scale pairs, minima, code words of
    // the lane's four tokens (t0, t0+1, t0+8, t0+9).
    constexpr int NW = BITS == 1 ? 4 : 8;        // code words per token the lane uses
    struct StepRegs { uint32_t pp0, pp1, zb0, zb1; uint4 s0, s1; uint32_t cw[4][NW]; };
    auto load_step = [&](int kq, StepRegs& R) {
      const int t0 = warp * QTOK + kq * 16 + 2 * c;   // token (in tile) of the lane's first k pair
      R.pp0 = lds32(lg_b + (uint32_t)t0 * 2u);
      R.pp1 = lds32(lg_b + (uint32_t)(t0 + 8) * 2u);
      // scale pairs of tokens (t0, t0+1) and (t0+8, t0+9), one register per channel group
      R.s0 = lds128(vs_b + (uint32_t)t0 * 8u);
      R.s1 = lds128(vs_b + (uint32_t)(t0 + 8) * 8u);
      R.zb0 = lds32(vmn_b + (uint32_t)t0 * 8u + zoff);
      R.zb1 = lds32(vmn_b + (uint32_t)(t0 + 8) * 8u + zoff);
      const uint32_t tb = code_b + (uint32_t)t0 * TOK_BYTES;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const uint32_t row = tb + (uint32_t)((r & 1) + 8 * (r >> 1)) * TOK_BYTES;
        if (BITS == 4) {
          // rows of tokens t0, t0+1, t0+8, t0+9 all carry the chunk XOR c (64-byte swizzle: chunk ^= (row / 2) % 4).
          // Per 32-channel group q the lane reads the two words (2hi, 2hi+1) of chunk q: m-tiles 2q and 2q+1.
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint2 w = lds64(row + (uint32_t)((q ^ c) << 4) + (uint32_t)(g >> 2) * 8u);
            R.cw[r][2 * q] = w.x; R.cw[r][2 * q + 1] = w.y;
          }
        } else {
#pragma unroll
          for (int part = 0; part < BITS; ++part) {      // 16 bytes of the token row at a time
            // 2 bits: 32-byte swizzle, chunk ^= (row / 4) % 2 = c / 2 for all four tokens
            const uint32_t po = BITS == 2 ? (uint32_t)((part ^ (c >> 1)) << 4) : (uint32_t)(part * 16);
            const uint4 w = lds128(row + po);
            R.cw[r][4 * part] = w.x; R.cw[r][4 * part + 1] = w.y; R.cw[r][4 * part + 2] = w.z; R.cw[r][4 * part + 3] = w.w;
          }
        }
      }
    };
    auto compute_step = [&](const StepRegs& R) {
      uint32_t pp0 = R.pp0, pp1 = R.pp1;
      if (g >= dm.n_rep) { pp0 = 0u; pp1 = 0u; }
      uint32_t bA[4], bB[4];
      bA[0] = hmul2_u32(pp0, R.s0.x); bA[1] = hmul2_u32(pp0, R.s0.y); bA[2] = hmul2_u32(pp0, R.s0.z); bA[3] = hmul2_u32(pp0, R.s0.w);
      bB[0] = hmul2_u32(pp1, R.s1.x); bB[1] = hmul2_u32(pp1, R.s1.y); bB[2] = hmul2_u32(pp1, R.s1.z); bB[3] = hmul2_u32(pp1, R.s1.w);
      // minima + row sum: A = p (rows = heads), B column n = g: n<4 -> vmn[.][n], n==4 -> 1
      mma_f16(cb, pp0, 0u, pp1, 0u, (R.zb0 & z_and) | z_or, (R.zb1 & z_and) | z_or);
      if (BITS == 1) {        // word m = channels 32m .. 32m+31 = m-tiles 2m, 2m+1, one byte permute for both
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const uint32_t x01 = prmt(R.cw[0][m], R.cw[1][m], sel[0]), x89 = prmt(R.cw[2][m], R.cw[3][m], sel[0]);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            mma_f16(acc[2 * m + i], x01 & m0[i], x01 & m1[i], x89 & m0[i], x89 & m1[i], bA[m], bB[m]);
        }
      } else {                // 2 bits: m-tile j = word j of the row; 4 bits: m-tiles 2q, 2q+1 = the pair loaded for q
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t x01 = prmt(R.cw[0][j], R.cw[1][j], sel[0]), x89 = prmt(R.cw[2][j], R.cw[3][j], sel[0]);
          mma_f16(acc[j], x01 & m0[0], x01 & m1[0], x89 & m0[0], x89 & m1[0], bA[j >> 1], bB[j >> 1]);
        }
      }
    };
    StepRegs R[2];
    load_step(0, R[0]);
#pragma unroll
    for (int kq = 0; kq < QTOK / 16; ++kq) {
      if (warp * QTOK + kq * 16 >= nt_tile) break;
      if (kq + 1 < QTOK / 16) load_step(kq + 1, R[(kq + 1) & 1]);
      compute_step(R[kq & 1]);
    }
    // the stage has been read: hand it back to the producer
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }
  if (failed) return;
  if (seg_pair >= 0) flush();
}

// =================================================================================================
// K3: combine
// =================================================================================================
// K3_LANES slot-parallel groups of 128 channel threads: 4 when a row has many partials to merge (long
// contexts), 1 when it has a handful (then four times as many rows fit on an SM at once)
template <typename T, int K3_LANES>
__global__ void __launch_bounds__(kHeadDim * K3_LANES)
k3_combine(Dims dm, const float* partial, const float2* ml,   // written by overlapping launches: plain loads only
           T* __restrict__ out) {
  __shared__ float o_s[K3_LANES][kHeadDim];
  __shared__ float l_s[K3_LANES];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x & (kHeadDim - 1), sl = threadIdx.x >> 7;
  const float2* r = ml + row * dm.n_slots;
  const int n_live = dm.n_chunks + (live_t_fp(dm) + 127) / 128;   // visual chunks, then fp chunks
  // common maximum: the lanes of every warp share the slots, one or two loads each
  float M = -INFINITY;
  for (int i = threadIdx.x & 31; i < n_live; i += 32) M = fmaxf(M, r[i].x);
  M = warp_max(M);
  float L = 0.f, o = 0.f;
  const float* p = partial + row * dm.n_slots * kHeadDim + d;
#pragma unroll 8
  for (int i = sl; i < n_live; i += K3_LANES) {
    const float2 mlv = r[i];
    if (mlv.x == -INFINITY) continue;      // an empty slot (its run of tiles was accumulated into an earlier one)
    const float w = exp2f((mlv.x - M) * LOG2E);
    L = fmaf(mlv.y, w, L);
    o = fmaf(p[(int64_t)i * kHeadDim], w, o);
  }
  o_s[sl][d] = o;
  if (d == 0) l_s[sl] = L;
  __syncthreads();
  if (sl == 0) {
#pragma unroll
    for (int j = 1; j < K3_LANES; ++j) { o += o_s[j][d]; L += l_s[j]; }
    out[row * kHeadDim + d] = Elem<T>::from_f(dm.raw ? o : o / L);
  }
}

// =================================================================================================
// host side
// =================================================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// rows x cols matrix (cols contiguous), box = box_cols columns x 128 rows.
// A decode loop asks for the same few descriptors at every step (one cache per layer), so the encoded
// maps are remembered per host thread: a descriptor is a pure function of the key below.
static bool make_map(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elem_bytes,
                     uint64_t cols, uint64_t rows, CUtensorMapSwizzle sw, uint32_t box_cols, uint32_t box_rows = 128) {
  struct Entry { const void* base; uint64_t cols, rows; int dt, sw; uint32_t box_cols, box_rows; CUtensorMap map; };
  constexpr int N = 256;
  thread_local Entry cache[N];
  thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i) {
    const Entry& e = cache[i];
    if (e.base == base && e.cols == cols && e.rows == rows && e.dt == (int)dt && e.sw == (int)sw && e.box_cols == box_cols &&
        e.box_rows == box_rows) {
      *m = e.map;
      return true;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  Entry& e = cache[next];
  e.base = base; e.cols = cols; e.rows = rows; e.dt = (int)dt; e.sw = (int)sw; e.box_cols = box_cols; e.box_rows = box_rows; e.map = *m;
  next = (next + 1) % N;
  if (used < N) ++used;
  return true;
}

// The value codes of the attn.V kernel at 2 and 4 bits: [tokens of all KV heads][4*BITS words], boxes of 256 token
// rows swizzled over the row width (32 or 64 bytes).  At 1 bit the kernel copies the rows untiled and ignores the map.
template <int BITS>
static bool make_v_map(CUtensorMap* tm_v, const void* code, uint64_t tokens) {
  if (BITS == 1) { memset(tm_v, 0, sizeof(*tm_v)); return true; }
  return make_map(tm_v, code, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, 4 * BITS, tokens,
                  BITS == 4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B, 4 * BITS, 256);
}

// The three tensor maps of the score kernel: code words (boxes of at most 128 bytes per channel row, swizzled
// over their width), scales and minima (one box of tile_g values per channel row, swizzled over its width).
template <int BITS>
static bool make_k_maps(CUtensorMap* tm_code, CUtensorMap* tm_ks, CUtensorMap* tm_kmn, const void* code,
                        const void* ks, const void* kmn, uint64_t n_groups, uint64_t rows) {
  constexpr int row = k1_code_row_bytes(BITS);
  constexpr int TILE_G = tile_g(BITS);
  const CUtensorMapSwizzle sw_ks = TILE_G * 2 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  return make_map(tm_code, code, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, n_groups * BITS, rows,
                  row == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, row / 4) &&
         make_map(tm_ks, ks, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, n_groups, rows, sw_ks, TILE_G) &&
         make_map(tm_kmn, kmn, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, n_groups, rows, sw_ks, TILE_G);
}

struct Layout {
  size_t status_off, scores_off, mm_off, ml_off, partial_off, total;
};

static Dims make_dims(const cq_decode_args* a) {
  Dims d;
  d.batch = a->batch; d.hq = a->n_q_heads; d.hkv = a->n_kv_heads; d.n_rep = d.hq / d.hkv;
  d.t_vis = a->t_vis; d.t_fp = a->t_fp; d.calibrate = a->calibrate ? 1 : 0;
  d.n_groups = d.t_vis / 32;
  d.n_ktiles = (d.n_groups + tile_g(a->bits) - 1) / tile_g(a->bits);
  // the large tiles only when they give every resident CTA a few of them (measured on the 7B step's shape, batch
  // 16 x 3328 tokens: 18.4 us with three to four large tiles per CTA against 19.4 us with five to six small
  // ones), and never at 4 bits, where a ring of large tiles leaves room for one CTA per SM only (the small ones:
  // three stages, two CTAs)
  d.chunk_tok = a->bits != 4 && (int64_t)d.batch * d.hkv * ((d.t_vis + VT_LARGE - 1) / VT_LARGE) >= 2 * K2_RESIDENT
                    ? VT_LARGE : VT_SMALL;
  d.n_chunks = (d.t_vis + d.chunk_tok - 1) / d.chunk_tok;
  d.n_fp_chunks = (d.t_fp + 127) / 128;
  d.n_slots = d.n_chunks + d.n_fp_chunks;
  d.pitch = (d.t_vis + d.t_fp + 7) / 8 * 8;
  d.n_mm = d.n_ktiles * K1_WARPS;
  d.fp_stride_b = a->fp_stride_b; d.fp_stride_h = a->fp_stride_h;
  d.t_fp_dev = a->t_fp_dev;
  d.raw = 0;
  d.mask = a->mask; d.mask_stride_b = a->mask_stride_b; d.t_sys = a->t_sys;
  return d;
}

static Layout make_layout(const Dims& d) {
  Layout l;
  const size_t rows = (size_t)d.batch * d.hq;
  l.status_off = 0;
  l.scores_off = 256;
  l.mm_off = l.scores_off + align_up(rows * (size_t)d.pitch * 2, 256);
  l.ml_off = l.mm_off + align_up(rows * (size_t)d.n_mm * sizeof(float2), 256);
  l.partial_off = l.ml_off + align_up(rows * (size_t)d.n_slots * sizeof(float2), 256);
  l.total = l.partial_off + rows * (size_t)d.n_slots * kHeadDim * sizeof(float);
  return l;
}

static int sm_count() {      // of the current device
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  return v;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may begin (up to its pdl_wait())
// while the previous kernel of the stream drains.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// A side stream and two events per host thread and device: the launch for the full-precision tokens depends on
// nothing the other launches of a step write, so it is forked off the caller's stream before the score launch and
// joined before the combine launch (a pattern that stream capture records as two parallel branches).
struct ForkSet { cudaStream_t side = nullptr; cudaEvent_t fork = nullptr, join = nullptr; };
static ForkSet* fork_set(int dev) {
  thread_local ForkSet sets[64];
  ForkSet& f = sets[dev];
  if (!f.side) {
    if (cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking) != cudaSuccess) { f.side = nullptr; return nullptr; }
    if (cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&f.join, cudaEventDisableTiming) != cudaSuccess) {
      cudaStreamDestroy(f.side);
      f.side = nullptr;
      return nullptr;
    }
  }
  return &f;
}

template <typename T, int BITS, int VT>
static int run_shape(const cq_decode_args* a, const Dims& d, const Layout& l, unsigned char* ws, cudaStream_t st,
                     cudaEvent_t* ev, int* status_word) {
  int* status = status_word ? status_word : reinterpret_cast<int*>(ws + l.status_off);
  T* scores = reinterpret_cast<T*>(ws + l.scores_off);
  float2* mm = reinterpret_cast<float2*>(ws + l.mm_off);
  float2* ml = reinterpret_cast<float2*>(ws + l.ml_off);
  float* partial = reinterpret_cast<float*>(ws + l.partial_off);
  const int n_pairs = d.batch * d.hkv;

  // token counts that are not a multiple of 256: row pitches a tensor map cannot describe (see k1_scores)
  const bool ldg = d.t_vis % 256 != 0;
  auto k1 = ldg ? (d.n_rep <= 4 ? k1_scores<T, BITS, true, true> : k1_scores<T, BITS, false, true>)
                : (d.n_rep <= 4 ? k1_scores<T, BITS, true> : k1_scores<T, BITS, false>);
  auto k2 = k2_attn_v<T, BITS, VT>;
  const int smem1 = k1_stages(BITS) * k1_stage_bytes(BITS) + 1024;
  const int smem2 = k2_smem_bytes(BITS, VT);
  static bool configured_dev[64][4] = {};   // per template instance, device and score-kernel variant
  static int occ1_dev[64][4], occ2_dev[64][4];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CQ_ERR_LAUNCH;
  static std::mutex config_mu;                // host threads may share a device
  std::lock_guard<std::mutex> config_lock(config_mu);
  const int variant = (d.n_rep <= 4 ? 1 : 0) + (ldg ? 2 : 0);
  bool& configured = configured_dev[dev][variant];
  int& occ1 = occ1_dev[dev][variant];
  int& occ2 = occ2_dev[dev][variant];
  if (!configured) {
    if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1) != cudaSuccess) return CQ_ERR_LAUNCH;
    if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) != cudaSuccess) return CQ_ERR_LAUNCH;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ1, k1, K1_THREADS, smem1) != cudaSuccess || occ1 < 1) return CQ_ERR_LAUNCH;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ2, k2, K2_THREADS, smem2) != cudaSuccess || occ2 < 1) return CQ_ERR_LAUNCH;
    configured = true;
  }
  // `ev` (profiling entry point only): five events recorded around the four launches, which then run one after
  // the other on the caller's stream
  auto mark = [&](int i) { if (ev) cudaEventRecord(ev[i], st); };
  auto launch_fp = [&](cudaStream_t s) -> int {
    k2_fp_tokens<T><<<n_pairs * d.n_fp_chunks, THREADS, 0, s>>>(d, static_cast<const T*>(a->q), static_cast<const T*>(a->k_fp),
                                                               static_cast<const T*>(a->v_fp), partial, ml);
    return check_launch();
  };
  ForkSet* fk = nullptr;
  if (d.n_fp_chunks > 0 && !ev) {
    fk = fork_set(dev);
    if (!fk) return CQ_ERR_LAUNCH;
    if (cudaEventRecord(fk->fork, st) != cudaSuccess || cudaStreamWaitEvent(fk->side, fk->fork, 0) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    const int rc = launch_fp(fk->side);
    if (rc != CQ_OK) return rc;
    if (cudaEventRecord(fk->join, fk->side) != cudaSuccess) return CQ_ERR_LAUNCH;
  }
  mark(0);
  if (d.t_vis > 0) {
    CUtensorMap tm_code, tm_ks, tm_kmn;
    const uint64_t rows = (uint64_t)n_pairs * kHeadDim;
    if (ldg) {
      memset(&tm_code, 0, sizeof(tm_code)); memset(&tm_ks, 0, sizeof(tm_ks)); memset(&tm_kmn, 0, sizeof(tm_kmn));
    } else if (!make_k_maps<BITS>(&tm_code, &tm_ks, &tm_kmn, a->k_code, a->k_scale, a->k_mn, (uint64_t)d.n_groups, rows)) {
      return CQ_ERR_LAUNCH;
    }
    const int items1 = n_pairs * d.n_ktiles;
    const int grid1 = max(1, min(items1, sm_count() * occ1));
    if (launch_pdl(k1, dim3(grid1), dim3(K1_THREADS), smem1, st, tm_code, tm_ks, tm_kmn, d, static_cast<const T*>(a->q),
                   scores, mm, status, a->k_code, static_cast<const T*>(a->k_scale),
                   static_cast<const T*>(a->k_mn)) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    int rc = check_launch();
    if (rc != CQ_OK) return rc;
  }
  mark(1);
  {
    const int items2 = n_pairs * d.n_chunks;
    const int grid2 = max(1, min(items2, sm_count() * occ2));
    CUtensorMap tm_v;
    if (!make_v_map<BITS>(&tm_v, a->v_code, (uint64_t)n_pairs * d.t_vis)) return CQ_ERR_LAUNCH;
    if (launch_pdl(k2, dim3(grid2), dim3(K2_THREADS), smem2, st, tm_v, d, static_cast<const T*>(scores),
                   static_cast<const float2*>(mm), a->v_code, static_cast<const T*>(a->v_scale),
                   static_cast<const T*>(a->v_mn), partial, ml, status) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    int rc = check_launch();
    if (rc != CQ_OK) return rc;
    mark(2);
    if (d.n_fp_chunks > 0) {
      if (fk) {
        if (cudaStreamWaitEvent(st, fk->join, 0) != cudaSuccess) return CQ_ERR_LAUNCH;
      } else {
        rc = launch_fp(st);
        if (rc != CQ_OK) return rc;
      }
    }
    mark(3);
  }
  cudaError_t e3;
  if (d.n_slots >= 16)
    e3 = launch_pdl(k3_combine<T, 4>, dim3(d.batch * d.hq), dim3(kHeadDim * 4), 0, st, d, static_cast<const float*>(partial),
                    static_cast<const float2*>(ml), static_cast<T*>(a->out));
  else
    e3 = launch_pdl(k3_combine<T, 1>, dim3(d.batch * d.hq), dim3(kHeadDim), 0, st, d, static_cast<const float*>(partial),
                    static_cast<const float2*>(ml), static_cast<T*>(a->out));
  if (e3 != cudaSuccess) return CQ_ERR_LAUNCH;
  const int rc3 = check_launch();
  mark(4);
  return rc3;
}

template <typename T, int BITS>
static int run(const cq_decode_args* a, const Dims& d, const Layout& l, unsigned char* ws, cudaStream_t st,
               cudaEvent_t* ev, int* status_word) {
  return d.chunk_tok == VT_LARGE ? run_shape<T, BITS, VT_LARGE>(a, d, l, ws, st, ev, status_word)
                                 : run_shape<T, BITS, VT_SMALL>(a, d, l, ws, st, ev, status_word);
}

}  // namespace mma

bool mma_path_eligible(const cq_decode_args* a) {
  if (a->t_vis <= 0 || a->t_vis % 32 != 0) return false;
  if (a->bits != 1 && a->bits != 2 && a->bits != 4) return false;
  const void* ptrs[] = {a->q, a->k_code, a->k_scale, a->k_mn, a->v_code, a->v_scale, a->v_mn};
  for (const void* p : ptrs)
    if (!aligned16(p)) return false;
  if (a->t_fp > 0 && (!aligned16(a->k_fp) || !aligned16(a->v_fp))) return false;
  return mma::encode_fn() != nullptr;
}

// ---- the stand-alone quantized product on the same kernels ----------------------------------------
// out[b,h,n] = sum_k fA[b,h,k] * (scale[k, n/32] * code[k, n] + zero[k, n/32]) with the codes packed along n.
//   K == 128, N % 256 == 0 ("q.K": rows = channels, n = tokens)   -> the score launch, rounding only
//   N == 128, K % 256 == 0 ("att.V": rows = tokens, n = channels) -> the attn.V launch on given weights,
//                                                                     then the merge without normalisation
static bool qbmm_ptrs_ok(const void* fA, const void* qB, const void* s, const void* z, const void* out) {
  return aligned16(fA) && aligned16(qB) && aligned16(s) && aligned16(z) && aligned16(out) && mma::encode_fn() != nullptr;
}

int mma_qbmm_kind(const void* fA, const void* qB, const void* scales, const void* zeros, const void* out,
                  int n_q_heads, int n_kv_heads, int64_t K, int64_t N) {
  if (!qbmm_ptrs_ok(fA, qB, scales, zeros, out)) return 0;
  if (n_q_heads / n_kv_heads > kMaxRep || K > 0x3fffffff || N > 0x3fffffff) return 0;
  if (K == kHeadDim && N % 256 == 0) return 1;
  if (N == kHeadDim && K % 256 == 0) return 2;
  return 0;
}

static mma::Dims qbmm_dims(int kind, int batch, int hq, int hkv, int64_t K, int64_t N) {
  cq_decode_args a = {};
  a.batch = batch; a.n_q_heads = hq; a.n_kv_heads = hkv;
  a.t_vis = (int)(kind == 1 ? N : K);
  mma::Dims d = mma::make_dims(&a);
  d.raw = 1;
  d.pitch = a.t_vis;                       // the caller's rows are dense
  d.calibrate = 0;
  return d;
}

size_t mma_qbmm_workspace_bytes(int batch, int n_q_heads, int64_t K, int64_t N) {
  // the attn.V route with the small work items (256 rows of k): one (acc[128], max, sum) partial per item
  if (N != kHeadDim || K % 256) return 256;
  const size_t rows = (size_t)batch * n_q_heads, slots = (size_t)(K / 256);
  return 256 + align_up(rows * slots * sizeof(float2), 256) + rows * slots * kHeadDim * sizeof(float);
}

template <typename T, int BITS>
static int qbmm_run_t(int kind, const mma::Dims& d_in, const void* fA, const int32_t* qB, const void* scales,
                      const void* zeros, void* out, unsigned char* ws, cudaStream_t st) {
  using namespace mma;
  Dims d = d_in;                       // built without the bit width: the K tiling depends on it
  d.n_ktiles = (d.n_groups + tile_g(BITS) - 1) / tile_g(BITS);
  d.n_mm = d.n_ktiles * K1_WARPS;
  int* status = reinterpret_cast<int*>(ws);
  const int n_pairs = d.batch * d.hkv;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CQ_ERR_LAUNCH;
  if (kind == 1) {
    const int variant = d.n_rep <= 4 ? 1 : 0;
    auto k1 = variant ? k1_scores<T, BITS, true> : k1_scores<T, BITS, false>;
    const int smem1 = k1_stages(BITS) * k1_stage_bytes(BITS) + 1024;
    static bool configured[64][2] = {};
    static int occ[64][2];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[dev][variant]) {
      if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1) != cudaSuccess) return CQ_ERR_LAUNCH;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ[dev][variant], k1, K1_THREADS, smem1) != cudaSuccess || occ[dev][variant] < 1) return CQ_ERR_LAUNCH;
      configured[dev][variant] = true;
    }
    CUtensorMap tm_code, tm_ks, tm_kmn;
    const uint64_t rows = (uint64_t)n_pairs * kHeadDim;
    if (!make_k_maps<BITS>(&tm_code, &tm_ks, &tm_kmn, qB, scales, zeros, (uint64_t)d.n_groups, rows)) return CQ_ERR_LAUNCH;
    const int grid = max(1, min(n_pairs * d.n_ktiles, sm_count() * occ[dev][variant]));
    k1<<<grid, K1_THREADS, smem1, st>>>(tm_code, tm_ks, tm_kmn, d, static_cast<const T*>(fA),
                                        static_cast<T*>(out), nullptr, status, nullptr, nullptr, nullptr);
    return check_launch();
  }
  float2* ml = reinterpret_cast<float2*>(ws + 256);
  const size_t rows = (size_t)d.batch * d.hq;
  float* partial = reinterpret_cast<float*>(ws + 256 + align_up(rows * (size_t)d.n_slots * sizeof(float2), 256));
  auto launch_k2 = [&](auto k2, int smem2) -> int {
    static bool configured[64] = {};
    static int occ[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!configured[dev]) {
      if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) != cudaSuccess) return CQ_ERR_LAUNCH;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ[dev], k2, K2_THREADS, smem2) != cudaSuccess || occ[dev] < 1) return CQ_ERR_LAUNCH;
      configured[dev] = true;
    }
    const int grid = max(1, min(n_pairs * d.n_chunks, sm_count() * occ[dev]));
    CUtensorMap tm_v;
    if (!make_v_map<BITS>(&tm_v, qB, (uint64_t)n_pairs * d.t_vis)) return CQ_ERR_LAUNCH;
    k2<<<grid, K2_THREADS, smem2, st>>>(tm_v, d, static_cast<const T*>(fA), nullptr, qB, static_cast<const T*>(scales),
                                     static_cast<const T*>(zeros), partial, ml, status);
    return check_launch();
  };
  int rc;
  if (d.chunk_tok == VT_LARGE)
    rc = launch_k2(k2_attn_v<T, BITS, VT_LARGE>, k2_smem_bytes(BITS, VT_LARGE));
  else
    rc = launch_k2(k2_attn_v<T, BITS, VT_SMALL>, k2_smem_bytes(BITS, VT_SMALL));
  if (rc != CQ_OK) return rc;
  if (d.n_slots >= 16)
    k3_combine<T, 4><<<d.batch * d.hq, kHeadDim * 4, 0, st>>>(d, partial, ml, static_cast<T*>(out));
  else
    k3_combine<T, 1><<<d.batch * d.hq, kHeadDim, 0, st>>>(d, partial, ml, static_cast<T*>(out));
  return check_launch();
}

int mma_qbmm_run(int kind, const void* fA, const int32_t* qB, const void* scales, const void* zeros, void* out,
                 int batch, int n_q_heads, int n_kv_heads, int64_t K, int64_t N, int bits, int dtype,
                 void* workspace, cudaStream_t st) {
  const mma::Dims d = qbmm_dims(kind, batch, n_q_heads, n_kv_heads, K, N);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
#define CQ_QBMM(T)                                                                                          \
  (bits == 1 ? qbmm_run_t<T, 1>(kind, d, fA, qB, scales, zeros, out, ws, st)                                 \
   : bits == 2 ? qbmm_run_t<T, 2>(kind, d, fA, qB, scales, zeros, out, ws, st)                               \
               : qbmm_run_t<T, 4>(kind, d, fA, qB, scales, zeros, out, ws, st))
  return dtype == CQ_DTYPE_F16 ? CQ_QBMM(__half) : CQ_QBMM(__nv_bfloat16);
#undef CQ_QBMM
}

size_t mma_path_workspace_bytes(const cq_decode_args* a) {
  return mma::make_layout(mma::make_dims(a)).total;
}

int mma_path_run(const cq_decode_args* a, void* workspace, cudaStream_t st, cudaEvent_t* ev, int* status_word) {
  const mma::Dims d = mma::make_dims(a);
  const mma::Layout l = mma::make_layout(d);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  if (a->dtype == CQ_DTYPE_F16) {
    switch (a->bits) {
      case 1: return mma::run<__half, 1>(a, d, l, ws, st, ev, status_word);
      case 2: return mma::run<__half, 2>(a, d, l, ws, st, ev, status_word);
      default: return mma::run<__half, 4>(a, d, l, ws, st, ev, status_word);
    }
  }
  switch (a->bits) {
    case 1: return mma::run<__nv_bfloat16, 1>(a, d, l, ws, st, ev, status_word);
    case 2: return mma::run<__nv_bfloat16, 2>(a, d, l, ws, st, ev, status_word);
    default: return mma::run<__nv_bfloat16, 4>(a, d, l, ws, st, ev, status_word);
  }
}

}  // namespace cq
