// Dense causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One CTA = 128 queries of one (batch, query head).  Warp 8 (one elected lane) is the producer and
// the MMA issuer: it streams 128-key K/V tiles through a two-stage shared-memory ring with tiled
// TMA loads and issues
//     S = Q K^T       tcgen05.mma kind::f16, A = Q (K-major), B = K (K-major), D in TMEM columns
//                     [0,128) / [128,256) alternately, so S(j+1) is computed while tile j is in softmax
//     O += P V        A = P (K-major, written by the softmax warps into one of two shared-memory
//                     buffers), B = V (MN-major), D accumulates in TMEM columns [256,384) over all tiles
// Warps 0-7 are the softmax warps: thread = (query row, 64-column half).  They read S from TMEM once
// (tcgen05.ld), apply scale, causal mask and the online softmax (the row maximum of the two halves
// meets in shared memory) and write P (16-bit) into the swizzled A-operand layout.  The running
// maximum is lazy: a row keeps its reference maximum until the true one exceeds it by more than 2^8,
// and only then are that row's O columns in TMEM and its running sum rescaled (tcgen05.ld / st
// between two PV products); probabilities therefore stay below 256 and O is read back once, at the
// end.  All operand tiles use the 128-byte swizzle: a [128 rows x 64 elements] TMA box lands directly
// in the canonical UMMA layout (8-row atoms of 1024 bytes).
//
// Every mbarrier wait is bounded; on a timeout the CTA records CQ_ERR_TIMEOUT in the status word,
// stops issuing work, frees its TMEM and returns.
#include <cuda.h>
#include <stdlib.h>

#include "cq_common.cuh"
#include "cq_ptx.cuh"

namespace cq {
namespace prefill_tc {

using namespace ptx;

constexpr int BM = 128, BN = 128;
constexpr int PANEL_BYTES = 128 * 128;          // [128 rows][64 x 16-bit]
constexpr int TILE_BYTES = 2 * PANEL_BYTES;     // [128 rows][128 x 16-bit]
constexpr int SMEM_BYTES = TILE_BYTES * 7 + 1024;   // Q, K x2, V x2, P x2 (+ alignment slack)
constexpr int SOFTMAX_THREADS = 256, MMA_WARP = 8, THREADS = SOFTMAX_THREADS + 32;
constexpr uint32_t WAIT_TRIES = 1u << 22;
constexpr uint32_t TMEM_COLS = 512;          // S x2 (double-buffered) + O; allocations are powers of two
constexpr float RESCALE_LOG2 = 8.f;          // a row is rescaled when its maximum grew by more than 2^8

struct Params {
  void* out;
  int t_len, hq, hkv;
  int64_t o_sb, o_st, o_sh;
  float scale_log2;
  uint32_t idesc_s, idesc_pv;
  int is_bf16;
  int* status;
};

// ---- tcgen05 wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, int c0, int c1, int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (Blackwell).
// K-major operands: lbo is unused (1), sbo = 1024 B between 8-row atoms.
// MN-major operands: lbo = bytes between 64-element MN blocks, sbo = 1024 B between 8-row K groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;          // descriptor version
  d |= (uint64_t)2 << 61;          // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack16(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;
  unsigned char* k_s = q_s + TILE_BYTES;        // 2 stages
  unsigned char* v_s = k_s + 2 * TILE_BYTES;    // 2 stages
  unsigned char* p_s = v_s + 2 * TILE_BYTES;    // 2 buffers
  __shared__ __align__(8) uint64_t bar_q, bar_kv_full[2], bar_kv_free[2], bar_s[2], bar_p[2], bar_pv[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ float half_max_s[2][BM];           // per-row maximum of each 64-column half

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.hq / p.hkv);
  const int q0 = qt * BM;
  const int n_tiles = min((q0 + BM + BN - 1) / BN, (p.t_len + BN - 1) / BN);

  if (tid == 0) {
    mbar_init(&bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_kv_full[s], 1);
      mbar_init(&bar_kv_free[s], 1);
      mbar_init(&bar_s[s], 1);
      mbar_init(&bar_p[s], SOFTMAX_THREADS);    // P buffer s written (tiles s, s+2, ...)
      mbar_init(&bar_pv[s], 1);                 // the PV product that read P buffer s has completed
    }
    mbar_fence_init();
  }
  if (warp == MMA_WARP) tmem_alloc(&tmem_base_s, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_O = tmem + 256;           // S buffers at columns [0,128) and [128,256)

  if (warp == MMA_WARP) {
    // ================= producer + MMA issuer (one lane) =================
    if (lane == 0) {
      auto load_kv = [&](int j) {
        const int s = j & 1;
        mbar_expect_tx(&bar_kv_full[s], 2 * TILE_BYTES);
        tma_load_4d(k_s + s * TILE_BYTES, &tm_k, 0, hk, j * BN, b, &bar_kv_full[s]);
        tma_load_4d(k_s + s * TILE_BYTES + PANEL_BYTES, &tm_k, 64, hk, j * BN, b, &bar_kv_full[s]);
        tma_load_4d(v_s + s * TILE_BYTES, &tm_v, 0, hk, j * BN, b, &bar_kv_full[s]);
        tma_load_4d(v_s + s * TILE_BYTES + PANEL_BYTES, &tm_v, 64, hk, j * BN, b, &bar_kv_full[s]);
      };
      const uint32_t qa = smem_u32(q_s);
      auto issue_s = [&](int j) -> bool {       // S(j) = Q K(j)^T into S buffer j&1
        const int s = j & 1;
        if (!mbar_wait_bounded(&bar_kv_full[s], (uint32_t)((j >> 1) & 1), WAIT_TRIES)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(k_s + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {        // 16 channels per step; panel = ks/4, 32 B per step
          const uint32_t off = (uint32_t)((ks >> 2) * PANEL_BYTES + (ks & 3) * 32);
          umma(tmem + (uint32_t)s * 128u, smem_desc(qa + off, 16, 1024), smem_desc(ka + off, 16, 1024),
               p.idesc_s, ks > 0);
        }
        umma_commit(&bar_s[s]);
        return true;
      };
      mbar_expect_tx(&bar_q, TILE_BYTES);
      tma_load_4d(q_s, &tm_q, 0, h, q0, b, &bar_q);
      tma_load_4d(q_s + PANEL_BYTES, &tm_q, 64, h, q0, b, &bar_q);
      load_kv(0);
      if (n_tiles > 1) load_kv(1);
      bool ok = mbar_wait_bounded(&bar_q, 0, WAIT_TRIES);
      ok = ok && issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        // S(j+1) goes to the other S buffer as soon as its K tile is there: the softmax warps
        // released that buffer when they signalled P(j-1), which was waited for last iteration
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        ok = mbar_wait_bounded(&bar_p[s], (uint32_t)((j >> 1) & 1), WAIT_TRIES);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(v_s + s * TILE_BYTES), pa = smem_u32(p_s + s * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {        // O += P(j) V(j): 16 keys per step
          const uint64_t ad = smem_desc(pa + (uint32_t)((ks >> 2) * PANEL_BYTES + (ks & 3) * 32), 16, 1024);
          const uint64_t bd = smem_desc(va + (uint32_t)(ks * 2048), PANEL_BYTES, 1024);
          umma(tmem_O, ad, bd, p.idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&bar_pv[s]);
        umma_commit(&bar_kv_free[s]);
        if (j + 2 < n_tiles) {                  // refill this stage once its MMAs have drained
          ok = mbar_wait_bounded(&bar_kv_free[s], (uint32_t)((j >> 1) & 1), WAIT_TRIES);
          if (!ok) break;
          load_kv(j + 2);
        }
      }
      if (!ok) atomicExch(p.status, CQ_ERR_TIMEOUT);
    }
    __syncwarp();
  } else {
    // ===== softmax: thread = (query row, 64-column half); 8 warps =====
    const int quarter = warp & 3, half = warp >> 2;
    const int r_in = quarter * 32 + lane;               // row inside the tile = TMEM lane
    const int row = q0 + r_in;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t col0 = (uint32_t)half * 64u;
    float m_ref = -INFINITY, l_run = 0.f;               // reference maximum (log2 units); sum over this thread's columns
    // Once a bounded wait has run out, `ok` stays false and all later waits are skipped, but every
    // thread still walks all tiles so that the named barrier below always sees its 256 arrivals.
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int key0 = j * BN + (int)col0;
      const bool need_mask = (j * BN + BN - 1 > q0) || (j * BN + BN > p.t_len);
      const uint32_t tS = tmem + (uint32_t)(j & 1) * 128u + lane_off + col0;
      if (ok) ok = mbar_wait_bounded(&bar_s[j & 1], (uint32_t)((j >> 1) & 1), WAIT_TRIES);
      tc_fence_after();
      uint32_t sv[2][32];                               // this thread's 64 logits, read once
      tmem_ld32_nowait(tS, sv[0]);
      tmem_ld32_nowait(tS + 32, sv[1]);
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (need_mask) {
            const int key = key0 + cc * 32 + i;
            if (key > row || key >= p.t_len) sv[cc][i] = 0xff800000u;   // -inf
          }
          mx = fmaxf(mx, __uint_as_float(sv[cc][i]));
        }
      half_max_s[half][r_in] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS) : "memory");
      mx = fmaxf(mx, half_max_s[half ^ 1][r_in]);
      const float m_true = fmaxf(m_ref, mx * p.scale_log2);
      // both threads of a row see the same m_ref and m_true, hence take the same decision
      const bool grow = m_true - m_ref > RESCALE_LOG2;  // also true for the first tile (m_ref = -inf)
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O holds PV(0..j-1); the product that last wrote it read P buffer (j-1)&1
        if (ok) ok = mbar_wait_bounded(&bar_pv[(j - 1) & 1], (uint32_t)(((j - 1) >> 1) & 1), WAIT_TRIES);
        tc_fence_after();
        const float alpha = grow ? exp2f(m_ref - m_true) : 1.f;    // 0 when m_ref was -inf
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t r[32];
          tmem_ld32(tmem_O + lane_off + col0 + cc * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st32(tmem_O + lane_off + col0 + cc * 32, r);
        }
        tmem_st_wait();
        l_run *= alpha;
      }
      if (grow) m_ref = m_true;
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      // the P buffer of this tile was last read by PV(j-2)
      if (j >= 2 && ok) ok = mbar_wait_bounded(&bar_pv[j & 1], (uint32_t)(((j - 2) >> 1) & 1), WAIT_TRIES);
      float rs = 0.f;
      unsigned char* prow = p_s + (j & 1) * TILE_BYTES + half * PANEL_BYTES + r_in * 128;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          // masked logits are -inf: ex2 gives 0
          const float p0 = ex2_approx(fmaf(__uint_as_float(sv[cc][i]), p.scale_log2, -m_use));
          const float p1 = ex2_approx(fmaf(__uint_as_float(sv[cc][i + 1]), p.scale_log2, -m_use));
          rs += p0 + p1;
          w[i >> 1] = pack16(p0, p1, p.is_bf16);
        }
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          const int chunk = (cc * 4 + qd) ^ (r_in & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(w[4 * qd], w[4 * qd + 1], w[4 * qd + 2], w[4 * qd + 3]);
        }
      }
      l_run += rs;
      fence_proxy_async_smem();        // P (generic-proxy writes) must be visible to the MMA (async proxy)
      tc_fence_before();
      mbar_arrive(&bar_p[j & 1]);
    }
    // the row sum is split over the two halves
    half_max_s[half][r_in] = l_run;
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_THREADS) : "memory");
    const float l_tot = l_run + half_max_s[half ^ 1][r_in];
    if (ok) ok = mbar_wait_bounded(&bar_pv[(n_tiles - 1) & 1], (uint32_t)(((n_tiles - 1) >> 1) & 1), WAIT_TRIES);
    if (!ok) {
      atomicExch(p.status, CQ_ERR_TIMEOUT);
    } else {
      tc_fence_after();
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      unsigned char* dst = reinterpret_cast<unsigned char*>(p.out) +
                           2 * ((int64_t)b * p.o_sb + (int64_t)row * p.o_st + (int64_t)h * p.o_sh) + col0 * 2;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t r[32];
        tmem_ld32(tmem_O + lane_off + col0 + cc * 32, r);     // warp-collective: rows past the end load too
        if (row < p.t_len) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv, p.is_bf16);
            w.y = pack16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv, p.is_bf16);
            w.z = pack16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv, p.is_bf16);
            w.w = pack16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv, p.is_bf16);
            *reinterpret_cast<uint4*>(dst + (cc * 32 + i) * 2) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) tmem_dealloc(tmem, TMEM_COLS);
}

// ---- host ---------------------------------------------------------------------------------------
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

// [B, T, H, D] with element strides (sb, st, sh), D contiguous -> 4-D map (d, h, t, b), box 64 x 1 x 128 x 1
static bool make_map(CUtensorMap* m, const void* base, int is_bf16, int batch, int t_len, int heads,
                     const int64_t* strides) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {128, (cuuint64_t)heads, (cuuint64_t)t_len, (cuuint64_t)batch};
  cuuint64_t gstr[3] = {(cuuint64_t)strides[2] * 2, (cuuint64_t)strides[1] * 2, (cuuint64_t)strides[0] * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(m, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
            const_cast<void*>(base), dims, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static uint32_t make_idesc(int is_bf16, int b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;                               // D format: f32
  d |= (uint32_t)(is_bf16 ? 1 : 0) << 7;      // A format
  d |= (uint32_t)(is_bf16 ? 1 : 0) << 10;     // B format
  d |= (uint32_t)(b_mn_major ? 1 : 0) << 16;  // B major (A stays K-major)
  d |= (uint32_t)(BN >> 3) << 17;             // N
  d |= (uint32_t)(BM >> 4) << 24;             // M
  return d;
}

}  // namespace prefill_tc

bool prefill_tc_eligible(const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os) {
  static const bool disabled = []() { const char* e = getenv("CQ_PREFILL_GENERAL"); return e && e[0] == '1'; }();
  if (disabled || !prefill_tc::encode_fn()) return false;
  const int64_t* all[] = {qs, ks, vs, os};
  for (const int64_t* s : all)
    for (int i = 0; i < 3; ++i)
      if (s[i] % 8 || s[i] <= 0) return false;
  return true;
}

int prefill_tc_run(const void* q, const void* k, const void* v, void* out, int batch, int t_len, int hq, int hkv,
                   const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, int is_bf16,
                   int* status, cudaStream_t st) {
  using namespace prefill_tc;
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q, is_bf16, batch, t_len, hq, qs) || !make_map(&tk, k, is_bf16, batch, t_len, hkv, ks) ||
      !make_map(&tv, v, is_bf16, batch, t_len, hkv, vs))
    return CQ_ERR_LAUNCH;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CQ_ERR_LAUNCH;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    configured[dev] = true;
  }
  Params p;
  p.out = out; p.t_len = t_len; p.hq = hq; p.hkv = hkv;
  p.o_sb = os[0]; p.o_st = os[1]; p.o_sh = os[2];
  p.scale_log2 = 1.4426950408889634f / sqrtf(128.f);
  p.idesc_s = make_idesc(is_bf16, 0);
  p.idesc_pv = make_idesc(is_bf16, 1);
  p.is_bf16 = is_bf16;
  p.status = status;
  dim3 grid((unsigned)((t_len + BM - 1) / BM), (unsigned)hq, (unsigned)batch);
  prefill_tc_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(tq, tk, tv, p);
  return check_launch();
}

}  // namespace cq
