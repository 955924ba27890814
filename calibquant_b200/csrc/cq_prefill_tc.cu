// Dense causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One work item = 256 queries of one (batch, query head), as two 128-row tiles A and B that share the
// K/V stream.  One CTA per SM; it starts with the item of its own block index and then takes over blocks of the
// grid that have not been launched yet (cluster launch control), so tensor memory, barriers and the pipeline
// are set up once per SM and the hardware's launch order and load balance are kept.  Roles:
//   warp 9 (one lane)  TMA producer: the item's Q tiles, then its 128-key K/V tiles through a two-stage ring
//                        that runs on across items; asks for the next block when an item's loads are issued
//   warp 8 (one lane)  MMA issuer:
//        S_X = Q_X K^T   tcgen05.mma kind::f16, A = Q_X and B = K from shared memory (K-major), D in the
//                        tile's 128 TMEM columns
//        O_X += P_X V    A = P_X read from TENSOR MEMORY (16-bit pairs the softmax warps stored over the
//                        first 64 columns of S_X), B = V from shared memory (MN-major), D accumulates in
//                        the tile's O columns over all key tiles
//   warps 0-3 / 4-7    softmax of tile A / B: thread = one query row (= TMEM lane).  It reads its 128
//                        logits once (tcgen05.ld), applies scale, causal mask and the online softmax
//                        with a lazy maximum, and stores P back to TMEM (tcgen05.st).  No cross-thread
//                        exchange: the two tiles run out of phase, so one tile's
//                        exponentials overlap the other tile's products on the tensor pipe.
// Lazy maximum: a row keeps its reference maximum until the true one exceeds it by more than 2^8, and
// only then are that row's O columns and running sum rescaled (tcgen05.ld / st between two PV
// products); probabilities stay below 256 and O is read back once, at the end.
// Epilogue: the normalised rows of a tile are staged in shared memory (swizzled box layout) and written
// with two tiled TMA stores, which also clip the rows past the end of the sequence.
// TMEM columns: S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512).  Operand tiles in shared
// memory use the 128-byte swizzle: a [128 rows x 64 elements] TMA box lands directly in the
// canonical UMMA layout (8-row atoms of 1024 bytes).
// Measured on B200: one M128 N128 K16 product takes 85 cycles of the tensor pipe whether A comes from shared or
// tensor memory (98 with the softmax warps' TMEM traffic beside it), so the 32 products of a key tile bound a
// CTA at ~3100 cycles per key tile; the loop runs at ~3400.
//
// Every mbarrier wait is bounded; on a timeout the CTA records CQ_ERR_TIMEOUT in the status word,
// skips its remaining waits, frees its TMEM and returns.
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
constexpr int SMEM_BYTES = TILE_BYTES * 7 + 1024;   // Q x2, K x2, V x2, output staging (+ alignment slack)
constexpr int SOFTMAX_THREADS = 256, MMA_WARP = 8, TMA_WARP = 9, THREADS = SOFTMAX_THREADS + 64;
constexpr uint32_t WAIT_TRIES = 1u << 22;
constexpr long long WAIT_CYCLES = 1ll << 30;     // ~0.5 s: bound of the waits on the S / P hand-offs
constexpr uint32_t TMEM_COLS = 512;
constexpr float RESCALE_LOG2 = 8.f;          // a row is rescaled when its maximum grew by more than 2^8

struct Params {
  int t_len, hq, hkv;
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
// the same product with the A operand in tensor memory (16-bit elements, two per 32-bit column)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
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

// 4-D tiled store shared -> global (rows past the tensor's extent are clipped), tracked by the thread's bulk group
__device__ __forceinline__ void tma_store_4d(const void* tmap, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
      ::"l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(src))
      : "memory");
}
// closes the thread's bulk group and waits until its stores have read their shared-memory source
__device__ __forceinline__ void tma_store_commit_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Cluster launch control: a running CTA asks for the grid's next CTA that has not been launched yet.  On success
// that CTA is never launched and the 16-byte response names its block index, so the caller does its work: the
// hardware's own launch order and load balance, without the launch gap and the set-up of a new CTA.
// After a request has failed (nothing left to cancel) no further request may be issued.
__device__ __forceinline__ void clc_try_cancel(void* resp, uint64_t* bar) {
  asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
               ::"r"(smem_u32(resp)), "r"(smem_u32(bar)) : "memory");
}
// decodes a response; false: the request failed, there is no further work
__device__ __forceinline__ bool clc_read(const void* resp, int& bx, int& by, int& bz) {
  uint32_t valid = 0, x = 0, y = 0, z = 0;
  asm volatile(
      "{\n\t.reg .pred p1;\n\t.reg .b128 r;\n\t"
      "ld.shared.b128 r, [%4];\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p1, r;\n\t"
      "selp.u32 %3, 1, 0, p1;\n\t"
      "@p1 clusterlaunchcontrol.query_cancel.get_first_ctaid.v4.b32.b128 {%0, %1, %2, _}, r;\n\t}"
      : "+r"(x), "+r"(y), "+r"(z), "+r"(valid)
      : "r"(smem_u32(resp))
      : "memory");
  fence_proxy_async_smem();       // the slot is written again through the async proxy
  bx = (int)x; by = (int)y; bz = (int)z;
  return valid != 0;
}
// A use counter in shared memory (monotonic, so a waiter may be any number of uses behind or ahead, which the
// parity of an mbarrier phase cannot express): bounded wait until it has reached `target`.
__device__ __forceinline__ bool wait_count(const uint32_t* ctr, uint32_t target, uint32_t max_tries) {
  for (uint32_t i = 0; i < max_tries; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(ctr)) : "memory");
    if (v >= target) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void publish_count(uint32_t* ctr, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(ctr)), "r"(v) : "memory");
}
// barrier among the four softmax warps of one query tile that also tells whether ALL of them passed `flag`
__device__ __forceinline__ bool tile_all(int id, bool flag) {
  uint32_t out;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, %2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(out) : "r"((uint32_t)flag), "r"(id) : "memory");
  return out != 0;
}
// barrier among the four softmax warps of one query tile
__device__ __forceinline__ void tile_barrier(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

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

// sm_100 arithmetic that halves the instruction count of the softmax: 3-input maximum, and fp32
// operations on register pairs
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (x0, x1) = (a0, a1) * (b, b) + (c, c)
__device__ __forceinline__ void fma_pair(float& x0, float& x1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(x0), "=f"(x1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (s0, s1) += (a0, a1)
__device__ __forceinline__ void add_pair(float& s0, float& s1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rs;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rs, {%0, %1};\n\t"
      "add.rn.f32x2 rs, rs, ra;\n\tmov.b64 {%0, %1}, rs;\n\t}"
      : "+f"(s0), "+f"(s1) : "f"(a0), "f"(a1));
}

template <bool IS_BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if (IS_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// One work item = 256 queries of one (batch, query head) = one block index of the grid (x: 256-query block,
// longest rows first; y: query head; z: batch row).  A CTA starts with its own index and then takes over blocks
// that have not been launched yet (cluster launch control).  Measured, the CTAs running at the same time keep
// working on the query blocks and heads of a few KV heads, whose K/V tiles stay in L2, as with one CTA per block;
// a static assignment of items sorted by length lost that and ran 6 % slower.
struct Item {
  int h, b, hk, q0, n_a, n_b, n_max;
};
__device__ __forceinline__ Item decode_item(const Params& p, int bx, int by, int bz) {
  Item w;
  const int qt = (int)gridDim.x - 1 - bx;         // longest rows first
  w.h = by;
  w.b = bz;
  w.hk = w.h / (p.hq / p.hkv);
  w.q0 = qt * 2 * BM;
  const int t_tiles = (p.t_len + BN - 1) / BN;
  // key tiles of query tile X = 0 (A), 1 (B); B may lie wholly past the end
  w.n_a = min((w.q0 + BM + BN - 1) / BN, t_tiles);
  w.n_b = w.q0 + BM < p.t_len ? min((w.q0 + 2 * BM + BN - 1) / BN, t_tiles) : 0;
  w.n_max = max(w.n_a, w.n_b);
  return w;
}

template <bool IS_BF16>
__global__ void __launch_bounds__(THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o, Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* q_s = smem;                    // tiles A, B
  unsigned char* k_s = q_s + 2 * TILE_BYTES;    // 2 stages
  unsigned char* v_s = k_s + 2 * TILE_BYTES;    // 2 stages
  unsigned char* o_s = v_s + 2 * TILE_BYTES;    // output staging, used by the two tiles in turn
  // Barriers.  Their phases run on across the CTA's items: every role keeps the count of completions it has seen.
  //   bar_q[X]       Q_X of an item has landed                         (once per item)
  //   bar_q_free[X]  the last S_X of an item has completed: Q_X may be overwritten   (once per item)
  //   bar_kv_full/free[stage]   K/V ring                               (once per key tile of the CTA)
  //   bar_s[X]       S_X ready;  bar_p[X][half]  P_X of keys 0-63 / 64-127 stored (128 arrivals);
  //   bar_pv[X]      O_X += P_X V done                                 (once per key tile of X)
  //   stage_done     (a counter, not a barrier) uses of the staging buffer whose stores have read it
  //   bar_clc_full/free[slot]   the response naming the CTA's next item has arrived / has been read by the MMA
  //                  thread and the eight softmax warps (item i's successor travels through slot i % 2)
  __shared__ __align__(8) uint64_t bar_q[2], bar_q_free[2], bar_kv_full[2], bar_kv_free[2], bar_s[2], bar_p[2][2],
      bar_pv[2], bar_clc_full[2], bar_clc_free[2];
  __shared__ __align__(16) uint4 clc_resp[2];
  __shared__ uint32_t stage_done;
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_q[s], 1);
      mbar_init(&bar_q_free[s], 1);
      mbar_init(&bar_kv_full[s], 1);
      mbar_init(&bar_kv_free[s], 1);
      mbar_init(&bar_s[s], 1);
      mbar_init(&bar_p[s][0], SOFTMAX_THREADS / 2);
      mbar_init(&bar_p[s][1], SOFTMAX_THREADS / 2);
      mbar_init(&bar_pv[s], 1);
      mbar_init(&bar_clc_full[s], 1);
      mbar_init(&bar_clc_free[s], 1 + SOFTMAX_THREADS / 32);
    }
    stage_done = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) tmem_alloc(&tmem_base_s, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (warp == TMA_WARP) {
    // ================= TMA producer (one lane) =================
    if (lane == 0) {
      bool ok = true;
      uint32_t kv = 0;                          // K/V tiles this CTA has loaded so far
      int bx = blockIdx.x, by = blockIdx.y, bz = blockIdx.z;
      for (uint32_t it = 0; ok; ++it) {         // items of this CTA
        const Item w = decode_item(p, bx, by, bz);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          // Q_x of the previous item is read until its last S_x has completed
          if (it > 0) ok = ok && mbar_wait_bounded(&bar_q_free[x], (it - 1) & 1, WAIT_TRIES);
          if (!ok) break;
          mbar_expect_tx(&bar_q[x], TILE_BYTES);
          tma_load_4d(q_s + x * TILE_BYTES, &tm_q, 0, w.h, w.q0 + x * BM, w.b, &bar_q[x]);
          tma_load_4d(q_s + x * TILE_BYTES + PANEL_BYTES, &tm_q, 64, w.h, w.q0 + x * BM, w.b, &bar_q[x]);
        }
        for (int j = 0; j < w.n_max && ok; ++j, ++kv) {
          const uint32_t s = kv & 1;
          if (kv >= 2) ok = mbar_wait_bounded(&bar_kv_free[s], ((kv - 2) >> 1) & 1, WAIT_TRIES);
          if (!ok) break;
          mbar_expect_tx(&bar_kv_full[s], 2 * TILE_BYTES);
          tma_load_4d(k_s + s * TILE_BYTES, &tm_k, 0, w.hk, j * BN, w.b, &bar_kv_full[s]);
          tma_load_4d(k_s + s * TILE_BYTES + PANEL_BYTES, &tm_k, 64, w.hk, j * BN, w.b, &bar_kv_full[s]);
          tma_load_4d(v_s + s * TILE_BYTES, &tm_v, 0, w.hk, j * BN, w.b, &bar_kv_full[s]);
          tma_load_4d(v_s + s * TILE_BYTES + PANEL_BYTES, &tm_v, 64, w.hk, j * BN, w.b, &bar_kv_full[s]);
        }
        if (!ok) break;
        // All loads of this item are on their way (the other roles are about two key tiles behind): ask for the
        // item's successor now, not earlier, so that a CTA does not sit on a block another CTA could start.
        const uint32_t slot = it & 1;
        if (it >= 2) ok = mbar_wait_bounded(&bar_clc_free[slot], ((it >> 1) - 1) & 1, WAIT_TRIES);
        if (!ok) break;
        mbar_expect_tx(&bar_clc_full[slot], 16);
        clc_try_cancel(&clc_resp[slot], &bar_clc_full[slot]);
        ok = mbar_wait_bounded(&bar_clc_full[slot], (it >> 1) & 1, WAIT_TRIES);
        if (!ok || !clc_read(&clc_resp[slot], bx, by, bz)) break;
      }
      if (!ok) atomicExch(p.status, CQ_ERR_TIMEOUT);
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    // ================= MMA issuer (one lane) =================
    if (lane == 0) {
      // descriptors of the operand tiles; a k-step only moves the start address (14-bit field of
      // 16-byte units in the low word, which cannot carry: shared memory ends below 256 KB)
      const uint64_t qd[2] = {smem_desc(smem_u32(q_s), 16, 1024), smem_desc(smem_u32(q_s + TILE_BYTES), 16, 1024)};
      const uint64_t kd[2] = {smem_desc(smem_u32(k_s), 16, 1024), smem_desc(smem_u32(k_s + TILE_BYTES), 16, 1024)};
      const uint64_t vd[2] = {smem_desc(smem_u32(v_s), PANEL_BYTES, 1024),
                              smem_desc(smem_u32(v_s + TILE_BYTES), PANEL_BYTES, 1024)};
      auto issue_s = [&](int x, uint32_t stage) {   // S_x = Q_x K^T on the K tile of that stage, known to be there
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {        // 16 channels per step; panel = ks/4, 32 B per step
          const uint64_t off = (uint64_t)(((ks >> 2) * PANEL_BYTES + (ks & 3) * 32) >> 4);
          umma(tmem + (uint32_t)x * 128u, qd[x] + off, kd[stage] + off, p.idesc_s, ks > 0);
        }
        umma_commit(&bar_s[x]);
      };
      bool ok = true;
      uint32_t kv = 0, cnt[2] = {0, 0};           // K/V tiles, key tiles of A / B done so far
      int bx = blockIdx.x, by = blockIdx.y, bz = blockIdx.z;
      for (uint32_t it = 0; ok; ++it) {
        const Item w = decode_item(p, bx, by, bz);
        const int n_x[2] = {w.n_a, w.n_b};
        ok = mbar_wait_bounded(&bar_kv_full[kv & 1], (kv >> 1) & 1, WAIT_TRIES);
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          ok = ok && mbar_wait_bounded(&bar_q[x], it & 1, WAIT_TRIES);
          if (!ok) break;
          tc_fence_after();
          if (n_x[x] > 0) issue_s(x, kv & 1);
          if (n_x[x] <= 1) umma_commit(&bar_q_free[x]);     // that was the item's last S_x (or it has none)
        }
        for (int j = 0; j < w.n_max && ok; ++j) {
          const uint32_t s = (kv + j) & 1;
          bool next_k_ready = false;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            if (j >= n_x[x]) continue;
            // O_x += P_x(j) V(j), 16 keys = 8 TMEM columns per step; the first four steps start as soon as
            // the probabilities of keys 0-63 are stored, while the softmax warps work on keys 64-127
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              ok = mbar_wait_cycles(&bar_p[x][hf], (cnt[x] + j) & 1, WAIT_CYCLES);
              if (!ok) break;
              tc_fence_after();
#pragma unroll
              for (int ks = 4 * hf; ks < 4 * hf + 4; ++ks)
                umma_ts(tmem + 256u + (uint32_t)x * 128u, tmem + (uint32_t)x * 128u + (uint32_t)ks * 8u,
                        vd[s] + (uint64_t)(ks * 2048 >> 4), p.idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
            }
            if (!ok) break;
            umma_commit(&bar_pv[x]);
            // S_x(j+1) overwrites the columns P_x(j) lives in; the tensor pipe runs in issue order
            if (j + 1 < n_x[x]) {
              if (!next_k_ready) {
                ok = mbar_wait_bounded(&bar_kv_full[s ^ 1], ((kv + j + 1) >> 1) & 1, WAIT_TRIES);
                if (!ok) break;
                tc_fence_after();
                next_k_ready = true;
              }
              issue_s(x, s ^ 1);
              if (j + 2 == n_x[x]) umma_commit(&bar_q_free[x]);   // the item's last S_x
            }
          }
          if (!ok) break;
          umma_commit(&bar_kv_free[s]);             // K(j), V(j) are free once everything issued so far has drained
        }
        kv += (uint32_t)w.n_max;
        cnt[0] += (uint32_t)w.n_a;
        cnt[1] += (uint32_t)w.n_b;
        if (!ok) break;
        ok = mbar_wait_bounded(&bar_clc_full[it & 1], (it >> 1) & 1, WAIT_TRIES);
        if (!ok) break;
        const bool more = clc_read(&clc_resp[it & 1], bx, by, bz);
        mbar_arrive(&bar_clc_free[it & 1]);
        if (!more) break;
      }
      if (!ok) atomicExch(p.status, CQ_ERR_TIMEOUT);
    }
    __syncwarp();
  } else {
    // ===== softmax: warps 0-3 tile A, 4-7 tile B; thread = one query row =====
    const int x = warp >> 2, quarter = warp & 3;
    const int r_in = quarter * 32 + lane;               // row inside the tile = TMEM lane
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + (uint32_t)x * 128u + lane_off;
    const uint32_t tO = tmem + 256u + (uint32_t)x * 128u + lane_off;
    bool ok = true;                                     // stays false after a timeout; later waits are skipped
    uint32_t cnt = 0, uses = 0;                         // key tiles of this tile / uses of the staging buffer so far
    int bx = blockIdx.x, by = blockIdx.y, bz = blockIdx.z;
    for (uint32_t it = 0;; ++it) {
      const Item w = decode_item(p, bx, by, bz);
      const int n_x = x == 0 ? w.n_a : w.n_b;
      const int qx0 = w.q0 + x * BM;
      const int row = qx0 + r_in;
      float m_ref = -INFINITY, l_run = 0.f;             // reference maximum (log2 units), row sum
      for (int j = 0; j < n_x; ++j) {
        const int key0 = j * BN;
        const bool need_mask = (key0 + BN - 1 > qx0) || (key0 + BN > p.t_len);
        if (ok) ok = mbar_wait_cycles(&bar_s[x], (cnt + j) & 1, WAIT_CYCLES);
        tc_fence_after();
        uint32_t sv[4][32];                             // this row's 128 logits, read once
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld32_nowait(tS + cc * 32, sv[cc]);
        tmem_ld_wait();
        if (need_mask) {                                // diagonal and last key tiles only
          const int lim = min(row, p.t_len - 1) - key0; // columns above lim are masked
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cc * 32 + i > lim) sv[cc][i] = 0xff800000u;   // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sv[cc][i]), __uint_as_float(sv[cc][i + 1]));
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_true = fmaxf(m_ref, mx * p.scale_log2);
        const bool grow = m_true - m_ref > RESCALE_LOG2;  // also true for the first tile (m_ref = -inf)
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // O_x holds the products of tiles 0..j-1; the last of them must have completed
          if (ok) ok = mbar_wait_bounded(&bar_pv[x], (cnt + j - 1) & 1, WAIT_TRIES);
          tc_fence_after();
          const float alpha = grow ? exp2f(m_ref - m_true) : 1.f;
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld32(tO + cc * 32, r);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO + cc * 32, r);
          }
          l_run *= alpha;
        }
        if (grow) m_ref = m_true;
        const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
        float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int cc = 0; cc < 4; cc += 2) {
          uint32_t wv[32];                              // 64 probabilities as 16-bit pairs = 32 TMEM columns
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            // masked logits are -inf: ex2 gives 0
            float x0, x1;
            fma_pair(x0, x1, __uint_as_float(sv[cc + (i >> 5)][i & 31]), __uint_as_float(sv[cc + (i >> 5)][(i & 31) + 1]),
                     p.scale_log2, -m_use);
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            add_pair(rs4[i & 2], rs4[(i & 2) + 1], p0, p1);
            wv[i >> 1] = pack16<IS_BF16>(p0, p1);
          }
          tmem_st32(tS + (cc >> 1) * 32, wv);           // over the first 64 columns of S_x
          tmem_st_wait();
          tc_fence_before();
          mbar_arrive(&bar_p[x][cc >> 1]);
        }
        l_run += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      }
      if (n_x > 0) {
        if (ok) ok = mbar_wait_bounded(&bar_pv[x], (cnt + n_x - 1) & 1, WAIT_TRIES);
        // the staging buffer is used by A, then B, of every item: wait until the use before this one has been read
        const uint32_t use = uses + (x == 1 && w.n_a > 0 ? 1u : 0u);
        if (ok) ok = wait_count(&stage_done, use, WAIT_TRIES);
        if (ok) {
          tc_fence_after();
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          // The normalised rows go through shared memory in the layout of a 128-byte-swizzled TMA box and leave
          // as two tiled stores: a thread's row is 256 contiguous bytes in global memory, but the 32 rows of a
          // warp are a row pitch apart, and direct 16-byte stores from the registers cost the CTA ~5000 cycles.
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld32(tO + cc * 32, r);
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 wq;
              wq.x = pack16<IS_BF16>(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              wq.y = pack16<IS_BF16>(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              wq.z = pack16<IS_BF16>(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              wq.w = pack16<IS_BF16>(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              const int chunk = (cc & 1) * 4 + (i >> 3);        // 16-byte chunk of the 128-byte panel row
              *reinterpret_cast<uint4*>(o_s + (cc >> 1) * PANEL_BYTES + r_in * 128 + ((chunk ^ (r_in & 7)) << 4)) = wq;
            }
          }
        }
        tc_fence_before();                              // O_x has been read: the next item's first P.V may overwrite it
        fence_proxy_async_smem();
        tile_barrier(1 + x);
        if (quarter == 0 && lane == 0) {
          if (ok) {
            tma_store_4d(&tm_o, o_s, 0, w.h, qx0, w.b);
            tma_store_4d(&tm_o, o_s + PANEL_BYTES, 64, w.h, qx0, w.b);
            tma_store_commit_wait_read();
          } else {
            atomicExch(p.status, CQ_ERR_TIMEOUT);
          }
          publish_count(&stage_done, use + 1);          // also after a timeout, so that nobody waits for this use
        }
      }
      cnt += (uint32_t)n_x;
      uses += (w.n_a > 0 ? 1u : 0u) + (w.n_b > 0 ? 1u : 0u);
      // the next item, if there is one
      if (ok) ok = mbar_wait_bounded(&bar_clc_full[it & 1], (it >> 1) & 1, WAIT_TRIES);
      bool more = ok && clc_read(&clc_resp[it & 1], bx, by, bz);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_clc_free[it & 1]);
      more = tile_all(1 + x, more);                     // the tile's four warps go on, or leave, together
      if (!more) break;
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
  if (!prefill_tc::encode_fn()) return false;
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
  CUtensorMap tq, tk, tv, to;
  if (!make_map(&tq, q, is_bf16, batch, t_len, hq, qs) || !make_map(&tk, k, is_bf16, batch, t_len, hkv, ks) ||
      !make_map(&tv, v, is_bf16, batch, t_len, hkv, vs) || !make_map(&to, out, is_bf16, batch, t_len, hq, os))
    return CQ_ERR_LAUNCH;
  static bool configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return CQ_ERR_LAUNCH;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return CQ_ERR_LAUNCH;
    configured[dev] = true;
  }
  Params p;
  p.t_len = t_len; p.hq = hq; p.hkv = hkv;
  p.scale_log2 = 1.4426950408889634f / sqrtf(128.f);
  p.idesc_s = make_idesc(is_bf16, 0);
  p.idesc_pv = make_idesc(is_bf16, 1);
  p.is_bf16 = is_bf16;
  p.status = status;
  dim3 grid((unsigned)((t_len + 2 * BM - 1) / (2 * BM)), (unsigned)hq, (unsigned)batch);
  if (is_bf16) prefill_tc_kernel<true><<<grid, THREADS, SMEM_BYTES, st>>>(tq, tk, tv, to, p);
  else prefill_tc_kernel<false><<<grid, THREADS, SMEM_BYTES, st>>>(tq, tk, tv, to, p);
  return check_launch();
}

}  // namespace cq
