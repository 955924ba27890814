// Dense causal prefill attention with GQA head sharing -- warp-level MMA version.
//
// Replaces the flash_attn calls of the reference prefill (patch_internvl.py:464-468 in 1024-query
// chunks, :606-609): o = softmax(q k^T / sqrt(D) + causal mask) v over unquantized K/V.
// One CTA = 64 queries of one (batch, query head); four warps of 16 query rows; K/V tiles of 64
// keys double-buffered in shared memory with 16-byte async copies; online softmax in registers;
// S = QK^T and O += PV on m16n8k16 tensor-core MMAs with fp32 accumulation.
// This is the general kernel (any T, fp16 or bf16); the tcgen05 kernel takes over for the shapes
// it supports.
#include "cq_common.cuh"
#include "cq_ptx.cuh"

namespace cq {
namespace prefill {

using namespace ptx;

constexpr int BM = 64, BN = 64, THREADS = 128;
constexpr int TILE_BYTES = BN * kHeadDim * 2;   // 16 KB

struct Args {
  const void *q, *k, *v;
  void* out;
  int batch, t_len, hq, hkv;
  int64_t q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh, o_sb, o_st, o_sh;
  float scale_log2;   // log2(e) / sqrt(D)
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <typename T> struct Mma;
template <> struct Mma<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) { mma_f16(d, a0, a1, a2, a3, b0, b1); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

// byte offset of 16-byte chunk `ch` (0..15) of row `r` in a [rows][128] 16-bit tile, XOR-swizzled
__device__ __forceinline__ uint32_t tile_off(int r, int ch) { return (uint32_t)(r * 256 + ((ch ^ (r & 7)) << 4)); }

template <typename T>
__device__ __forceinline__ void load_tile(uint32_t dst, const T* base, int64_t row_stride, int row0, int n_rows,
                                          int tid) {
  // 64 rows x 16 chunks = 1024 copies, 8 per thread
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = tid + i * THREADS;
    const int r = idx >> 4, ch = idx & 15;
    const bool ok = row0 + r < n_rows;
    const T* src = base + (int64_t)(ok ? row0 + r : 0) * row_stride + ch * 8;
    cp_async16(dst + tile_off(r, ch), src, ok);
  }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
prefill_kernel(Args a) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  const uint32_t q_s = smem_u32(smem);                    // [64][128]
  const uint32_t k_s = q_s + TILE_BYTES;                   // 2 x [64][128]
  const uint32_t v_s = k_s + 2 * TILE_BYTES;               // 2 x [64][128]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  const int qt = gridDim.x - 1 - blockIdx.x;              // heavy (late) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.hq / a.hkv);
  const int q0 = qt * BM;
  const T* qb = static_cast<const T*>(a.q) + b * a.q_sb + h * a.q_sh;
  const T* kb = static_cast<const T*>(a.k) + b * a.k_sb + hk * a.k_sh;
  const T* vb = static_cast<const T*>(a.v) + b * a.v_sb + hk * a.v_sh;
  const int n_kv_tiles = min((q0 + BM + BN - 1) / BN, (a.t_len + BN - 1) / BN);

  load_tile<T>(q_s, qb, a.q_st, q0, a.t_len, tid);
  load_tile<T>(k_s, kb, a.k_st, 0, a.t_len, tid);
  load_tile<T>(v_s, vb, a.v_st, 0, a.t_len, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  // Q fragments: 8 k-tiles x 4 registers
  uint32_t qf[8][4];
  {
    const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
    for (int kt = 0; kt < 8; ++kt) ldmatrix_x4(q_s + tile_off(r, 2 * kt + (lane >> 4)), qf[kt][0], qf[kt][1], qf[kt][2], qf[kt][3]);
  }

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_g = q0 + warp * 16 + g;     // query index of accumulator rows g (and +8)

  for (int j = 0; j < n_kv_tiles; ++j) {
    const int buf = j & 1;
    if (j + 1 < n_kv_tiles) {   // prefetch next tile into the other buffer
      load_tile<T>(k_s + (buf ^ 1) * TILE_BYTES, kb, a.k_st, (j + 1) * BN, a.t_len, tid);
      load_tile<T>(v_s + (buf ^ 1) * TILE_BYTES, vb, a.v_st, (j + 1) * BN, a.t_len, tid);
    }
    cp_async_commit();
    const uint32_t kt_s = k_s + buf * TILE_BYTES, vt_s = v_s + buf * TILE_BYTES;

    // ---- S = Q K^T (16 x 64 per warp)
    float s[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const int r = nt * 8 + (lane & 7);
#pragma unroll
      for (int kp = 0; kp < 4; ++kp) {    // two k-tiles per ldmatrix.x4
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kt_s + tile_off(r, 4 * kp + (lane >> 3)), b0, b1, b2, b3);
        Mma<T>::run(s[nt], qf[2 * kp][0], qf[2 * kp][1], qf[2 * kp][2], qf[2 * kp][3], b0, b1);
        Mma<T>::run(s[nt], qf[2 * kp + 1][0], qf[2 * kp + 1][1], qf[2 * kp + 1][2], qf[2 * kp + 1][3], b2, b3);
      }
    }
    // ---- scale, mask, online softmax
    const int key0 = j * BN;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + 2 * c + (e & 1);
        const int row = row_g + 8 * (e >> 1);
        float v = s[nt][e] * a.scale_log2;
        if (key > row || key >= a.t_len) v = -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float alpha[2], m_new[2];
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      mx[r2] = fmaxf(mx[r2], __shfl_xor_sync(0xffffffffu, mx[r2], 1));
      mx[r2] = fmaxf(mx[r2], __shfl_xor_sync(0xffffffffu, mx[r2], 2));
      m_new[r2] = fmaxf(m_run[r2], mx[r2]);
      const float m_use = m_new[r2] == -INFINITY ? 0.f : m_new[r2];
      alpha[r2] = exp2f(m_run[r2] - m_use);
      m_run[r2] = m_new[r2];
      m_new[r2] = m_use;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[8][2];   // P as 16-bit pairs: [nt][row half]
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - m_new[0]), p1 = exp2f(s[nt][1] - m_new[0]);
      const float p2 = exp2f(s[nt][2] - m_new[1]), p3 = exp2f(s[nt][3] - m_new[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[nt][0] = Mma<T>::pack(p0, p1);
      pf[nt][1] = Mma<T>::pack(p2, p3);
    }
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) l_run[r2] = l_run[r2] * alpha[r2] + rs[r2];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    // ---- O += P V : k-tile kk = keys 16kk..16kk+15, n-tile = 8 channels
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const int r = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int np = 0; np < 8; ++np) {    // two n-tiles per ldmatrix.x4.trans
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vt_s + tile_off(r, 2 * np + (lane >> 4)), b0, b1, b2, b3);
        Mma<T>::run(o[2 * np], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b0, b1);
        Mma<T>::run(o[2 * np + 1], pf[2 * kk][0], pf[2 * kk][1], pf[2 * kk + 1][0], pf[2 * kk + 1][1], b2, b3);
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  }

  // ---- normalise and store
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 1);
    l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 2);
  }
  T* ob = static_cast<T*>(a.out) + b * a.o_sb + h * a.o_sh;
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    const int row = row_g + 8 * r2;
    if (row >= a.t_len) continue;
    const float inv = l_run[r2] > 0.f ? 1.f / l_run[r2] : 0.f;
    T* orow = ob + (int64_t)row * a.o_st;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t w = Mma<T>::pack(o[i][2 * r2] * inv, o[i][2 * r2 + 1] * inv);
      *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * c) = w;
    }
  }
}

template <typename T>
int launch(const Args& a, cudaStream_t st) {
  const int smem = 5 * TILE_BYTES + 128;
  auto kern = prefill_kernel<T>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return CQ_ERR_LAUNCH;
  dim3 grid((unsigned)((a.t_len + BM - 1) / BM), (unsigned)a.hq, (unsigned)a.batch);
  kern<<<grid, THREADS, smem, st>>>(a);
  return check_launch();
}

}  // namespace prefill
}  // namespace cq

namespace cq {
bool prefill_tc_eligible(const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os);
int prefill_tc_run(const void* q, const void* k, const void* v, void* out, int batch, int t_len, int hq, int hkv,
                   const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, int is_bf16,
                   int* status, cudaStream_t st);

// Sticky status of the tcgen05 prefill kernel (it has no workspace to report into).
static __device__ int g_prefill_status;
static int* prefill_status_ptr() {
  static int* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_prefill_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}
}  // namespace cq

extern "C" int cq_prefill_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, cq::g_prefill_status, sizeof(int)) != cudaSuccess) return CQ_ERR_LAUNCH;
  return v;
}

extern "C" int cq_prefill_attn(const void* q, const void* k, const void* v, void* out, int batch, int t_len,
                               int n_q_heads, int n_kv_heads, int head_dim, const int64_t* q_strides,
                               const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                               int dtype, void* stream) {
  if (!q || !k || !v || !out || !q_strides || !k_strides || !v_strides || !o_strides) return CQ_ERR_BAD_ARG;
  if (batch < 0 || t_len < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (head_dim != cq::kHeadDim) return CQ_ERR_UNSUPPORTED;
  if (batch == 0 || t_len == 0) return CQ_OK;
  if (batch > 65535 || n_q_heads > 65535) return CQ_ERR_UNSUPPORTED;
  const void* ptrs[] = {q, k, v, out};
  for (const void* p : ptrs)
    if (!cq::aligned16(p)) return CQ_ERR_BAD_ARG;
  const int64_t* strides[] = {q_strides, k_strides, v_strides, o_strides};
  for (const int64_t* s : strides)
    for (int i = 0; i < 3; ++i)
      if (s[i] % 8) return CQ_ERR_BAD_ARG;
  if (cq::prefill_tc_eligible(q_strides, k_strides, v_strides, o_strides)) {
    int* status = cq::prefill_status_ptr();
    if (status)
      return cq::prefill_tc_run(q, k, v, out, batch, t_len, n_q_heads, n_kv_heads, q_strides, k_strides,
                                v_strides, o_strides, dtype == CQ_DTYPE_BF16, status,
                                static_cast<cudaStream_t>(stream));
  }
  cq::prefill::Args a;
  a.q = q; a.k = k; a.v = v; a.out = out;
  a.batch = batch; a.t_len = t_len; a.hq = n_q_heads; a.hkv = n_kv_heads;
  a.q_sb = q_strides[0]; a.q_st = q_strides[1]; a.q_sh = q_strides[2];
  a.k_sb = k_strides[0]; a.k_st = k_strides[1]; a.k_sh = k_strides[2];
  a.v_sb = v_strides[0]; a.v_st = v_strides[1]; a.v_sh = v_strides[2];
  a.o_sb = o_strides[0]; a.o_st = o_strides[1]; a.o_sh = o_strides[2];
  a.scale_log2 = 1.4426950408889634f / sqrtf((float)head_dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16) return cq::prefill::launch<__half>(a, st);
  return cq::prefill::launch<__nv_bfloat16>(a, st);
}
