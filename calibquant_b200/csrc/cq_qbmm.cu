// Stand-alone quantized vector-matrix product over the group format (M == 1):
//   out[b,h,n] = sum_k fA[b,h,k] * (scale[b,hk,k,n/32]*code[b,hk,k,n] + zero[b,hk,k,n/32])
// Semantics of qjl/csrc/quantization.cu:108-123 of the reference (fp32 dequantise, fp32
// accumulate, round once to the activation dtype), but the packed operand is read once per KV
// head for all of its query heads, in its stored layout (no transposed copies), and 1-bit works.
//
// Work split: thread = output column n, CTA = 128 columns x one chunk of KCHUNK rows of k,
// partial sums land in an fp32 workspace [k_chunks][B*Hq][N]; a second kernel adds the chunks.
// The two shapes the attention path calls the product with (K == 128 with N % 256 == 0, and N == 128
// with K % 256 == 0) run instead on the tensor-core kernels of the decode step (cq_decode_mma.cu),
// where the operand sides round to fp16 before the product (relative error about 2^-11 per term).
#include "cq_common.cuh"
#include "cq_decode_shared.cuh"

namespace cq {

constexpr int QB_NT = 128;      // output columns per CTA
constexpr int QB_KCHUNK = 256;  // reduction rows per CTA

template <typename T, int BITS>
__global__ void __launch_bounds__(QB_NT)
qbmm_partial_kernel(const T* __restrict__ fA, const int32_t* __restrict__ qB,
                    const T* __restrict__ scales, const T* __restrict__ zeros,
                    float* __restrict__ partial, int n_rep, int n_q_rows, int64_t K, int64_t N) {
  constexpr int FPI = 32 / BITS;
  constexpr unsigned MASK = (1u << BITS) - 1u;
  __shared__ float a_s[kMaxRep][QB_KCHUNK];

  const int bhk = blockIdx.z;
  const int64_t k0 = (int64_t)blockIdx.y * QB_KCHUNK;
  const int kn = (int)min((int64_t)QB_KCHUNK, K - k0);
  const int64_t n = (int64_t)blockIdx.x * QB_NT + threadIdx.x;

  for (int i = threadIdx.x; i < n_rep * QB_KCHUNK; i += blockDim.x) {
    const int r = i / QB_KCHUNK, kk = i % QB_KCHUNK;
    a_s[r][kk] = kk < kn ? Elem<T>::to_f(fA[((int64_t)bhk * n_rep + r) * K + k0 + kk]) : 0.f;
  }
  __syncthreads();
  if (n >= N) return;

  const int64_t words_per_row = N / FPI, groups_per_row = N / kGroup;
  const int32_t* wp = qB + ((int64_t)bhk * K + k0) * words_per_row + n / FPI;
  const T* sp = scales + ((int64_t)bhk * K + k0) * groups_per_row + n / kGroup;
  const T* zp = zeros + ((int64_t)bhk * K + k0) * groups_per_row + n / kGroup;
  const int shift = (int)(n % FPI) * BITS;

  float acc[kMaxRep];
#pragma unroll
  for (int r = 0; r < kMaxRep; ++r) acc[r] = 0.f;
  for (int kk = 0; kk < kn; ++kk) {
    const unsigned w = (unsigned)__ldg(wp + (int64_t)kk * words_per_row);
    const float s = Elem<T>::to_f(__ldg(sp + (int64_t)kk * groups_per_row));
    const float z = Elem<T>::to_f(__ldg(zp + (int64_t)kk * groups_per_row));
    const float deq = fmaf(s, (float)((w >> shift) & MASK), z);
#pragma unroll
    for (int r = 0; r < kMaxRep; ++r)
      if (r < n_rep) acc[r] = fmaf(deq, a_s[r][kk], acc[r]);
  }
  for (int r = 0; r < n_rep; ++r)
    partial[((int64_t)blockIdx.y * n_q_rows + (int64_t)bhk * n_rep + r) * N + n] = acc[r];
}

template <typename T>
__global__ void qbmm_finalize_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                     int k_chunks, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int c = 0; c < k_chunks; ++c) s += partial[(int64_t)c * total + i];
  out[i] = Elem<T>::from_f(s);
}

template <typename T>
int launch_qbmm(const void* fA, const int32_t* qB, const void* scales, const void* zeros,
                void* out, int batch, int hq, int hkv, int64_t K, int64_t N, int bits,
                float* ws, cudaStream_t st) {
  const int n_rep = hq / hkv;
  const int k_chunks = (int)((K + QB_KCHUNK - 1) / QB_KCHUNK);
  dim3 grid((unsigned)((N + QB_NT - 1) / QB_NT), (unsigned)k_chunks, (unsigned)(batch * hkv));
  const T* a = static_cast<const T*>(fA);
  const T* s = static_cast<const T*>(scales);
  const T* z = static_cast<const T*>(zeros);
  const int rows = batch * hq;
  switch (bits) {
    case 1: qbmm_partial_kernel<T, 1><<<grid, QB_NT, 0, st>>>(a, qB, s, z, ws, n_rep, rows, K, N); break;
    case 2: qbmm_partial_kernel<T, 2><<<grid, QB_NT, 0, st>>>(a, qB, s, z, ws, n_rep, rows, K, N); break;
    default: qbmm_partial_kernel<T, 4><<<grid, QB_NT, 0, st>>>(a, qB, s, z, ws, n_rep, rows, K, N); break;
  }
  int rc = check_launch();
  if (rc != CQ_OK) return rc;
  const int64_t total = (int64_t)rows * N;
  qbmm_finalize_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(ws, static_cast<T*>(out), k_chunks, total);
  return check_launch();
}

}  // namespace cq

extern "C" size_t cq_qbmm_workspace_bytes(int batch, int n_q_heads, int64_t K, int64_t N) {
  if (batch <= 0 || n_q_heads <= 0 || K <= 0 || N <= 0) return 0;
  const size_t k_chunks = (size_t)((K + cq::QB_KCHUNK - 1) / cq::QB_KCHUNK);
  // [status word, padded to 256 bytes][fp32 partial sums]
  const size_t general = 256 + k_chunks * (size_t)batch * (size_t)n_q_heads * (size_t)N * sizeof(float);
  const size_t fast = cq::mma_qbmm_workspace_bytes(batch, n_q_heads, K, N);
  return general > fast ? general : fast;
}

extern "C" int cq_qbmm(const void* fA, const int32_t* qB, const void* scales, const void* zeros,
                       void* out, int batch, int n_q_heads, int n_kv_heads, int64_t K, int64_t N,
                       int group_size, int bits, int dtype, void* workspace,
                       size_t workspace_bytes, void* stream) {
  if (!fA || !qB || !scales || !zeros || !out) return CQ_ERR_BAD_ARG;
  if (batch < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || K < 0 || N < 0) return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (n_q_heads % n_kv_heads != 0) return CQ_ERR_BAD_ARG;
  if (bits != 1 && bits != 2 && bits != 4) return CQ_ERR_UNSUPPORTED;
  if (group_size != cq::kGroup || N % 32 != 0) return CQ_ERR_UNSUPPORTED;
  if (n_q_heads / n_kv_heads > cq::kMaxRep) return CQ_ERR_UNSUPPORTED;
  if (batch == 0 || N == 0) return CQ_OK;
  if ((int64_t)batch * n_kv_heads > 65535) return CQ_ERR_UNSUPPORTED;
  if (K == 0) {
    cudaError_t e = cudaMemsetAsync(out, 0, (size_t)batch * n_q_heads * N * 2,
                                    static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
  }
  if (!workspace || workspace_bytes < cq_qbmm_workspace_bytes(batch, n_q_heads, K, N))
    return CQ_ERR_WORKSPACE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the two shapes of the attention path run on the tensor-core kernels of the decode step
  const int kind = cq::mma_qbmm_kind(fA, qB, scales, zeros, out, n_q_heads, n_kv_heads, K, N);
  if (kind != 0 && cq::aligned16(workspace))
    return cq::mma_qbmm_run(kind, fA, qB, scales, zeros, out, batch, n_q_heads, n_kv_heads, K, N, bits, dtype,
                            workspace, st);
  float* ws = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + 256);   // after the status word
  if (dtype == CQ_DTYPE_F16)
    return cq::launch_qbmm<__half>(fA, qB, scales, zeros, out, batch, n_q_heads, n_kv_heads, K, N, bits, ws, st);
  return cq::launch_qbmm<__nv_bfloat16>(fA, qB, scales, zeros, out, batch, n_q_heads, n_kv_heads, K, N, bits, ws, st);
}

// ------------------------------------------------------------------------------------------
// Allocation-free variant: the fp32 partial sums live in a fixed array inside the library image.
//
// Who needs it: a serving process that has handed every remaining byte of HBM to its KV-cache
// pool, or that must not stall its other streams, cannot call cudaMalloc in the decode loop
// (the call can fail for lack of memory, and it synchronises the whole device).  Such a caller
// still owns its inputs and outputs; only the scratch is taken off its hands.
//
// Cost: every GPU that loads this library keeps QB_STATIC_BYTES (8 MiB) of device memory until
// the process exits, whether or not this entry point is ever called.
// ------------------------------------------------------------------------------------------
#include <mutex>

namespace cq {

constexpr size_t QB_STATIC_BYTES = (size_t)8 << 20;   // 8 MiB = 2 Mi fp32 partial sums
constexpr int QB_MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char qbmm_static_scratch[QB_STATIC_BYTES];

// In host code `qbmm_static_scratch` is only a handle for the runtime, not a device address,
// so the address is asked for once per device (with that device current) and cached.
static int static_scratch_address(float** out) {
  static std::mutex mu;
  static void* cached[QB_MAX_DEVICES] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= QB_MAX_DEVICES) return CQ_ERR_LAUNCH;
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, qbmm_static_scratch) != cudaSuccess || !p) return CQ_ERR_LAUNCH;
    cached[dev] = p;
  }
  *out = static_cast<float*>(cached[dev]);
  return CQ_OK;
}

}  // namespace cq

extern "C" size_t cq_qbmm_static_capacity_bytes(void) { return cq::QB_STATIC_BYTES; }

extern "C" int cq_qbmm_static_status(void* stream) {
  float* scratch = nullptr;
  const int rc = cq::static_scratch_address(&scratch);
  if (rc != CQ_OK) return rc;
  return cq_workspace_status(scratch, stream);
}

extern "C" int cq_qbmm_static(const void* fA, const int32_t* qB, const void* scales,
                              const void* zeros, void* out, int batch, int n_q_heads,
                              int n_kv_heads, int64_t K, int64_t N, int group_size, int bits,
                              int dtype, void* stream) {
  if (batch > 0 && n_q_heads > 0 && K > 0 && N > 0 &&
      cq_qbmm_workspace_bytes(batch, n_q_heads, K, N) > cq::QB_STATIC_BYTES)
    return CQ_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = cq::static_scratch_address(&scratch);
  if (rc != CQ_OK) return rc;
  return cq_qbmm(fA, qB, scales, zeros, out, batch, n_q_heads, n_kv_heads, K, N, group_size, bits,
                 dtype, scratch, cq::QB_STATIC_BYTES, stream);
}
