// One-shot all-reduce / all-gather for the tensor-parallel decode step, over peer memory on NVLink.
//
// A decode step of a model sharded over G GPUs (one process per GPU) ends each sharded block with a
// [batch, hidden] partial sum per rank that every rank needs the total of: 128 KB at batch 16, far too
// small for a bandwidth-oriented collective.  Here every rank owns a receive buffer that its peers can
// write (CUDA IPC), and the collective is two halves that ride on kernels the step runs anyway:
//   push   : the producer copies its partial into slot `rank` of every rank's buffer with plain stores
//            over NVLink, fences, and stores the collective's sequence number into a flag word there;
//   reduce : the consumer -- the residual-add + RMSNorm kernel that follows, or a plain gather --
//            polls its own flag words until all G carry the sequence number, then sums the G slots.
// cq_comm_allreduce_add_rmsnorm does both halves in one launch, row by row (a CTA pushes its row, then waits
// for the same row of every peer), which saves a launch and a grid-wide hand-over per collective.
// Buffers are double-buffered on the parity of the sequence number: a rank can run at most one collective
// ahead of a peer (its reduce of collective c needs the peer's push of c, which follows the peer's reduce
// of c-1 in stream order), so slot c+1 never overwrites data a peer still reads.  The sequence number
// lives in the buffer itself and advances on the device, so a captured CUDA graph replays the step.
// Every poll is bounded by the global timer; a timeout stores CQ_ERR_TIMEOUT in the status word of the
// buffer and the kernel returns without touching its outputs.  No multicast loads, no multimem.
#include <string.h>

#include "cq_common.cuh"

namespace cq {
namespace comm {

constexpr int MAX_WORLD = 8;
constexpr int MAX_ROWS = 64;           // rows of a fused all-reduce (one flag word per row, rank and parity)
constexpr size_t FLAGS_OFF = 0;        // uint32 flags[2][MAX_ROWS][MAX_WORLD]: sequence number of the data in slot
                                       // [parity][rank], per row for the fused all-reduce, row 0 for push / gather
constexpr size_t CTRL_OFF = 4096;      // uint32 {sequence, done ticket, status, pad, push tickets[MAX_WORLD]}
constexpr size_t DATA_OFF = 4096 + 256;   // [2][world][slot_bytes]
constexpr unsigned long long WAIT_NS = 2000000000ull;   // give up on a peer after two seconds

struct Peers {
  unsigned char* base[MAX_WORLD];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// grid (chunks, world): CTA (x, p) copies chunk x of `src` into this rank's slot of peer p's buffer; the
// last CTA of a peer to finish publishes the flag (with one chunk per peer no ticket is needed).
__global__ void __launch_bounds__(1024)
push_kernel(const uint4* __restrict__ src, int n16, Peers peers, int rank, int world, size_t slot_bytes) {
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(peers.base[rank] + CTRL_OFF);
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(ctrl);
  const int p = blockIdx.y;
  uint4* dst = reinterpret_cast<uint4*>(peers.base[p] + DATA_OFF + ((size_t)(seq & 1u) * world + rank) * slot_bytes);
  uint32_t* flag = reinterpret_cast<uint32_t*>(peers.base[p] + FLAGS_OFF) + (seq & 1u) * (MAX_ROWS * MAX_WORLD) + rank;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) dst[i] = src[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    if (gridDim.x == 1) {
      st_release_sys(flag, seq);          // orders the CTA's stores (seen through the barrier) before the flag
    } else {
      __threadfence_system();
      const uint32_t old = atomicAdd(&ctrl[4 + p], 1u);
      if (old == gridDim.x - 1) {
        ctrl[4 + p] = 0u;
        st_release_sys(flag, seq);
      }
    }
  }
}

// Wait until all `world` slots of the current collective have landed in this rank's buffer.  Called by the
// first `world` threads of a CTA; returns false on a timeout (after recording it).
__device__ __forceinline__ bool wait_slot(unsigned char* base, uint32_t seq, int q, int row = 0) {
  const uint32_t* flag = reinterpret_cast<const uint32_t*>(base + FLAGS_OFF) + ((seq & 1u) * MAX_ROWS + row) * MAX_WORLD + q;
  if (ld_acquire_sys(flag) == seq) return true;
  if (*(reinterpret_cast<volatile int*>(base + CTRL_OFF) + 2) != 0) return false;   // an earlier wait already gave up
  const unsigned long long t0 = global_ns();
  for (;;) {
    if (ld_acquire_sys(flag) == seq) return true;
    if (global_ns() - t0 > WAIT_NS) {
      atomicExch(reinterpret_cast<int*>(base + CTRL_OFF) + 2, CQ_ERR_TIMEOUT);
      return false;
    }
    __nanosleep(100);
  }
}

// The last CTA of a consumer kernel to finish advances the sequence number.
__device__ __forceinline__ void finish_collective(unsigned char* base, uint32_t seq) {
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(base + CTRL_OFF);
  __threadfence();
  const uint32_t old = atomicAdd(&ctrl[1], 1u);
  if (old == gridDim.x - 1) {
    ctrl[1] = 0u;
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(ctrl) = seq + 1u;
  }
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_VEC = 8;
constexpr int NORM_MAXV = 8;

// residual += sum over ranks of the pushed partial rows (fp32 sum, one rounding), then RMSNorm as
// cq_add_rmsnorm: out = weight * (r_fp32 * rsqrt(mean(r^2) + eps)).to(dtype).  One CTA per row.
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
reduce_add_rmsnorm_kernel(unsigned char* base, int world, size_t slot_bytes, T* __restrict__ residual,
                          const T* __restrict__ weight, T* __restrict__ out, int hidden, float eps) {
  __shared__ int ok_s;
  __shared__ float part[NORM_THREADS / 32];
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(base + CTRL_OFF);
  const int tid = threadIdx.x;
  if (tid == 0) ok_s = 1;
  __syncthreads();
  if (tid < world && !wait_slot(base, seq, tid)) ok_s = 0;
  __syncthreads();
  if (!ok_s) return;
  const int64_t row = blockIdx.x;
  const int n_vec = hidden / NORM_VEC;
  T* res = residual + row * hidden;
  const unsigned char* slots = base + DATA_OFF + (size_t)(seq & 1u) * world * slot_bytes;
  float v[NORM_MAXV][NORM_VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int iv = tid + k * NORM_THREADS;
    if (iv < n_vec) {
      float acc[NORM_VEC];
#pragma unroll
      for (int e = 0; e < NORM_VEC; ++e) acc[e] = 0.f;
      for (int q = 0; q < world; ++q) {
        const uint4 draw = *reinterpret_cast<const uint4*>(slots + q * slot_bytes + (row * hidden + iv * NORM_VEC) * sizeof(T));
        const T* d = reinterpret_cast<const T*>(&draw);
#pragma unroll
        for (int e = 0; e < NORM_VEC; ++e) acc[e] += Elem<T>::to_f(d[e]);
      }
      const uint4 raw = *reinterpret_cast<const uint4*>(res + iv * NORM_VEC);
      const T* r = reinterpret_cast<const T*>(&raw);
      uint4 sum;
      T* s = reinterpret_cast<T*>(&sum);
#pragma unroll
      for (int e = 0; e < NORM_VEC; ++e) {
        s[e] = Elem<T>::from_f(Elem<T>::to_f(r[e]) + acc[e]);
        v[k][e] = Elem<T>::to_f(s[e]);
        ss = fmaf(v[k][e], v[k][e], ss);
      }
      *reinterpret_cast<uint4*>(res + iv * NORM_VEC) = sum;
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) part[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NORM_THREADS / 32; ++w) tot += part[w];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  if (out) {
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
        for (int e = 0; e < NORM_VEC; ++e) r[e] = Elem<T>::from_f(Elem<T>::to_f(w[e]) * rnd<T>(v[k][e] * inv));
        *reinterpret_cast<uint4*>(o + iv * NORM_VEC) = res4;
      }
    }
  }
  __syncthreads();
  if (tid == 0) finish_collective(base, seq);
}

// The whole collective in one launch: CTA = row.  The CTA stores its row of this rank's partial into slot
// `rank` of every peer's buffer and publishes the row's flag there, waits for the same row of every peer in
// its own buffer, then residual += sum over the ranks (in rank order on every rank, so all ranks hold the same
// bits; this rank's own term comes straight from `src`) and RMSNorm as above.
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
allreduce_add_rmsnorm_kernel(const T* __restrict__ src, Peers peers, int rank, int world, size_t slot_bytes,
                             T* __restrict__ residual, const T* __restrict__ weight, T* __restrict__ out,
                             int hidden, float eps) {
  __shared__ int ok_s;
  __shared__ float part[NORM_THREADS / 32];
  unsigned char* base = peers.base[rank];
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(base + CTRL_OFF);
  const int tid = threadIdx.x;
  const int row = blockIdx.x;
  const int n_vec = hidden / NORM_VEC;
  const size_t row_off = (size_t)row * hidden * sizeof(T);
  const uint4* srow = reinterpret_cast<const uint4*>(src + (size_t)row * hidden);
  if (tid == 0) ok_s = 1;
  // ---- this rank's row to every peer
  for (int i = tid; i < (world - 1) * n_vec; i += NORM_THREADS) {
    const int pi = i / n_vec, iv = i % n_vec;
    const int p = pi + (pi >= rank ? 1 : 0);
    reinterpret_cast<uint4*>(peers.base[p] + DATA_OFF + ((size_t)(seq & 1u) * world + rank) * slot_bytes + row_off)[iv] = srow[iv];
  }
  __syncthreads();
  if (tid < world && tid != rank)
    st_release_sys(reinterpret_cast<uint32_t*>(peers.base[tid] + FLAGS_OFF) + ((seq & 1u) * MAX_ROWS + row) * MAX_WORLD + rank, seq);
  // ---- the peers' rows
  if (tid < world && tid != rank && !wait_slot(base, seq, tid, row)) ok_s = 0;
  __syncthreads();
  if (!ok_s) return;
  T* res = residual + (size_t)row * hidden;
  const unsigned char* slots = base + DATA_OFF + (size_t)(seq & 1u) * world * slot_bytes + row_off;
  float v[NORM_MAXV][NORM_VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NORM_MAXV; ++k) {
    const int iv = tid + k * NORM_THREADS;
    if (iv < n_vec) {
      float acc[NORM_VEC];
#pragma unroll
      for (int e = 0; e < NORM_VEC; ++e) acc[e] = 0.f;
      for (int q = 0; q < world; ++q) {
        const uint4 draw = q == rank ? srow[iv] : *reinterpret_cast<const uint4*>(slots + q * slot_bytes + (size_t)iv * 16);
        const T* d = reinterpret_cast<const T*>(&draw);
#pragma unroll
        for (int e = 0; e < NORM_VEC; ++e) acc[e] += Elem<T>::to_f(d[e]);
      }
      const uint4 raw = *reinterpret_cast<const uint4*>(res + iv * NORM_VEC);
      const T* r = reinterpret_cast<const T*>(&raw);
      uint4 sum;
      T* sm = reinterpret_cast<T*>(&sum);
#pragma unroll
      for (int e = 0; e < NORM_VEC; ++e) {
        sm[e] = Elem<T>::from_f(Elem<T>::to_f(r[e]) + acc[e]);
        v[k][e] = Elem<T>::to_f(sm[e]);
        ss = fmaf(v[k][e], v[k][e], ss);
      }
      *reinterpret_cast<uint4*>(res + iv * NORM_VEC) = sum;
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) part[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < NORM_THREADS / 32; ++w) tot += part[w];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  if (out) {
    T* o = out + (size_t)row * hidden;
#pragma unroll
    for (int k = 0; k < NORM_MAXV; ++k) {
      const int iv = tid + k * NORM_THREADS;
      if (iv < n_vec) {
        const uint4 wraw = *reinterpret_cast<const uint4*>(weight + iv * NORM_VEC);
        const T* w = reinterpret_cast<const T*>(&wraw);
        uint4 res4;
        T* r = reinterpret_cast<T*>(&res4);
#pragma unroll
        for (int e = 0; e < NORM_VEC; ++e) r[e] = Elem<T>::from_f(Elem<T>::to_f(w[e]) * rnd<T>(v[k][e] * inv));
        *reinterpret_cast<uint4*>(o + iv * NORM_VEC) = res4;
      }
    }
  }
  __syncthreads();
  if (tid == 0) finish_collective(base, seq);
}

// out[q][:] = slot q, for all ranks q: the all-gather of the pushed rows.
__global__ void __launch_bounds__(256)
gather_kernel(unsigned char* base, int world, size_t slot_bytes, uint4* __restrict__ out, int n16) {
  __shared__ int ok_s;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(base + CTRL_OFF);
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < world && !wait_slot(base, seq, threadIdx.x)) ok_s = 0;
  __syncthreads();
  if (!ok_s) return;
  const unsigned char* slots = base + DATA_OFF + (size_t)(seq & 1u) * world * slot_bytes;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < world * n16; i += gridDim.x * blockDim.x) {
    const int q = i / n16, j = i % n16;
    out[i] = *reinterpret_cast<const uint4*>(slots + q * slot_bytes + (size_t)j * 16);
  }
  __syncthreads();
  if (threadIdx.x == 0) finish_collective(base, seq);
}

static bool fill_peers(Peers* p, void* const* peer_buffers, int rank, int world) {
  if (!peer_buffers || world < 1 || world > MAX_WORLD || rank < 0 || rank >= world) return false;
  for (int i = 0; i < MAX_WORLD; ++i) p->base[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    if (!peer_buffers[i] || (reinterpret_cast<uintptr_t>(peer_buffers[i]) & 255u)) return false;
    p->base[i] = static_cast<unsigned char*>(peer_buffers[i]);
  }
  return true;
}

}  // namespace comm
}  // namespace cq

using namespace cq;

extern "C" size_t cq_comm_buffer_bytes(int world, size_t slot_bytes) {
  if (world < 1 || world > comm::MAX_WORLD) return 0;
  return comm::DATA_OFF + 2 * (size_t)world * align_up(slot_bytes, 256);
}

extern "C" int cq_comm_alloc(size_t bytes, void** buffer, void* ipc_handle) {
  if (!buffer || !ipc_handle || bytes < comm::DATA_OFF) return CQ_ERR_BAD_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return CQ_ERR_LAUNCH;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return CQ_ERR_LAUNCH; }
  const uint32_t one = 1u;        // sequence numbers start at 1: a zeroed flag never matches
  if (cudaMemcpy(static_cast<unsigned char*>(p) + comm::CTRL_OFF, &one, sizeof(one), cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(ipc_handle), p) != cudaSuccess) {
    cudaFree(p);
    return CQ_ERR_LAUNCH;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  *buffer = p;
  return CQ_OK;
}

extern "C" int cq_comm_open(const void* ipc_handle, void** buffer) {
  if (!ipc_handle || !buffer) return CQ_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  return cudaIpcOpenMemHandle(buffer, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_comm_close(void* buffer) {
  return buffer && cudaIpcCloseMemHandle(buffer) == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

extern "C" int cq_comm_free(void* buffer) { return buffer && cudaFree(buffer) == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH; }

extern "C" int cq_comm_status(const void* buffer, void* stream) {
  if (!buffer) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int word = 0;
  if (cudaMemcpyAsync(&word, static_cast<const unsigned char*>(buffer) + comm::CTRL_OFF + 8, sizeof(int),
                      cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return CQ_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return CQ_ERR_LAUNCH;
  return word == 0 ? CQ_OK : CQ_ERR_TIMEOUT;
}

extern "C" int cq_comm_push(const void* src, size_t bytes, void* const* peer_buffers, int rank, int world,
                            size_t slot_bytes, void* stream) {
  comm::Peers peers;
  if (!src || !comm::fill_peers(&peers, peer_buffers, rank, world)) return CQ_ERR_BAD_ARG;
  slot_bytes = align_up(slot_bytes, 256);
  if (bytes == 0 || bytes % 16 || bytes > slot_bytes || !aligned16(src)) return CQ_ERR_BAD_ARG;
  const int n16 = (int)(bytes / 16);
  const int chunks = n16 > 16384 ? (n16 + 16383) / 16384 : 1;      // one CTA of 1024 threads per 256 KB and peer
  const int threads = n16 >= 1024 ? 1024 : (n16 + 31) / 32 * 32;
  comm::push_kernel<<<dim3(chunks, world), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), n16, peers, rank, world, slot_bytes);
  return check_launch();
}

extern "C" int cq_comm_reduce_add_rmsnorm(void* buffer, int world, size_t slot_bytes, void* residual,
                                          const void* weight, void* out, int64_t rows, int hidden, float eps,
                                          int dtype, void* stream) {
  if (!buffer || !residual || world < 1 || world > comm::MAX_WORLD || rows <= 0 || hidden <= 0 || (out && !weight))
    return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (hidden % comm::NORM_VEC || hidden > comm::NORM_THREADS * comm::NORM_VEC * comm::NORM_MAXV) return CQ_ERR_UNSUPPORTED;
  slot_bytes = align_up(slot_bytes, 256);
  if ((size_t)rows * hidden * 2 > slot_bytes || rows > 0x7fffffff) return CQ_ERR_BAD_ARG;
  if (!aligned16(residual) || !aligned16(weight) || !aligned16(out)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* base = static_cast<unsigned char*>(buffer);
  if (dtype == CQ_DTYPE_F16)
    comm::reduce_add_rmsnorm_kernel<__half><<<(unsigned)rows, comm::NORM_THREADS, 0, st>>>(
        base, world, slot_bytes, static_cast<__half*>(residual), static_cast<const __half*>(weight),
        static_cast<__half*>(out), hidden, eps);
  else
    comm::reduce_add_rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, comm::NORM_THREADS, 0, st>>>(
        base, world, slot_bytes, static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight),
        static_cast<__nv_bfloat16*>(out), hidden, eps);
  return check_launch();
}

extern "C" int cq_comm_gather(void* buffer, int world, size_t slot_bytes, void* out, size_t bytes, void* stream) {
  if (!buffer || !out || world < 1 || world > comm::MAX_WORLD) return CQ_ERR_BAD_ARG;
  slot_bytes = align_up(slot_bytes, 256);
  if (bytes == 0 || bytes % 16 || bytes > slot_bytes || !aligned16(out)) return CQ_ERR_BAD_ARG;
  const int n16 = (int)(bytes / 16);
  const int grid = (world * n16 + 255) / 256 < 32 ? (world * n16 + 255) / 256 : 32;
  comm::gather_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned char*>(buffer), world, slot_bytes, static_cast<uint4*>(out), n16);
  return check_launch();
}

extern "C" int cq_comm_allreduce_add_rmsnorm(const void* src, void* const* peer_buffers, int rank, int world,
                                             size_t slot_bytes, void* residual, const void* weight, void* out,
                                             int64_t rows, int hidden, float eps, int dtype, void* stream) {
  comm::Peers peers;
  if (!src || !residual || !comm::fill_peers(&peers, peer_buffers, rank, world) || rows <= 0 || hidden <= 0 ||
      (out && !weight))
    return CQ_ERR_BAD_ARG;
  if (dtype != CQ_DTYPE_F16 && dtype != CQ_DTYPE_BF16) return CQ_ERR_BAD_ARG;
  if (hidden % comm::NORM_VEC || hidden > comm::NORM_THREADS * comm::NORM_VEC * comm::NORM_MAXV) return CQ_ERR_UNSUPPORTED;
  if (rows > comm::MAX_ROWS) return CQ_ERR_UNSUPPORTED;
  slot_bytes = align_up(slot_bytes, 256);
  if ((size_t)rows * hidden * 2 > slot_bytes) return CQ_ERR_BAD_ARG;
  if (!aligned16(src) || !aligned16(residual) || !aligned16(weight) || !aligned16(out)) return CQ_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CQ_DTYPE_F16)
    comm::allreduce_add_rmsnorm_kernel<__half><<<(unsigned)rows, comm::NORM_THREADS, 0, st>>>(
        static_cast<const __half*>(src), peers, rank, world, slot_bytes, static_cast<__half*>(residual),
        static_cast<const __half*>(weight), static_cast<__half*>(out), hidden, eps);
  else
    comm::allreduce_add_rmsnorm_kernel<__nv_bfloat16><<<(unsigned)rows, comm::NORM_THREADS, 0, st>>>(
        static_cast<const __nv_bfloat16*>(src), peers, rank, world, slot_bytes, static_cast<__nv_bfloat16*>(residual),
        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), hidden, eps);
  return check_launch();
}
