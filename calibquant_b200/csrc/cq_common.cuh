// Shared device/host helpers for the calibquant_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/calibquant_b200.h"

#ifndef __CUDA_ARCH__
#define CQ_HOST_ONLY 1
#endif

namespace cq {

constexpr int kHeadDim = 128;
constexpr int kGroup = 32;
constexpr int kMaxRep = 8;  // query heads per KV head supported by the kernels

// ---- element-type traits -------------------------------------------------------------
// The reference computes in fp16/bf16 tensors whose every torch op is "compute in fp32,
// round to the tensor dtype".  rnd() is that rounding step.
template <typename T>
struct Elem;

template <>
struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__half2 v) { return __half22float2(v); }
  static __device__ __forceinline__ float lowest() { return -65504.f; }
};

template <>
struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 v) { return __bfloat1622float2(v); }
  static __device__ __forceinline__ float lowest() { return -3.3895313892515355e38f; }
};

template <typename T>
__device__ __forceinline__ float rnd(float v) {
  return Elem<T>::to_f(Elem<T>::from_f(v));
}

// ---- warp helpers ------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- host helpers ----------------------------------------------------------------------
inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? CQ_OK : CQ_ERR_LAUNCH;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace cq
