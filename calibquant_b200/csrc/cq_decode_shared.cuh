// Interface between the decode entry point (cq_decode.cu) and the tensor-core fast path
// (cq_decode_mma.cu).
#pragma once

#include "cq_common.cuh"

namespace cq {

// True when the fast path implements this request (t_vis % 256 == 0, 16-byte aligned operands).
bool mma_path_eligible(const cq_decode_args* args);
size_t mma_path_workspace_bytes(const cq_decode_args* args);
// The first 4 bytes of `workspace` are a sticky device status word (CQ_ERR_TIMEOUT when a bounded
// wait ran out); the caller zeroes the workspace once after allocating it.
// `events`, when given, are five events recorded before the first launch and after each of the four
// launches (scores, attn.V, attn.V of the full-precision tokens, combine).
// `status_word`, when given, replaces the workspace's first word as the place a timed-out wait is reported
// (a device-visible address, e.g. mapped page-locked host memory).
int mma_path_run(const cq_decode_args* args, void* workspace, cudaStream_t stream, cudaEvent_t* events = nullptr,
                 int* status_word = nullptr);


// The stand-alone quantized product (cq_qbmm) on the same kernels.  mma_qbmm_kind returns 0 when the
// shapes or pointers are not ones the fast kernels take, 1 for the "q.K" use (K == 128) and 2 for the
// "att.V" use (N == 128); workspace as mma_qbmm_workspace_bytes says, its first word a status word.
int mma_qbmm_kind(const void* fA, const void* qB, const void* scales, const void* zeros, const void* out,
                  int n_q_heads, int n_kv_heads, int64_t K, int64_t N);
size_t mma_qbmm_workspace_bytes(int batch, int n_q_heads, int64_t K, int64_t N);
int mma_qbmm_run(int kind, const void* fA, const int32_t* qB, const void* scales, const void* zeros, void* out,
                 int batch, int n_q_heads, int n_kv_heads, int64_t K, int64_t N, int bits, int dtype,
                 void* workspace, cudaStream_t stream);

}  // namespace cq
