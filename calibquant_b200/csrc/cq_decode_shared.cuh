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
int mma_path_run(const cq_decode_args* args, void* workspace, cudaStream_t stream);

}  // namespace cq
