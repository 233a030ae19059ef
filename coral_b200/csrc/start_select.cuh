// Entry-point selection (see start_select.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace coral {

// Writes M entry points to h_out (host): h_out[0] = first, then farthest-point sampling over BFS
// hop counts.  Allocates and frees its own scratch (16 bytes per node); synchronises `stream`.
cudaError_t select_start_ids(const int32_t* d_adj, int64_t n, int deg_pad, int first, int M, int32_t* h_out,
                             int sm_count, cudaStream_t stream, int64_t* launches);

}  // namespace coral
