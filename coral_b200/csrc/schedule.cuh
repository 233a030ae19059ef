// Query scheduling pre-pass (see schedule.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace coral {

// Copies the frontier rows vecs[d_ids[f]] into fvecs[F][dim] and their squared norms into fnorm[F].
cudaError_t gather_frontier(const float* vecs, const int32_t* d_ids, int F, int dim, float* fvecs, float* fnorm,
                            cudaStream_t stream);

// d_order[0..Q) <- the queries grouped by their best frontier node (d_keys[Q] and d_bins[F] are scratch).
// Four kernels on `stream`, no synchronisation.
cudaError_t schedule_queries(const float* d_queries, int Q, int dim, int metric, const float* fvecs, const float* fnorm,
                             int F, int* d_keys, int* d_bins, int32_t* d_order, int sm_count, cudaStream_t stream);

}  // namespace coral
