// Query scheduling pre-pass (see schedule.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace coral {

// Copies the frontier rows vecs[d_ids[f]] into fvecs[F][dim] and their squared norms into fnorm[F].
cudaError_t gather_frontier(const float* vecs, const int32_t* d_ids, int F, int dim, float* fvecs, float* fnorm,
                            cudaStream_t stream);

// keys[q] = the frontier row closest to query q, by fp32 SIMT tiles (one kernel).
cudaError_t frontier_keys_simt(const float* d_queries, int Q, int dim, int metric, const float* fvecs, const float* fnorm,
                               int F, int* d_keys, cudaStream_t stream);

// keys[q] = ids[q * stride] clamped to [0, F) (takes the first column of a k-NN result).
cudaError_t keys_from_ids(const int32_t* d_ids, int Q, int stride, int F, int* d_keys, int sm_count, cudaStream_t stream);

// d_order[0..Q) <- the queries sorted by key, equal keys in query order (deterministic).  d_bins[F] and
// d_scratch[sort_scratch_ints(Q, F)] are scratch.  Four kernels on `stream`, no synchronisation.
size_t sort_scratch_ints(int Q, int F);
cudaError_t sort_queries_by_key(const int* d_keys, int Q, int F, int* d_bins, int* d_scratch, int32_t* d_order,
                                int sm_count, cudaStream_t stream);

}  // namespace coral
