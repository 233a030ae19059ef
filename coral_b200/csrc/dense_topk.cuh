// Dense scores on the 5th-generation tensor cores with a fused per-row top-k' selection, and the
// exact fp32 re-rank that turns the selection into exact nearest neighbours (see dense_topk.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace coral {

constexpr int kDenseTileM = 128;   // query rows per CTA tile (= TMEM lanes)
constexpr int kDenseTileN = 256;   // base rows per accumulator tile (= TMEM columns per buffer)
constexpr int kDenseTileK = 32;    // floats per k-block: one 128-byte swizzle row
constexpr int kDenseRowCap = 512;  // candidate keys a (query, split) pair can hold between compactions
constexpr int kDenseMaxKeep = 256; // largest k' (= kDenseRowCap - kDenseTileN)
constexpr int kDenseMaxSplit = 32;

// Workspace of one dense_knn call sequence; sized by dense_workspace_bytes and carved by the caller.
struct DenseWorkspace {
    float* a_split = nullptr;      // [2][q_cap][dim]: queries split into tf32 high and low parts
    float* b_split = nullptr;      // [2][b_cap][dim]: one chunk of base rows, same split
    float* b_norm = nullptr;       // [b_cap]: squared norms of the chunk's rows (L2 only)
    uint64_t* keys = nullptr;      // [q_cap * n_split][kDenseRowCap]
    int32_t* cnt = nullptr;        // [q_cap * n_split]
    float* thr = nullptr;          // [q_cap * n_split]
    int* err = nullptr;            // [4]: bounded-wait flag, uncertified count, ...
    int q_cap = 0, b_cap = 0, n_split = 1;
};

size_t dense_workspace_bytes(int q_cap, int b_cap, int dim, int n_split);
void dense_workspace_carve(void* base, int q_cap, int b_cap, int dim, int n_split, DenseWorkspace& w);

// One pass over `n_rows` base rows starting at global row `row0` (vecs points at row0) for the Q
// queries whose split form is already in w.a_split: the approximate scores (inner product, or
// 2 q.b - |b|^2 for L2; larger = closer) of every (query, row) pair are formed on the tensor cores
// in `passes` tf32 passes (1: plain tf32; 3: high*high + high*low + low*high, fp32-grade) and the
// keep best of every query are retained in the workspace.  Several calls accumulate over chunks.
cudaError_t dense_scan_chunk(const DenseWorkspace& w, const float* d_queries_unused, int Q, const float* d_vecs,
                             int64_t row0, int n_rows, int dim, int metric, int passes, int keep, int sm_count,
                             cudaStream_t stream, int64_t* launches);

// Splits Q query rows into w.a_split and resets the per-(query, split) selection state.
cudaError_t dense_begin(const DenseWorkspace& w, const float* d_queries, int Q, int dim, cudaStream_t stream,
                        int64_t* launches);

// Merges the splits, re-ranks the keep best of every query with the exact fp32 distance in the
// reference's sequential order (include/utils.cuh:254-275,:307-323) against `d_vecs` (the whole base,
// row 0 first), and writes the k closest by (distance, id).  certified_out[q] (nullable) = 1 when the
// exact k-th distance beats the best score any unselected row can have.
cudaError_t dense_finish(const DenseWorkspace& w, const float* d_queries, int Q, const float* d_vecs, int dim,
                         int metric, int passes, int keep, int k, int32_t* d_ids_out, float* d_dists_out,
                         int32_t* d_certified_out, cudaStream_t stream, int64_t* launches);

}  // namespace coral
