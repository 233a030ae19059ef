// Graph build kernels: neighbourhood-aware projection and connectivity enhancement (see build.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace coral {

// The graph under construction.  adj doubles as the search adjacency (valid ids first, -1 padding);
// ndist holds the distance of every stored edge (the reference's Slot::dists, include/disk_graph.h:34);
// rows are kept closest-first.  claim[n] is scratch for the lowest-index-wins rules (all 0x7f bytes
// between batches).
struct BuildGraph {
    const float* vecs = nullptr;
    int32_t* adj = nullptr;
    float* ndist = nullptr;
    int32_t* deg = nullptr;
    uint32_t* claim = nullptr;
    int64_t n = 0;
    int dim = 0, deg_pad = 0, max_degree = 0, metric = 0;
};

// Scratch of one nap_batch call: the lists' distance matrices and the staged rows.
size_t nap_scratch_bytes(int batch, int kb, int max_degree);

// One batch of B lists of kb base ids (device): four kernels on `st`.
cudaError_t nap_batch(const BuildGraph& g, const int32_t* d_lists, int B, int kb, void* scratch, cudaStream_t st,
                      int64_t* launches);

// One batch of n_iso isolated nodes with their kb search results (ids < 0 = padding): reverse edges,
// then the isolated nodes' own rows.  Three kernels on `st`.
cudaError_t ce_batch(const BuildGraph& g, const int32_t* d_iso_ids, int n_iso, const int32_t* d_res_ids,
                     const float* d_res_dists, int kb, cudaStream_t st, int64_t* launches);

// out[r] = vecs[d_ids[r]] for r < count.
cudaError_t gather_rows(const float* vecs, const int32_t* d_ids, int count, int dim, float* out, cudaStream_t st);

}  // namespace coral
