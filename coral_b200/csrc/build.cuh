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
// then the isolated nodes' own rows.  Three kernels on `st`.  mode bit 0: candidate distances are
// recomputed instead of taken from d_res_dists (the insert path, src/update.cu:139); bit 1: rows are
// filled with every kept candidate first, then pruned ones (src/update.cu:530-577).
cudaError_t ce_batch(const BuildGraph& g, const int32_t* d_iso_ids, int n_iso, const int32_t* d_res_ids,
                     const float* d_res_dists, int kb, cudaStream_t st, int64_t* launches, int mode = 0);

// ndist and deg of a graph given as adjacency only (every edge distance one sequential chain).
cudaError_t edge_dists(const BuildGraph& g, cudaStream_t st);

// Delete with repair (src/update.cu:674-771).  mark_deleted sets the bits and pos_of[id] = position in
// the id list; innbr_scan counts (fill == nullptr) or fills the deleted nodes' live in-neighbours;
// sort_innbr_lists orders every list ascending and writes the deleted node of every pivot;
// delete_batch repairs one batch of (deleted node, in-neighbour) pivots.  max_degree <= 64.
cudaError_t mark_deleted(const int32_t* d_ids, int count, int64_t n, uint32_t* bits, int32_t* pos_of, cudaStream_t st);
cudaError_t innbr_scan(const BuildGraph& g, const uint32_t* bits, const int32_t* pos_of, int* counts, const int* offsets,
                       int32_t* fill, cudaStream_t st);
cudaError_t sort_innbr_lists(int32_t* lists, const int* offsets, int n_lists, int32_t* piv_del, const int32_t* d_del_ids,
                             cudaStream_t st);
cudaError_t delete_batch(const BuildGraph& g, const uint32_t* bits, const int32_t* piv_del, const int32_t* piv_in, int n_piv,
                         cudaStream_t st, int64_t* launches);

// out[r] = vecs[d_ids[r]] for r < count.
cudaError_t gather_rows(const float* vecs, const int32_t* d_ids, int count, int dim, float* out, cudaStream_t st);

}  // namespace coral
