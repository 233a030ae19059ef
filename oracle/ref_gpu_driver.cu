// REFERENCE-KERNEL HARNESS (test infrastructure, not product code).
//
// Calls the reference's own GPUFuncs::search_gpu (src/search_gpu.cu:835-886) -- and through it the
// reference's beam_search_kernel (bitset overload, src/search_gpu.cu:347-580) with the reference's
// distance functions, BP, Slot and BCD types (include/utils.cuh, include/uni.h,
// include/disk_graph.h) -- all compiled unmodified from the reference tree by oracle/Makefile.
// What this file adds is what the reference does around that call in code that cannot be built
// here (it needs Faiss and a header the reference does not ship): the Slot upload of Graph::Graph
// (include/graph.cuh:240-261), the scratch of Search_Data (include/gpufuncs.cuh:557-564) and the
// BP fields set by GPUFuncs::search_prepare (src/search.cu:400-402).
//
// Only the overload without the deleted bitset is driven.  The overload with it
// (src/search_gpu.cu:582-833) loops `while (s_i < k)` with no bound and reads sh_beams[-1] once
// the beam runs out of live entries, so it is not run on a shared GPU.
//
// The reference kernel reads out of range in release builds when a query reaches fewer than
// beam_capacity nodes (src/search_gpu.cu:444, :466-467): callers must only pass cases whose every
// query fills its beam (the CPU oracle reports that per query).
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <vector>

#include "gpufuncs.cuh"

using namespace efanna2e;

namespace {
struct Cleanup {
    std::vector<void*> dev;
    cudaStream_t stream = nullptr;
    ~Cleanup() {
        for (void* p : dev) cudaFree(p);
        if (stream) cudaStreamDestroy(stream);
    }
    template <typename T>
    bool alloc(T** p, size_t bytes) {
        if (cudaMalloc(p, bytes) != cudaSuccess) return false;
        dev.push_back(*p);
        return true;
    }
};
}  // namespace

// The index as the reference holds it on the device: Slot records and the row array.
struct coral_ref_gpu {
    Cleanup c;
    Slot* d_slots = nullptr;
    float* d_vecs = nullptr;
    int64_t n = 0;
    int dim = 0, max_degree = 0, metric = 0;
    std::vector<int> starts;
};

// adj: [n][deg_pad] int32, valid ids first, -1 padding.  metric: 0 = L2, 1 = IP.
// Uploads the graph and the vectors once; returns nullptr on failure.
extern "C" coral_ref_gpu* coral_ref_gpu_open(const float* h_vecs, int64_t n, int dim, const int32_t* adj, int deg_pad,
                                             int max_degree, int metric, const int32_t* start_ids, int M) {
    if (!h_vecs || !adj || !start_ids || n <= 0 || M <= 0) return nullptr;
    if (max_degree > 64 || max_degree > deg_pad) return nullptr;  // Slot::nbrs has 64 entries (include/disk_graph.h:33)
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return nullptr;
    coral_ref_gpu* r = new coral_ref_gpu;
    if (cudaStreamCreate(&r->c.stream) != cudaSuccess) {
        delete r;
        return nullptr;
    }
    std::vector<Slot> slots((size_t)n);
    for (int64_t i = 0; i < n; ++i) {
        Slot& s = slots[(size_t)i];
        std::memset(&s, 0, sizeof(Slot));
        s.node_id = (int)i;
        int deg = 0;
        for (int j = 0; j < max_degree; ++j) {
            const int v = adj[(size_t)i * deg_pad + j];
            if (v < 0) break;
            s.nbrs[deg++] = v;
        }
        s.deg = deg;
    }
    if (!r->c.alloc(&r->d_slots, slots.size() * sizeof(Slot)) || !r->c.alloc(&r->d_vecs, (size_t)n * dim * sizeof(float)) ||
        cudaMemcpy(r->d_slots, slots.data(), slots.size() * sizeof(Slot), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(r->d_vecs, h_vecs, (size_t)n * dim * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
        delete r;
        return nullptr;
    }
    r->n = n;
    r->dim = dim;
    r->max_degree = max_degree;
    r->metric = metric;
    r->starts.assign(start_ids, start_ids + M);
    return r;
}

extern "C" void coral_ref_gpu_close(coral_ref_gpu* r) { delete r; }

// One call of the reference's GPUFuncs::search_gpu with its own scratch (Search_Data) sized for the
// batch, as GPUFuncs::search_prepare does.  Returns 0 on success; ids_out [Q][k], dists_out [Q][k]
// (may be null), total hops and the reference's timed window in seconds.
extern "C" int coral_ref_gpu_run(coral_ref_gpu* r, const float* h_queries, int Q, int L, int k, int32_t* ids_out,
                                 float* dists_out, int64_t* total_hops_out, double* seconds_out) {
    if (!r || !h_queries || !ids_out || Q <= 0 || k <= 0 || k > L) return -1;
    Cleanup c;   // per-call scratch; the stream stays with the handle
    float *d_queries = nullptr, *d_dists = nullptr;
    int* d_ids = nullptr;
    if (!c.alloc(&d_queries, (size_t)Q * r->dim * sizeof(float)) || !c.alloc(&d_ids, (size_t)Q * k * sizeof(int)) ||
        !c.alloc(&d_dists, (size_t)Q * k * sizeof(float)))
        return -5;
    cudaMemcpy(d_queries, h_queries, (size_t)Q * r->dim * sizeof(float), cudaMemcpyHostToDevice);

    GPUFuncs f;
    f.bp = BP(r->dim, r->max_degree, (int)r->n, Q, k, L, r->metric == 0 ? DIST_METRIC::L2_ : DIST_METRIC::IP_);
    f.bp.beam_capacity = L;                       // src/search.cu:401
    f.bp.beam_size = L * r->max_degree;           // src/search.cu:402
    Graph g(r->d_slots, r->d_vecs);
    f.graph = &g;
    f.streams["search"].stream = r->c.stream;
    Search_Data<Beam_Data> sd;                    // include/gpufuncs.cuh:557-564
    sd.Q_ = Q;
    sd.batch_ = Q < 4096 ? Q : 4096;              // min(SEARCH_BATCH * 2, Q), SEARCH_BATCH = 2048
    if (!c.alloc(&sd.d_beams_, sizeof(BCD) * (size_t)sd.batch_ * f.bp.beam_size) ||
        !c.alloc(&sd.d_visited_, sizeof(uint32_t) * (size_t)sd.batch_ * f.bp.visit_n))
        return -5;
    f.search_data.push_back(&sd);

    Test_Result tr = f.search_gpu(d_queries, d_ids, d_dists, Q, k, r->starts, false, r->c.stream);
    if (cudaStreamSynchronize(r->c.stream) != cudaSuccess) return -6;
    cudaMemcpy(ids_out, d_ids, (size_t)Q * k * sizeof(int), cudaMemcpyDeviceToHost);
    if (dists_out) cudaMemcpy(dists_out, d_dists, (size_t)Q * k * sizeof(float), cudaMemcpyDeviceToHost);
    if (total_hops_out) *total_hops_out = (int64_t)tr.get_hops();
    if (seconds_out) *seconds_out = tr.get_time();
    f.search_data.clear();
    return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

// One-shot form of the three calls above.
extern "C" int coral_ref_gpu_search(const float* h_vecs, int64_t n, int dim, const int32_t* adj, int deg_pad,
                                    int max_degree, int metric, const int32_t* start_ids, int M,
                                    const float* h_queries, int Q, int L, int k, int32_t* ids_out,
                                    float* dists_out, int64_t* total_hops_out, double* seconds_out) {
    if (!h_queries || !ids_out || Q <= 0 || k <= 0 || k > L) return -1;
    coral_ref_gpu* r = coral_ref_gpu_open(h_vecs, n, dim, adj, deg_pad, max_degree, metric, start_ids, M);
    if (!r) return -2;
    const int rc = coral_ref_gpu_run(r, h_queries, Q, L, k, ids_out, dists_out, total_hops_out, seconds_out);
    coral_ref_gpu_close(r);
    return rc;
}
