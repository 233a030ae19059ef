// CPU BASELINE HARNESS (test/benchmark infrastructure, not product code).
//
// Drives the reference's own CPU best-first search building blocks -- its
// NeighborPriorityQueue (include/efanna2e/neighbor.h:148-237) and its AVX-512
// DistanceL2 (include/efanna2e/distance.h:39-89), both compiled from the
// reference tree via -I<reference>/include -- with a loop that follows
// GPUFuncs::search_in_cpu (src/search_in_cpu.cpp:23-119) statement by
// statement.  That translation unit itself cannot be compiled (it includes
// gpufuncs.cuh, which needs Faiss and a header the reference does not ship),
// so the device copies at :29-31 and :113-115 become plain pointers and the
// 400-byte Slot becomes a row of a padded adjacency array.
//
// This is a timed baseline, NOT a parity oracle: best-first search visits a
// different node set than the GPU kernel's full expansion.
#include <omp.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#include "efanna2e/distance.h"
#include "efanna2e/neighbor.h"

extern "C" int coral_cpu_search(const float* h_base, int64_t base_n, int dim, const int32_t* adj,
                                int deg_pad, const int32_t* start_node_ids, int M,
                                const float* queries, int Q, int beam_capacity, int k,
                                int32_t* ids_res, float* dists_res, int64_t* total_hops_out,
                                double* seconds_out, int n_threads) {
    using namespace efanna2e;
    if (!h_base || !adj || !start_node_ids || !queries || !ids_res || base_n <= 0 || M <= 0) return -1;
    if (n_threads <= 0) n_threads = omp_get_max_threads();
    for (size_t i = 0; i < (size_t)Q * k; ++i) ids_res[i] = -1;  // :33
    if (dists_res)
        for (size_t i = 0; i < (size_t)Q * k; ++i) dists_res[i] = std::numeric_limits<float>::infinity();

    // :43-48 one visited byte-array and tag per thread
    std::vector<std::vector<uint8_t>> visited_buffers(n_threads, std::vector<uint8_t>((size_t)base_n, 0));
    std::vector<uint8_t> visited_tags(n_threads, 1);

    int64_t total_hop = 0;
    double time = 0.0;
    Distance* distance_ = new DistanceL2();  // :52 -- L2 whatever the index metric is

#pragma omp parallel num_threads(n_threads) reduction(+ : total_hop)
    {
        const int tid = omp_get_thread_num();
        std::vector<uint8_t>& visited = visited_buffers[tid];
        uint8_t& visited_tag = visited_tags[tid];
        auto s = std::chrono::steady_clock::now();

#pragma omp for schedule(dynamic, 1)
        for (int qi = 0; qi < Q; qi++) {  // :62-108
            NeighborPriorityQueue search_queue(beam_capacity);
            const float* query = queries + (size_t)qi * dim;
            if (++visited_tag == 0) {
                std::memset(visited.data(), 0, (size_t)base_n);
                visited_tag = 1;
            }
            for (int i = 0; i < M; i++) {
                const int id = start_node_ids[i];
                const float dist = distance_->compare(h_base + (size_t)id * dim, query, dim);
                search_queue.insert({id, dist, false});
                visited[id] = visited_tag;
            }
            uint32_t hops = M;
            while (search_queue.has_unexpanded_node()) {
                auto cur = search_queue.closest_unexpanded();
                const int32_t* nbrs = adj + (size_t)cur.id * deg_pad;
                ++hops;
                for (int i = 0; i < deg_pad; i++) {
                    const int nbr_id = nbrs[i];
                    if (nbr_id < 0) break;  // end of the slot's nbrs[0..deg)
                    if (visited[nbr_id] == visited_tag) continue;
                    const float dist = distance_->compare(h_base + (size_t)nbr_id * dim, query, dim);
                    search_queue.insert({nbr_id, dist, false});
                    visited[nbr_id] = visited_tag;
                }
            }
            total_hop += hops;
            const int topk = std::min<int>(k, (int)search_queue.size());
            for (int i = 0; i < topk; i++) {
                ids_res[(size_t)qi * k + i] = search_queue[i].id;
                if (dists_res) dists_res[(size_t)qi * k + i] = search_queue[i].distance;
            }
        }
        double t = std::chrono::duration<double>(std::chrono::steady_clock::now() - s).count();
#pragma omp critical
        if (t > time) time = t;  // :110 wall time of the parallel search loop
    }
    delete distance_;
    if (total_hops_out) *total_hops_out = total_hop;
    if (seconds_out) *seconds_out = time;
    return 0;
}

extern "C" int coral_cpu_search_kind(void) { return 1; }  // 1 = built on the reference's headers
