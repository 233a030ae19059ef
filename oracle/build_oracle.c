/*
 * CPU ORACLE for the stages around the search path (test infrastructure, not product code):
 * exact k-nearest neighbours, and -- further down -- the graph build (neighbourhood-aware
 * projection and connectivity enhancement).  Only tests and the benchmark's checker may load it.
 *
 * Exact k-NN.  The reference gets the k_b nearest base points of every training query, and its
 * ground truth, from Faiss' flat GPU index (src/knn.cu:174-193, include/myfaiss.h:17-29,
 * tests/comp_gt.cpp:121-155).  Faiss is a third-party dependency that is not vendored and whose
 * version CMakeLists.txt:40 does not pin; its flat search is exhaustive, so the published
 * algorithm is "the k rows with the smallest squared L2 distance / largest inner product".
 * Here the distance is the reference's own device function (include/utils.cuh:254-275, :307-323:
 * one sequential fp32 fused chain) and ties order by the smaller id.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_L2 0
#define ORACLE_IP 1
#define FMA_CLONES __attribute__((target_clones("fma", "default")))

float coral_oracle_dist_seq(const float* row, const float* q, int dim, int metric);

/* "closer" == smaller key */
static inline uint32_t ord_of(float d, int metric) {
    if (metric == ORACLE_IP) d = -d;
    uint32_t u;
    memcpy(&u, &d, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

static int cmp_u64(const void* a, const void* b) {
    const uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
    return x < y ? -1 : (x > y ? 1 : 0);
}

/* ids_out [Q][k], dists_out [Q][k] (nullable): the k closest rows by (distance, id). */
int coral_oracle_exact_knn(const float* base, int64_t n, int dim, const float* queries, int Q, int k, int metric,
                           int32_t* ids_out, float* dists_out) {
    if (!base || !queries || !ids_out || n <= 0 || Q < 0 || k <= 0 || k > n) return -1;
#pragma omp parallel
    {
        uint64_t* keys = (uint64_t*)malloc((size_t)n * sizeof(uint64_t));
#pragma omp for schedule(dynamic, 1)
        for (int q = 0; q < Q; ++q) {
            const float* qv = queries + (size_t)q * dim;
            for (int64_t i = 0; i < n; ++i)
                keys[i] = ((uint64_t)ord_of(coral_oracle_dist_seq(base + (size_t)i * dim, qv, dim, metric), metric) << 32) |
                          (uint32_t)i;
            qsort(keys, (size_t)n, sizeof(uint64_t), cmp_u64);
            for (int j = 0; j < k; ++j) {
                const int32_t id = (int32_t)(uint32_t)keys[j];
                ids_out[(size_t)q * k + j] = id;
                if (dists_out) dists_out[(size_t)q * k + j] = coral_oracle_dist_seq(base + (size_t)id * dim, qv, dim, metric);
            }
        }
        free(keys);
    }
    return 0;
}
