/*
 * CPU BASELINE PORT (test/benchmark infrastructure, not product code).
 *
 * A self-contained restatement of the reference's CPU best-first search,
 * GPUFuncs::search_in_cpu (src/search_in_cpu.cpp:23-119), for machines where
 * the harness built on the reference's own headers cannot run (those headers
 * need AVX-512).  Same algorithm: per-thread byte-tag visited array (:43-48,
 * :68-71), M entry points (:74-79), pop the closest unexpanded entry, scan its
 * neighbour list, sorted insert into a capacity-L queue ordered by
 * (distance, id) with equal ids dropped (include/efanna2e/neighbor.h:39-41,
 * :162-195), first k entries out (:103-107).  Distance is squared L2 whatever
 * the index metric (:52); the summation order of the reference's AVX-512
 * kernel is not reproduced (this is a timing baseline, not a parity oracle).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef struct {
    int id;
    float dist;
    int flag;
} nb_t;

static inline int nb_less(const nb_t* a, const nb_t* b) {
    return a->dist < b->dist || (a->dist == b->dist && a->id < b->id);
}

typedef struct {
    size_t size, cap, cur;
    nb_t* data;
} pq_t;

static void pq_insert(pq_t* q, nb_t nbr) { /* neighbor.h:162-195 */
    if (q->size == q->cap && nb_less(&q->data[q->size - 1], &nbr)) return;
    size_t lo = 0, hi = q->size;
    while (lo < hi) {
        size_t mid = (lo + hi) >> 1;
        if (nb_less(&nbr, &q->data[mid]))
            hi = mid;
        else if (q->data[mid].id == nbr.id)
            return;
        else
            lo = mid + 1;
    }
    if (lo < q->cap) memmove(&q->data[lo + 1], &q->data[lo], (q->size - lo) * sizeof(nb_t));
    q->data[lo] = nbr;
    q->data[lo].flag = 0;
    if (q->size < q->cap) q->size++;
    if (lo < q->cur) q->cur = lo;
}

static nb_t pq_closest_unexpanded(pq_t* q) { /* neighbor.h:197-204 */
    q->data[q->cur].flag = 1;
    size_t pre = q->cur;
    while (q->cur < q->size && q->data[q->cur].flag) q->cur++;
    return q->data[pre];
}

__attribute__((target_clones("avx2,fma", "default"))) static float l2sq(const float* x, const float* y,
                                                                      int d) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int i = 0;
    for (; i + 8 <= d; i += 8)
        for (int j = 0; j < 8; ++j) {
            float t = x[i + j] - y[i + j];
            acc[j] += t * t;
        }
    float s = 0.f;
    for (int j = 0; j < 8; ++j) s += acc[j];
    for (; i < d; ++i) {
        float t = x[i] - y[i];
        s += t * t;
    }
    return s;
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

int coral_cpu_search(const float* h_base, int64_t base_n, int dim, const int32_t* adj, int deg_pad,
                     const int32_t* start_node_ids, int M, const float* queries, int Q,
                     int beam_capacity, int k, int32_t* ids_res, float* dists_res,
                     int64_t* total_hops_out, double* seconds_out, int n_threads) {
    if (!h_base || !adj || !start_node_ids || !queries || !ids_res || base_n <= 0 || M <= 0) return -1;
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_max_threads();
#else
    n_threads = 1;
#endif
    for (size_t i = 0; i < (size_t)Q * k; ++i) ids_res[i] = -1;
    if (dists_res)
        for (size_t i = 0; i < (size_t)Q * k; ++i) dists_res[i] = INFINITY;
    int64_t total_hop = 0;
    double time = 0.0;

#pragma omp parallel num_threads(n_threads) reduction(+ : total_hop)
    {
        uint8_t* visited = (uint8_t*)calloc((size_t)base_n, 1);
        uint8_t tag = 1;
        pq_t pq;
        pq.cap = (size_t)beam_capacity;
        pq.data = (nb_t*)malloc(sizeof(nb_t) * (pq.cap + 1));
        double s = now_s();
#pragma omp for schedule(dynamic, 1)
        for (int qi = 0; qi < Q; ++qi) {
            const float* query = queries + (size_t)qi * dim;
            pq.size = 0;
            pq.cur = 0;
            if (++tag == 0) {
                memset(visited, 0, (size_t)base_n);
                tag = 1;
            }
            for (int i = 0; i < M; ++i) {
                int id = start_node_ids[i];
                nb_t nb = {id, l2sq(h_base + (size_t)id * dim, query, dim), 0};
                pq_insert(&pq, nb);
                visited[id] = tag;
            }
            uint32_t hops = (uint32_t)M;
            while (pq.cur < pq.size) {
                nb_t cur = pq_closest_unexpanded(&pq);
                const int32_t* nbrs = adj + (size_t)cur.id * deg_pad;
                ++hops;
                for (int i = 0; i < deg_pad; ++i) {
                    int v = nbrs[i];
                    if (v < 0) break;
                    if (visited[v] == tag) continue;
                    nb_t nb = {v, l2sq(h_base + (size_t)v * dim, query, dim), 0};
                    pq_insert(&pq, nb);
                    visited[v] = tag;
                }
            }
            total_hop += hops;
            int topk = k < (int)pq.size ? k : (int)pq.size;
            for (int i = 0; i < topk; ++i) {
                ids_res[(size_t)qi * k + i] = pq.data[i].id;
                if (dists_res) dists_res[(size_t)qi * k + i] = pq.data[i].dist;
            }
        }
        double t = now_s() - s;
#pragma omp critical
        if (t > time) time = t;
        free(visited);
        free(pq.data);
    }
    if (total_hops_out) *total_hops_out = total_hop;
    if (seconds_out) *seconds_out = time;
    return 0;
}

int coral_cpu_search_kind(void) { return 0; } /* 0 = self-contained port */
