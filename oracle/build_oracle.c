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
#define _GNU_SOURCE
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

/* ------------------------------------------------------------------------------------------------
 * Graph build: neighbourhood-aware projection (NAP) and connectivity enhancement (CE).
 *
 *   NAP   GPUFuncs::gpu_neibor_aware          src/upd_gpu.cu:260-303
 *           pair_dist_compute_kernel          src/upd_gpu.cu:12-78     candidates of every list member
 *           segmented sort by distance        src/utils.cu:340-346     (IP: descending)
 *           candidate_ignore_kernel           src/upd_gpu.cu:203-247   occlusion pruning
 *           update_new_nbrs_kernel            src/upd_gpu.cu:88-167    need_discard = 1 (config.json:15)
 *   CE    GPUFuncs::gpu_connect_enhance       src/enhance.cu:728-861   enhance_mode 0, isolated nodes
 *           build_candidate_kernel            src/enhance.cu:136-212   candidates + reverse edges
 *           candidate_ignore_kernel_for_iso   src/enhance.cu:344-389
 *           update_iso_nbrs_kernel            src/enhance.cu:528-580
 *
 * The graph is held as in the CUDA library: adj[n][deg_pad] (-1 padding), ndist[n][deg_pad] (the
 * reference's Slot::dists), deg[n].  Rows are kept closest-first, as the reference keeps them.
 *
 * Where the reference lets thread arrival order decide, this restatement (and the CUDA path) fix
 * the lowest index:
 *   - a node that is a member of several lists of one batch is updated by its FIRST occurrence in
 *     the batch (reference: whichever thread wins atomicTestAndSetBit, src/upd_gpu.cu:102);
 *   - a node found by several isolated nodes of one CE batch receives the reverse edge of the first
 *     (isolated node, result rank) pair (reference: src/enhance.cu:166);
 *   - the segmented sorts are stable (equal distances keep their candidate order).
 * Every other step is deterministic in the reference and restated literally.
 * ------------------------------------------------------------------------------------------------ */

enum { S_INVALID = 0, S_INITIAL = 1, S_DISCARDED = 2, S_RETAINED = 3, S_REPEATED = 4 };  /* include/uni.h:140-146 */

typedef struct {
    int id;
    int col;      /* position in the unsorted candidate row (stable sort key) */
    int status;
    float dist;
} Cand;

static inline float farthest_of(int metric) { return metric == ORACLE_L2 ? 3.402823466e+38f : -3.402823466e+38f; }
/* include/utils.cuh:380-382: true when d1 is closer than d0 */
static inline int closer(float d0, float d1, int metric) { return metric == ORACLE_L2 ? d0 > d1 : d0 < d1; }

static int cmp_cand(const void* a, const void* b, void* metric_p) {
    const Cand* x = (const Cand*)a;
    const Cand* y = (const Cand*)b;
    const int metric = *(const int*)metric_p;
    const uint32_t ox = ord_of(x->dist, metric), oy = ord_of(y->dist, metric);
    if (ox != oy) return ox < oy ? -1 : 1;
    return x->col < y->col ? -1 : (x->col > y->col ? 1 : 0);
}

/* src/upd_gpu.cu:203-247 (and src/enhance.cu:344-389, the same rule run by a block). */
static void occlusion_prune(const float* base, int dim, int metric, Cand* c, int n_cand, int max_degree) {
    int nbr_num = 0;
    for (int i = 0; i < n_cand && nbr_num < max_degree; ++i) {
        if (c[i].status == S_INVALID) break;
        if (c[i].status == S_INITIAL) {
            c[i].status = S_RETAINED;
            ++nbr_num;
            const float* vi = base + (size_t)c[i].id * dim;
            for (int j = i + 1; j < n_cand; ++j) {
                if (c[j].status == S_INVALID) break;
                if (c[j].id == c[i].id)
                    c[j].status = S_REPEATED;
                else if (c[j].status == S_INITIAL) {
                    const float dij = coral_oracle_dist_seq(vi, base + (size_t)c[j].id * dim, dim, metric);
                    if (closer(c[j].dist, dij, metric)) c[j].status = S_DISCARDED;
                }
            }
        } else if (c[i].status == S_DISCARDED) {
            for (int j = i + 1; j < n_cand; ++j) {
                if (c[j].id == c[i].id)
                    c[j].status = S_REPEATED;
                else if (c[j].status == S_INVALID)
                    break;
            }
        }
    }
}

/* src/upd_gpu.cu:106-135 / src/enhance.cu:544-570: kept first, then pruned ones to fill the row. */
static int fill_row(const Cand* c, int n_cand, int max_degree, int32_t* nbrs, float* dists) {
    int retained = 0;
    for (int i = 0; i < n_cand; ++i) {
        if (c[i].status == S_RETAINED) ++retained;
        else if (c[i].status == S_INVALID) break;
    }
    int discarded_need = max_degree - retained, nbr_num = 0;
    for (int j = 0; j < n_cand && nbr_num < max_degree; ++j) {
        if (c[j].status == S_RETAINED) {
            nbrs[nbr_num] = c[j].id;
            dists[nbr_num++] = c[j].dist;
        } else if (c[j].status == S_DISCARDED && (discarded_need--) > 0) {
            nbrs[nbr_num] = c[j].id;
            dists[nbr_num++] = c[j].dist;
        } else if (c[j].status == S_INVALID)
            break;
    }
    return nbr_num;
}

/* One NAP batch: B lists of kb base ids; every pivot sees the graph as it was before the batch. */
int coral_oracle_nap_batch(const float* base, int64_t n, int dim, int metric, int max_degree, int deg_pad,
                           int32_t* adj, float* ndist, int32_t* deg, const int32_t* lists, int B, int kb) {
    if (!base || !adj || !ndist || !deg || !lists || B < 0 || kb < 2 || max_degree > deg_pad) return -1;
    const int cand_size = kb + max_degree;
    const int64_t pivots = (int64_t)B * kb;
    /* first occurrence of every node in the batch */
    int64_t* first = (int64_t*)malloc((size_t)n * sizeof(int64_t));
    for (int64_t i = 0; i < n; ++i) first[i] = -1;
    for (int64_t p = 0; p < pivots; ++p) {
        const int id = lists[p];
        if (id < 0 || id >= n) { free(first); return -2; }
        if (first[id] < 0) first[id] = p;
    }
    int32_t* new_nbrs = (int32_t*)malloc((size_t)pivots * max_degree * sizeof(int32_t));
    float* new_dists = (float*)malloc((size_t)pivots * max_degree * sizeof(float));
    int32_t* new_deg = (int32_t*)malloc((size_t)pivots * sizeof(int32_t));
#pragma omp parallel
    {
        Cand* c = (Cand*)malloc((size_t)cand_size * sizeof(Cand));
#pragma omp for schedule(dynamic, 16)
        for (int64_t p = 0; p < pivots; ++p) {
            new_deg[p] = -1;
            const int row_id = lists[p];
            if (first[row_id] != p) continue;                       /* src/upd_gpu.cu:102 */
            const int32_t* ids = lists + (p / kb) * kb;
            const int i = (int)(p % kb);
            const int row_deg = deg[row_id];
            for (int col = 0; col < cand_size; ++col) {             /* src/upd_gpu.cu:36-73 */
                Cand* e = &c[col];
                e->col = col;
                e->id = -1;
                e->status = S_INVALID;
                e->dist = farthest_of(metric);
                if (col >= kb + row_deg || col == i) continue;
                if (col >= kb) {
                    e->id = adj[(size_t)row_id * deg_pad + (col - kb)];
                    e->dist = ndist[(size_t)row_id * deg_pad + (col - kb)];
                    e->status = S_INITIAL;
                } else {
                    const int col_id = ids[col];
                    if (col_id == row_id) continue;
                    if (row_deg > 0 && deg[col_id] > 0) continue;
                    e->id = col_id;
                    e->dist = coral_oracle_dist_seq(base + (size_t)row_id * dim, base + (size_t)col_id * dim, dim, metric);
                    e->status = S_INITIAL;
                }
            }
            qsort_r(c, (size_t)cand_size, sizeof(Cand), cmp_cand, &metric);
            occlusion_prune(base, dim, metric, c, cand_size, max_degree);
            new_deg[p] = fill_row(c, cand_size, max_degree, new_nbrs + (size_t)p * max_degree, new_dists + (size_t)p * max_degree);
        }
        free(c);
    }
    for (int64_t p = 0; p < pivots; ++p) {
        if (new_deg[p] < 0) continue;
        const int id = lists[p];
        for (int j = 0; j < deg_pad; ++j) {
            adj[(size_t)id * deg_pad + j] = j < new_deg[p] ? new_nbrs[(size_t)p * max_degree + j] : -1;
            ndist[(size_t)id * deg_pad + j] = j < new_deg[p] ? new_dists[(size_t)p * max_degree + j] : 0.f;
        }
        deg[id] = new_deg[p];
    }
    free(first); free(new_nbrs); free(new_dists); free(new_deg);
    return 0;
}

/* One CE batch (src/enhance.cu:640-668): n_iso isolated nodes with their kb search results
 * (res_ids < 0 = padding).  Reverse edges first (src/enhance.cu:136-212), then every isolated node's
 * own row from its pruned results. */
int coral_oracle_ce_batch(const float* base, int64_t n, int dim, int metric, int max_degree, int deg_pad,
                          int32_t* adj, float* ndist, int32_t* deg, const int32_t* iso_ids, int n_iso,
                          const int32_t* res_ids, const float* res_dists, int kb) {
    if (!base || !adj || !ndist || !deg || !iso_ids || !res_ids || !res_dists || n_iso < 0 || kb < 1) return -1;
    /* first (isolated node, rank) pair that names each found node */
    int64_t* first = (int64_t*)malloc((size_t)n * sizeof(int64_t));
    for (int64_t i = 0; i < n; ++i) first[i] = -1;
    for (int64_t e = 0; e < (int64_t)n_iso * kb; ++e) {
        const int id = res_ids[e];
        if (id >= 0 && id < n && first[id] < 0) first[id] = e;
    }
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < (int64_t)n_iso * kb; ++e) {
        const int knn_id = res_ids[e];
        if (knn_id < 0 || knn_id >= n || first[knn_id] != e) continue;
        const int iso_id = iso_ids[e / kb];
        const float knn_dist = res_dists[e];
        const float* iso_vec = base + (size_t)iso_id * dim;
        int32_t* nb = adj + (size_t)knn_id * deg_pad;
        float* ds = ndist + (size_t)knn_id * deg_pad;
        const int d = deg[knn_id];
        int pos = 0, valid = 1, out_pos;
        for (; pos < d; ++pos) {
            if (closer(knn_dist, ds[pos], metric)) {
                if (valid && closer(knn_dist, coral_oracle_dist_seq(iso_vec, base + (size_t)nb[pos] * dim, dim, metric), metric))
                    valid = 0;
            } else
                break;
        }
        if (d == max_degree) {
            if (!valid || pos >= d) continue;
            out_pos = d - 1;
            for (; out_pos >= pos; --out_pos)
                if (closer(ds[out_pos], coral_oracle_dist_seq(iso_vec, base + (size_t)nb[out_pos] * dim, dim, metric), metric))
                    break;
            if (out_pos < pos) out_pos = d - 1;
        } else {
            out_pos = d;
            deg[knn_id] = d + 1;
        }
        for (int j = out_pos; j > pos; --j) {
            nb[j] = nb[j - 1];
            ds[j] = ds[j - 1];
        }
        nb[pos] = iso_id;
        ds[pos] = knn_dist;
    }
    free(first);
#pragma omp parallel
    {
        Cand* c = (Cand*)malloc((size_t)kb * sizeof(Cand));
        int32_t* row_n = (int32_t*)malloc((size_t)max_degree * sizeof(int32_t));
        float* row_d = (float*)malloc((size_t)max_degree * sizeof(float));
#pragma omp for schedule(dynamic, 16)
        for (int i = 0; i < n_iso; ++i) {
            for (int r = 0; r < kb; ++r) {
                const int id = res_ids[(size_t)i * kb + r];
                c[r].col = r;
                c[r].id = id >= 0 && id < n ? id : -1;
                c[r].status = c[r].id >= 0 ? S_INITIAL : S_INVALID;
                c[r].dist = c[r].id >= 0 ? res_dists[(size_t)i * kb + r] : farthest_of(metric);
            }
            qsort_r(c, (size_t)kb, sizeof(Cand), cmp_cand, &metric);
            occlusion_prune(base, dim, metric, c, kb, max_degree);
            const int nd = fill_row(c, kb, max_degree, row_n, row_d);
            const int id = iso_ids[i];
            for (int j = 0; j < deg_pad; ++j) {
                adj[(size_t)id * deg_pad + j] = j < nd ? row_n[j] : -1;
                ndist[(size_t)id * deg_pad + j] = j < nd ? row_d[j] : 0.f;
            }
            deg[id] = nd;
        }
        free(c); free(row_n); free(row_d);
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------------
 * Update: delete with topology repair, insert.
 *
 *   delete   IndexGPU::Delete                  src/index_gpu.cpp:138-206 (batches of INNBR_BATCH in-neighbours)
 *            Graph::get_del_innbrs             src/graph.cpp:155-195
 *            GPUFuncs::vector_delete           src/update.cu:674-771
 *              vector_deletion_patch_kernel    src/update.cu:312-391   candidates of every in-neighbour
 *              candidate_ignore_kernel         src/upd_gpu.cu:203-247
 *              update_and_collect_nbrs_kernel  src/update.cu:499-583   kept ones, THEN pruned ones
 *   insert   IndexGPU::Insert                  src/index_gpu.cpp:207-224 (batches of insert_batch)
 *            GPUFuncs::vector_insert           src/update.cu:880-959, upd_type 1 (neighbours from the search)
 *              k_plus_ones_build_kernel        src/update.cu:101-197   candidates + reverse edges
 *              candidate_ignore_kernel_for_ins src/update.cu:585-629
 *              update_and_collect_nbrs_kernel  src/update.cu:499-583
 *
 * Fixed where the reference leaves it open or is plainly off:
 *   - in-neighbours of a deleted node are taken in ascending id order (the reference iterates a
 *     std::unordered_set, include/graph.cuh:536);
 *   - an in-neighbour named by several deleted nodes of one batch is repaired by its first
 *     occurrence (reference: thread arrival, src/update.cu:514);
 *   - both sorts are closest-first for either metric (the reference sorts ascending by value without
 *     the inner-product flag here, src/update.cu:728,:930, i.e. farthest-first for inner product);
 *   - a deleted node's out-neighbour that is the in-neighbour being repaired is skipped (the
 *     reference would propose the node to itself at distance 0).
 * ------------------------------------------------------------------------------------------------ */

static inline int bit_test(const uint32_t* bits, int i) { return (bits[i >> 5] >> (i & 31)) & 1u; }

/* src/update.cu:530-577: every kept candidate in order, then pruned ones while the row has room. */
static int fill_row_kept_then_pruned(const Cand* c, int n_cand, int max_degree, int32_t* nbrs, float* dists) {
    int nbr_num = 0;
    for (int i = 0; i < n_cand && nbr_num < max_degree; ++i) {
        if (c[i].status == S_RETAINED) {
            nbrs[nbr_num] = c[i].id;
            dists[nbr_num++] = c[i].dist;
        } else if (c[i].status == S_INVALID)
            break;
    }
    for (int j = 0; j < n_cand && nbr_num < max_degree; ++j) {
        if (c[j].status == S_DISCARDED) {
            nbrs[nbr_num] = c[j].id;
            dists[nbr_num++] = c[j].dist;
        } else if (c[j].status == S_INVALID)
            break;
    }
    return nbr_num;
}

/* One repair batch: pivots p = (deleted node del_of[p], in-neighbour innbr[p]), n_piv of them.
 * `deleted` already has every deleted id of the whole Delete call marked. */
int coral_oracle_delete_batch(const float* base, int64_t n, int dim, int metric, int max_degree, int deg_pad,
                              int32_t* adj, float* ndist, int32_t* deg, const uint32_t* deleted, const int32_t* del_of,
                              const int32_t* innbr, int n_piv) {
    if (!base || !adj || !ndist || !deg || !deleted || !del_of || !innbr || n_piv < 0) return -1;
    const int cand_size = 2 * max_degree;
    int64_t* first = (int64_t*)malloc((size_t)n * sizeof(int64_t));
    for (int64_t i = 0; i < n; ++i) first[i] = -1;
    for (int p = 0; p < n_piv; ++p)
        if (first[innbr[p]] < 0) first[innbr[p]] = p;
    int32_t* new_nbrs = (int32_t*)malloc((size_t)n_piv * max_degree * sizeof(int32_t));
    float* new_dists = (float*)malloc((size_t)n_piv * max_degree * sizeof(float));
    int32_t* new_deg = (int32_t*)malloc((size_t)n_piv * sizeof(int32_t));
#pragma omp parallel
    {
        Cand* c = (Cand*)malloc((size_t)cand_size * sizeof(Cand));
#pragma omp for schedule(dynamic, 16)
        for (int p = 0; p < n_piv; ++p) {
            new_deg[p] = -1;
            const int I = innbr[p], D = del_of[p];
            if (first[I] != p) continue;
            int nc = 0;
            for (int j = 0; j < deg[I]; ++j) {                                   /* src/update.cu:357-365 */
                const int id = adj[(size_t)I * deg_pad + j];
                if (bit_test(deleted, id)) continue;
                c[nc].id = id; c[nc].col = nc; c[nc].status = S_INITIAL; c[nc].dist = ndist[(size_t)I * deg_pad + j];
                ++nc;
            }
            for (int j = 0; j < deg[D]; ++j) {                                   /* src/update.cu:366-373 */
                const int id = adj[(size_t)D * deg_pad + j];
                if (bit_test(deleted, id) || id == I) continue;
                c[nc].id = id; c[nc].col = nc; c[nc].status = S_INITIAL;
                c[nc].dist = coral_oracle_dist_seq(base + (size_t)I * dim, base + (size_t)id * dim, dim, metric);
                ++nc;
            }
            const int valid = nc;
            for (; nc < cand_size; ++nc) { c[nc].id = -1; c[nc].col = nc; c[nc].status = S_INVALID; c[nc].dist = farthest_of(metric); }
            qsort_r(c, (size_t)valid, sizeof(Cand), cmp_cand, &metric);
            occlusion_prune(base, dim, metric, c, cand_size, max_degree);
            new_deg[p] = fill_row_kept_then_pruned(c, cand_size, max_degree, new_nbrs + (size_t)p * max_degree,
                                                   new_dists + (size_t)p * max_degree);
        }
        free(c);
    }
    for (int p = 0; p < n_piv; ++p) {
        if (new_deg[p] < 0) continue;
        const int id = innbr[p];
        for (int j = 0; j < deg_pad; ++j) {
            adj[(size_t)id * deg_pad + j] = j < new_deg[p] ? new_nbrs[(size_t)p * max_degree + j] : -1;
            ndist[(size_t)id * deg_pad + j] = j < new_deg[p] ? new_dists[(size_t)p * max_degree + j] : 0.f;
        }
        deg[id] = new_deg[p];
    }
    free(first); free(new_nbrs); free(new_dists); free(new_deg);
    return 0;
}

/* One insert batch: n_ins new nodes with their kb search results (ids < 0 = padding).  The same two
 * steps as a CE batch with the insert path's differences: candidate distances are recomputed
 * (src/update.cu:139) and the row is filled kept-first (src/update.cu:530-577). */
int coral_oracle_insert_batch(const float* base, int64_t n, int dim, int metric, int max_degree, int deg_pad,
                              int32_t* adj, float* ndist, int32_t* deg, const int32_t* ins_ids, int n_ins,
                              const int32_t* res_ids, int kb) {
    if (!base || !adj || !ndist || !deg || !ins_ids || !res_ids || n_ins < 0 || kb < 1) return -1;
    float* res_d = (float*)malloc((size_t)n_ins * kb * sizeof(float));
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < (int64_t)n_ins * kb; ++e) {
        const int id = res_ids[e];
        res_d[e] = id >= 0 && id < n ? coral_oracle_dist_seq(base + (size_t)ins_ids[e / kb] * dim, base + (size_t)id * dim, dim, metric)
                                     : farthest_of(metric);
    }
    /* reverse edges: identical rule to the CE batch (src/update.cu:143-191 == src/enhance.cu:166-211) */
    int64_t* first = (int64_t*)malloc((size_t)n * sizeof(int64_t));
    for (int64_t i = 0; i < n; ++i) first[i] = -1;
    for (int64_t e = 0; e < (int64_t)n_ins * kb; ++e) {
        const int id = res_ids[e];
        if (id >= 0 && id < n && first[id] < 0) first[id] = e;
    }
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t e = 0; e < (int64_t)n_ins * kb; ++e) {
        const int knn_id = res_ids[e];
        if (knn_id < 0 || knn_id >= n || first[knn_id] != e) continue;
        const int ins_id = ins_ids[e / kb];
        const float knn_dist = res_d[e];
        const float* ins_vec = base + (size_t)ins_id * dim;
        int32_t* nb = adj + (size_t)knn_id * deg_pad;
        float* ds = ndist + (size_t)knn_id * deg_pad;
        const int d = deg[knn_id];
        int pos = 0, valid = 1, out_pos;
        for (; pos < d; ++pos) {
            if (closer(knn_dist, ds[pos], metric)) {
                if (valid && closer(knn_dist, coral_oracle_dist_seq(ins_vec, base + (size_t)nb[pos] * dim, dim, metric), metric))
                    valid = 0;
            } else
                break;
        }
        if (d == max_degree) {
            if (!valid || pos >= d) continue;
            out_pos = d - 1;
            for (; out_pos >= pos; --out_pos)
                if (closer(ds[out_pos], coral_oracle_dist_seq(ins_vec, base + (size_t)nb[out_pos] * dim, dim, metric), metric))
                    break;
            if (out_pos < pos) out_pos = d - 1;
        } else {
            out_pos = d;
            deg[knn_id] = d + 1;
        }
        for (int j = out_pos; j > pos; --j) {
            nb[j] = nb[j - 1];
            ds[j] = ds[j - 1];
        }
        nb[pos] = ins_id;
        ds[pos] = knn_dist;
    }
    free(first);
#pragma omp parallel
    {
        Cand* c = (Cand*)malloc((size_t)kb * sizeof(Cand));
        int32_t* row_n = (int32_t*)malloc((size_t)max_degree * sizeof(int32_t));
        float* row_d = (float*)malloc((size_t)max_degree * sizeof(float));
#pragma omp for schedule(dynamic, 16)
        for (int i = 0; i < n_ins; ++i) {
            for (int r = 0; r < kb; ++r) {
                const int id = res_ids[(size_t)i * kb + r];
                c[r].col = r;
                c[r].id = id >= 0 && id < n ? id : -1;
                c[r].status = c[r].id >= 0 ? S_INITIAL : S_INVALID;
                c[r].dist = res_d[(size_t)i * kb + r];
            }
            qsort_r(c, (size_t)kb, sizeof(Cand), cmp_cand, &metric);
            occlusion_prune(base, dim, metric, c, kb, max_degree);
            const int nd = fill_row_kept_then_pruned(c, kb, max_degree, row_n, row_d);
            const int id = ins_ids[i];
            for (int j = 0; j < deg_pad; ++j) {
                adj[(size_t)id * deg_pad + j] = j < nd ? row_n[j] : -1;
                ndist[(size_t)id * deg_pad + j] = j < nd ? row_d[j] : 0.f;
            }
            deg[id] = nd;
        }
        free(c); free(row_n); free(row_d);
    }
    free(res_d);
    return 0;
}

/* Distances of the stored edges (one sequential chain each) and the degrees of a padded adjacency. */
int coral_oracle_edge_dists(const float* base, int64_t n, int dim, int metric, const int32_t* adj, int deg_pad,
                            float* ndist, int32_t* deg) {
    if (!base || !adj || !ndist || !deg) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int cnt = 0;
        for (int j = 0; j < deg_pad; ++j) {
            const int id = adj[(size_t)i * deg_pad + j];
            const int ok = id >= 0 && id < n;
            ndist[(size_t)i * deg_pad + j] = ok ? coral_oracle_dist_seq(base + (size_t)i * dim, base + (size_t)id * dim, dim, metric) : 0.f;
            cnt += ok;
        }
        deg[i] = cnt;
    }
    return 0;
}
