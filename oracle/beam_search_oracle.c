/*
 * CPU ORACLE (test infrastructure, not product code).
 *
 * Restates, for one CPU thread per query, what CORAL's GPU "full expansion"
 * beam search computes per query:
 *
 *   reference kernel          src/search_gpu.cu:347-580 (bitset-visited overload)
 *   neighbour distances       include/utils.cuh:254-275 (L2), :307-323 (IP)
 *   seed distances            src/search_gpu.cu:14-23 (lane-strided + shuffle tree)
 *   closer-than predicate     include/utils.cuh:380-382
 *   sentinels                 include/uni.h:65-68
 *
 * Parity status: PINNED to the reference's own kernel.  The reference ships no
 * golden vector or known-answer test for this path, so the pin is the
 * reference's search sources themselves (src/search_gpu.cu, src/utils.cu,
 * src/uni.cpp, src/fileout.cpp), compiled unmodified for sm_100a by
 * oracle/Makefile (target ref_gpu) and run on a B200: this file's ids, distance
 * bits and hop counts equal that kernel's on every case of
 * tests/test_gpu_ref_pin.py, and the kernel's outputs are committed as
 * tests/golden/ref_kernel_small.npz, which tests/test_oracle.py checks on CPU.
 * Where the reference kernel leaves an outcome to thread arrival order (equal
 * distances at the cut, src/search_gpu.cu:530-532) the lowest id wins here.
 * Only tests, the smoke check and the benchmark's checker may load this file.
 *
 * Semantics restated (per query):
 *   beam <- the M entry points (duplicates kept, as src/search_gpu.cu:392-407
 *   ignores the test-and-set result), worst <- "farthest" sentinel.
 *   round: every beam entry not yet expanded is marked and its neighbour list
 *   scanned; a neighbour that enters the exact visited set for the first time
 *   gets a distance (src/search_gpu.cu:430-431) and becomes a candidate iff it
 *   is STRICTLY closer than `worst` as it stood at round start (:432).
 *   no candidates -> stop (:442).  |beam|+|cand| <= L -> append, worst
 *   unchanged (:477-483).  Otherwise beam <- the L closest of beam U cand and
 *   worst <- the farthest kept distance (:525-576; the `total > 2L` branch at
 *   :486 cannot be reached because total <= |beam| + L).
 *   Output: the k closest beam entries, closest first (:447-472).
 *
 * Floating point: the reference is compiled with nvcc's default -fmad=true, so
 * `sum += diff*diff` is one fused multiply-add per element.  Neighbour
 * distances are a single sequential chain over d = 0..dim-1; seed distances
 * are 32 lane-strided chains combined by the shfl_down tree 16,8,4,2,1.  Both
 * orders are reproduced bit for bit here (fmaf is correctly rounded).
 *
 * Ties: the reference resolves equal distances by thread/slot position, which
 * is not deterministic.  This oracle (and the CUDA path) use one fixed total
 * order instead -- (distance, id) -- which is one of the outcomes the
 * reference can produce.
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

#define ST_OK 0
#define ST_BEAM_UNDERFULL 1

/* stats row: status, n_dist, n_exp, rounds, hops, n_scan, max_cand, reserved */
#define STATS_W 8

#define FMA_CLONES __attribute__((target_clones("fma", "default")))

/* include/utils.cuh:254-275 / :307-323 -- one sequential fused chain. */
FMA_CLONES
float coral_oracle_dist_seq(const float* row, const float* q, int dim, int metric) {
    float sum = 0.0f;
    if (metric == ORACLE_L2) {
        for (int d = 0; d < dim; ++d) {
            float diff = row[d] - q[d];
            sum = fmaf(diff, diff, sum);
        }
    } else {
        for (int d = 0; d < dim; ++d) sum = fmaf(row[d], q[d], sum);
    }
    return sum;
}

/* src/search_gpu.cu:14-23 -- lane l sums d = l, l+32, ...; then
 * sum += shfl_down(sum, off) for off = 16,8,4,2,1; lane 0 is returned.
 * shfl_down from a lane >= 32 yields the caller's own value; those lanes never
 * feed lane 0, so only the in-range adds are modelled. */
FMA_CLONES
float coral_oracle_dist_tree(const float* row, const float* q, int dim, int metric) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float sum = 0.0f;
        if (metric == ORACLE_L2) {
            for (int d = l; d < dim; d += 32) {
                float diff = q[d] - row[d];
                sum = fmaf(diff, diff, sum);
            }
        } else {
            for (int d = l; d < dim; d += 32) sum = fmaf(q[d], row[d], sum);
        }
        lane[l] = sum;
    }
    for (int off = 16; off > 0; off >>= 1)
        for (int l = 0; l + off < 32 && l < off; ++l) lane[l] = lane[l] + lane[l + off];
    return lane[0];
}

static inline float farthest_of(int metric) { return metric == ORACLE_L2 ? 3.402823466e+38f : -3.402823466e+38f; }

/* include/utils.cuh:380-382: true when d1 is closer than d0. */
static inline int closer(float d0, float d1, int metric) { return metric == ORACLE_L2 ? d0 > d1 : d0 < d1; }

/* Order-preserving map float -> uint32 so that "closer" == smaller. */
static inline uint32_t ord_of(float d, int metric) {
    if (metric == ORACLE_IP) d = -d;
    uint32_t u;
    memcpy(&u, &d, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
static inline float dist_of(uint32_t o, int metric) {
    uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    float d;
    memcpy(&d, &u, 4);
    return metric == ORACLE_IP ? -d : d;
}
/* key = ord(dist) : id : expanded-bit.  ids are unique in a beam (apart from
 * duplicated entry points), so the expanded bit never decides an ordering. */
static inline uint64_t make_key(float d, int id, int expanded, int metric) {
    return ((uint64_t)ord_of(d, metric) << 32) | ((uint64_t)(uint32_t)id << 1) | (uint64_t)(expanded & 1);
}
static int cmp_u64(const void* a, const void* b) {
    uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
    return x < y ? -1 : (x > y ? 1 : 0);
}

typedef struct {
    uint32_t* bits;   /* N-bit exact visited set (the reference's bitset) */
    int* touched;     /* ids set this query, for O(visited) clearing */
    int n_touched, cap_touched;
    uint64_t* beam;   /* <= L keys, sorted */
    uint64_t* cand;   /* candidates of the current round */
    int cap_cand;
} scratch_t;

static int test_and_set(scratch_t* s, int id) {
    uint32_t m = 1u << (id & 31), *w = s->bits + (id >> 5);
    if (*w & m) return 1;
    *w |= m;
    if (s->n_touched == s->cap_touched) {
        s->cap_touched *= 2;
        s->touched = (int*)realloc(s->touched, sizeof(int) * (size_t)s->cap_touched);
    }
    s->touched[s->n_touched++] = id;
    return 0;
}

/*
 * order: 0 = the reference's orders (seeds: lane tree; neighbours: sequential)
 *        1 = lane tree for every distance (what a warp-cooperative reduction
 *            would give; used only to measure how often the order matters)
 * adj:   int32[n][deg_pad], entries < 0 are padding (the reference stores
 *        deg + nbrs[0..deg), include/disk_graph.h:30-35).
 * Returns 0, or -1 on bad arguments.
 */
int coral_oracle_search(const float* base, int64_t n, int dim, const int32_t* adj, int deg_pad,
                        const int32_t* start_ids, int M, const float* queries, int Q, int L, int k,
                        int metric, int order, int32_t* ids_out, float* dists_out,
                        int32_t* stats_out, int n_threads) {
    if (!base || !adj || !start_ids || !queries || n <= 0 || dim <= 0 || deg_pad <= 0 || M <= 0 ||
        M > L || k <= 0 || k > L || Q < 0)
        return -1;
    for (int i = 0; i < M; ++i)
        if (start_ids[i] < 0 || start_ids[i] >= n) return -1;
#ifdef _OPENMP
    if (n_threads <= 0) n_threads = omp_get_max_threads();
#else
    n_threads = 1;
#endif
    const size_t words = (size_t)((n + 31) / 32);
    const float far0 = farthest_of(metric);

#pragma omp parallel num_threads(n_threads)
    {
        scratch_t s;
        s.bits = (uint32_t*)calloc(words, 4);
        s.cap_touched = 1 << 16;
        s.touched = (int*)malloc(sizeof(int) * (size_t)s.cap_touched);
        s.beam = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(L + 1));
        s.cap_cand = L * deg_pad + 1;
        s.cand = (uint64_t*)malloc(sizeof(uint64_t) * ((size_t)s.cap_cand + (size_t)L));

#pragma omp for schedule(dynamic, 1)
        for (int qi = 0; qi < Q; ++qi) {
            const float* q = queries + (size_t)qi * dim;
            int nbeam = 0, n_dist = 0, n_exp = 0, rounds = 0, hops = 0, n_scan = 0, max_cand = 0;
            float worst = far0;
            s.n_touched = 0;

            for (int i = 0; i < M; ++i) { /* src/search_gpu.cu:392-407 */
                int id = start_ids[i];
                (void)test_and_set(&s, id);
                float d = coral_oracle_dist_tree(base + (size_t)id * dim, q, dim, metric);
                s.beam[nbeam++] = make_key(d, id, 0, metric);
                ++n_dist;
            }
            qsort(s.beam, (size_t)nbeam, 8, cmp_u64);

            for (;;) {
                ++rounds;
                int nc = 0;
                for (int bi = 0; bi < nbeam; ++bi) { /* src/search_gpu.cu:415-438 */
                    if (s.beam[bi] & 1u) continue;
                    s.beam[bi] |= 1u;
                    ++n_exp;
                    int id = (int)((uint32_t)(s.beam[bi] & 0xffffffffu) >> 1);
                    const int32_t* nb = adj + (size_t)id * deg_pad;
                    for (int j = 0; j < deg_pad; ++j) {
                        int v = nb[j];
                        if (v < 0) continue;
                        ++n_scan;
                        if (test_and_set(&s, v)) continue;
                        const float* row = base + (size_t)v * dim;
                        float d = order == 0 ? coral_oracle_dist_seq(row, q, dim, metric)
                                             : coral_oracle_dist_tree(row, q, dim, metric);
                        ++n_dist;
                        if (closer(worst, d, metric)) s.cand[nc++] = make_key(d, v, 0, metric);
                    }
                }
                if (nc > max_cand) max_cand = nc;
                if (nc == 0) break; /* :442 */
                hops += nc;         /* :481,:574 */
                if (nbeam + nc <= L) { /* :477-483 */
                    memcpy(s.beam + nbeam, s.cand, 8 * (size_t)nc);
                    nbeam += nc;
                    qsort(s.beam, (size_t)nbeam, 8, cmp_u64);
                } else { /* :525-576 -> the L closest of the union */
                    memcpy(s.cand + nc, s.beam, 8 * (size_t)nbeam);
                    qsort(s.cand, (size_t)(nc + nbeam), 8, cmp_u64);
                    memcpy(s.beam, s.cand, 8 * (size_t)L);
                    nbeam = L;
                    worst = dist_of((uint32_t)(s.beam[L - 1] >> 32), metric);
                }
            }

            for (int i = 0; i < k; ++i) { /* :447-472 */
                if (i < nbeam) {
                    ids_out[(size_t)qi * k + i] = (int32_t)((uint32_t)(s.beam[i] & 0xffffffffu) >> 1);
                    if (dists_out) dists_out[(size_t)qi * k + i] = dist_of((uint32_t)(s.beam[i] >> 32), metric);
                } else {
                    ids_out[(size_t)qi * k + i] = -1;
                    if (dists_out) dists_out[(size_t)qi * k + i] = far0;
                }
            }
            if (stats_out) {
                int32_t* st = stats_out + (size_t)qi * STATS_W;
                st[0] = nbeam < L ? ST_BEAM_UNDERFULL : ST_OK; /* the reference asserts this, :444 */
                st[1] = n_dist;
                st[2] = n_exp;
                st[3] = rounds;
                st[4] = hops;
                st[5] = n_scan;
                st[6] = max_cand;
                st[7] = s.n_touched;
            }
            for (int i = 0; i < s.n_touched; ++i) s.bits[s.touched[i] >> 5] = 0;
        }
        free(s.bits);
        free(s.touched);
        free(s.beam);
        free(s.cand);
    }
    return 0;
}

/* Exact k-way merge of per-shard results, the definition the shard-merge
 * kernel is checked against: input keys[G][Q][k] as (id, dist) pairs, output
 * the k closest per query by (distance, id); ids < 0 are padding. */
int coral_oracle_merge_shards(const int32_t* ids, const float* dists, int G, int Q, int k, int metric,
                              int32_t* ids_out, float* dists_out) {
    if (G <= 0 || Q < 0 || k <= 0) return -1;
    uint64_t* buf = (uint64_t*)malloc(8 * (size_t)G * (size_t)k);
    const float far0 = farthest_of(metric);
    for (int qi = 0; qi < Q; ++qi) {
        int m = 0;
        for (int g = 0; g < G; ++g)
            for (int i = 0; i < k; ++i) {
                size_t o = ((size_t)g * Q + qi) * k + i;
                if (ids[o] < 0) continue;
                buf[m++] = make_key(dists[o], ids[o], 0, metric);
            }
        qsort(buf, (size_t)m, 8, cmp_u64);
        for (int i = 0; i < k; ++i) {
            if (i < m) {
                ids_out[(size_t)qi * k + i] = (int32_t)((uint32_t)(buf[i] & 0xffffffffu) >> 1);
                dists_out[(size_t)qi * k + i] = dist_of((uint32_t)(buf[i] >> 32), metric);
            } else {
                ids_out[(size_t)qi * k + i] = -1;
                dists_out[(size_t)qi * k + i] = far0;
            }
        }
    }
    free(buf);
    return 0;
}

/* tests/test_search_pipeline.cpp:25-39 */
double coral_oracle_recall(const int32_t* res, const int32_t* gt, int Q, int k, int gt_dim) {
    long hit = 0;
    for (int qi = 0; qi < Q; ++qi)
        for (int j = 0; j < k; ++j) {
            int p = gt[(size_t)qi * gt_dim + j];
            for (int i = 0; i < k; ++i)
                if (res[(size_t)qi * k + i] == p) {
                    ++hit;
                    break;
                }
        }
    return Q > 0 ? (double)hit / ((double)k * Q) : 0.0;
}

/* Entry-point selection: farthest-point sampling over BFS hop counts, restating
 * Graph::FPS (src/start.cu:72-145) with its helpers bfs (:53-70), bfs_expand_kernel
 * (:31-51), update_min_hop_kernel (:20-29) and the ArgMax at :122-126.  The reference draws
 * the first node from std::random_device (:77-86); here the caller names it (`first`, which
 * must have out-degree > 0 like the reference insists), so the result is reproducible.
 * min_hops starts at INT_MAX; after every BFS a node keeps the smallest hop count seen, a
 * node never reached yet becomes -1, and the next start is the FIRST index holding the
 * largest min_hops (CUB ArgMax returns the lowest index among equals).
 * Returns the number of ids written (== M), or -1 on bad arguments. */
int coral_oracle_select_start_ids(const int32_t* adj, int64_t n, int deg_pad, int first, int M, int32_t* out) {
    if (!adj || !out || n <= 0 || deg_pad <= 0 || M <= 0 || first < 0 || first >= n) return -1;
    int* hops = (int*)malloc(sizeof(int) * (size_t)n);
    int* min_hops = (int*)malloc(sizeof(int) * (size_t)n);
    int* queue = (int*)malloc(sizeof(int) * (size_t)n);
    for (int64_t i = 0; i < n; ++i) min_hops[i] = 2147483647;
    int start = first, count = 0;
    out[count++] = start;
    while (count < M) {
        for (int64_t i = 0; i < n; ++i) hops[i] = -1;
        int head = 0, tail = 0;
        hops[start] = 0;
        queue[tail++] = start;
        while (head < tail) { /* level-synchronous BFS == FIFO BFS for hop counts */
            int u = queue[head++];
            const int32_t* nb = adj + (size_t)u * deg_pad;
            for (int j = 0; j < deg_pad; ++j) {
                int v = nb[j];
                if (v < 0 || v >= n) continue;
                if (hops[v] == -1) {
                    hops[v] = hops[u] + 1;
                    queue[tail++] = v;
                }
            }
        }
        int best = -2147483647 - 1, best_i = 0;
        for (int64_t i = 0; i < n; ++i) {
            int h = hops[i];
            if (h >= 0) {
                if (h < min_hops[i] || min_hops[i] < 0) min_hops[i] = h;
            } else if (min_hops[i] == 2147483647) {
                min_hops[i] = -1;
            }
            if (min_hops[i] > best) {
                best = min_hops[i];
                best_i = (int)i;
            }
        }
        start = best_i;
        out[count++] = start;
    }
    free(hops);
    free(min_hops);
    free(queue);
    return count;
}
