// C ABI of the beam-search path: handle management, shared-memory planning,
// host<->device staging, the small companion kernels (hit count, shard merge,
// id mapping).  There is no CPU fallback: without a CUDA device every entry
// point that needs one returns CORAL_ERR_NOGPU.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../include/coral_b200.h"
#include "build.cuh"
#include "dense_topk.cuh"
#include "plan.cuh"
#include "schedule.cuh"
#include "search_kernel.cuh"
#include "start_select.cuh"

using coral::SearchArgs;
using coral::SearchPlan;

namespace {

thread_local std::string g_create_error;

// Control block shared with the kernel: word 0 = query counter | error flag, word 1 = hop
// total, words 4..8 = record of the first failed index check (self-checking build only).
constexpr int kCtrlWords = 16;
constexpr int kMaxFrontier = 4096;   // entry points' neighbours used by the scheduling pre-pass

struct Options {
    // Defaults from a sweep on 10M x 512 (one B200): many small CTAs beat few large ones, one
    // 256-byte stage per warp beats deeper rings, and shared memory spent on more resident
    // CTAs beats spending it on a shared-memory visited table.
    int ctas_per_sm = 0;  // 0 = as many as shared memory allows (at most 8)
    int warps = 0;        // 0 = 3..6, whichever keeps most warps resident per SM
    int chunk_bytes = 0;   // bytes of a row moved by one bulk copy: 0 = automatic (about 256, see make_plan)
    int stages = 0;  // 0 = one stage when ctas_per_sm is automatic, else as many as fit (at most 6)
    int smem_hash_bits = 0;
    int ghash_factor = 8;  // global visited table entries >= factor * L * deg_pad
    int ghash_entries = 0; // explicit table size (power of two >= 64), 0 = from ghash_factor
    int max_rounds = 1 << 16;
    int cluster_size = 0;  // CTAs sharing one query in small batches: 0 = automatic, 1 = never, else 2/4/8/16
    int scout_ids = 0;     // neighbour ids per lane per scout step: 0 = automatic (4; 1 in cluster mode), else 1..4
    int visit_cache_bits = 0;  // shared-memory cache of recently seen ids in front of the visited table (log2 entries)
    int sort_tile = 0;     // candidate sort tile in keys: 0 = automatic (about twice the beam capacity)
    int probe_carry = 1;   // carry ids the first probe pair leaves open into the next scout step (0 = settle them at once)
    int gather = -1;       // row chunks to shared memory: 0 = one bulk copy per row chunk, 1 = 16-byte unit copies,
                           // 2 = tensor copies gathering four rows each, -1 = automatic (2 when the driver encodes tensor maps)
    int schedule = 0;      // order large batches for L2 locality: 0 = automatic (batches >= 8192), 1 = always, -1 = never
    int schedule_tc = 1;   // scheduling keys on the tensor cores (1) or by the fp32 SIMT tile kernel (0)
    int dense_passes = 3;  // tf32 passes of the dense scans behind coral_exact_knn: 3 = fp32-grade, 1 = plain tf32
};

}  // namespace

struct coral_index {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    int64_t n = 0;
    int64_t live_n = 0;   // rows [0, live_n) are part of the index; the rest wait to be inserted
    int dim = 0, max_degree = 0, deg_pad = 0, metric = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_t0 = nullptr, ev_k0 = nullptr, ev_k1 = nullptr, ev_t1 = nullptr;

    float* d_vecs = nullptr;
    bool own_vecs = false;
    int32_t* d_adj = nullptr;
    int32_t* d_start = nullptr;
    int M = 0;
    uint32_t* d_deleted = nullptr;

    Options opt;
    bool prepared = false;
    int max_q = 0, max_L = 0, max_k = 0;
    int grid_cap = 0;
    uint32_t gh_entries = 0;
    uint32_t epoch_base = 0;
    uint64_t* d_ghash = nullptr;
    uint64_t* d_gcand = nullptr;
    coral::ClusterCtl* d_cctl = nullptr;  // small-batch (cluster) mode: per-cluster round state
    int32_t* d_gexp = nullptr;            // and expansion lists
    int last_cluster_size = 1;
    // locality scheduling: the entry points' neighbours ("frontier") and per-batch scratch
    std::vector<int32_t> h_start;
    bool frontier_dirty = true;
    int n_front = 0;
    int32_t* d_front_ids = nullptr;
    float* d_front_vecs = nullptr;
    float* d_front_norm = nullptr;
    int* d_keys = nullptr;
    int* d_bins = nullptr;
    int32_t* d_order = nullptr;
    int* d_sort_scratch = nullptr;
    void* d_sched_ws = nullptr;      // dense-scan workspace of the scheduling pre-pass
    int sched_q_cap = 0, sched_split = 1;
    int32_t* d_sched_ids = nullptr;  // [sched_q_cap] best frontier row of each query of a chunk
    int last_scheduled = 0;
    int last_plan_key = -1;   // plans[] key of the most recent search or prepare
    size_t cand_cap_alloc = 0;
    float* d_queries = nullptr;
    int32_t* d_ids = nullptr;
    float* d_dists = nullptr;
    int32_t* d_stats = nullptr;
    unsigned long long* d_ctrl = nullptr;  // [0] q_counter(int) | err(int), [1] hops_total
    unsigned long long* h_ctrl = nullptr;  // pinned mirror
    int64_t* d_hits = nullptr;
    std::map<int, std::pair<SearchPlan, int>> plans;  // L -> (plan, CTAs per SM)

    // graph build (NAP + CE): distances of the stored edges, degrees, claim words, batch scratch
    float* d_ndist = nullptr;
    int32_t* d_deg = nullptr;
    uint32_t* d_claim = nullptr;
    void* d_nap_scratch = nullptr;
    size_t nap_scratch_bytes = 0;
    bool building = false;

    // dense tensor-core scans (exact k-NN): workspace kept between calls
    void* d_dense = nullptr;
    size_t dense_bytes = 0;
    float last_dense_ms = 0.f;
    double last_dense_flops = 0.0;

    float last_kernel_ms = 0.f, last_total_ms = 0.f;
    int64_t launches = 0;
    std::string err;
};

namespace {

int fail(coral_index* h, int code, const std::string& msg) {
    if (h)
        h->err = msg;
    else
        g_create_error = msg;
    return code;
}

#define CK(call)                                                                                  \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            cudaGetLastError();                                                                   \
            return fail(h, CORAL_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_));   \
        }                                                                                         \
    } while (0)

bool is_device_ptr(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

int next_pow2(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

coral::PlanOptions plan_options(const Options& o) {
    coral::PlanOptions p;
    p.ctas_per_sm = o.ctas_per_sm;
    p.warps = o.warps;
    p.chunk_bytes = o.chunk_bytes;
    p.stages = o.stages;
    p.smem_hash_bits = o.smem_hash_bits;
    p.visit_cache_bits = o.visit_cache_bits;
    p.sort_tile = o.sort_tile;
    p.probe_carry = o.probe_carry;
    p.gather = o.gather < 0 ? (coral::row_gather_available() ? 2 : 0) : o.gather;
    return p;
}

// `small_batch`: the batch cannot fill the GPU, so latency per query matters more than
// resident warps per SM: 8-warp CTAs (faster merges, more scouts per query) measured best for
// batches of 1..512 on 10M x 512 (batch 1: 377 us against 601 us with the throughput plan).
int get_plan(coral_index* h, int L, SearchPlan& p, int& per_sm, bool small_batch = false) {
    const bool tuned = h->opt.warps > 0 || h->opt.ctas_per_sm > 0;
    const int key = 2 * L + ((small_batch && !tuned) ? 1 : 0);
    auto it = h->plans.find(key);
    h->last_plan_key = key;
    if (it != h->plans.end()) {
        p = it->second.first;
        per_sm = it->second.second;
        return CORAL_OK;
    }
    const char* why = "no plan";
    const coral::PlanOptions po = plan_options(h->opt);
    const bool ok = (key & 1) ? coral::make_plan_warps(h->dim, h->smem_optin, po, L, 8, p, &why)
                              : coral::make_plan(h->dim, h->smem_optin, po, L, p, &why);
    if (!ok) return fail(h, CORAL_ERR_ARG, why);
    per_sm = coral::beam_search_occupancy(p, h->metric);
    if (per_sm <= 0) return fail(h, CORAL_ERR_CUDA, "kernel does not fit an SM with this plan");
    per_sm = std::min(per_sm, p.ctas_per_sm);
    h->plans[key] = {p, per_sm};
    return CORAL_OK;
}

// ------------------------------------------------------------------ companion kernels

__global__ void count_hits_kernel(const int32_t* __restrict__ res, const int32_t* __restrict__ gt, int Q, int k,
                                  int gt_dim, unsigned long long* hits) {
    unsigned long long local = 0;
    const long long total = (long long)Q * k;
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
         t += (long long)gridDim.x * blockDim.x) {
        const int q = (int)(t / k), j = (int)(t % k);
        const int p = gt[(size_t)q * gt_dim + j];
        const int32_t* r = res + (size_t)q * k;
        for (int i = 0; i < k; ++i)
            if (r[i] == p) {
                ++local;
                break;
            }
    }
    for (int off = 16; off > 0; off >>= 1) local += __shfl_down_sync(0xffffffffu, local, off);
    if ((threadIdx.x & 31) == 0 && local) atomicAdd(hits, local);
}

__device__ __forceinline__ uint32_t ord32(float d, int metric) {
    if (metric == 1) d = -d;
    uint32_t u = __float_as_uint(d);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unord32(uint32_t o, int metric) {
    uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    float d = __uint_as_float(u);
    return metric == 1 ? -d : d;
}

// One warp per query: the G*k per-shard results are sorted by (distance, id) in
// shared memory and the first k written out.
__global__ void merge_shards_kernel(const int32_t* __restrict__ ids, const float* __restrict__ dists, int G,
                                    int Q, int k, long long g_stride, int n2, int metric,
                                    int32_t* __restrict__ ids_out, float* __restrict__ dists_out) {
    extern __shared__ unsigned long long msm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    unsigned long long* s = msm + (size_t)warp * n2;
    for (int q = blockIdx.x * wpb + warp; q < Q; q += gridDim.x * wpb) {
        for (int i = lane; i < n2; i += 32) {
            unsigned long long key = ~0ull;
            if (i < G * k) {
                const int g = i / k, j = i - g * k;
                const size_t o = (size_t)g * g_stride + (size_t)q * k + j;
                const int id = ids[o];
                if (id >= 0) key = ((unsigned long long)ord32(dists[o], metric) << 32) | (uint32_t)id;
            }
            s[i] = key;
        }
        __syncwarp();
        for (int kk = 2; kk <= n2; kk <<= 1)
            for (int j = kk >> 1; j > 0; j >>= 1) {
                for (int i = lane; i < n2; i += 32) {
                    const int ixj = i ^ j;
                    if (ixj > i) {
                        const unsigned long long a = s[i], b = s[ixj];
                        if ((a > b) == ((i & kk) == 0)) {
                            s[i] = b;
                            s[ixj] = a;
                        }
                    }
                }
                __syncwarp();
            }
        for (int i = lane; i < k; i += 32) {
            const unsigned long long key = s[i];
            if (key == ~0ull) {
                ids_out[(size_t)q * k + i] = -1;
                dists_out[(size_t)q * k + i] = metric == 0 ? 3.402823466e+38f : -3.402823466e+38f;
            } else {
                ids_out[(size_t)q * k + i] = (int32_t)(uint32_t)key;
                dists_out[(size_t)q * k + i] = unord32((uint32_t)(key >> 32), metric);
            }
        }
        __syncwarp();
    }
}

__global__ void map_ids_kernel(int32_t* ids, long long count, const int32_t* __restrict__ id_map) {
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < count;
         t += (long long)gridDim.x * blockDim.x) {
        const int v = ids[t];
        if (v >= 0) ids[t] = id_map[v];
    }
}

int ensure_device(coral_index* h) {
    CK(cudaSetDevice(h->device));
    return CORAL_OK;
}

void free_search(coral_index* h) {
    cudaFree(h->d_ghash);   h->d_ghash = nullptr;
    cudaFree(h->d_gcand);   h->d_gcand = nullptr;
    cudaFree(h->d_cctl);    h->d_cctl = nullptr;
    cudaFree(h->d_gexp);    h->d_gexp = nullptr;
    cudaFree(h->d_keys);    h->d_keys = nullptr;
    cudaFree(h->d_bins);    h->d_bins = nullptr;
    cudaFree(h->d_order);   h->d_order = nullptr;
    cudaFree(h->d_sort_scratch); h->d_sort_scratch = nullptr;
    cudaFree(h->d_sched_ws);     h->d_sched_ws = nullptr;
    cudaFree(h->d_sched_ids);    h->d_sched_ids = nullptr;
    cudaFree(h->d_queries); h->d_queries = nullptr;
    cudaFree(h->d_ids);     h->d_ids = nullptr;
    cudaFree(h->d_dists);   h->d_dists = nullptr;
    cudaFree(h->d_stats);   h->d_stats = nullptr;
    h->prepared = false;
    h->plans.clear();
}

}  // namespace

extern "C" {

int coral_version(void) { return 200; }

int coral_plan(int dim, int L, int smem_optin_bytes, int* out8) {
    if (dim <= 0 || dim % 4 != 0 || L <= 0 || L > 4096 || smem_optin_bytes <= 0 || !out8) return CORAL_ERR_ARG;
    SearchPlan p;
    const char* why = nullptr;
    if (!coral::make_plan(dim, smem_optin_bytes, coral::PlanOptions{}, L, p, &why)) return CORAL_ERR_LIMIT;
    out8[0] = p.warps;
    out8[1] = p.ctas_per_sm;
    out8[2] = p.chunk_bytes;
    out8[3] = p.n_chunks;
    out8[4] = p.stages;
    out8[5] = p.smem_bytes;
    out8[6] = p.tile_max;
    out8[7] = p.LP;
    return CORAL_OK;
}

// Test hook (not part of the declared ABI): index of the (device, metric, kernel variant) slot in
// the per-device cache of granted shared-memory sizes, -1 when the device is not cached.
int coral_internal_grant_slot(int device, int metric, int cluster) {
    static int table[coral::kMaxGrantDevices * 4];
    int* s = coral::granted_slot(table, device, metric, cluster != 0);
    return s ? (int)(s - table) : -1;
}
int coral_compiled_sm(void) { return 100; }

const char* coral_last_error(coral_index_t* h) { return h ? h->err.c_str() : g_create_error.c_str(); }

int coral_index_create(coral_index_t** out, int device, int64_t n, int dim, int max_degree, int metric) {
    coral_index* h = nullptr;
    if (!out) return fail(h, CORAL_ERR_ARG, "out is null");
    *out = nullptr;
    if (n <= 0 || n > 0x7fffffffll) return fail(h, CORAL_ERR_ARG, "n must be in [1, 2^31)");
    if (dim <= 0 || dim % 4 != 0) return fail(h, CORAL_ERR_ARG, "dim must be a positive multiple of 4");
    if (max_degree <= 0 || max_degree > 128) return fail(h, CORAL_ERR_ARG, "max_degree must be in [1, 128]");
    if (metric != CORAL_L2 && metric != CORAL_IP) return fail(h, CORAL_ERR_ARG, "metric must be CORAL_L2 or CORAL_IP");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(h, CORAL_ERR_NOGPU, "no CUDA device: this library has no CPU fallback");
    }
    if (device < 0 || device >= count) return fail(h, CORAL_ERR_ARG, "device index out of range");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        cudaGetLastError();
        return fail(h, CORAL_ERR_CUDA, "cudaGetDeviceProperties failed");
    }
    if (prop.major != 10) return fail(h, CORAL_ERR_NOGPU, "kernels are built for sm_100a only");
    h = new (std::nothrow) coral_index();
    if (!h) return fail(nullptr, CORAL_ERR_CUDA, "out of host memory");
    h->device = device;
    h->sm_count = prop.multiProcessorCount;
    h->smem_optin = (int)prop.sharedMemPerBlockOptin;
    h->n = n;
    h->live_n = n;
    h->dim = dim;
    h->max_degree = max_degree;
    h->deg_pad = max_degree <= 32 ? 32 : (max_degree <= 64 ? 64 : 128);
    h->metric = metric;
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&h->ev_t0);
    if (e == cudaSuccess) e = cudaEventCreate(&h->ev_k0);
    if (e == cudaSuccess) e = cudaEventCreate(&h->ev_k1);
    if (e == cudaSuccess) e = cudaEventCreate(&h->ev_t1);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_ctrl, kCtrlWords * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMallocHost(&h->h_ctrl, kCtrlWords * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMalloc(&h->d_hits, sizeof(int64_t));
    if (e != cudaSuccess) {
        cudaGetLastError();
        std::string msg = std::string("handle set-up: ") + cudaGetErrorString(e);
        coral_index_destroy(h);
        return fail(nullptr, CORAL_ERR_CUDA, msg);
    }
    *out = h;
    return CORAL_OK;
}

int coral_index_destroy(coral_index_t* h) {
    if (!h) return CORAL_OK;
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    free_search(h);
    if (h->own_vecs) cudaFree(h->d_vecs);
    cudaFree(h->d_adj);
    cudaFree(h->d_start);
    cudaFree(h->d_deleted);
    cudaFree(h->d_front_ids);
    cudaFree(h->d_front_vecs);
    cudaFree(h->d_front_norm);
    cudaFree(h->d_ctrl);
    cudaFree(h->d_hits);
    cudaFree(h->d_dense);
    cudaFree(h->d_ndist);
    cudaFree(h->d_deg);
    cudaFree(h->d_claim);
    cudaFree(h->d_nap_scratch);
    if (h->h_ctrl) cudaFreeHost(h->h_ctrl);
    if (h->ev_t0) cudaEventDestroy(h->ev_t0);
    if (h->ev_k0) cudaEventDestroy(h->ev_k0);
    if (h->ev_k1) cudaEventDestroy(h->ev_k1);
    if (h->ev_t1) cudaEventDestroy(h->ev_t1);
    if (h->stream) cudaStreamDestroy(h->stream);
    cudaGetLastError();
    delete h;
    return CORAL_OK;
}

int coral_index_set_vectors(coral_index_t* h, const float* vecs) {
    if (!h || !vecs) return fail(h, CORAL_ERR_ARG, "null argument");
    if (int rc = ensure_device(h)) return rc;
    const size_t bytes = (size_t)h->n * h->dim * sizeof(float);
    if (h->own_vecs) cudaFree(h->d_vecs);
    h->d_vecs = nullptr;
    h->own_vecs = false;
    CK(cudaMalloc(&h->d_vecs, bytes));
    h->own_vecs = true;
    h->frontier_dirty = true;
    CK(cudaMemcpyAsync(h->d_vecs, vecs, bytes, cudaMemcpyDefault, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    return CORAL_OK;
}

int coral_index_write_vectors(coral_index_t* h, int64_t first_row, int64_t count, const float* vecs) {
    if (!h || !vecs || first_row < 0 || count < 0 || first_row + count > h->n) return fail(h, CORAL_ERR_ARG, "rows out of range");
    if (int rc = ensure_device(h)) return rc;
    if (!h->d_vecs) {
        CK(cudaMalloc(&h->d_vecs, (size_t)h->n * h->dim * sizeof(float)));
        h->own_vecs = true;
    }
    if (!h->own_vecs) return fail(h, CORAL_ERR_STATE, "attached vectors are written by their owner");
    CK(cudaMemcpyAsync(h->d_vecs + (size_t)first_row * h->dim, vecs, (size_t)count * h->dim * sizeof(float), cudaMemcpyDefault,
                       h->stream));
    CK(cudaStreamSynchronize(h->stream));
    h->frontier_dirty = true;
    return CORAL_OK;
}

int coral_index_attach_vectors(coral_index_t* h, const float* dev_vecs) {
    if (!h || !dev_vecs) return fail(h, CORAL_ERR_ARG, "null argument");
    if (((uintptr_t)dev_vecs & 15) != 0) return fail(h, CORAL_ERR_ARG, "vectors must be 16-byte aligned");
    if (!is_device_ptr(dev_vecs)) return fail(h, CORAL_ERR_ARG, "attach needs a device pointer");
    if (int rc = ensure_device(h)) return rc;
    if (h->own_vecs) cudaFree(h->d_vecs);
    h->d_vecs = const_cast<float*>(dev_vecs);
    h->own_vecs = false;
    h->frontier_dirty = true;
    return CORAL_OK;
}

int coral_index_set_adjacency(coral_index_t* h, const int32_t* adj, int deg_pad) {
    if (!h || !adj) return fail(h, CORAL_ERR_ARG, "null argument");
    if (deg_pad != h->deg_pad) return fail(h, CORAL_ERR_ARG, "deg_pad must be max_degree rounded up to 32/64/128");
    if (int rc = ensure_device(h)) return rc;
    const size_t bytes = (size_t)h->n * deg_pad * sizeof(int32_t);
    if (!h->d_adj) CK(cudaMalloc(&h->d_adj, bytes));
    CK(cudaMemcpyAsync(h->d_adj, adj, bytes, cudaMemcpyDefault, h->stream));
    h->frontier_dirty = true;
    CK(cudaStreamSynchronize(h->stream));
    return CORAL_OK;
}

int coral_index_set_slots(coral_index_t* h, const int32_t* degs, size_t deg_stride, const int32_t* nbrs,
                          size_t nbr_stride) {
    if (!h || !degs || !nbrs || deg_stride == 0 || nbr_stride == 0) return fail(h, CORAL_ERR_ARG, "null argument");
    std::vector<int32_t> adj((size_t)h->n * h->deg_pad, -1);
    for (int64_t i = 0; i < h->n; ++i) {
        int deg = degs[(size_t)i * deg_stride];
        if (deg < 0) deg = 0;
        if (deg > h->max_degree) deg = h->max_degree;  // src/graph.cu:723-727
        const int32_t* nb = nbrs + (size_t)i * nbr_stride;
        int32_t* row = adj.data() + (size_t)i * h->deg_pad;
        int w = 0;
        for (int j = 0; j < deg; ++j)
            if (nb[j] >= 0 && (int64_t)nb[j] < h->n) row[w++] = nb[j];
    }
    return coral_index_set_adjacency(h, adj.data(), h->deg_pad);
}

int coral_index_set_start_ids(coral_index_t* h, const int32_t* ids, int M) {
    if (!h || !ids || M <= 0 || M > 4096) return fail(h, CORAL_ERR_ARG, "start ids: need 1..4096 ids");
    for (int i = 0; i < M; ++i)
        if (ids[i] < 0 || (int64_t)ids[i] >= h->n) return fail(h, CORAL_ERR_ARG, "start id out of range");
    if (int rc = ensure_device(h)) return rc;
    cudaFree(h->d_start);
    h->d_start = nullptr;
    CK(cudaMalloc(&h->d_start, (size_t)M * sizeof(int32_t)));
    CK(cudaMemcpyAsync(h->d_start, ids, (size_t)M * sizeof(int32_t), cudaMemcpyHostToDevice, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    h->M = M;
    h->h_start.assign(ids, ids + M);
    h->frontier_dirty = true;
    return CORAL_OK;
}

void* coral_index_stream(coral_index_t* h) { return h ? (void*)h->stream : nullptr; }

int coral_index_get_adjacency(coral_index_t* h, int32_t* adj_out) {
    if (!h || !adj_out) return fail(h, CORAL_ERR_ARG, "null argument");
    if (!h->d_adj) return fail(h, CORAL_ERR_STATE, "no adjacency set");
    if (int rc = ensure_device(h)) return rc;
    CK(cudaMemcpyAsync(adj_out, h->d_adj, (size_t)h->n * h->deg_pad * sizeof(int32_t), cudaMemcpyDefault, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    return CORAL_OK;
}

int coral_index_get_start_ids(coral_index_t* h, int32_t* ids_out, int capacity) {
    if (!h) return -1;
    if (ids_out)
        for (int i = 0; i < h->M && i < capacity; ++i) ids_out[i] = h->h_start[(size_t)i];
    return h->M;
}

int coral_index_select_start_ids(coral_index_t* h, int first_id, int M, int32_t* ids_out) {
    if (!h || M <= 0 || M > 4096) return fail(h, CORAL_ERR_ARG, "select start ids: need 1..4096 ids");
    if (first_id < 0 || (int64_t)first_id >= h->n) return fail(h, CORAL_ERR_ARG, "first id out of range");
    if (!h->d_adj) return fail(h, CORAL_ERR_STATE, "select start ids: no adjacency set");
    if (int rc = ensure_device(h)) return rc;
    std::vector<int32_t> row((size_t)h->deg_pad);
    CK(cudaMemcpyAsync(row.data(), h->d_adj + (size_t)first_id * h->deg_pad, row.size() * sizeof(int32_t),
                       cudaMemcpyDeviceToHost, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    bool has_edge = false;
    for (int32_t v : row) has_edge |= v >= 0 && (int64_t)v < h->n;
    if (!has_edge) return fail(h, CORAL_ERR_ARG, "first id has no out-edges");
    std::vector<int32_t> ids((size_t)M);
    CK(coral::select_start_ids(h->d_adj, h->n, h->deg_pad, first_id, M, ids.data(), h->sm_count, h->stream,
                               &h->launches));
    if (ids_out) std::copy(ids.begin(), ids.end(), ids_out);
    return coral_index_set_start_ids(h, ids.data(), M);
}

int coral_index_set_deleted(coral_index_t* h, const uint32_t* bits) {
    if (!h) return CORAL_ERR_ARG;
    if (int rc = ensure_device(h)) return rc;
    if (!bits) {
        cudaFree(h->d_deleted);
        h->d_deleted = nullptr;
        return CORAL_OK;
    }
    const size_t bytes = (size_t)((h->n + 31) / 32) * sizeof(uint32_t);
    if (!h->d_deleted) CK(cudaMalloc(&h->d_deleted, bytes));
    CK(cudaMemcpyAsync(h->d_deleted, bits, bytes, cudaMemcpyDefault, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    return CORAL_OK;
}

int coral_set_option(coral_index_t* h, const char* name, int value) {
    if (!h || !name) return CORAL_ERR_ARG;
    Options& o = h->opt;
    std::string s(name);
    if (s == "ctas_per_sm") o.ctas_per_sm = value;
    else if (s == "warps") o.warps = value;
    else if (s == "chunk_bytes") o.chunk_bytes = value;
    else if (s == "stages") o.stages = value;
    else if (s == "smem_hash_bits") o.smem_hash_bits = value;
    else if (s == "ghash_factor") o.ghash_factor = value;
    else if (s == "ghash_entries") o.ghash_entries = value;
    else if (s == "max_rounds") o.max_rounds = value;
    else if (s == "cluster_size") o.cluster_size = value;
    else if (s == "scout_ids") o.scout_ids = value;
    else if (s == "schedule") o.schedule = value;
    else if (s == "sort_tile") o.sort_tile = value;
    else if (s == "visit_cache_bits") o.visit_cache_bits = value;
    else if (s == "gather") o.gather = value;
    else if (s == "probe_carry") o.probe_carry = value;
    else if (s == "dense_passes") o.dense_passes = value;
    else if (s == "schedule_tc") o.schedule_tc = value;
    else return fail(h, CORAL_ERR_ARG, "unknown option " + s);
    h->plans.clear();
    return CORAL_OK;
}

int coral_get_option(coral_index_t* h, const char* name, int* value) {
    if (!h || !name || !value) return CORAL_ERR_ARG;
    const Options& o = h->opt;
    std::string s(name);
    if (s == "ctas_per_sm") *value = o.ctas_per_sm;
    else if (s == "warps") *value = o.warps;
    else if (s == "chunk_bytes") *value = o.chunk_bytes;
    else if (s == "stages") *value = o.stages;
    else if (s == "smem_hash_bits") *value = o.smem_hash_bits;
    else if (s == "ghash_factor") *value = o.ghash_factor;
    else if (s == "ghash_entries") *value = (int)h->gh_entries;
    else if (s == "max_rounds") *value = o.max_rounds;
    else if (s == "cluster_size") *value = o.cluster_size;
    else if (s == "last_cluster_size") *value = h->last_cluster_size;
    else if (s == "schedule") *value = o.schedule;
    else if (s == "gather") *value = o.gather < 0 ? (coral::row_gather_available() ? 2 : 0) : o.gather;
    else if (s == "probe_carry") *value = o.probe_carry;
    else if (s == "dense_passes") *value = o.dense_passes;
    else if (s == "schedule_tc") *value = o.schedule_tc;
    else if (s == "sort_tile") *value = o.sort_tile;
    else if (s == "scout_ids") *value = o.scout_ids;
    else if (s == "visit_cache_bits") *value = o.visit_cache_bits;
    else if (s == "last_scheduled") *value = h->last_scheduled;
    else if (s == "frontier_size") *value = h->n_front;
    else if (s == "grid_cap") *value = h->grid_cap;
    else if (s == "deg_pad") *value = h->deg_pad;
    else if (s == "dim") *value = h->dim;
    else if (s.rfind("plan_", 0) == 0 && h->plans.count(h->last_plan_key)) {  // plan of the most recent search
        const auto& entry = h->plans[h->last_plan_key];
        const SearchPlan& p = entry.first;
        if (s == "plan_stages") *value = p.stages;
        else if (s == "plan_warps") *value = p.warps;
        else if (s == "plan_chunk_bytes") *value = p.chunk_bytes;
        else if (s == "plan_smem_bytes") *value = p.smem_bytes;
        else if (s == "plan_hash_bits") *value = p.hs_bits;
        else if (s == "plan_ctas_per_sm") *value = entry.second;
        else return fail(h, CORAL_ERR_ARG, "unknown option " + s);
    } else return fail(h, CORAL_ERR_ARG, "unknown option " + s);
    return CORAL_OK;
}

int coral_search_free(coral_index_t* h) {
    if (!h) return CORAL_ERR_ARG;
    if (int rc = ensure_device(h)) return rc;
    cudaStreamSynchronize(h->stream);
    free_search(h);
    return CORAL_OK;
}

int coral_search_prepare(coral_index_t* h, int max_queries, int max_L, int max_k) {
    if (!h || max_queries <= 0 || max_L <= 0 || max_k <= 0 || max_k > max_L || max_L > 4096)
        return fail(h, CORAL_ERR_ARG, "prepare: need max_queries > 0 and 0 < max_k <= max_L <= 4096");
    if (int rc = ensure_device(h)) return rc;
    cudaStreamSynchronize(h->stream);
    free_search(h);
    SearchPlan p;
    int per_sm = 0;
    if (int rc = get_plan(h, max_L, p, per_sm)) return rc;
    // smaller L never needs more CTAs than ctas_per_sm allows
    h->grid_cap = h->sm_count * (h->opt.ctas_per_sm <= 0 ? 8 : std::max(per_sm, h->opt.ctas_per_sm));
    h->max_q = max_queries;
    h->max_L = max_L;
    h->max_k = max_k;
    uint64_t want = (uint64_t)std::max(h->opt.ghash_factor, 2) * (uint64_t)max_L * (uint64_t)h->deg_pad;
    uint32_t ent = 1u << 14;
    while (ent < want && ent < (1u << 24)) ent <<= 1;
    if (h->opt.ghash_entries >= 64) {
        ent = 64;
        while (ent < (uint32_t)h->opt.ghash_entries && ent < (1u << 24)) ent <<= 1;
    }
    h->gh_entries = ent;
    h->cand_cap_alloc = (size_t)max_L * h->deg_pad;
    CK(cudaMalloc(&h->d_ghash, (size_t)h->grid_cap * ent * sizeof(uint64_t)));
    CK(cudaMemsetAsync(h->d_ghash, 0, (size_t)h->grid_cap * ent * sizeof(uint64_t), h->stream));
    h->epoch_base = 0;
    CK(cudaMalloc(&h->d_gcand, (size_t)h->grid_cap * h->cand_cap_alloc * sizeof(uint64_t)));
    CK(cudaMalloc(&h->d_cctl, (size_t)h->sm_count * sizeof(coral::ClusterCtl)));
    CK(cudaMalloc(&h->d_gexp, (size_t)h->sm_count * max_L * sizeof(int32_t)));
    CK(cudaMalloc(&h->d_keys, (size_t)max_queries * sizeof(int)));
    CK(cudaMalloc(&h->d_order, (size_t)max_queries * sizeof(int32_t)));
    CK(cudaMalloc(&h->d_bins, (size_t)kMaxFrontier * sizeof(int)));
    CK(cudaMalloc(&h->d_sort_scratch, coral::sort_scratch_ints(max_queries, kMaxFrontier) * sizeof(int)));
    if (h->opt.schedule >= 0 && max_queries >= 4096 && h->opt.schedule_tc != 0) {
        // tensor-core pre-pass: queries in chunks of one CTA per SM, the frontier as the "base"
        h->sched_q_cap = std::min(max_queries, h->sm_count * coral::kDenseTileM);
        const int q_tiles = (h->sched_q_cap + coral::kDenseTileM - 1) / coral::kDenseTileM;
        h->sched_split = std::max(1, std::min(kMaxFrontier / coral::kDenseTileN, h->sm_count / q_tiles));
        CK(cudaMalloc(&h->d_sched_ws, coral::dense_workspace_bytes(h->sched_q_cap, kMaxFrontier, h->dim, h->sched_split)));
        CK(cudaMalloc(&h->d_sched_ids, (size_t)h->sched_q_cap * sizeof(int32_t)));
    }
    CK(cudaMalloc(&h->d_queries, (size_t)max_queries * h->dim * sizeof(float)));
    CK(cudaMalloc(&h->d_ids, (size_t)max_queries * max_k * sizeof(int32_t)));
    CK(cudaMalloc(&h->d_dists, (size_t)max_queries * max_k * sizeof(float)));
    CK(cudaMalloc(&h->d_stats, (size_t)max_queries * CORAL_STATS_W * sizeof(int32_t)));
    CK(cudaStreamSynchronize(h->stream));
    h->prepared = true;
    return CORAL_OK;
}

// The frontier of the first expansion round -- the distinct neighbours of the entry points -- as
// a contiguous block of vectors for the scheduling pre-pass.  Rebuilt when vectors, graph or
// entry points change.  Synchronises h->stream (set-up path, not the search path).
static int ensure_frontier(coral_index* h) {
    if (!h->frontier_dirty) return CORAL_OK;
    h->frontier_dirty = false;
    h->n_front = 0;
    if (h->M > 64) return CORAL_OK;   // many entry points: the frontier would not be a cheap predictor
    std::vector<int32_t> rows((size_t)h->M * h->deg_pad);
    for (int i = 0; i < h->M; ++i)
        CK(cudaMemcpy(rows.data() + (size_t)i * h->deg_pad, h->d_adj + (size_t)h->h_start[i] * h->deg_pad,
                      (size_t)h->deg_pad * sizeof(int32_t), cudaMemcpyDeviceToHost));
    std::sort(rows.begin(), rows.end());
    rows.erase(std::unique(rows.begin(), rows.end()), rows.end());
    std::vector<int32_t> ids;
    for (int32_t v : rows)
        if (v >= 0 && (int64_t)v < h->n && (int)ids.size() < kMaxFrontier) ids.push_back(v);
    if (ids.size() < 2) return CORAL_OK;
    cudaFree(h->d_front_ids);
    cudaFree(h->d_front_vecs);
    cudaFree(h->d_front_norm);
    h->d_front_ids = nullptr;
    h->d_front_vecs = h->d_front_norm = nullptr;
    CK(cudaMalloc(&h->d_front_ids, ids.size() * sizeof(int32_t)));
    CK(cudaMalloc(&h->d_front_vecs, ids.size() * (size_t)h->dim * sizeof(float)));
    CK(cudaMalloc(&h->d_front_norm, ids.size() * sizeof(float)));
    CK(cudaMemcpyAsync(h->d_front_ids, ids.data(), ids.size() * sizeof(int32_t), cudaMemcpyHostToDevice, h->stream));
    CK(coral::gather_frontier(h->d_vecs, h->d_front_ids, (int)ids.size(), h->dim, h->d_front_vecs, h->d_front_norm,
                              h->stream));
    h->launches += 1;
    CK(cudaStreamSynchronize(h->stream));
    h->n_front = (int)ids.size();
    return CORAL_OK;
}

// h->d_order[0..Q) <- the batch ordered by each query's closest frontier row.  The scores are formed
// on the tensor cores (one tf32 pass of the dense scan, the 8 best re-ranked exactly, so the key is
// the exact nearest frontier row and does not depend on tensor-core rounding); option
// "schedule_tc" = 0 selects the fp32 SIMT tile kernel instead.
static int query_order(coral_index* h, const float* d_queries, int Q, cudaStream_t st) {
    if (h->d_sched_ws && h->opt.schedule_tc != 0) {
        coral::DenseWorkspace w;
        coral::dense_workspace_carve(h->d_sched_ws, h->sched_q_cap, kMaxFrontier, h->dim, h->sched_split, w);
        const int keep = 8;
        for (int q0 = 0; q0 < Q; q0 += h->sched_q_cap) {
            const int nq = std::min(h->sched_q_cap, Q - q0);
            const float* q = d_queries + (size_t)q0 * h->dim;
            CK(coral::dense_begin(w, q, nq, h->dim, st, &h->launches));
            CK(coral::dense_scan_chunk(w, q, nq, h->d_front_vecs, 0, h->n_front, h->dim, h->metric, 1, keep, h->sm_count, st,
                                       &h->launches));
            CK(coral::dense_finish(w, q, nq, h->d_front_vecs, h->dim, h->metric, 1, keep, 1, h->d_sched_ids, nullptr, nullptr,
                                   st, &h->launches));
            CK(coral::keys_from_ids(h->d_sched_ids, nq, 1, h->n_front, h->d_keys + q0, h->sm_count, st));
            h->launches += 1;
        }
    } else {
        CK(coral::frontier_keys_simt(d_queries, Q, h->dim, h->metric, h->d_front_vecs, h->d_front_norm, h->n_front, h->d_keys,
                                     st));
        h->launches += 1;
    }
    CK(coral::sort_queries_by_key(h->d_keys, Q, h->n_front, h->d_bins, h->d_sort_scratch, h->d_order, h->sm_count, st));
    h->launches += 4;
    return CORAL_OK;
}

static int enqueue_search(coral_index* h, const float* d_queries, int Q, int L, int k, int32_t* d_ids,
                          float* d_dists, int32_t* d_stats, cudaStream_t st) {
    if (!h->d_vecs || !h->d_adj || !h->d_start) return fail(h, CORAL_ERR_STATE, "vectors, graph and start ids must be set first");
    if (!h->prepared) return fail(h, CORAL_ERR_STATE, "coral_search_prepare has not been called");
    if (Q < 0 || L <= 0 || k <= 0 || k > L) return fail(h, CORAL_ERR_ARG, "need Q >= 0 and 0 < k <= L");
    if (h->M > L) return fail(h, CORAL_ERR_ARG, "more start ids than beam capacity L");
    if (Q > h->max_q || L > h->max_L || k > h->max_k) return fail(h, CORAL_ERR_LIMIT, "request exceeds coral_search_prepare sizes");
    SearchPlan p;
    int per_sm = 0;
    if (int rc = get_plan(h, L, p, per_sm, Q <= 4 * h->sm_count)) return rc;
    CK(cudaMemsetAsync(h->d_ctrl, 0, kCtrlWords * sizeof(unsigned long long), st));
    if (Q == 0) return CORAL_OK;
    if ((uint64_t)h->epoch_base + (uint64_t)Q + 2ull >= 0xFFFFFFFFull) {  // epochs would wrap: start over
        CK(cudaMemsetAsync(h->d_ghash, 0, (size_t)h->grid_cap * h->gh_entries * sizeof(uint64_t), st));
        h->epoch_base = 0;
    }
    SearchArgs a{};
    a.vecs = h->d_vecs;
    a.adj = h->d_adj;
    a.queries = d_queries;
    a.start_ids = h->d_start;
    a.deleted = h->d_deleted;
    a.ids_out = d_ids;
    a.dists_out = d_dists;
    a.stats_out = d_stats;
    a.q_counter = reinterpret_cast<int*>(h->d_ctrl);
    a.err_flag = reinterpret_cast<int*>(h->d_ctrl) + 1;
#ifdef CORAL_CHECKED
    a.dbg = reinterpret_cast<long long*>(h->d_ctrl + 4);
#else
    a.dbg = nullptr;
#endif
    a.hops_total = h->d_ctrl + 1;
    a.ghash = h->d_ghash;
    a.gcand = h->d_gcand;
    a.n = h->n;
    a.dim = h->dim;
    a.deg_pad = h->deg_pad;
    a.deg_shift = h->deg_pad == 32 ? 5 : (h->deg_pad == 64 ? 6 : 7);
    a.M = h->M;
    a.Q = Q;
    a.L = L;
    a.k = k;
    a.epoch_base = h->epoch_base;
    a.gh_mask = h->gh_entries - 1;
    a.cand_cap = (int)std::min<size_t>((size_t)L * h->deg_pad, h->cand_cap_alloc);
    a.max_rounds = h->opt.max_rounds;
    a.ids_per_lane = h->opt.scout_ids > 0 ? h->opt.scout_ids : 4;
    a.plan = p;
    int grid = std::min(Q, std::min(h->sm_count * per_sm, h->grid_cap));
    // Small batches leave most SMs idle with one CTA per query: let a thread-block cluster of
    // 2..16 CTAs share each query instead (needs the visited set entirely in the global table).
    int cs = 1;
    const int slots = h->sm_count * per_sm;   // CTAs resident at once
    if (h->opt.cluster_size != 1 && p.hs_bits == 0 && Q <= std::min(slots / 2, h->sm_count)) {
        // automatic: the largest cluster that still keeps every query's cluster resident
        cs = h->opt.cluster_size > 1 ? h->opt.cluster_size : 16;
        while (cs > 1 && (cs > 16 || (cs & (cs - 1)) != 0 || (h->opt.cluster_size <= 1 && Q * cs > slots))) cs >>= 1;
        int room = 0;
        while (cs > 1 && ((room = coral::beam_search_max_clusters(p, h->metric, cs)) < 1 ||
                          (h->opt.cluster_size <= 1 && room < Q)))
            cs >>= 1;
        if (cs > 1) {
            const int groups = std::min(Q, std::min(room, h->sm_count));
            grid = groups * cs;
            CK(cudaMemsetAsync(h->d_cctl, 0, (size_t)groups * sizeof(coral::ClusterCtl), st));
            a.cctl = h->d_cctl;
            a.gexp = h->d_gexp;
            // a round's short expansion list must spread over all the cluster's warps
            if (h->opt.scout_ids <= 0) a.ids_per_lane = 1;
        }
    }
    h->last_cluster_size = cs;
    // Large batches: run the queries grouped by their best frontier node (see schedule.cu).
    h->last_scheduled = 0;
    if (cs == 1 && h->opt.schedule >= 0 && (h->opt.schedule > 0 || Q >= 8192)) {
        if (int rc = ensure_frontier(h)) return rc;
        if (h->n_front >= 2) {
            if (int rc = query_order(h, d_queries, Q, st)) return rc;
            a.order = h->d_order;
            h->last_scheduled = 1;
        }
    }
    alignas(64) CUtensorMap row_map;
    const CUtensorMap* row_map_ptr = nullptr;
    if (p.gather == 2) {
        if (!coral::make_row_gather_map(&row_map, h->d_vecs, h->n, h->dim, p.chunk_bytes / 4))
            return fail(h, CORAL_ERR_CUDA, "could not encode the tensor map of the row array (gather = 2)");
        row_map_ptr = &row_map;
    }
    CK(coral::launch_beam_search(a, h->metric, grid, st, cs, row_map_ptr));
    h->launches += 1;
    h->epoch_base += (uint32_t)Q;
    CK(cudaMemcpyAsync(h->h_ctrl, h->d_ctrl, kCtrlWords * sizeof(unsigned long long), cudaMemcpyDeviceToHost, st));
    return CORAL_OK;
}

int coral_search_async(coral_index_t* h, const float* d_queries, int Q, int L, int k, int32_t* d_ids_out,
                       float* d_dists_out, int32_t* d_stats_out, void* stream) {
    if (!h || (!d_queries && Q > 0) || (!d_ids_out && Q > 0)) return fail(h, CORAL_ERR_ARG, "null argument");
    if (int rc = ensure_device(h)) return rc;
    cudaStream_t st = stream ? (cudaStream_t)stream : h->stream;
    return enqueue_search(h, d_queries, Q, L, k, d_ids_out, d_dists_out, d_stats_out, st);
}

int coral_query_order(coral_index_t* h, const float* d_queries, int Q, int32_t* d_order_out, void* stream) {
    if (!h || !d_queries || !d_order_out || Q <= 0) return fail(h, CORAL_ERR_ARG, "bad argument");
    if (!h->prepared) return fail(h, CORAL_ERR_STATE, "coral_search_prepare has not been called");
    if (Q > h->max_q) return fail(h, CORAL_ERR_LIMIT, "request exceeds coral_search_prepare sizes");
    if (int rc = ensure_device(h)) return rc;
    cudaStream_t st = stream ? (cudaStream_t)stream : h->stream;
    if (int rc = ensure_frontier(h)) return rc;
    if (h->n_front < 2) return fail(h, CORAL_ERR_STATE, "no frontier to order by (more than 64 entry points, or no edges)");
    if (int rc = query_order(h, d_queries, Q, st)) return rc;
    CK(cudaMemcpyAsync(d_order_out, h->d_order, (size_t)Q * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
    return CORAL_OK;
}

int coral_search_check(coral_index_t* h) {
    if (!h) return CORAL_ERR_ARG;
    const int err = reinterpret_cast<int*>(h->h_ctrl)[1];
    if (err) return fail(h, CORAL_ERR_KERNEL, "a bounded wait in the search kernel ran out; results are invalid");
#ifdef CORAL_CHECKED
    const long long* dbg = reinterpret_cast<const long long*>(h->h_ctrl + 4);
    if (dbg[0] != 0) {
        char msg[256];
        std::snprintf(msg, sizeof msg, "index check %lld failed: v0=%lld v1=%lld (0x%llx) query=%lld cta=%lld", dbg[0],
                      dbg[1], dbg[2], (unsigned long long)dbg[2], dbg[3], dbg[4]);
        return fail(h, CORAL_ERR_KERNEL, msg);
    }
#endif
    return CORAL_OK;
}

int coral_search(coral_index_t* h, const float* queries, int Q, int L, int k, int32_t* ids_out,
                 float* dists_out, int32_t* stats_out, int64_t* total_hops_out) {
    if (!h || (Q > 0 && (!queries || !ids_out))) return fail(h, CORAL_ERR_ARG, "null argument");
    if (int rc = ensure_device(h)) return rc;
    if (!h->prepared) return fail(h, CORAL_ERR_STATE, "coral_search_prepare has not been called");
    if (Q > h->max_q || k > h->max_k) return fail(h, CORAL_ERR_LIMIT, "request exceeds coral_search_prepare sizes");
    cudaStream_t st = h->stream;
    const bool q_dev = Q > 0 && is_device_ptr(queries);
    const bool i_dev = Q > 0 && is_device_ptr(ids_out);
    const bool d_dev = dists_out && is_device_ptr(dists_out);
    const bool s_dev = stats_out && is_device_ptr(stats_out);
    const float* dq = q_dev ? queries : h->d_queries;
    int32_t* di = i_dev ? ids_out : h->d_ids;
    float* dd = dists_out ? (d_dev ? dists_out : h->d_dists) : nullptr;
    int32_t* ds = stats_out ? (s_dev ? stats_out : h->d_stats) : nullptr;

    CK(cudaEventRecord(h->ev_t0, st));
    if (Q > 0 && !q_dev)
        CK(cudaMemcpyAsync(h->d_queries, queries, (size_t)Q * h->dim * sizeof(float), cudaMemcpyHostToDevice, st));
    CK(cudaEventRecord(h->ev_k0, st));
    if (int rc = enqueue_search(h, dq, Q, L, k, di, dd, ds, st)) return rc;
    CK(cudaEventRecord(h->ev_k1, st));
    if (Q > 0) {
        if (!i_dev) CK(cudaMemcpyAsync(ids_out, di, (size_t)Q * k * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        if (dists_out && !d_dev)
            CK(cudaMemcpyAsync(dists_out, dd, (size_t)Q * k * sizeof(float), cudaMemcpyDeviceToHost, st));
        if (stats_out && !s_dev)
            CK(cudaMemcpyAsync(stats_out, ds, (size_t)Q * CORAL_STATS_W * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    }
    CK(cudaEventRecord(h->ev_t1, st));
    CK(cudaStreamSynchronize(st));
    CK(cudaEventElapsedTime(&h->last_kernel_ms, h->ev_k0, h->ev_k1));
    CK(cudaEventElapsedTime(&h->last_total_ms, h->ev_t0, h->ev_t1));
    if (total_hops_out) *total_hops_out = Q > 0 ? (int64_t)h->h_ctrl[1] : 0;
    if (Q > 0)
        if (int rc = coral_search_check(h)) return rc;
    return CORAL_OK;
}

float coral_last_kernel_ms(coral_index_t* h) { return h ? h->last_kernel_ms : 0.f; }
float coral_last_total_ms(coral_index_t* h) { return h ? h->last_total_ms : 0.f; }
int64_t coral_launch_count(coral_index_t* h) { return h ? h->launches : 0; }

int coral_count_hits(coral_index_t* h, const int32_t* res, const int32_t* gt, int Q, int k, int gt_dim,
                     int64_t* hits_out) {
    if (!h || !res || !gt || !hits_out || Q < 0 || k <= 0 || gt_dim < k) return fail(h, CORAL_ERR_ARG, "bad argument");
    if (int rc = ensure_device(h)) return rc;
    *hits_out = 0;
    if (Q == 0) return CORAL_OK;
    cudaStream_t st = h->stream;
    int32_t *d_res = nullptr, *d_gt = nullptr;
    const bool r_dev = is_device_ptr(res), g_dev = is_device_ptr(gt);
    int rc = CORAL_OK;
    cudaError_t e = cudaSuccess;
    if (!r_dev) {
        e = cudaMalloc(&d_res, (size_t)Q * k * 4);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_res, res, (size_t)Q * k * 4, cudaMemcpyHostToDevice, st);
    }
    if (e == cudaSuccess && !g_dev) {
        e = cudaMalloc(&d_gt, (size_t)Q * gt_dim * 4);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_gt, gt, (size_t)Q * gt_dim * 4, cudaMemcpyHostToDevice, st);
    }
    if (e == cudaSuccess) e = cudaMemsetAsync(h->d_hits, 0, sizeof(int64_t), st);
    if (e == cudaSuccess) {
        const int blocks = (int)std::min<long long>(((long long)Q * k + 255) / 256, 4096);
        count_hits_kernel<<<blocks, 256, 0, st>>>(r_dev ? res : d_res, g_dev ? gt : d_gt, Q, k, gt_dim,
                                                  reinterpret_cast<unsigned long long*>(h->d_hits));
        h->launches += 1;
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(hits_out, h->d_hits, sizeof(int64_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        cudaGetLastError();
        rc = fail(h, CORAL_ERR_CUDA, std::string("count_hits: ") + cudaGetErrorString(e));
    }
    cudaFree(d_res);
    cudaFree(d_gt);
    return rc;
}

// Exact k-NN of `Q` queries over `n_rows` rows at d_rows (device), ids relative to d_rows.
static int exact_knn_over(coral_index* h, const float* d_rows, int64_t n_rows, const float* queries, int Q, int k,
                          int passes, int32_t* ids_out, float* dists_out, int64_t* uncertified_out) {
    if (k <= 0 || (int64_t)k > n_rows) return fail(h, CORAL_ERR_ARG, "exact knn: need 0 < k <= number of rows");
    int keep = k + 28;                                   // slack between the selection and the k that are returned
    if (keep > coral::kDenseMaxKeep) keep = coral::kDenseMaxKeep;
    if (k > keep) return fail(h, CORAL_ERR_LIMIT, "exact knn: k must not exceed 256");
    if (uncertified_out) *uncertified_out = 0;
    if (Q == 0) return CORAL_OK;
    cudaStream_t st = h->stream;
    const int q_chunk = h->sm_count * coral::kDenseTileM;          // one CTA per SM and query tile
    const int q_cap = std::min(Q, q_chunk);
    const int q_tiles = (q_cap + coral::kDenseTileM - 1) / coral::kDenseTileM;
    // base rows per scan launch: bounded by 2 GiB of split operands
    int64_t b_cap = std::min<int64_t>(n_rows, std::max<int64_t>(coral::kDenseTileN, ((int64_t)1 << 28) / h->dim));
    const int col_tiles = (int)((b_cap + coral::kDenseTileN - 1) / coral::kDenseTileN);
    int n_split = std::max(1, std::min(std::min(coral::kDenseMaxSplit, h->sm_count / q_tiles), col_tiles));
    const size_t need = coral::dense_workspace_bytes(q_cap, (int)b_cap, h->dim, n_split);
    if (need > h->dense_bytes) {
        cudaFree(h->d_dense);
        h->d_dense = nullptr;
        h->dense_bytes = 0;
        CK(cudaMalloc(&h->d_dense, need));
        h->dense_bytes = need;
    }
    coral::DenseWorkspace w;
    coral::dense_workspace_carve(h->d_dense, q_cap, (int)b_cap, h->dim, n_split, w);
    const bool q_dev = is_device_ptr(queries), i_dev = is_device_ptr(ids_out);
    const bool d_dev = dists_out && is_device_ptr(dists_out);
    float* dq = nullptr;
    int32_t* di = nullptr;
    float* dd = nullptr;
    int32_t* d_cert = nullptr;
    if (!q_dev) CK(cudaMalloc(&dq, (size_t)q_cap * h->dim * sizeof(float)));
    if (!i_dev) CK(cudaMalloc(&di, (size_t)q_cap * k * sizeof(int32_t)));
    if (dists_out && !d_dev) CK(cudaMalloc(&dd, (size_t)q_cap * k * sizeof(float)));
    int rc = CORAL_OK;
    int64_t bad = 0;
    cudaError_t e = cudaEventRecord(h->ev_k0, st);
    for (int q0 = 0; q0 < Q && e == cudaSuccess; q0 += q_cap) {
        const int nq = std::min(q_cap, Q - q0);
        const float* qsrc = queries + (size_t)q0 * h->dim;
        if (!q_dev) {
            e = cudaMemcpyAsync(dq, qsrc, (size_t)nq * h->dim * sizeof(float), cudaMemcpyHostToDevice, st);
            qsrc = dq;
        }
        if (e == cudaSuccess) e = coral::dense_begin(w, qsrc, nq, h->dim, st, &h->launches);
        // Rows are scanned in launches of at most 131072 (the first of a query block 16384).  The
        // epilogue's work differs from CTA to CTA while the per-row thresholds are loose; on a long
        // launch the CTAs drift apart until they no longer share operand tiles in L2 and each reads
        // the rows from DRAM (measured: 235 GB of DRAM reads for a 2 GB operand, half speed).  A
        // launch boundary lines them up again and costs microseconds.
        for (int64_t r0 = 0; r0 < n_rows && e == cudaSuccess;) {
            int nr = (int)std::min<int64_t>(b_cap, n_rows - r0);
            const int cap = r0 == 0 ? 16384 : 131072;
            if (nr > cap + cap / 2) nr = cap;
            e = coral::dense_scan_chunk(w, qsrc, nq, d_rows + (size_t)r0 * h->dim, r0, nr, h->dim, h->metric, passes, keep,
                                        h->sm_count, st, &h->launches);
            r0 += nr;
        }
        int32_t* io = i_dev ? ids_out + (size_t)q0 * k : di;
        float* dox = dists_out ? (d_dev ? dists_out + (size_t)q0 * k : dd) : nullptr;
        if (e == cudaSuccess)
            e = coral::dense_finish(w, qsrc, nq, d_rows, h->dim, h->metric, passes, keep, k, io, dox, d_cert, st, &h->launches);
        int flags[4] = {0, 0, 0, 0};
        if (e == cudaSuccess) e = cudaMemcpyAsync(flags, w.err, sizeof flags, cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess && !i_dev)
            e = cudaMemcpyAsync(ids_out + (size_t)q0 * k, di, (size_t)nq * k * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess && dists_out && !d_dev)
            e = cudaMemcpyAsync(dists_out + (size_t)q0 * k, dd, (size_t)nq * k * sizeof(float), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e == cudaSuccess && flags[0]) {
            rc = fail(h, CORAL_ERR_KERNEL, "a bounded wait in the dense scan kernel ran out; results are invalid");
            break;
        }
        bad += flags[1];
    }
    if (e == cudaSuccess && rc == CORAL_OK) {
        e = cudaEventRecord(h->ev_k1, st);
        if (e == cudaSuccess) e = cudaEventSynchronize(h->ev_k1);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&h->last_dense_ms, h->ev_k0, h->ev_k1);
        h->last_dense_flops = 2.0 * (passes == 1 ? 1.0 : 3.0) * (double)Q * (double)n_rows * (double)h->dim;
    }
    cudaFree(dq);
    cudaFree(di);
    cudaFree(dd);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, CORAL_ERR_CUDA, std::string("exact knn: ") + cudaGetErrorString(e));
    }
    if (uncertified_out) *uncertified_out = bad;
    return rc;
}

int coral_exact_knn(coral_index_t* h, const float* queries, int Q, int k, int32_t* ids_out, float* dists_out,
                    int64_t* uncertified_out) {
    if (!h || Q < 0 || (Q > 0 && (!queries || !ids_out))) return fail(h, CORAL_ERR_ARG, "null argument");
    if (!h->d_vecs) return fail(h, CORAL_ERR_STATE, "exact knn: no vectors set");
    if (int rc = ensure_device(h)) return rc;
    return exact_knn_over(h, h->d_vecs, h->live_n, queries, Q, k, h->opt.dense_passes == 1 ? 1 : 3, ids_out, dists_out,
                          uncertified_out);
}

float coral_last_dense_ms(coral_index_t* h) { return h ? h->last_dense_ms : 0.f; }
double coral_last_dense_flops(coral_index_t* h) { return h ? h->last_dense_flops : 0.0; }

// ------------------------------------------------------------------ graph build

static coral::BuildGraph build_view(coral_index* h) {
    coral::BuildGraph g;
    g.vecs = h->d_vecs;
    g.adj = h->d_adj;
    g.ndist = h->d_ndist;
    g.deg = h->d_deg;
    g.claim = h->d_claim;
    g.n = h->n;
    g.dim = h->dim;
    g.deg_pad = h->deg_pad;
    g.max_degree = h->max_degree;
    g.metric = h->metric;
    return g;
}

int coral_build_begin(coral_index_t* h) {
    if (!h) return CORAL_ERR_ARG;
    if (!h->d_vecs) return fail(h, CORAL_ERR_STATE, "build: set the vectors first");
    if (int rc = ensure_device(h)) return rc;
    const size_t cells = (size_t)h->n * h->deg_pad;
    if (!h->d_adj) CK(cudaMalloc(&h->d_adj, cells * sizeof(int32_t)));
    if (!h->d_ndist) CK(cudaMalloc(&h->d_ndist, cells * sizeof(float)));
    if (!h->d_deg) CK(cudaMalloc(&h->d_deg, (size_t)h->n * sizeof(int32_t)));
    if (!h->d_claim) CK(cudaMalloc(&h->d_claim, (size_t)h->n * sizeof(uint32_t)));
    CK(cudaMemsetAsync(h->d_adj, 0xff, cells * sizeof(int32_t), h->stream));
    CK(cudaMemsetAsync(h->d_ndist, 0, cells * sizeof(float), h->stream));
    CK(cudaMemsetAsync(h->d_deg, 0, (size_t)h->n * sizeof(int32_t), h->stream));
    CK(cudaMemsetAsync(h->d_claim, 0x7f, (size_t)h->n * sizeof(uint32_t), h->stream));
    CK(cudaStreamSynchronize(h->stream));
    h->building = true;
    h->frontier_dirty = true;
    return CORAL_OK;
}

int coral_build_set_graph(coral_index_t* h, const int32_t* adj, const float* dists, const int32_t* degs) {
    if (!h || !adj || !dists || !degs) return fail(h, CORAL_ERR_ARG, "null argument");
    if (!h->building) return fail(h, CORAL_ERR_STATE, "build: coral_build_begin has not been called");
    if (int rc = ensure_device(h)) return rc;
    const size_t cells = (size_t)h->n * h->deg_pad;
    CK(cudaMemcpyAsync(h->d_adj, adj, cells * sizeof(int32_t), cudaMemcpyDefault, h->stream));
    CK(cudaMemcpyAsync(h->d_ndist, dists, cells * sizeof(float), cudaMemcpyDefault, h->stream));
    CK(cudaMemcpyAsync(h->d_deg, degs, (size_t)h->n * sizeof(int32_t), cudaMemcpyDefault, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    h->frontier_dirty = true;
    return CORAL_OK;
}

int coral_build_get_graph(coral_index_t* h, int32_t* adj_out, float* dists_out, int32_t* degs_out) {
    if (!h) return CORAL_ERR_ARG;
    if (!h->building) return fail(h, CORAL_ERR_STATE, "build: coral_build_begin has not been called");
    if (int rc = ensure_device(h)) return rc;
    const size_t cells = (size_t)h->n * h->deg_pad;
    if (adj_out) CK(cudaMemcpyAsync(adj_out, h->d_adj, cells * sizeof(int32_t), cudaMemcpyDefault, h->stream));
    if (dists_out) CK(cudaMemcpyAsync(dists_out, h->d_ndist, cells * sizeof(float), cudaMemcpyDefault, h->stream));
    if (degs_out) CK(cudaMemcpyAsync(degs_out, h->d_deg, (size_t)h->n * sizeof(int32_t), cudaMemcpyDefault, h->stream));
    CK(cudaStreamSynchronize(h->stream));
    return CORAL_OK;
}

int coral_build_nap(coral_index_t* h, const int32_t* lists, int T, int kb, int batch) {
    if (!h || (T > 0 && !lists) || T < 0) return fail(h, CORAL_ERR_ARG, "null argument");
    if (!h->building) return fail(h, CORAL_ERR_STATE, "build: coral_build_begin has not been called");
    if (kb < 2 || kb > 128 || kb + h->max_degree > 256) return fail(h, CORAL_ERR_LIMIT, "build: need 2 <= k_b <= 128 and k_b + max_degree <= 256");
    if (batch <= 0) batch = 1024;                                    // config.json:5
    if (int rc = ensure_device(h)) return rc;
    if (T == 0) return CORAL_OK;
    batch = std::min(batch, T);
    const size_t need = coral::nap_scratch_bytes(batch, kb, h->max_degree) + (size_t)batch * kb * sizeof(int32_t);
    if (need > h->nap_scratch_bytes) {
        cudaFree(h->d_nap_scratch);
        h->d_nap_scratch = nullptr;
        h->nap_scratch_bytes = 0;
        CK(cudaMalloc(&h->d_nap_scratch, need));
        h->nap_scratch_bytes = need;
    }
    const bool dev = is_device_ptr(lists);
    int32_t* d_stage = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(h->d_nap_scratch) +
                                                  coral::nap_scratch_bytes(batch, kb, h->max_degree));
    const coral::BuildGraph g = build_view(h);
    for (int s = 0; s < T; s += batch) {                              // src/index_gpu.cpp:555-560: batch after batch
        const int B = std::min(batch, T - s);
        const int32_t* src = lists + (size_t)s * kb;
        if (!dev) {
            CK(cudaMemcpyAsync(d_stage, src, (size_t)B * kb * sizeof(int32_t), cudaMemcpyHostToDevice, h->stream));
            src = d_stage;
        }
        CK(coral::nap_batch(g, src, B, kb, h->d_nap_scratch, h->stream, &h->launches));
        if (!dev) CK(cudaStreamSynchronize(h->stream));              // the staging buffer is reused
    }
    CK(cudaStreamSynchronize(h->stream));
    h->frontier_dirty = true;
    return CORAL_OK;
}

int coral_build_connect_enhance(coral_index_t* h, int kb, int L, int search_batch, int nap_batch, int M,
                                int64_t* n_isolated_out) {
    if (!h) return CORAL_ERR_ARG;
    if (!h->building) return fail(h, CORAL_ERR_STATE, "build: coral_build_begin has not been called");
    if (kb < 1 || kb > 128) return fail(h, CORAL_ERR_LIMIT, "build: need 1 <= k_b <= 128");
    if (L <= 0) L = 256;                                              // src/enhance.cu:783
    if (search_batch <= 0) search_batch = 524288;                     // config.json:7
    if (nap_batch <= 0) nap_batch = 4096;                             // config.json:6
    if (M <= 0) M = 16;                                               // config.json:29
    if (kb > L || M > L) return fail(h, CORAL_ERR_ARG, "build: need k_b <= L and M <= L");
    if (int rc = ensure_device(h)) return rc;
    std::vector<int32_t> degs((size_t)h->n);
    CK(cudaMemcpy(degs.data(), h->d_deg, degs.size() * sizeof(int32_t), cudaMemcpyDeviceToHost));
    std::vector<int32_t> iso;                                         // src/enhance.cu:582-607, ascending ids
    int first_connected = -1;
    for (int64_t i = 0; i < h->live_n; ++i) {
        if (degs[(size_t)i] == 0) iso.push_back((int32_t)i);
        else if (first_connected < 0) first_connected = (int)i;
    }
    std::vector<int32_t>().swap(degs);
    if (n_isolated_out) *n_isolated_out = (int64_t)iso.size();
    if (iso.empty()) return CORAL_OK;
    if (first_connected < 0) return fail(h, CORAL_ERR_STATE, "build: no node has an out-edge yet");
    const int qmax = (int)std::min<size_t>((size_t)search_batch, iso.size());
    if (int rc = coral_search_prepare(h, qmax, L, kb)) return rc;
    int32_t *d_iso = nullptr, *d_res_ids = nullptr;
    float *d_res_d = nullptr, *d_q = nullptr;
    cudaError_t e = cudaMalloc(&d_iso, iso.size() * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&d_res_ids, (size_t)qmax * kb * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&d_res_d, (size_t)qmax * kb * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&d_q, (size_t)qmax * h->dim * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(d_iso, iso.data(), iso.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
    int rc = CORAL_OK;
    const coral::BuildGraph g = build_view(h);
    for (size_t s = 0; s < iso.size() && e == cudaSuccess && rc == CORAL_OK; s += (size_t)search_batch) {
        const int nq = (int)std::min<size_t>((size_t)search_batch, iso.size() - s);
        // entry points of this search batch (src/enhance.cu:793): farthest-point sampling from the
        // lowest-numbered node with an out-edge
        rc = coral_index_select_start_ids(h, first_connected, M, nullptr);
        if (rc != CORAL_OK) break;
        e = coral::gather_rows(h->d_vecs, d_iso + s, nq, h->dim, d_q, h->stream);
        h->launches += 1;
        if (e != cudaSuccess) break;
        rc = enqueue_search(h, d_q, nq, L, kb, d_res_ids, d_res_d, nullptr, h->stream);   // src/enhance.cu:794
        if (rc != CORAL_OK) break;
        e = cudaStreamSynchronize(h->stream);
        if (e != cudaSuccess) break;
        rc = coral_search_check(h);
        if (rc != CORAL_OK) break;
        for (int j = 0; j < nq && e == cudaSuccess; j += nap_batch) {                       // src/enhance.cu:795-800
            const int nb = std::min(nap_batch, nq - j);
            e = coral::ce_batch(g, d_iso + s + j, nb, d_res_ids + (size_t)j * kb, d_res_d + (size_t)j * kb, kb, h->stream,
                                &h->launches);
        }
        if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
        h->frontier_dirty = true;
    }
    cudaFree(d_iso);
    cudaFree(d_res_ids);
    cudaFree(d_res_d);
    cudaFree(d_q);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, CORAL_ERR_CUDA, std::string("build: ") + cudaGetErrorString(e));
    }
    return rc;
}

int coral_index_set_live(coral_index_t* h, int64_t live) {
    if (!h || live < 1 || live > h->n) return fail(h, CORAL_ERR_ARG, "live count must be in [1, n]");
    h->live_n = live;
    return CORAL_OK;
}

int coral_build_begin_from_graph(coral_index_t* h) {
    if (!h) return CORAL_ERR_ARG;
    if (!h->d_vecs || !h->d_adj) return fail(h, CORAL_ERR_STATE, "update: vectors and graph must be set first");
    if (int rc = ensure_device(h)) return rc;
    if (h->building) return CORAL_OK;           // still in build mode: the edge distances are there
    const size_t cells = (size_t)h->n * h->deg_pad;
    if (!h->d_ndist) CK(cudaMalloc(&h->d_ndist, cells * sizeof(float)));
    if (!h->d_deg) CK(cudaMalloc(&h->d_deg, (size_t)h->n * sizeof(int32_t)));
    if (!h->d_claim) CK(cudaMalloc(&h->d_claim, (size_t)h->n * sizeof(uint32_t)));
    CK(cudaMemsetAsync(h->d_claim, 0x7f, (size_t)h->n * sizeof(uint32_t), h->stream));
    CK(coral::edge_dists(build_view(h), h->stream));
    h->launches += 1;
    CK(cudaStreamSynchronize(h->stream));
    h->building = true;
    return CORAL_OK;
}

// Lowest-numbered live node that has an out-edge and is not deleted (host scan of degrees and bits).
static int first_usable_node(coral_index* h, int* out) {
    std::vector<int32_t> degs((size_t)h->live_n);
    std::vector<uint32_t> bits((size_t)((h->n + 31) / 32), 0u);
    CK(cudaMemcpy(degs.data(), h->d_deg, degs.size() * sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (h->d_deleted) CK(cudaMemcpy(bits.data(), h->d_deleted, bits.size() * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    *out = -1;
    for (int64_t i = 0; i < h->live_n; ++i)
        if (degs[(size_t)i] > 0 && !((bits[(size_t)(i >> 5)] >> (i & 31)) & 1u)) {
            *out = (int)i;
            break;
        }
    return CORAL_OK;
}

int coral_delete(coral_index_t* h, const int32_t* ids, int count, int M) {
    if (!h || (count > 0 && !ids) || count < 0) return fail(h, CORAL_ERR_ARG, "null argument");
    if (!h->building) return fail(h, CORAL_ERR_STATE, "update: coral_build_begin_from_graph has not been called");
    if (h->max_degree > 64) return fail(h, CORAL_ERR_LIMIT, "update: max_degree must not exceed 64");
    if (int rc = ensure_device(h)) return rc;
    if (count == 0) return CORAL_OK;
    for (int i = 0; i < count; ++i)
        if (ids[i] < 0 || (int64_t)ids[i] >= h->live_n) return fail(h, CORAL_ERR_ARG, "deleted id out of range");
    cudaStream_t st = h->stream;
    const size_t words = (size_t)((h->n + 31) / 32);
    if (!h->d_deleted) {
        CK(cudaMalloc(&h->d_deleted, words * sizeof(uint32_t)));
        CK(cudaMemsetAsync(h->d_deleted, 0, words * sizeof(uint32_t), st));
    }
    int32_t *d_ids = nullptr, *d_pos = nullptr, *d_lists = nullptr, *d_piv_del = nullptr;
    int *d_counts = nullptr, *d_offsets = nullptr;
    cudaError_t e = cudaMalloc(&d_ids, (size_t)count * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&d_pos, (size_t)h->n * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&d_counts, (size_t)count * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&d_offsets, ((size_t)count + 1) * sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyAsync(d_ids, ids, (size_t)count * sizeof(int32_t), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_pos, 0xff, (size_t)h->n * sizeof(int32_t), st);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_counts, 0, (size_t)count * sizeof(int), st);
    const coral::BuildGraph g = build_view(h);
    // src/update.cu:660-672: every id of the call is marked before any repair
    if (e == cudaSuccess) e = coral::mark_deleted(d_ids, count, h->n, h->d_deleted, d_pos, st);
    // src/graph.cpp:155-195: the live in-neighbours of every deleted node
    if (e == cudaSuccess) e = coral::innbr_scan(g, h->d_deleted, d_pos, d_counts, nullptr, nullptr, st);
    std::vector<int> counts((size_t)count), offsets((size_t)count + 1, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync(counts.data(), d_counts, counts.size() * sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e == cudaSuccess) {
        for (int i = 0; i < count; ++i) offsets[(size_t)i + 1] = offsets[(size_t)i] + counts[(size_t)i];
        const int total = offsets[(size_t)count];
        if (total > 0) {
            e = cudaMalloc(&d_lists, (size_t)total * sizeof(int32_t));
            if (e == cudaSuccess) e = cudaMalloc(&d_piv_del, (size_t)total * sizeof(int32_t));
            if (e == cudaSuccess) e = cudaMemcpyAsync(d_offsets, offsets.data(), offsets.size() * sizeof(int), cudaMemcpyHostToDevice, st);
            if (e == cudaSuccess) e = cudaMemsetAsync(d_counts, 0, (size_t)count * sizeof(int), st);
            if (e == cudaSuccess) e = coral::innbr_scan(g, h->d_deleted, d_pos, d_counts, d_offsets, d_lists, st);
            if (e == cudaSuccess) e = coral::sort_innbr_lists(d_lists, d_offsets, count, d_piv_del, d_ids, st);
            h->launches += 4;
            // src/index_gpu.cpp:170-194: deleted nodes are taken in order until their in-neighbours
            // would exceed INNBR_BATCH = 4096 * 32 (include/uni.h:61)
            const int kInnbrBatch = 4096 * 32;
            int b0 = 0;
            while (b0 < count && e == cudaSuccess) {
                int b1 = b0, num = 0;
                while (b1 < count && (num == 0 || num + counts[(size_t)b1] <= kInnbrBatch)) num += counts[(size_t)b1++];
                if (num > 0)
                    e = coral::delete_batch(g, h->d_deleted, d_piv_del + offsets[(size_t)b0], d_lists + offsets[(size_t)b0], num,
                                            st, &h->launches);
                b0 = b1;
            }
        }
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_ids);
    cudaFree(d_pos);
    cudaFree(d_counts);
    cudaFree(d_offsets);
    cudaFree(d_lists);
    cudaFree(d_piv_del);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, CORAL_ERR_CUDA, std::string("delete: ") + cudaGetErrorString(e));
    }
    h->frontier_dirty = true;
    // entry points must not be deleted nodes (Graph::update_start_ids, src/graph.cpp:229): choose them
    // again from the lowest-numbered usable node
    int first = -1;
    if (int rc = first_usable_node(h, &first)) return rc;
    if (first < 0) return fail(h, CORAL_ERR_STATE, "delete: no connected node is left");
    return coral_index_select_start_ids(h, first, M > 0 ? M : (h->M > 0 ? h->M : 16), nullptr);
}

int coral_insert(coral_index_t* h, int64_t first_id, int count, int kb, int L, int batch, int M) {
    if (!h || count < 0) return CORAL_ERR_ARG;
    if (!h->building) return fail(h, CORAL_ERR_STATE, "update: coral_build_begin_from_graph has not been called");
    if (first_id != h->live_n || first_id + count > h->n)
        return fail(h, CORAL_ERR_ARG, "insert: the new rows must follow the live rows and fit the index");
    if (kb < 1 || kb > 128) return fail(h, CORAL_ERR_LIMIT, "insert: need 1 <= k_b <= 128");
    if (L <= 0) L = 512;                                              // config.json:28 test_beam_capacity
    if (batch <= 0) batch = 2048;                                     // config.json:36 insert_batch
    if (M <= 0) M = 16;
    if (kb > L || M > L) return fail(h, CORAL_ERR_ARG, "insert: need k_b <= L and M <= L");
    if (int rc = ensure_device(h)) return rc;
    if (count == 0) return CORAL_OK;
    batch = std::min(batch, count);
    if (int rc = coral_search_prepare(h, batch, L, kb)) return rc;
    int32_t *d_ins = nullptr, *d_res_ids = nullptr;
    float* d_res_d = nullptr;
    std::vector<int32_t> ins((size_t)count);
    for (int i = 0; i < count; ++i) ins[(size_t)i] = (int32_t)(first_id + i);
    cudaError_t e = cudaMalloc(&d_ins, (size_t)count * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&d_res_ids, (size_t)batch * kb * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&d_res_d, (size_t)batch * kb * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(d_ins, ins.data(), ins.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
    int rc = CORAL_OK;
    const coral::BuildGraph g = build_view(h);
    for (int s = 0; s < count && e == cudaSuccess && rc == CORAL_OK; s += batch) {        // src/index_gpu.cpp:212-216
        const int nb = std::min(batch, count - s);
        int first = -1;
        rc = first_usable_node(h, &first);
        if (rc != CORAL_OK) break;
        if (first < 0) {
            rc = fail(h, CORAL_ERR_STATE, "insert: no connected node to search from");
            break;
        }
        rc = coral_index_select_start_ids(h, first, M, nullptr);                           // src/update.cu:777
        if (rc != CORAL_OK) break;
        // the new vectors are rows of the vector array: they are their own queries (src/update.cu:813)
        rc = enqueue_search(h, h->d_vecs + (size_t)(first_id + s) * h->dim, nb, L, kb, d_res_ids, d_res_d, nullptr, h->stream);
        if (rc != CORAL_OK) break;
        e = cudaStreamSynchronize(h->stream);
        if (e != cudaSuccess) break;
        rc = coral_search_check(h);
        if (rc != CORAL_OK) break;
        e = coral::ce_batch(g, d_ins + s, nb, d_res_ids, d_res_d, kb, h->stream, &h->launches, 3);   // src/update.cu:904-940
        if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
        h->live_n = first_id + s + nb;
        h->frontier_dirty = true;
    }
    cudaFree(d_ins);
    cudaFree(d_res_ids);
    cudaFree(d_res_d);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, CORAL_ERR_CUDA, std::string("insert: ") + cudaGetErrorString(e));
    }
    return rc;
}

int coral_build_end(coral_index_t* h) {
    if (!h) return CORAL_ERR_ARG;
    if (int rc = ensure_device(h)) return rc;
    cudaStreamSynchronize(h->stream);
    cudaFree(h->d_ndist);        h->d_ndist = nullptr;
    cudaFree(h->d_deg);          h->d_deg = nullptr;
    cudaFree(h->d_claim);        h->d_claim = nullptr;
    cudaFree(h->d_nap_scratch);  h->d_nap_scratch = nullptr;
    h->nap_scratch_bytes = 0;
    h->building = false;
    return CORAL_OK;
}

int coral_merge_shards(coral_index_t* h, const int32_t* d_ids, const float* d_dists, int G, int Q, int k,
                       int32_t* d_ids_out, float* d_dists_out, void* stream) {
    return coral_merge_shards_strided(h, d_ids, d_dists, G, Q, k, (int64_t)Q * k, d_ids_out, d_dists_out, stream);
}

int coral_merge_shards_strided(coral_index_t* h, const int32_t* d_ids, const float* d_dists, int G, int Q, int k,
                               int64_t shard_stride, int32_t* d_ids_out, float* d_dists_out, void* stream) {
    if (!h || !d_ids || !d_dists || !d_ids_out || !d_dists_out || G <= 0 || Q < 0 || k <= 0 ||
        shard_stride < (int64_t)Q * k)
        return fail(h, CORAL_ERR_ARG, "bad argument");
    if ((long long)G * k > 4096) return fail(h, CORAL_ERR_LIMIT, "G*k must not exceed 4096");
    if (int rc = ensure_device(h)) return rc;
    if (Q == 0) return CORAL_OK;
    cudaStream_t st = stream ? (cudaStream_t)stream : h->stream;
    const int n2 = next_pow2(std::max(G * k, 32));
    const int wpb = std::max(1, std::min(8, 8192 / n2));
    const size_t smem = (size_t)wpb * n2 * 8;
    CK(cudaFuncSetAttribute(merge_shards_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int blocks = std::min((Q + wpb - 1) / wpb, h->sm_count * 8);
    merge_shards_kernel<<<blocks, wpb * 32, smem, st>>>(d_ids, d_dists, G, Q, k, (long long)shard_stride, n2, h->metric,
                                                        d_ids_out, d_dists_out);
    h->launches += 1;
    CK(cudaGetLastError());
    return CORAL_OK;
}

int coral_map_ids(coral_index_t* h, int32_t* d_ids, int64_t count, const int32_t* d_id_map, void* stream) {
    if (!h || !d_ids || !d_id_map || count < 0) return fail(h, CORAL_ERR_ARG, "bad argument");
    if (int rc = ensure_device(h)) return rc;
    if (count == 0) return CORAL_OK;
    cudaStream_t st = stream ? (cudaStream_t)stream : h->stream;
    const int blocks = (int)std::min<long long>((count + 255) / 256, (long long)h->sm_count * 16);
    map_ids_kernel<<<blocks, 256, 0, st>>>(d_ids, count, d_id_map);
    h->launches += 1;
    CK(cudaGetLastError());
    return CORAL_OK;
}

}  // extern "C"
