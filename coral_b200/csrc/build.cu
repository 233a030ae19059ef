// Graph build on the GPU: neighbourhood-aware projection (NAP) of the training queries' nearest
// neighbour lists onto the base set, and connectivity enhancement (CE) of the nodes no list reached.
//
//   NAP   GPUFuncs::gpu_neibor_aware         src/upd_gpu.cu:260-303
//   CE    GPUFuncs::gpu_connect_enhance      src/enhance.cu:728-812 (enhance_mode 0), batches :640-668
//
// What is kept from the reference: the candidate sets, the sort by distance, the occlusion rule
// (a candidate j is pruned when a kept candidate i is closer to it than the pivot is), "kept first,
// then pruned ones to fill the row", the reverse-edge insertion rule, and every distance as one
// sequential fp32 fused chain (include/utils.cuh:254-275, :307-323) so rows come out bit-identical.
//
// What is different:
//   * the pairwise distances of a list's members are computed ONCE per list (a k_b x k_b matrix in
//     L2-resident scratch) and looked up by all k_b pivots of the list; the reference recomputes
//     them per pivot and per kept candidate inside candidate_ignore_kernel (one thread per pivot);
//   * one warp per pivot sorts in shared memory and prunes with its lanes over the later candidates,
//     instead of a global CUB segmented sort of 16-byte records and a serial thread per pivot;
//   * where the reference lets thread arrival order decide (which occurrence of a node in a batch
//     updates it, src/upd_gpu.cu:102; which isolated node gets to add the reverse edge,
//     src/enhance.cu:166) the lowest index wins, found with atomicMin before the update runs; new
//     rows are staged and committed by a separate kernel so every pivot of a batch sees the graph
//     as it was before the batch, as in the reference.
#include "build.cuh"

#include <cstdint>

namespace coral {

namespace {

constexpr int kCandMax = 256;        // k_b + max_degree candidates per pivot
constexpr uint32_t kUnclaimed = 0x7f7f7f7fu;

enum : uint8_t { S_INVALID = 0, S_INITIAL = 1, S_DISCARDED = 2, S_RETAINED = 3, S_REPEATED = 4 };

__device__ __forceinline__ uint32_t ord_of(float d, int metric) {
    if (metric == 1) d = -d;
    const uint32_t u = __float_as_uint(d);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float dist_of(uint32_t o, int metric) {
    const float d = __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
    return metric == 1 ? -d : d;
}
// include/utils.cuh:380-382: true when d1 is closer than d0
__device__ __forceinline__ bool closer(float d0, float d1, int metric) { return metric == 0 ? d0 > d1 : d0 < d1; }

// One sequential fused chain over d = 0..dim-1 (dim % 4 == 0).
__device__ __forceinline__ float dist_seq(const float* __restrict__ a, const float* __restrict__ b, int dim, int metric) {
    const float4* x = reinterpret_cast<const float4*>(a);
    const float4* y = reinterpret_cast<const float4*>(b);
    float acc = 0.f;
    for (int v = 0; v < dim / 4; ++v) {
        const float4 p = __ldg(x + v), q = __ldg(y + v);
        if (metric == 0) {
            float t;
            t = p.x - q.x; acc = fmaf(t, t, acc);
            t = p.y - q.y; acc = fmaf(t, t, acc);
            t = p.z - q.z; acc = fmaf(t, t, acc);
            t = p.w - q.w; acc = fmaf(t, t, acc);
        } else {
            acc = fmaf(p.x, q.x, acc);
            acc = fmaf(p.y, q.y, acc);
            acc = fmaf(p.z, q.z, acc);
            acc = fmaf(p.w, q.w, acc);
        }
    }
    return acc;
}

// Warp-wide bitonic sort of 256 keys in shared memory, ascending.
__device__ void warp_sort256(uint64_t* s, int lane) {
    for (int k = 2; k <= kCandMax; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = lane; i < kCandMax; i += 32) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const uint64_t a = s[i], b = s[ixj];
                    if ((a > b) == ((i & k) == 0)) {
                        s[i] = b;
                        s[ixj] = a;
                    }
                }
            }
            __syncwarp();
        }
}

__global__ void claim_kernel(const int32_t* __restrict__ ids, long long count, int64_t n, uint32_t* __restrict__ claim) {
    for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x; p < count; p += (long long)gridDim.x * blockDim.x) {
        const int id = ids[p];
        if (id >= 0 && (int64_t)id < n) atomicMin(&claim[id], (uint32_t)p);
    }
}
__global__ void unclaim_kernel(const int32_t* __restrict__ ids, long long count, int64_t n, uint32_t* __restrict__ claim) {
    for (long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x; p < count; p += (long long)gridDim.x * blockDim.x) {
        const int id = ids[p];
        if (id >= 0 && (int64_t)id < n) claim[id] = kUnclaimed;
    }
}

// One CTA per list: gram[list][i][j] = distance between members i and j, every entry one sequential
// chain over the whole dimension (the vectors pass through shared memory 32 floats at a time; the
// partial sums live in shared memory between chunks).
__global__ void __launch_bounds__(256) nap_gram_kernel(const float* __restrict__ vecs, int dim, int metric,
                                                       const int32_t* __restrict__ lists, int kb, float* __restrict__ gram) {
    extern __shared__ float gsm[];
    float* D = gsm;                       // [kb][kb]
    float* stage = gsm + kb * kb;         // [kb][33]
    __shared__ int sid[128];
    const int tid = threadIdx.x;
    const int32_t* ids = lists + (size_t)blockIdx.x * kb;
    for (int i = tid; i < kb; i += 256) sid[i] = ids[i];
    for (int e = tid; e < kb * kb; e += 256) D[e] = 0.f;
    __syncthreads();
    for (int d0 = 0; d0 < dim; d0 += 32) {
        const int w = dim - d0 < 32 ? dim - d0 : 32;
        for (int e = tid; e < kb * 32; e += 256) {
            const int r = e >> 5, c = e & 31;
            stage[r * 33 + c] = c < w ? __ldg(vecs + (size_t)sid[r] * dim + d0 + c) : 0.f;
        }
        __syncthreads();
        for (int e = tid; e < kb * kb; e += 256) {
            const int i = e / kb, j = e - i * kb;
            if (j <= i) continue;
            float acc = D[e];
            const float* a = stage + i * 33;
            const float* b = stage + j * 33;
            if (metric == 0) {
                for (int c = 0; c < w; ++c) {
                    const float t = a[c] - b[c];
                    acc = fmaf(t, t, acc);
                }
            } else {
                for (int c = 0; c < w; ++c) acc = fmaf(a[c], b[c], acc);
            }
            D[e] = acc;
        }
        __syncthreads();
    }
    float* out = gram + (size_t)blockIdx.x * kb * kb;
    for (int e = tid; e < kb * kb; e += 256) {
        const int i = e / kb, j = e - i * kb;
        out[e] = j > i ? D[e] : (j < i ? D[j * kb + i] : 0.f);
    }
}

struct PruneScratch {
    uint64_t keys[kCandMax];     // ord(dist) : col, sorted ascending = closest first
    int32_t id_by_col[kCandMax];
    uint8_t status[kCandMax];    // by sorted position
};

// Occlusion pruning (src/upd_gpu.cu:203-247) by one warp.  Sorted position -> (id, dist, col).
// member_of(col) >= 0 names a row of the list's distance matrix, else the pair is computed.
template <typename PairDist>
__device__ void warp_prune(PruneScratch& S, int n_cand, int max_degree, int metric, int lane, PairDist pair_dist) {
    int nbr_num = 0;
    for (int i = 0; i < n_cand && nbr_num < max_degree; ++i) {
        const uint8_t st = S.status[i];
        if (st == S_INVALID) break;
        const int col_i = (int)(uint32_t)(S.keys[i] & 0xffffffffu);
        const int id_i = S.id_by_col[col_i];
        if (st == S_INITIAL) {
            ++nbr_num;
            for (int j = i + 1 + lane; j < n_cand; j += 32) {
                const uint8_t sj = S.status[j];
                if (sj == S_INVALID) continue;    // the reference breaks here; entries are sorted, so nothing valid follows
                const int col_j = (int)(uint32_t)(S.keys[j] & 0xffffffffu);
                const int id_j = S.id_by_col[col_j];
                if (id_j == id_i) {
                    S.status[j] = S_REPEATED;
                } else if (sj == S_INITIAL) {
                    const float dj = dist_of((uint32_t)(S.keys[j] >> 32), metric);
                    if (closer(dj, pair_dist(col_i, id_i, col_j, id_j), metric)) S.status[j] = S_DISCARDED;
                }
            }
            __syncwarp();
            if (lane == 0) S.status[i] = S_RETAINED;
        } else if (st == S_DISCARDED) {
            for (int j = i + 1 + lane; j < n_cand; j += 32) {
                if (S.status[j] == S_INVALID) continue;
                const int col_j = (int)(uint32_t)(S.keys[j] & 0xffffffffu);
                if (S.id_by_col[col_j] == id_i) S.status[j] = S_REPEATED;
            }
        }
        __syncwarp();
    }
}

// src/update.cu:530-577 (the update path's fill): every kept candidate in order, THEN pruned ones
// while the row has room.  Lane 0 only.
__device__ int fill_row_kept_first(const PruneScratch& S, int n_cand, int max_degree, int metric, int32_t* nbrs,
                                   float* dists) {
    int nbr_num = 0;
    for (int pass = 0; pass < 2; ++pass) {
        const uint8_t want = pass == 0 ? S_RETAINED : S_DISCARDED;
        for (int j = 0; j < n_cand && nbr_num < max_degree; ++j) {
            const uint8_t st = S.status[j];
            if (st == S_INVALID) break;
            if (st == want) {
                nbrs[nbr_num] = S.id_by_col[(int)(uint32_t)(S.keys[j] & 0xffffffffu)];
                dists[nbr_num] = dist_of((uint32_t)(S.keys[j] >> 32), metric);
                ++nbr_num;
            }
        }
    }
    return nbr_num;
}

// src/upd_gpu.cu:106-135: kept first, then pruned ones while the row has room.  Lane 0 only.
__device__ int fill_row(const PruneScratch& S, int n_cand, int max_degree, int metric, int32_t* nbrs, float* dists) {
    int retained = 0;
    for (int i = 0; i < n_cand; ++i) {
        if (S.status[i] == S_RETAINED) ++retained;
        else if (S.status[i] == S_INVALID) break;
    }
    int discarded_need = max_degree - retained, nbr_num = 0;
    for (int j = 0; j < n_cand && nbr_num < max_degree; ++j) {
        const uint8_t st = S.status[j];
        if (st == S_INVALID) break;
        if (st == S_RETAINED || (st == S_DISCARDED && (discarded_need--) > 0)) {
            nbrs[nbr_num] = S.id_by_col[(int)(uint32_t)(S.keys[j] & 0xffffffffu)];
            dists[nbr_num] = dist_of((uint32_t)(S.keys[j] >> 32), metric);
            ++nbr_num;
        }
    }
    return nbr_num;
}

// One warp per pivot (list member); only the first occurrence of a node in the batch works.
__global__ void __launch_bounds__(128) nap_prune_kernel(const float* __restrict__ vecs, int dim, int metric,
                                                        const int32_t* __restrict__ adj, const float* __restrict__ ndist,
                                                        const int32_t* __restrict__ deg, int deg_pad, int max_degree,
                                                        const int32_t* __restrict__ lists, long long pivots, int kb,
                                                        const float* __restrict__ gram, const uint32_t* __restrict__ claim,
                                                        int32_t* __restrict__ new_nbrs, float* __restrict__ new_dists,
                                                        int32_t* __restrict__ new_deg) {
    __shared__ PruneScratch scratch[4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    PruneScratch& S = scratch[warp];
    const long long p = (long long)blockIdx.x * 4 + warp;
    if (p >= pivots) return;
    const int row_id = lists[p];
    if (lane == 0) new_deg[p] = -1;
    if (claim[row_id] != (uint32_t)p) return;                       // src/upd_gpu.cu:102
    const long long list = p / kb;
    const int me = (int)(p - list * kb);
    const int32_t* ids = lists + list * kb;
    const float* G = gram + (size_t)list * kb * kb + (size_t)me * kb;
    const int row_deg = deg[row_id];
    const int cand_size = kb + max_degree;
    for (int col = lane; col < kCandMax; col += 32) {               // src/upd_gpu.cu:36-73
        uint64_t key = ~0ull;
        int id = -1;
        if (col < cand_size && col != me && col < kb + row_deg) {
            if (col >= kb) {
                id = adj[(size_t)row_id * deg_pad + (col - kb)];
                key = ((uint64_t)ord_of(ndist[(size_t)row_id * deg_pad + (col - kb)], metric) << 32) | (uint32_t)col;
            } else {
                const int col_id = ids[col];
                if (col_id != row_id && !(row_deg > 0 && deg[col_id] > 0)) {
                    id = col_id;
                    key = ((uint64_t)ord_of(G[col], metric) << 32) | (uint32_t)col;
                }
            }
        }
        S.keys[col] = key;
        S.id_by_col[col] = id;
    }
    __syncwarp();
    warp_sort256(S.keys, lane);
    for (int i = lane; i < kCandMax; i += 32) S.status[i] = S.keys[i] == ~0ull ? S_INVALID : S_INITIAL;
    __syncwarp();
    const float* Gl = gram + (size_t)list * kb * kb;
    warp_prune(S, cand_size, max_degree, metric, lane, [&](int col_i, int id_i, int col_j, int id_j) {
        if (col_i < kb && col_j < kb) return Gl[(size_t)col_i * kb + col_j];
        return dist_seq(vecs + (size_t)id_i * dim, vecs + (size_t)id_j * dim, dim, metric);
    });
    if (lane == 0)
        new_deg[p] = fill_row(S, cand_size, max_degree, metric, new_nbrs + (size_t)p * max_degree,
                              new_dists + (size_t)p * max_degree);
}

__global__ void nap_commit_kernel(const int32_t* __restrict__ lists, long long pivots, int max_degree, int deg_pad,
                                  const int32_t* __restrict__ new_nbrs, const float* __restrict__ new_dists,
                                  const int32_t* __restrict__ new_deg, int32_t* __restrict__ adj,
                                  float* __restrict__ ndist, int32_t* __restrict__ deg, uint32_t* __restrict__ claim) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long p = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < pivots; p += warps) {
        const int nd = new_deg[p];
        if (nd < 0) continue;
        const int id = lists[p];
        for (int j = lane; j < deg_pad; j += 32) {
            adj[(size_t)id * deg_pad + j] = j < nd ? new_nbrs[(size_t)p * max_degree + j] : -1;
            ndist[(size_t)id * deg_pad + j] = j < nd ? new_dists[(size_t)p * max_degree + j] : 0.f;
        }
        if (lane == 0) {
            deg[id] = nd;
            claim[id] = kUnclaimed;
        }
    }
}

// ------------------------------------------------------------------------------------------- CE

__global__ void gather_rows_kernel(const float* __restrict__ vecs, const int32_t* __restrict__ ids, int count, int dim,
                                   float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < count; r += warps) {
        const float4* src = reinterpret_cast<const float4*>(vecs + (size_t)ids[r] * dim);
        float4* dst = reinterpret_cast<float4*>(out + (size_t)r * dim);
        for (int v = lane; v < dim / 4; v += 32) dst[v] = __ldg(src + v);
    }
}

constexpr int kCeRowFloats = 68;                          // 64 floats of a row chunk + 4 of padding (bank spread)
constexpr int kCeStageBytes = 32 * kCeRowFloats * 4;      // one chunk of 32 rows per warp

// Reverse edges (src/enhance.cu:136-212): one warp per (isolated node, result rank) pair that won
// the found node.  The lanes evaluate, for every position of the found node's row, the three
// comparisons the reference's loops make (each needs the distance between the isolated node and the
// stored neighbour: one sequential chain per lane); lane 0 then walks the flags in the reference's
// order and shifts the row.
__global__ void __launch_bounds__(128) ce_reverse_kernel(const float* __restrict__ vecs, int dim, int metric,
                                                         int32_t* __restrict__ adj, float* __restrict__ ndist,
                                                         int32_t* __restrict__ deg, int deg_pad, int max_degree,
                                                         const int32_t* __restrict__ iso_ids, int n_iso,
                                                         const int32_t* __restrict__ res_ids,
                                                         const float* __restrict__ res_dists, int kb, int64_t n,
                                                         const uint32_t* __restrict__ claim, int mode) {
    __shared__ uint8_t flags[4][128];   // bit 0: stored neighbour closer to the node than the isolated node is
                                        // bit 1: ... and closer to the isolated node than the node is (occludes it)
                                        // bit 2: the isolated node occludes the stored neighbour
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long e = (long long)blockIdx.x * 4 + warp;
    if (e >= (long long)n_iso * kb) return;
    const int knn_id = res_ids[e];
    if (knn_id < 0 || (int64_t)knn_id >= n || claim[knn_id] != (uint32_t)e) return;
    const int iso_id = iso_ids[e / kb];
    const float* iso_vec = vecs + (size_t)iso_id * dim;
    // insert path (src/update.cu:139): the candidate's distance is recomputed, not taken from the search
    const float knn_dist = (mode & 1) ? dist_seq(iso_vec, vecs + (size_t)knn_id * dim, dim, metric) : res_dists[e];
    int32_t* nb = adj + (size_t)knn_id * deg_pad;
    float* ds = ndist + (size_t)knn_id * deg_pad;
    const int d = deg[knn_id];
    // Distances from the isolated node to the stored neighbours: lane o owns neighbour o's chain
    // (same order as dist_seq), but the rows are staged through shared memory 64 floats at a time
    // by the whole warp (two rows per load instruction, whole lines), instead of every lane walking
    // its own row through L1 sixteen bytes at a time.
    extern __shared__ __align__(16) unsigned char ce_smem[];
    float* s_iso = reinterpret_cast<float*>(ce_smem + (size_t)warp * ((size_t)dim * 4 + kCeStageBytes));
    float* s_rows = s_iso + dim;
    for (int v = lane; v < dim / 4; v += 32)
        reinterpret_cast<float4*>(s_iso)[v] = __ldg(reinterpret_cast<const float4*>(iso_vec) + v);
    for (int o0 = 0; o0 < d; o0 += 32) {
        const int rows = d - o0 < 32 ? d - o0 : 32;
        const int o = o0 + lane;
        float acc = 0.f;
        for (int c0 = 0; c0 < dim; c0 += 64) {
            const int units = (dim - c0 < 64 ? dim - c0 : 64) / 4;       // float4 units of this chunk
            __syncwarp();
            // all of the chunk's loads are in flight before the first one is stored (a 32-row chunk is 16
            // loads per lane: two rows per warp-wide load)
            float4 tmp[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int r = 2 * k + (lane >> 4), u = lane & 15;
                if (r < rows && u < units)
                    tmp[k] = __ldg(reinterpret_cast<const float4*>(vecs + (size_t)nb[o0 + r] * dim + c0) + u);
            }
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int r = 2 * k + (lane >> 4), u = lane & 15;
                if (r < rows && u < units) *reinterpret_cast<float4*>(s_rows + r * kCeRowFloats + u * 4) = tmp[k];
            }
            __syncwarp();
            if (lane < rows) {
                const float4* y = reinterpret_cast<const float4*>(s_rows + lane * kCeRowFloats);
                const float4* x = reinterpret_cast<const float4*>(s_iso + c0);
                for (int u = 0; u < units; ++u) {
                    const float4 p = x[u], q = y[u];
                    if (metric == 0) {
                        float t;
                        t = p.x - q.x; acc = fmaf(t, t, acc);
                        t = p.y - q.y; acc = fmaf(t, t, acc);
                        t = p.z - q.z; acc = fmaf(t, t, acc);
                        t = p.w - q.w; acc = fmaf(t, t, acc);
                    } else {
                        acc = fmaf(p.x, q.x, acc);
                        acc = fmaf(p.y, q.y, acc);
                        acc = fmaf(p.z, q.z, acc);
                        acc = fmaf(p.w, q.w, acc);
                    }
                }
            }
        }
        if (lane < rows) {
            const float dso = ds[o], dio = acc;
            uint8_t f = 0;
            if (closer(knn_dist, dso, metric)) f |= 1;
            if (closer(knn_dist, dio, metric)) f |= 2;
            if (closer(dso, dio, metric)) f |= 4;
            flags[warp][o] = f;
        }
    }
    __syncwarp();
    // lane 0 walks the flags in the reference's order; the warp then shifts the row together
    int pos = 0, out_pos = -1, insert = 0;
    if (lane == 0) {
        const uint8_t* F = flags[warp];
        int valid = 1;
        for (; pos < d; ++pos) {                                   // :172-181
            if (F[pos] & 1) {
                if (valid && (F[pos] & 2)) valid = 0;
            } else
                break;
        }
        if (d == max_degree) {                                     // :183-191
            if (valid && pos < d) {
                out_pos = d - 1;
                for (; out_pos >= pos; --out_pos)
                    if (F[out_pos] & 4) break;
                if (out_pos < pos) out_pos = d - 1;
                insert = 1;
            }
        } else {
            out_pos = d;
            deg[knn_id] = d + 1;
            insert = 1;
        }
    }
    insert = __shfl_sync(0xffffffffu, insert, 0);
    if (!insert) return;
    pos = __shfl_sync(0xffffffffu, pos, 0);
    out_pos = __shfl_sync(0xffffffffu, out_pos, 0);
    // entries pos .. out_pos-1 move one place up, the isolated node takes place pos (:206-211)
    int32_t vn[4];
    float vd[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int j = lane + 32 * t;
        if (j > pos && j <= out_pos) {
            vn[t] = nb[j - 1];
            vd[t] = ds[j - 1];
        }
    }
    __syncwarp();
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int j = lane + 32 * t;
        if (j > pos && j <= out_pos) {
            nb[j] = vn[t];
            ds[j] = vd[t];
        } else if (j == pos) {
            nb[j] = iso_id;
            ds[j] = knn_dist;
        }
    }
}

// Every isolated node's own row from its pruned search results (src/enhance.cu:344-389, :528-580).
__global__ void __launch_bounds__(128) ce_prune_kernel(const float* __restrict__ vecs, int dim, int metric,
                                                       int32_t* __restrict__ adj, float* __restrict__ ndist,
                                                       int32_t* __restrict__ deg, int deg_pad, int max_degree,
                                                       const int32_t* __restrict__ iso_ids, int n_iso,
                                                       const int32_t* __restrict__ res_ids,
                                                       const float* __restrict__ res_dists, int kb, int64_t n,
                                                       uint32_t* __restrict__ claim, int mode) {
    __shared__ PruneScratch scratch[4];
    __shared__ int32_t row_n[4][128];
    __shared__ float row_d[4][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    PruneScratch& S = scratch[warp];
    const int i = blockIdx.x * 4 + warp;
    if (i >= n_iso) return;
    for (int col = lane; col < kCandMax; col += 32) {
        uint64_t key = ~0ull;
        int id = -1;
        if (col < kb) {
            id = res_ids[(size_t)i * kb + col];
            if (id >= 0 && (int64_t)id < n) {
                const float dc = (mode & 1) ? dist_seq(vecs + (size_t)iso_ids[i] * dim, vecs + (size_t)id * dim, dim, metric)
                                            : res_dists[(size_t)i * kb + col];
                key = ((uint64_t)ord_of(dc, metric) << 32) | (uint32_t)col;
                claim[id] = kUnclaimed;     // the reverse edges of this batch are in place: free the claim
            } else {
                id = -1;
            }
        }
        S.keys[col] = key;
        S.id_by_col[col] = id;
    }
    __syncwarp();
    warp_sort256(S.keys, lane);
    for (int j = lane; j < kCandMax; j += 32) S.status[j] = S.keys[j] == ~0ull ? S_INVALID : S_INITIAL;
    __syncwarp();
    warp_prune(S, kb, max_degree, metric, lane, [&](int, int id_i, int, int id_j) {
        return dist_seq(vecs + (size_t)id_i * dim, vecs + (size_t)id_j * dim, dim, metric);
    });
    int nd = 0;
    if (lane == 0)
        nd = (mode & 2) ? fill_row_kept_first(S, kb, max_degree, metric, row_n[warp], row_d[warp])
                        : fill_row(S, kb, max_degree, metric, row_n[warp], row_d[warp]);
    nd = __shfl_sync(0xffffffffu, nd, 0);
    const int id = iso_ids[i];
    for (int j = lane; j < deg_pad; j += 32) {
        adj[(size_t)id * deg_pad + j] = j < nd ? row_n[warp][j] : -1;
        ndist[(size_t)id * deg_pad + j] = j < nd ? row_d[warp][j] : 0.f;
    }
    if (lane == 0) deg[id] = nd;
}

// ------------------------------------------------------------------------------------- update

// Distances of the stored edges and the degrees of a graph given as adjacency only.
__global__ void edge_dist_kernel(const float* __restrict__ vecs, int dim, int metric, const int32_t* __restrict__ adj,
                                 int deg_pad, int64_t n, float* __restrict__ ndist, int32_t* __restrict__ deg) {
    const int lane = threadIdx.x & 31;
    const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        int cnt = 0;
        for (int j = lane; j < deg_pad; j += 32) {
            const int id = adj[(size_t)i * deg_pad + j];
            const bool ok = id >= 0 && (int64_t)id < n;
            ndist[(size_t)i * deg_pad + j] = ok ? dist_seq(vecs + (size_t)i * dim, vecs + (size_t)id * dim, dim, metric) : 0.f;
            cnt += __popc(__ballot_sync(0xffffffffu, ok));
        }
        if (lane == 0) deg[i] = cnt;
    }
}

__global__ void mark_deleted_kernel(const int32_t* __restrict__ ids, int count, int64_t n, uint32_t* __restrict__ bits,
                                    int32_t* __restrict__ pos_of) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
        const int id = ids[i];
        if (id < 0 || (int64_t)id >= n) continue;
        atomicOr(bits + (id >> 5), 1u << (id & 31));
        pos_of[id] = i;
    }
}

// In-neighbours of the deleted nodes: first pass counts, second pass fills (fill != nullptr).
__global__ void innbr_scan_kernel(const int32_t* __restrict__ adj, const int32_t* __restrict__ deg, int deg_pad, int64_t n,
                                  const uint32_t* __restrict__ bits, const int32_t* __restrict__ pos_of,
                                  int* __restrict__ counts, const int* __restrict__ offsets, int32_t* __restrict__ fill) {
    const long long total = n * (long long)deg_pad;
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const long long i = t / deg_pad;
        const int j = (int)(t - i * deg_pad);
        if (j >= deg[i] || ((bits[i >> 5] >> (i & 31)) & 1u)) continue;       // deleted rows are not repaired
        const int id = adj[t];
        if (id < 0 || (int64_t)id >= n || !((bits[id >> 5] >> (id & 31)) & 1u)) continue;
        const int p = pos_of[id];
        if (p < 0) continue;                                                     // deleted by an earlier call: no longer anyone's neighbour
        const int slot = atomicAdd(&counts[p], 1);
        if (fill) fill[offsets[p] + slot] = (int32_t)i;
    }
}

// Ascending order inside every list (the fill order is arbitrary): one CTA per list, bitonic sort in
// shared memory in pieces of 4096 followed by a merge through global memory when a list is longer.
__global__ void __launch_bounds__(256) sort_lists_kernel(int32_t* __restrict__ lists, const int* __restrict__ offsets,
                                                         int n_lists, int32_t* __restrict__ piv_del,
                                                         const int32_t* __restrict__ del_ids) {
    __shared__ int32_t s[4096];
    for (int l = blockIdx.x; l < n_lists; l += gridDim.x) {
        const int lo = offsets[l], hi = offsets[l + 1], len = hi - lo;
        for (int i = threadIdx.x; i < len; i += 256) piv_del[lo + i] = del_ids[l];
        if (len <= 1) continue;
        if (len <= 4096) {
            int n2 = 2;
            while (n2 < len) n2 <<= 1;
            for (int i = threadIdx.x; i < n2; i += 256) s[i] = i < len ? lists[lo + i] : 0x7fffffff;
            __syncthreads();
            for (int k = 2; k <= n2; k <<= 1)
                for (int j = k >> 1; j > 0; j >>= 1) {
                    for (int i = threadIdx.x; i < n2; i += 256) {
                        const int ixj = i ^ j;
                        if (ixj > i) {
                            const int32_t a = s[i], b = s[ixj];
                            if ((a > b) == ((i & k) == 0)) {
                                s[i] = b;
                                s[ixj] = a;
                            }
                        }
                    }
                    __syncthreads();
                }
            for (int i = threadIdx.x; i < len; i += 256) lists[lo + i] = s[i];
            __syncthreads();
        } else if (threadIdx.x == 0) {
            // a hub with more than 4096 in-neighbours: heap sort in place by one thread (rare)
            int32_t* a = lists + lo;
            for (int start = len / 2 - 1; start >= 0; --start) {
                int root = start;
                for (;;) {
                    int child = 2 * root + 1;
                    if (child >= len) break;
                    if (child + 1 < len && a[child] < a[child + 1]) ++child;
                    if (a[root] >= a[child]) break;
                    const int32_t t = a[root]; a[root] = a[child]; a[child] = t;
                    root = child;
                }
            }
            for (int end = len - 1; end > 0; --end) {
                const int32_t t0 = a[0]; a[0] = a[end]; a[end] = t0;
                int root = 0;
                for (;;) {
                    int child = 2 * root + 1;
                    if (child >= end) break;
                    if (child + 1 < end && a[child] < a[child + 1]) ++child;
                    if (a[root] >= a[child]) break;
                    const int32_t t = a[root]; a[root] = a[child]; a[child] = t;
                    root = child;
                }
            }
        }
        __syncthreads();
    }
}

// Repair of one in-neighbour (src/update.cu:312-391, :499-583): one warp per (deleted node,
// in-neighbour) pair; the first pair of the batch that names an in-neighbour repairs it.
__global__ void __launch_bounds__(128) delete_prune_kernel(const float* __restrict__ vecs, int dim, int metric,
                                                           int32_t* __restrict__ adj, float* __restrict__ ndist,
                                                           int32_t* __restrict__ deg, int deg_pad, int max_degree,
                                                           const uint32_t* __restrict__ bits,
                                                           const int32_t* __restrict__ piv_del,
                                                           const int32_t* __restrict__ piv_in, int n_piv,
                                                           uint32_t* __restrict__ claim) {
    __shared__ PruneScratch scratch[4];
    __shared__ int32_t row_n[4][128];
    __shared__ float row_d[4][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    PruneScratch& S = scratch[warp];
    const int p = blockIdx.x * 4 + warp;
    if (p >= n_piv) return;
    const int I = piv_in[p], D = piv_del[p];
    if (claim[I] != (uint32_t)p) return;
    const int deg_i = deg[I], deg_d = deg[D];
    // candidates in the reference's order: the in-neighbour's surviving neighbours, then the deleted
    // node's surviving out-neighbours; column = position among the survivors (the stable sort key)
    int base_col = 0;
    for (int half = 0; half < 2; ++half) {
        const int src = half == 0 ? I : D, d = half == 0 ? deg_i : deg_d;
        for (int b0 = 0; b0 < d; b0 += 32) {
            const int j = b0 + lane;
            int id = -1;
            if (j < d) {
                id = adj[(size_t)src * deg_pad + j];
                if (id < 0 || ((bits[id >> 5] >> (id & 31)) & 1u) || (half == 1 && id == I)) id = -1;
            }
            const uint32_t m = __ballot_sync(0xffffffffu, id >= 0);
            if (id >= 0) {
                const int col = base_col + __popc(m & ((1u << lane) - 1u));
                const float dc = half == 0 ? ndist[(size_t)I * deg_pad + j]
                                           : dist_seq(vecs + (size_t)I * dim, vecs + (size_t)id * dim, dim, metric);
                S.keys[col] = ((uint64_t)ord_of(dc, metric) << 32) | (uint32_t)col;
                S.id_by_col[col] = id;
            }
            base_col += __popc(m);
        }
    }
    for (int col = base_col + lane; col < kCandMax; col += 32) {
        S.keys[col] = ~0ull;
        S.id_by_col[col] = -1;
    }
    __syncwarp();
    warp_sort256(S.keys, lane);
    for (int j = lane; j < kCandMax; j += 32) S.status[j] = S.keys[j] == ~0ull ? S_INVALID : S_INITIAL;
    __syncwarp();
    warp_prune(S, 2 * max_degree, max_degree, metric, lane, [&](int, int id_i, int, int id_j) {
        return dist_seq(vecs + (size_t)id_i * dim, vecs + (size_t)id_j * dim, dim, metric);
    });
    int nd = 0;
    if (lane == 0) nd = fill_row_kept_first(S, 2 * max_degree, max_degree, metric, row_n[warp], row_d[warp]);
    nd = __shfl_sync(0xffffffffu, nd, 0);
    for (int j = lane; j < deg_pad; j += 32) {
        adj[(size_t)I * deg_pad + j] = j < nd ? row_n[warp][j] : -1;
        ndist[(size_t)I * deg_pad + j] = j < nd ? row_d[warp][j] : 0.f;
    }
    if (lane == 0) {
        deg[I] = nd;
        claim[I] = kUnclaimed;
    }
}

int grid_for(long long items, int per_block, int cap) {
    long long b = (items + per_block - 1) / per_block;
    if (b < 1) b = 1;
    return (int)(b < cap ? b : cap);
}

}  // namespace

size_t nap_scratch_bytes(int batch, int kb, int max_degree) {
    const size_t pivots = (size_t)batch * kb;
    return (size_t)batch * kb * kb * 4 + pivots * max_degree * 8 + pivots * 4 + 1024;
}

cudaError_t nap_batch(const BuildGraph& g, const int32_t* d_lists, int B, int kb, void* scratch, cudaStream_t st,
                      int64_t* launches) {
    if (kb < 2 || kb > 128 || kb + g.max_degree > kCandMax || g.max_degree > 128) return cudaErrorInvalidValue;
    const long long pivots = (long long)B * kb;
    unsigned char* p = static_cast<unsigned char*>(scratch);
    float* gram = reinterpret_cast<float*>(p);            p += (size_t)B * kb * kb * 4;
    int32_t* new_nbrs = reinterpret_cast<int32_t*>(p);    p += (size_t)pivots * g.max_degree * 4;
    float* new_dists = reinterpret_cast<float*>(p);       p += (size_t)pivots * g.max_degree * 4;
    int32_t* new_deg = reinterpret_cast<int32_t*>(p);
    claim_kernel<<<grid_for(pivots, 256, 2048), 256, 0, st>>>(d_lists, pivots, g.n, g.claim);
    const size_t gsm = (size_t)kb * kb * 4 + (size_t)kb * 33 * 4;
    cudaError_t e = cudaFuncSetAttribute(nap_gram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gsm);
    if (e != cudaSuccess) return e;
    nap_gram_kernel<<<B, 256, gsm, st>>>(g.vecs, g.dim, g.metric, d_lists, kb, gram);
    nap_prune_kernel<<<(unsigned)((pivots + 3) / 4), 128, 0, st>>>(g.vecs, g.dim, g.metric, g.adj, g.ndist, g.deg, g.deg_pad,
                                                                   g.max_degree, d_lists, pivots, kb, gram, g.claim,
                                                                   new_nbrs, new_dists, new_deg);
    nap_commit_kernel<<<grid_for(pivots * 32, 256, 4096), 256, 0, st>>>(d_lists, pivots, g.max_degree, g.deg_pad, new_nbrs,
                                                                        new_dists, new_deg, g.adj, g.ndist, g.deg, g.claim);
    if (launches) *launches += 4;
    return cudaGetLastError();
}

cudaError_t ce_batch(const BuildGraph& g, const int32_t* d_iso_ids, int n_iso, const int32_t* d_res_ids,
                     const float* d_res_dists, int kb, cudaStream_t st, int64_t* launches, int mode) {
    if (kb < 1 || kb > 128 || g.max_degree > 128) return cudaErrorInvalidValue;
    const long long entries = (long long)n_iso * kb;
    claim_kernel<<<grid_for(entries, 256, 2048), 256, 0, st>>>(d_res_ids, entries, g.n, g.claim);
    const size_t rev_smem = 4 * ((size_t)g.dim * 4 + kCeStageBytes);
    if (rev_smem > 48 * 1024) {
        if (rev_smem > 200 * 1024) return cudaErrorInvalidValue;
        cudaError_t e = cudaFuncSetAttribute(ce_reverse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rev_smem);
        if (e != cudaSuccess) return e;
    }
    ce_reverse_kernel<<<(unsigned)((entries + 3) / 4), 128, rev_smem, st>>>(g.vecs, g.dim, g.metric, g.adj, g.ndist, g.deg, g.deg_pad,
                                                                     g.max_degree, d_iso_ids, n_iso, d_res_ids, d_res_dists,
                                                                     kb, g.n, g.claim, mode);
    ce_prune_kernel<<<(unsigned)((n_iso + 3) / 4), 128, 0, st>>>(g.vecs, g.dim, g.metric, g.adj, g.ndist, g.deg, g.deg_pad,
                                                                 g.max_degree, d_iso_ids, n_iso, d_res_ids, d_res_dists, kb,
                                                                 g.n, g.claim, mode);
    if (launches) *launches += 3;
    return cudaGetLastError();
}

cudaError_t edge_dists(const BuildGraph& g, cudaStream_t st) {
    edge_dist_kernel<<<grid_for(g.n * 32, 256, 8192), 256, 0, st>>>(g.vecs, g.dim, g.metric, g.adj, g.deg_pad, g.n, g.ndist,
                                                                     g.deg);
    return cudaGetLastError();
}

cudaError_t mark_deleted(const int32_t* d_ids, int count, int64_t n, uint32_t* bits, int32_t* pos_of, cudaStream_t st) {
    mark_deleted_kernel<<<grid_for(count, 256, 2048), 256, 0, st>>>(d_ids, count, n, bits, pos_of);
    return cudaGetLastError();
}

cudaError_t innbr_scan(const BuildGraph& g, const uint32_t* bits, const int32_t* pos_of, int* counts, const int* offsets,
                       int32_t* fill, cudaStream_t st) {
    innbr_scan_kernel<<<grid_for(g.n * (long long)g.deg_pad, 256, 16384), 256, 0, st>>>(g.adj, g.deg, g.deg_pad, g.n, bits,
                                                                                        pos_of, counts, offsets, fill);
    return cudaGetLastError();
}

cudaError_t sort_innbr_lists(int32_t* lists, const int* offsets, int n_lists, int32_t* piv_del, const int32_t* d_del_ids,
                             cudaStream_t st) {
    sort_lists_kernel<<<grid_for(n_lists, 1, 8192), 256, 0, st>>>(lists, offsets, n_lists, piv_del, d_del_ids);
    return cudaGetLastError();
}

cudaError_t delete_batch(const BuildGraph& g, const uint32_t* bits, const int32_t* piv_del, const int32_t* piv_in, int n_piv,
                         cudaStream_t st, int64_t* launches) {
    if (g.max_degree > 64) return cudaErrorInvalidValue;
    claim_kernel<<<grid_for(n_piv, 256, 2048), 256, 0, st>>>(piv_in, n_piv, g.n, g.claim);
    delete_prune_kernel<<<(unsigned)((n_piv + 3) / 4), 128, 0, st>>>(g.vecs, g.dim, g.metric, g.adj, g.ndist, g.deg, g.deg_pad,
                                                                     g.max_degree, bits, piv_del, piv_in, n_piv, g.claim);
    unclaim_kernel<<<grid_for(n_piv, 256, 2048), 256, 0, st>>>(piv_in, n_piv, g.n, g.claim);
    if (launches) *launches += 3;
    return cudaGetLastError();
}

cudaError_t gather_rows(const float* vecs, const int32_t* d_ids, int count, int dim, float* out, cudaStream_t st) {
    gather_rows_kernel<<<grid_for((long long)count * 32, 256, 4096), 256, 0, st>>>(vecs, d_ids, count, dim, out);
    return cudaGetLastError();
}

}  // namespace coral
