// Query scheduling for L2 locality.
//
// The first expansion round of the beam search is the same for every query: the
// M entry points are expanded and their neighbours (the "frontier", at most
// M * deg_pad nodes) get a distance.  Which frontier node a query likes best is
// a cheap, good predictor of where in the graph that query will spend its time,
// and queries that run at the same moment on neighbouring CTAs and like the same
// node re-read each other's rows from the 126 MB L2 instead of from HBM.
//
// So before a large batch is searched: (1) one dense pass, queries x frontier
// vectors, keeps the best frontier node per query -- on the tensor cores (the
// tcgen05 scan of dense_topk.cu, one tf32 pass, exact re-rank of the 8 best), with
// the fp32 SIMT tile kernel below as the variant for comparison; the key only
// orders the work, so nothing of it reaches a result -- (2) a stable counting
// sort by that node yields the order in which the persistent CTAs take the queries.
// Results are written at each query's own position: nothing observable changes
// except speed (10M x 512, 100k queries, L=64: 422k -> 492k queries/s).
#include <cuda_runtime.h>
#include <stdint.h>

#include "schedule.cuh"

namespace coral {

namespace {

constexpr int kTileQ = 64, kTileF = 64, kTileK = 32;

// keys[q] = argmax_f score(q, f); score = q.f (inner product) or 2 q.f - |f|^2 (L2, larger = closer).
__global__ void __launch_bounds__(256) frontier_argmax_kernel(const float* __restrict__ queries, int Q, int dim,
                                                              const float* __restrict__ fvecs,
                                                              const float* __restrict__ fnorm, int F, int metric,
                                                              int* __restrict__ keys) {
    __shared__ float As[kTileK][kTileQ + 1];
    __shared__ float Bs[kTileK][kTileF + 1];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int q0 = blockIdx.x * kTileQ;
    float best[4];
    int best_f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        best[i] = -3.402823466e+38f;
        best_f[i] = 0;
    }
    for (int f0 = 0; f0 < F; f0 += kTileF) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        for (int k0 = 0; k0 < dim; k0 += kTileK) {
            // 64 rows x 32 columns per operand, 256 threads: 8 elements each, coalesced along k
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int e = tid + 256 * t, r = e >> 5, c = e & 31;
                const int q = q0 + r, f = f0 + r, k = k0 + c;
                As[c][r] = (q < Q && k < dim) ? queries[(size_t)q * dim + k] : 0.f;
                Bs[c][r] = (f < F && k < dim) ? fvecs[(size_t)f * dim + k] : 0.f;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < kTileK; ++kk) {
                float a4[4], b4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a4[i] = As[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) b4[j] = Bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int f = f0 + tx * 4 + j;
            if (f < F) {
                const float nf = metric == 0 ? fnorm[f] : 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float s = metric == 0 ? 2.f * acc[i][j] - nf : acc[i][j];
                    if (s > best[i]) {
                        best[i] = s;
                        best_f[i] = f;
                    }
                }
            }
        }
    }
    // the 16 threads of a row sit in one half-warp: butterfly over tx
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best[i], off);
            const int of = __shfl_xor_sync(0xffffffffu, best_f[i], off);
            if (ov > best[i] || (ov == best[i] && of < best_f[i])) {
                best[i] = ov;
                best_f[i] = of;
            }
        }
        const int q = q0 + ty * 4 + i;
        if (tx == 0 && q < Q) keys[q] = best_f[i];
    }
}

__global__ void gather_frontier_kernel(const float* __restrict__ vecs, const int32_t* __restrict__ ids, int F, int dim,
                                       float* __restrict__ fvecs, float* __restrict__ fnorm) {
    const int f = blockIdx.x;
    if (f >= F) return;
    const float* src = vecs + (size_t)ids[f] * dim;
    float s = 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        const float v = src[d];
        fvecs[(size_t)f * dim + d] = v;
        s = fmaf(v, v, s);
    }
    __shared__ float red[32];
    for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x + 31) / 32; ++w) t += red[w];
        fnorm[f] = t;
    }
}

// ---- deterministic counting sort of the batch by key (stable: equal keys keep their query order,
// so every GPU that sorts the same batch gets the same order).
constexpr int kSortChunk = 1024;

// One block per chunk of 1024 queries: rank of every query among the chunk's earlier queries with
// the same key, and the chunk's count per key.
__global__ void __launch_bounds__(kSortChunk) chunk_rank_kernel(const int* __restrict__ keys, int Q, int F,
                                                                int* __restrict__ rank_in_chunk,
                                                                int* __restrict__ chunk_counts) {
    __shared__ int sk[kSortChunk];
    const int q = blockIdx.x * kSortChunk + threadIdx.x;
    const int key = q < Q ? keys[q] : -1;
    sk[threadIdx.x] = key;
    __syncthreads();
    if (q >= Q) return;
    int r = 0;
    for (int i = 0; i < (int)threadIdx.x; ++i) r += sk[i] == key;
    rank_in_chunk[q] = r;
    atomicAdd(&chunk_counts[(size_t)blockIdx.x * F + key], 1);
}

// One thread per key: chunk_counts[c][key] -> exclusive prefix over the chunks; bins[key] = total.
__global__ void column_scan_kernel(int* __restrict__ chunk_counts, int n_chunks, int F, int* __restrict__ bins) {
    const int key = blockIdx.x * blockDim.x + threadIdx.x;
    if (key >= F) return;
    int run = 0;
    for (int c = 0; c < n_chunks; ++c) {
        const int v = chunk_counts[(size_t)c * F + key];
        chunk_counts[(size_t)c * F + key] = run;
        run += v;
    }
    bins[key] = run;
}

// One block: bins[0..F) -> exclusive prefix in place.
__global__ void exclusive_scan_kernel(int* __restrict__ bins, int F) {
    __shared__ int carry;
    __shared__ int part[1024];
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < F; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < F ? bins[i] : 0;
        part[threadIdx.x] = v;
        __syncthreads();
        for (int off = 1; off < 1024; off <<= 1) {
            const int add = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
            __syncthreads();
            part[threadIdx.x] += add;
            __syncthreads();
        }
        if (i < F) bins[i] = carry + part[threadIdx.x] - v;
        __syncthreads();
        if (threadIdx.x == 0) carry += part[1023];
        __syncthreads();
    }
}

__global__ void place_kernel(const int* __restrict__ keys, int Q, int F, const int* __restrict__ bins,
                             const int* __restrict__ chunk_counts, const int* __restrict__ rank_in_chunk,
                             int32_t* __restrict__ order) {
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < Q; q += gridDim.x * blockDim.x) {
        const int key = keys[q];
        order[bins[key] + chunk_counts[(size_t)(q / kSortChunk) * F + key] + rank_in_chunk[q]] = q;
    }
}

__global__ void first_column_kernel(const int32_t* __restrict__ ids, int Q, int stride, int F, int* __restrict__ keys) {
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < Q; q += gridDim.x * blockDim.x) {
        const int v = ids[(size_t)q * stride];
        keys[q] = v >= 0 && v < F ? v : 0;
    }
}

}  // namespace

cudaError_t gather_frontier(const float* vecs, const int32_t* d_ids, int F, int dim, float* fvecs, float* fnorm,
                            cudaStream_t stream) {
    gather_frontier_kernel<<<F, 128, 0, stream>>>(vecs, d_ids, F, dim, fvecs, fnorm);
    return cudaGetLastError();
}

size_t sort_scratch_ints(int Q, int F) {
    const size_t chunks = (size_t)(Q + kSortChunk - 1) / kSortChunk;
    return (size_t)Q + chunks * (size_t)F;
}

cudaError_t sort_queries_by_key(const int* d_keys, int Q, int F, int* d_bins, int* d_scratch, int32_t* d_order,
                                int sm_count, cudaStream_t stream) {
    const int n_chunks = (Q + kSortChunk - 1) / kSortChunk;
    int* rank_in_chunk = d_scratch;
    int* chunk_counts = d_scratch + Q;
    cudaError_t e = cudaMemsetAsync(chunk_counts, 0, (size_t)n_chunks * F * sizeof(int), stream);
    if (e != cudaSuccess) return e;
    chunk_rank_kernel<<<n_chunks, kSortChunk, 0, stream>>>(d_keys, Q, F, rank_in_chunk, chunk_counts);
    column_scan_kernel<<<(F + 255) / 256, 256, 0, stream>>>(chunk_counts, n_chunks, F, d_bins);
    exclusive_scan_kernel<<<1, 1024, 0, stream>>>(d_bins, F);
    const int blocks = sm_count * 4 < (Q + 255) / 256 ? sm_count * 4 : (Q + 255) / 256;
    place_kernel<<<blocks, 256, 0, stream>>>(d_keys, Q, F, d_bins, chunk_counts, rank_in_chunk, d_order);
    return cudaGetLastError();
}

cudaError_t keys_from_ids(const int32_t* d_ids, int Q, int stride, int F, int* d_keys, int sm_count, cudaStream_t stream) {
    const int blocks = sm_count * 4 < (Q + 255) / 256 ? sm_count * 4 : (Q + 255) / 256;
    first_column_kernel<<<blocks, 256, 0, stream>>>(d_ids, Q, stride, F, d_keys);
    return cudaGetLastError();
}

cudaError_t frontier_keys_simt(const float* d_queries, int Q, int dim, int metric, const float* fvecs, const float* fnorm,
                               int F, int* d_keys, cudaStream_t stream) {
    frontier_argmax_kernel<<<(Q + kTileQ - 1) / kTileQ, 256, 0, stream>>>(d_queries, Q, dim, fvecs, fnorm, F, metric, d_keys);
    return cudaGetLastError();
}

}  // namespace coral
