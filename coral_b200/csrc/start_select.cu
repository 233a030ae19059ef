// Entry-point selection on the device: farthest-point sampling over BFS hop counts
// (replaces Graph::FPS and its kernels, reference src/start.cu:10-145) on the padded
// adjacency.  The first node is given by the caller instead of std::random_device, so
// the same graph always yields the same entry points.
#include <cuda_runtime.h>
#include <stdint.h>

#include "start_select.cuh"

namespace coral {

namespace {

__global__ void fps_bfs_init(int* __restrict__ hops, int64_t n, int start, int* __restrict__ frontier) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        hops[i] = i == start ? 0 : -1;
    if (blockIdx.x == 0 && threadIdx.x == 0) frontier[0] = start;
}

// One warp per frontier node; a neighbour is claimed for this level by compare-and-swap on its
// hop count and appended to the next frontier (warp-aggregated).
__global__ void fps_bfs_expand(const int32_t* __restrict__ adj, int deg_pad, int64_t n, const int* __restrict__ frontier,
                               int frontier_size, int* __restrict__ next_frontier, int* __restrict__ next_size,
                               int* __restrict__ hops, int level) {
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, total = (gridDim.x * blockDim.x) >> 5;
    for (int i = warp; i < frontier_size; i += total) {
        const int u = frontier[i];
        for (int j = lane; j < deg_pad; j += 32) {
            const int v = adj[(size_t)u * deg_pad + j];
            const bool won = v >= 0 && (int64_t)v < n && atomicCAS(hops + v, -1, level) == -1;
            const unsigned m = __ballot_sync(0xffffffffu, won);
            if (m) {
                int base = 0;
                if (lane == 0) base = atomicAdd(next_size, __popc(m));
                base = __shfl_sync(0xffffffffu, base, 0);
                if (won) next_frontier[base + __popc(m & ((1u << lane) - 1u))] = v;
            }
        }
    }
}

// min_hops update (src/start.cu:20-31) fused with the arg-max of the updated values: the packed
// word (value biased to unsigned : inverted index) makes atomicMax pick the largest value and,
// among equals, the lowest index.
__global__ void fps_update_and_argmax(const int* __restrict__ hops, int* __restrict__ min_hops, int64_t n,
                                      unsigned long long* __restrict__ best) {
    unsigned long long local = 0ull;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int h = hops[i];
        int m = min_hops[i];
        if (h >= 0) {
            if (h < m || m < 0) m = h;
        } else if (m == 2147483647) {
            m = -1;
        }
        min_hops[i] = m;
        const unsigned long long key =
            ((unsigned long long)((unsigned)m ^ 0x80000000u) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
        if (key > local) local = key;
    }
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long o = __shfl_down_sync(0xffffffffu, local, off);
        if (o > local) local = o;
    }
    if ((threadIdx.x & 31) == 0) atomicMax(best, local);
}

__global__ void fps_fill(int* __restrict__ p, int64_t n, int value) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = value;
}

}  // namespace

cudaError_t select_start_ids(const int32_t* d_adj, int64_t n, int deg_pad, int first, int M, int32_t* h_out,
                             int sm_count, cudaStream_t stream, int64_t* launches) {
    int *hops = nullptr, *min_hops = nullptr, *fa = nullptr, *fb = nullptr, *sizes = nullptr;
    unsigned long long* best = nullptr;
    cudaError_t e = cudaMalloc(&hops, sizeof(int) * (size_t)n);
    if (e == cudaSuccess) e = cudaMalloc(&min_hops, sizeof(int) * (size_t)n);
    if (e == cudaSuccess) e = cudaMalloc(&fa, sizeof(int) * (size_t)n);
    if (e == cudaSuccess) e = cudaMalloc(&fb, sizeof(int) * (size_t)n);
    if (e == cudaSuccess) e = cudaMalloc(&sizes, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&best, sizeof(unsigned long long));
    const int blocks = sm_count * 8;
    int count = 0, start = first;
    if (e == cudaSuccess) {
        fps_fill<<<blocks, 256, 0, stream>>>(min_hops, n, 2147483647);
        ++*launches;
        h_out[count++] = start;
    }
    while (e == cudaSuccess && count < M) {
        fps_bfs_init<<<blocks, 256, 0, stream>>>(hops, n, start, fa);
        ++*launches;
        int fsize = 1, level = 1;
        int *cur = fa, *nxt = fb;
        while (e == cudaSuccess && fsize > 0 && level <= 1 << 24) {   // levels are bounded by n anyway
            e = cudaMemsetAsync(sizes, 0, sizeof(int), stream);
            if (e != cudaSuccess) break;
            const int warps_needed = fsize < blocks * 8 ? fsize : blocks * 8;
            fps_bfs_expand<<<(warps_needed + 7) / 8, 256, 0, stream>>>(d_adj, deg_pad, n, cur, fsize, nxt, sizes, hops, level);
            ++*launches;
            e = cudaMemcpyAsync(&fsize, sizes, sizeof(int), cudaMemcpyDeviceToHost, stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
            int* t = cur;
            cur = nxt;
            nxt = t;
            ++level;
        }
        if (e != cudaSuccess) break;
        e = cudaMemsetAsync(best, 0, sizeof(unsigned long long), stream);
        if (e != cudaSuccess) break;
        fps_update_and_argmax<<<blocks, 256, 0, stream>>>(hops, min_hops, n, best);
        ++*launches;
        unsigned long long h_best = 0ull;
        e = cudaMemcpyAsync(&h_best, best, sizeof(h_best), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) break;
        start = (int)(0xFFFFFFFFu - (unsigned)(h_best & 0xFFFFFFFFull));
        h_out[count++] = start;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    cudaFree(hops);
    cudaFree(min_hops);
    cudaFree(fa);
    cudaFree(fb);
    cudaFree(sizes);
    cudaFree(best);
    return e;
}

}  // namespace coral
