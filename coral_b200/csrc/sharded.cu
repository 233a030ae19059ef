// Multi-GPU layer at the C boundary: one handle per GPU, NCCL for the single exchange step.
//
// Sharded index (the base does not fit one GPU): every rank holds one shard with its own graph and
// entry points and searches ALL queries; the per-shard top-k (global ids, distances) are exchanged
// with ONE ncclAllGather and every rank merges only its own contiguous slice of the batch.  The
// reference is single-GPU (there is no NCCL/MPI call site in it); its tiers for large bases are
// host memory and SSD (include/uni.h:149, src/index_gpu.cpp:256-257), which sharding replaces.
//
// NCCL is loaded at first use with dlopen("libnccl.so.2") -- a process that already has NCCL loaded
// (one that imported a framework bundling it) gets that copy -- so the library itself loads and
// works on one GPU without NCCL installed.  Remote data always lands in this GPU's memory through
// NCCL before a kernel of this library reads it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../../include/coral_b200.h"

struct coral_comm {
    ncclComm_t comm = nullptr;
    int device = 0, world = 1, rank = 0;
    int32_t* d_send = nullptr;   // [2][Q][k]: this shard's global ids, then its distances as bits
    int32_t* d_recv = nullptr;   // [world][2][Q][k]
    size_t cap = 0;              // Q * k the two buffers are sized for
    int32_t* d_out_ids = nullptr;   // merged slice when the caller's buffers are on the host
    float* d_out_d = nullptr;
    size_t out_cap = 0;
    float* d_q = nullptr;           // queries staged from a host pointer
    size_t q_cap = 0;
    int32_t* d_id_map = nullptr;    // local -> global ids installed with coral_comm_set_id_map
    int64_t id_map_n = 0;
    std::string err;
};

namespace {

struct Nccl {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

Nccl& nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!n.lib) return;
        n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(dlsym(n.lib, "ncclGetUniqueId"));
        n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(dlsym(n.lib, "ncclCommInitRank"));
        n.CommInitAll = reinterpret_cast<decltype(n.CommInitAll)>(dlsym(n.lib, "ncclCommInitAll"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(n.lib, "ncclCommDestroy"));
        n.AllGather = reinterpret_cast<decltype(n.AllGather)>(dlsym(n.lib, "ncclAllGather"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(n.lib, "ncclGetErrorString"));
        n.ok = n.GetUniqueId && n.CommInitRank && n.CommInitAll && n.CommDestroy && n.AllGather && n.GetErrorString;
    });
    return n;
}

thread_local std::string g_comm_error;

int comm_fail(coral_comm* c, int code, const std::string& msg) {
    if (c) c->err = msg; else g_comm_error = msg;
    return code;
}

bool is_device_ptr(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

void free_buffers(coral_comm* c) {
    cudaFree(c->d_send);
    cudaFree(c->d_recv);
    cudaFree(c->d_out_ids);
    cudaFree(c->d_out_d);
    cudaFree(c->d_q);
    cudaFree(c->d_id_map);
    c->d_send = c->d_recv = c->d_out_ids = c->d_id_map = nullptr;
    c->d_out_d = c->d_q = nullptr;
    c->cap = c->out_cap = c->q_cap = 0;
    c->id_map_n = 0;
}

__global__ void pack_kernel(const int32_t* __restrict__ ids, const float* __restrict__ dists,
                            const int32_t* __restrict__ id_map, long long count, int32_t* __restrict__ send) {
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < count;
         t += (long long)gridDim.x * blockDim.x) {
        const int v = ids[t];
        send[t] = v >= 0 && id_map ? id_map[v] : v;
        send[count + t] = __float_as_int(dists[t]);
    }
}

}  // namespace

extern "C" {

const char* coral_comm_last_error(coral_comm_t* c) { return c ? c->err.c_str() : g_comm_error.c_str(); }

int coral_comm_unique_id(void* id128) {
    if (!id128) return comm_fail(nullptr, CORAL_ERR_ARG, "null argument");
    Nccl& n = nccl();
    if (!n.ok) return comm_fail(nullptr, CORAL_ERR_STATE, "NCCL (libnccl.so.2) could not be loaded");
    ncclUniqueId id;
    const ncclResult_t r = n.GetUniqueId(&id);
    if (r != ncclSuccess) return comm_fail(nullptr, CORAL_ERR_CUDA, std::string("ncclGetUniqueId: ") + n.GetErrorString(r));
    memcpy(id128, &id, sizeof id);
    return CORAL_OK;
}

int coral_comm_create(coral_comm_t** out, int device, int world, int rank, const void* id128) {
    if (!out || !id128 || world < 1 || rank < 0 || rank >= world) return comm_fail(nullptr, CORAL_ERR_ARG, "bad argument");
    *out = nullptr;
    Nccl& n = nccl();
    if (!n.ok) return comm_fail(nullptr, CORAL_ERR_STATE, "NCCL (libnccl.so.2) could not be loaded");
    if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        return comm_fail(nullptr, CORAL_ERR_NOGPU, "cudaSetDevice failed");
    }
    coral_comm* c = new coral_comm();
    c->device = device;
    c->world = world;
    c->rank = rank;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    const ncclResult_t r = n.CommInitRank(&c->comm, world, id, rank);
    if (r != ncclSuccess) {
        const std::string msg = std::string("ncclCommInitRank: ") + n.GetErrorString(r);
        delete c;
        return comm_fail(nullptr, CORAL_ERR_CUDA, msg);
    }
    *out = c;
    return CORAL_OK;
}

int coral_comm_create_all(coral_comm_t** out, const int* devices, int n_dev) {
    if (!out || !devices || n_dev < 1 || n_dev > 64) return comm_fail(nullptr, CORAL_ERR_ARG, "bad argument");
    Nccl& n = nccl();
    if (!n.ok) return comm_fail(nullptr, CORAL_ERR_STATE, "NCCL (libnccl.so.2) could not be loaded");
    ncclComm_t comms[64];
    const ncclResult_t r = n.CommInitAll(comms, n_dev, devices);
    if (r != ncclSuccess) return comm_fail(nullptr, CORAL_ERR_CUDA, std::string("ncclCommInitAll: ") + n.GetErrorString(r));
    for (int i = 0; i < n_dev; ++i) {
        coral_comm* c = new coral_comm();
        c->comm = comms[i];
        c->device = devices[i];
        c->world = n_dev;
        c->rank = i;
        out[i] = c;
    }
    return CORAL_OK;
}

int coral_comm_destroy(coral_comm_t* c) {
    if (!c) return CORAL_OK;
    cudaSetDevice(c->device);
    free_buffers(c);
    if (c->comm) nccl().CommDestroy(c->comm);
    cudaGetLastError();
    delete c;
    return CORAL_OK;
}

int coral_comm_set_id_map(coral_comm_t* c, const int32_t* ids, int64_t count) {
    if (!c || !ids || count <= 0) return comm_fail(c, CORAL_ERR_ARG, "bad argument");
    if (cudaSetDevice(c->device) != cudaSuccess) {
        cudaGetLastError();
        return comm_fail(c, CORAL_ERR_NOGPU, "cudaSetDevice failed");
    }
    cudaFree(c->d_id_map);
    c->d_id_map = nullptr;
    c->id_map_n = 0;
    if (cudaMalloc(&c->d_id_map, (size_t)count * sizeof(int32_t)) != cudaSuccess ||
        cudaMemcpy(c->d_id_map, ids, (size_t)count * sizeof(int32_t), cudaMemcpyDefault) != cudaSuccess) {
        cudaGetLastError();
        return comm_fail(c, CORAL_ERR_CUDA, "id map upload failed");
    }
    c->id_map_n = count;
    return CORAL_OK;
}

int coral_comm_world(coral_comm_t* c) { return c ? c->world : 0; }
int coral_comm_rank(coral_comm_t* c) { return c ? c->rank : -1; }

void coral_query_slice(int Q, int world, int rank, int* lo, int* hi) {
    if (lo) *lo = (int)((long long)rank * Q / world);
    if (hi) *hi = (int)((long long)(rank + 1) * Q / world);
}

int coral_search_sharded(coral_index_t* h, coral_comm_t* c, const int32_t* d_id_map, const float* d_queries, int Q,
                         int L, int k, int32_t* ids_out, float* dists_out, void* stream) {
    if (!h || !c || (Q > 0 && (!d_queries || !ids_out))) return comm_fail(c, CORAL_ERR_ARG, "null argument");
    if (Q < 0 || k <= 0 || (long long)c->world * k > 4096) return comm_fail(c, CORAL_ERR_LIMIT, "need world * k <= 4096");
    Nccl& n = nccl();
    if (!n.ok) return comm_fail(c, CORAL_ERR_STATE, "NCCL (libnccl.so.2) could not be loaded");
    if (cudaSetDevice(c->device) != cudaSuccess) {
        cudaGetLastError();
        return comm_fail(c, CORAL_ERR_NOGPU, "cudaSetDevice failed");
    }
    if (Q == 0) return CORAL_OK;
    if (d_id_map && !is_device_ptr(d_id_map)) return comm_fail(c, CORAL_ERR_ARG, "the id map must be a device pointer");
    if (!d_id_map) d_id_map = c->d_id_map;      // installed with coral_comm_set_id_map (NULL: ids are global already)
    cudaStream_t st = static_cast<cudaStream_t>(stream ? stream : coral_index_stream(h));
    if (!is_device_ptr(d_queries)) {            // host queries: staged on the stream
        int dim = 0;
        if (coral_get_option(h, "dim", &dim) != CORAL_OK || dim <= 0) return comm_fail(c, CORAL_ERR_STATE, "cannot read the index dimension");
        const size_t floats = (size_t)Q * dim;
        if (floats > c->q_cap) {
            cudaFree(c->d_q);
            c->d_q = nullptr;
            c->q_cap = 0;
            if (cudaMalloc(&c->d_q, floats * sizeof(float)) != cudaSuccess) {
                cudaGetLastError();
                return comm_fail(c, CORAL_ERR_CUDA, "sharded search buffers: out of memory");
            }
            c->q_cap = floats;
        }
        if (cudaMemcpyAsync(c->d_q, d_queries, floats * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess) {
            cudaGetLastError();
            return comm_fail(c, CORAL_ERR_CUDA, "sharded search: query copy failed");
        }
        d_queries = c->d_q;
    }
    const size_t cells = (size_t)Q * k;
    int lo = 0, hi = 0;
    coral_query_slice(Q, c->world, c->rank, &lo, &hi);
    const size_t out_cells = (size_t)(hi - lo) * k;
    cudaError_t e = cudaSuccess;
    if (cells > c->cap) {       // grown on demand, kept between calls: no allocation in steady state
        cudaFree(c->d_send);
        cudaFree(c->d_recv);
        c->d_send = c->d_recv = nullptr;
        c->cap = 0;
        e = cudaMalloc(&c->d_send, 4 * cells * sizeof(int32_t));       // [2][Q][k] packed + [2][Q][k] raw local results
        if (e == cudaSuccess) e = cudaMalloc(&c->d_recv, (size_t)c->world * 2 * cells * sizeof(int32_t));
        if (e == cudaSuccess) c->cap = cells;
    }
    const bool out_dev = is_device_ptr(ids_out);
    if (e == cudaSuccess && !out_dev && out_cells > c->out_cap) {
        cudaFree(c->d_out_ids);
        cudaFree(c->d_out_d);
        c->d_out_ids = nullptr;
        c->d_out_d = nullptr;
        c->out_cap = 0;
        e = cudaMalloc(&c->d_out_ids, out_cells * sizeof(int32_t));
        if (e == cudaSuccess) e = cudaMalloc(&c->d_out_d, out_cells * sizeof(float));
        if (e == cudaSuccess) c->out_cap = out_cells;
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return comm_fail(c, CORAL_ERR_CUDA, std::string("sharded search buffers: ") + cudaGetErrorString(e));
    }
    // 1. this shard's top-k of every query (shard-local ids)
    int32_t* raw_ids = c->d_send + 2 * cells;
    float* raw_d = reinterpret_cast<float*>(c->d_send + 3 * cells);
    int rc = coral_search_async(h, d_queries, Q, L, k, raw_ids, raw_d, nullptr, st);
    if (rc != CORAL_OK) return comm_fail(c, rc, coral_last_error(h));
    // 2. global ids and distance bits side by side: one buffer, one collective
    const int blocks = (int)((cells + 255) / 256 < 2048 ? (cells + 255) / 256 : 2048);
    pack_kernel<<<blocks, 256, 0, st>>>(raw_ids, raw_d, d_id_map, (long long)cells, c->d_send);
    const ncclResult_t r = n.AllGather(c->d_send, c->d_recv, 2 * cells, ncclInt32, c->comm, st);
    if (r != ncclSuccess) return comm_fail(c, CORAL_ERR_CUDA, std::string("ncclAllGather: ") + n.GetErrorString(r));
    // 3. merge this rank's slice of the batch only
    int32_t* mi = out_dev ? ids_out : c->d_out_ids;
    float* md = dists_out ? (out_dev ? dists_out : c->d_out_d) : c->d_out_d;
    if (!md) {   // device ids requested without distances: the merge still needs somewhere to put them
        if (out_cells > c->out_cap) {
            cudaFree(c->d_out_d);
            cudaFree(c->d_out_ids);
            c->d_out_ids = nullptr;
            c->d_out_d = nullptr;
            if (cudaMalloc(&c->d_out_ids, out_cells * sizeof(int32_t)) != cudaSuccess ||
                cudaMalloc(&c->d_out_d, out_cells * sizeof(float)) != cudaSuccess) {
                cudaGetLastError();
                return comm_fail(c, CORAL_ERR_CUDA, "sharded search buffers: out of memory");
            }
            c->out_cap = out_cells;
        }
        md = c->d_out_d;
    }
    if (hi > lo) {
        rc = coral_merge_shards_strided(h, c->d_recv + (size_t)lo * k, reinterpret_cast<const float*>(c->d_recv + cells + (size_t)lo * k),
                                        c->world, hi - lo, k, (int64_t)(2 * cells), mi, md, st);
        if (rc != CORAL_OK) return comm_fail(c, rc, coral_last_error(h));
        if (!out_dev) {
            e = cudaMemcpyAsync(ids_out, mi, out_cells * sizeof(int32_t), cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess && dists_out) e = cudaMemcpyAsync(dists_out, md, out_cells * sizeof(float), cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return comm_fail(c, CORAL_ERR_CUDA, std::string("sharded search copy: ") + cudaGetErrorString(e));
            }
        }
    }
    return CORAL_OK;
}

}  // extern "C"
