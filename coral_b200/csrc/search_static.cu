// coral_search_static: the beam search for callers that must not allocate.
//
// Some embedders of this library cannot call cudaMalloc when they want to
// search: a serving process whose memory pool already owns the whole device, a
// plugin running inside another framework's stream callback, code executing
// under a memory-budget guard that treats any allocation as a fault.  The
// regular path (coral_search_prepare) gives the kernel two scratch areas from
// cudaMalloc -- the global visited table and the per-round candidate buffers.
// This entry point runs the very same kernel with that scratch carved out of a
// fixed array that is part of the library image, so nothing is allocated or
// freed here: no cudaMalloc/cudaFree, no host containers, no library routine
// that allocates.
//
// Costs and rules:
//   * every GPU that loads the library holds the array (kStaticScratchBytes)
//     until the process exits, used or not;
//   * the array bounds the problem: L * deg_pad <= kMaxCandidates, and the
//     number of CTAs in flight is whatever fits, so it is slower than the
//     regular path on large beams;
//   * the first call on a device looks up the array's device address (once per
//     device); make that first call outside any stream capture;
//   * all calls share the one array.  The visited table is never cleared --
//     entries carry a per-query epoch that only grows -- and the few control
//     words that must start at zero are zeroed on the stream by every call.
//     Two calls that overlap on the same GPU race on the array: serialise them.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/coral_b200.h"
#include "plan.cuh"
#include "search_kernel.cuh"

namespace {

constexpr size_t kStaticScratchBytes = 64ull << 20;  // 64 MiB per GPU
constexpr int kMaxCandidates = 16384;                // L * deg_pad, e.g. L = 256 at degree 64
constexpr int kMaxDevices = 64;
constexpr size_t kCtrlBytes = 256;                   // control words at the start of the array

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct DeviceState {
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
    int smem_optin = 0;
    uint32_t epoch_base = 0;
    uint32_t last_entries = 0;  // carving of the previous call: a different one invalidates the tables
    int last_cand_cap = 0, last_grid = 0;
    int last_status = 0;        // worst per-query status of the previous call
};
DeviceState g_state[kMaxDevices];
std::mutex g_mutex;

// cudaPointerGetAttributes allocates nothing; a host pointer handed in by mistake is refused here
// instead of faulting in the kernel.
bool is_device_ptr(const void* p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged;
}

}  // namespace

extern "C" int coral_search_static(int device, void* stream, const float* d_vecs, const int32_t* d_adj,
                                   int64_t n, int dim, int deg_pad, int metric, const int32_t* d_start_ids,
                                   int M, const float* d_queries, int Q, int L, int k, int32_t* d_ids_out,
                                   float* d_dists_out) {
    if (!d_vecs || !d_adj || !d_start_ids || (Q > 0 && (!d_queries || !d_ids_out))) return CORAL_ERR_ARG;
    if (device < 0 || device >= kMaxDevices) return CORAL_ERR_ARG;
    if (n <= 0 || n > 0x7fffffffll || dim <= 0 || dim % 4 != 0) return CORAL_ERR_ARG;
    if (deg_pad != 32 && deg_pad != 64 && deg_pad != 128) return CORAL_ERR_ARG;
    if (metric != CORAL_L2 && metric != CORAL_IP) return CORAL_ERR_ARG;
    if (Q < 0 || L <= 0 || k <= 0 || k > L || M <= 0 || M > L) return CORAL_ERR_ARG;
    if ((((uintptr_t)d_vecs) & 15) != 0) return CORAL_ERR_ARG;
    // the fixed array bounds the beam: refuse rather than overrun
    if ((long long)L * deg_pad > kMaxCandidates) return CORAL_ERR_LIMIT;
    if (Q > (1 << 24)) return CORAL_ERR_LIMIT;
    if (Q == 0) return CORAL_OK;
    if (!is_device_ptr(d_vecs) || !is_device_ptr(d_adj) || !is_device_ptr(d_start_ids) || !is_device_ptr(d_queries) ||
        !is_device_ptr(d_ids_out) || (d_dists_out && !is_device_ptr(d_dists_out)))
        return CORAL_ERR_ARG;

    std::lock_guard<std::mutex> lock(g_mutex);
    if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        return CORAL_ERR_NOGPU;
    }
    DeviceState& ds = g_state[device];
    if (!ds.scratch) {  // once per device, with that device current
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return CORAL_ERR_CUDA;
        }
        int sms = 0, optin = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) {
            cudaGetLastError();
            return CORAL_ERR_CUDA;
        }
        ds.sm_count = sms;
        ds.smem_optin = optin;
        ds.epoch_base = 0;
        ds.scratch = static_cast<unsigned char*>(ptr);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // The same planner as the handle-based path, with its default options.
    coral::SearchPlan plan;
    const char* why = nullptr;
    if (!coral::make_plan(dim, ds.smem_optin, coral::PlanOptions{}, L, plan, &why)) return CORAL_ERR_LIMIT;
    int per_sm = coral::beam_search_occupancy(plan, metric);
    if (per_sm <= 0) return CORAL_ERR_CUDA;
    if (per_sm > plan.ctas_per_sm) per_sm = plan.ctas_per_sm;

    // carve the array: [control words | per-CTA visited tables | per-CTA candidate buffers]
    // The visited table gets 8 x L x deg_pad entries per CTA (what coral_search_prepare gives it)
    // when a full grid of such CTAs fits the array, else 4 x (never fewer than 4096).
    const int cand_cap = L * deg_pad;
    int grid = ds.sm_count * per_sm;
    if (grid > Q) grid = Q;
    uint32_t gh_entries = 1u << 12;
    while (gh_entries < 8u * (uint32_t)cand_cap) gh_entries <<= 1;
    size_t per_cta = (size_t)gh_entries * 8 + (size_t)cand_cap * 8;
    if ((size_t)grid * per_cta > kStaticScratchBytes - kCtrlBytes && gh_entries > (1u << 12) &&
        gh_entries / 2 >= 4u * (uint32_t)cand_cap) {
        gh_entries >>= 1;
        per_cta = (size_t)gh_entries * 8 + (size_t)cand_cap * 8;
    }
    const size_t fit = (kStaticScratchBytes - kCtrlBytes) / per_cta;
    if (fit < 1) return CORAL_ERR_LIMIT;
    if ((size_t)grid > fit) grid = (int)fit;

    const bool recarved = gh_entries != ds.last_entries || cand_cap != ds.last_cand_cap || grid != ds.last_grid;
    ds.last_entries = gh_entries;
    ds.last_cand_cap = cand_cap;
    ds.last_grid = grid;
    // The array keeps the previous call's bytes.  Old table entries are harmless (their epochs are
    // smaller), but after a different carving a table could overlap old candidate records, and when
    // epochs would wrap old entries could look current: wipe everything in both cases.
    if (recarved || (uint64_t)ds.epoch_base + (uint64_t)Q + 2ull >= 0xFFFFFFFFull) {
        if (cudaMemsetAsync(ds.scratch, 0, kStaticScratchBytes, st) != cudaSuccess) {
            cudaGetLastError();
            return CORAL_ERR_CUDA;
        }
        ds.epoch_base = 0;
    }
    if (cudaMemsetAsync(ds.scratch, 0, kCtrlBytes, st) != cudaSuccess) {  // query counter, error flag, hop total
        cudaGetLastError();
        return CORAL_ERR_CUDA;
    }

    coral::SearchArgs a{};
    a.vecs = d_vecs;
    a.adj = d_adj;
    a.queries = d_queries;
    a.start_ids = d_start_ids;
    a.deleted = nullptr;
    a.ids_out = d_ids_out;
    a.dists_out = d_dists_out;
    a.stats_out = nullptr;
    a.q_counter = reinterpret_cast<int*>(ds.scratch);
    a.err_flag = reinterpret_cast<int*>(ds.scratch) + 1;
    a.worst_status = reinterpret_cast<int*>(ds.scratch) + 4;
    a.hops_total = reinterpret_cast<unsigned long long*>(ds.scratch) + 1;
    a.ghash = reinterpret_cast<uint64_t*>(ds.scratch + kCtrlBytes);
    a.gcand = reinterpret_cast<uint64_t*>(ds.scratch + kCtrlBytes + (size_t)grid * gh_entries * 8);
    a.n = n;
    a.dim = dim;
    a.deg_pad = deg_pad;
    a.deg_shift = deg_pad == 32 ? 5 : (deg_pad == 64 ? 6 : 7);
    a.M = M;
    a.Q = Q;
    a.L = L;
    a.k = k;
    a.epoch_base = ds.epoch_base;
    a.gh_mask = gh_entries - 1;
    a.cand_cap = cand_cap;
    a.max_rounds = 1 << 16;
    a.plan = plan;
    if (coral::launch_beam_search(a, metric, grid, st) != cudaSuccess) {
        cudaGetLastError();
        return CORAL_ERR_CUDA;
    }
    ds.epoch_base += (uint32_t)Q;

    int ctrl[5] = {0, 0, 0, 0, 0};   // query counter, error flag, hop total (2 words), worst per-query status
    if (cudaMemcpyAsync(ctrl, ds.scratch, sizeof(ctrl), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess) {
        cudaGetLastError();
        return CORAL_ERR_CUDA;
    }
    ds.last_status = ctrl[4];
    if (ctrl[1]) return CORAL_ERR_KERNEL;
    return ctrl[4] >= CORAL_Q_HASH_OVERFLOW ? CORAL_ERR_QUERY : CORAL_OK;
}

extern "C" int coral_search_static_status(int device) {
    if (device < 0 || device >= kMaxDevices) return -1;
    std::lock_guard<std::mutex> lock(g_mutex);
    return g_state[device].last_status;
}
