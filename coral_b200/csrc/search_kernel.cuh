// Host/device shared declarations of the beam-search kernel (sm_100a).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace coral {

// Per-warp list of new ids waiting for a gather batch (ints): fewer than 64 left over when a scout
// step starts + up to 128 from the step, rounded up.  off_pend must reserve this much per warp.
constexpr int kPendCap = 224;

// Shared-memory plan of one CTA, computed on the host for (dim, L, deg_pad) and
// the tuning knobs; every offset is in bytes from the start of dynamic smem.
struct SearchPlan {
    int warps;        // warps per CTA; every warp runs its own gather/distance pipeline
    int stages;       // per-warp ring depth (stages of 32 row chunks)
    int chunk_bytes;  // bytes of one row chunk moved by one bulk copy (multiple of 16)
    int n_chunks;     // chunks per row (chunk_bytes * n_chunks == dim * 4; >= dim * 4 in gather mode 2)
    int row_stride;   // bytes between two rows inside a stage (padded against bank conflicts)
    int group_stride; // gather mode 2: bytes between two groups of four rows (multiple of 128)
    int tail_vec;     // 16-byte units of the last chunk that belong to the row (the rest reads as zeros)
    int stage_bytes;  // 32 * row_stride (8 * group_stride in gather mode 2)
    int hs_bits;      // log2 entries of the shared-memory visited hash, 0 = none
    int vc_bits;      // log2 entries of the shared-memory cache of recently seen ids, 0 = none
    int LP;           // beam array length: L rounded up to a power of two
    int tile_max;     // largest candidate tile sorted at once (power of two)
    int ctas_per_sm;
    int gather;       // how row chunks reach shared memory: 0 = one bulk copy per row chunk, 1 = 16-byte unit copies,
                      // 2 = tensor copies that gather the chunks of four rows each (needs the row map)
    int carry;        // 1 = an id its first probe pair does not settle is carried into the lane's next scout step
    int off_query, off_beam0, off_beam1, off_exp, off_hash, off_vcache, off_bar, off_pend, off_bids, off_stage;
    int smem_bytes;
};

// Round state shared by the CTAs of a thread-block cluster that work on one query
// (small-batch mode); lives in global memory, one block per cluster.
struct ClusterCtl {
    int exp_count, exp_next, cand_count, done;
    float worst;
    int n_dist, n_exp, n_scan, n_spill, status;
    int abort;   // the leader saw the launch's error flag: the cluster takes no further query
    int pad[5];
};

struct SearchArgs {
    const float* vecs;         // [n][dim]
    const int32_t* adj;        // [n][deg_pad]
    const float* queries;      // [Q][dim]
    const int32_t* start_ids;  // [M]
    const uint32_t* deleted;   // nullable bitset over n
    int32_t* ids_out;          // [Q][k]
    float* dists_out;          // nullable [Q][k]
    int32_t* stats_out;        // nullable [Q][8]
    unsigned long long* hops_total;  // sum of per-query hops
    uint64_t* ghash;           // [grid][gh_mask+1] spill table of the visited set, epoch-tagged
    uint64_t* gcand;           // [grid][cand_cap] candidates of the current round
    int* q_counter;            // next query to take
    int* err_flag;             // set when a bounded wait ran out
    int* worst_status;         // nullable: atomicMax of the per-query status words of the launch
    long long* dbg;            // self-checking build only: [0] first failed check, [1..4] its values
    ClusterCtl* cctl;          // cluster mode: [clusters] round state
    int32_t* gexp;             // cluster mode: [clusters][L] ids to expand this round
    const int32_t* order;      // nullable: order[i] = the i-th query to run (locality scheduling)
    int64_t n;
    int dim, deg_pad, deg_shift, M, Q, L, k;
    uint32_t epoch_base;       // epoch of query q is epoch_base + q + 1 (never 0)
    uint32_t gh_mask;
    int cand_cap;              // L * deg_pad
    int ids_per_lane;          // neighbour ids a lane examines per scout step, 1..4 (0 = 4)
    int max_rounds;
    SearchPlan plan;
};

// Cache of the opt-in shared-memory size granted per (device, metric, kernel variant): the slot of
// a [kMaxGrantDevices][2][2] table, or nullptr for a device the table does not cover.
constexpr int kMaxGrantDevices = 64;
int* granted_slot(int* table, int device, int metric, bool cluster);

// Launches the kernel for `metric` (0 = L2, 1 = IP) with `grid` CTAs on `stream`.  With
// cluster_size > 1 the grid is made of thread-block clusters of that many CTAs, each cluster
// working on one query at a time (grid must be a multiple of cluster_size).
// `row_map` (gather mode 2 only): the tensor map made by make_row_gather_map for a.vecs and this plan.
cudaError_t launch_beam_search(const SearchArgs& a, int metric, int grid, cudaStream_t stream, int cluster_size = 1,
                               const CUtensorMap* row_map = nullptr);
// Tensor map of the [n][dim] fp32 row array for gather mode 2: two dimensions, a box of one row by
// `box_floats` columns, no swizzle; columns past `dim` read as zeros.  False when the driver's
// encoder is not available or refuses the shape.
bool make_row_gather_map(CUtensorMap* map, const float* vecs, int64_t n, int dim, int box_floats);
// Whether the driver's tensor-map encoder can be reached at all (asked once per process).
bool row_gather_available();
// Registers the dynamic shared-memory size with the runtime and returns the
// number of CTAs of this plan that fit one SM (0 on failure).
int beam_search_occupancy(const SearchPlan& p, int metric);
// Number of clusters of `cluster_size` CTAs of this plan that can be resident at once (0 when
// that cluster size cannot be launched).
int beam_search_max_clusters(const SearchPlan& p, int metric, int cluster_size);

}  // namespace coral
