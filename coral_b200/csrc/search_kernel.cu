// Batched "full expansion" graph beam search for sm_100a.
//
// One CTA owns one query at a time (queries are pulled from an atomic counter,
// like the reference's persistent blocks, src/search_gpu.cu:379).  Inside a
// round every warp is an autonomous pipeline:
//
//   scout    read the adjacency rows of beam entries still to be expanded
//            (coalesced, 128 neighbour ids per step), test-and-set each id in
//            the exact visited set (an epoch-tagged global table; optionally a
//            shared-memory hash in front of it), keep the new ids.  The step is
//            split in two: the first half loads the first pair of probe slots
//            of every id and issues the compare-and-swaps, the second half reads
//            their answers only when the warp runs short of ids, so the
//            microseconds an atomic takes under load overlap with gathering;
//   gather   for 32 new ids at a time, bring the rows into shared memory chunk
//            by chunk with one bulk asynchronous copy (cp.async.bulk, completion
//            counted on an mbarrier) per row chunk, several stages in flight;
//   distance lane j owns row j and accumulates over the chunks in the order of
//            the reference's thread-per-neighbour loop (include/utils.cuh:254-275,
//            :307-323): one sequential fp32 fused chain over d = 0..dim-1, so the
//            distance is bit-identical to the reference's;
//   filter   strictly closer than the worst beam distance at round start
//            (src/search_gpu.cu:432) -> appended to the CTA's candidate buffer.
//
// At the end of a round the CTA merges beam and candidates into the L closest,
// kept sorted by (distance, id): candidates are sorted tile by tile (bitonic, in
// the idle staging memory) and merged by rank.  This replaces the reference's
// one-reduction-per-accepted-candidate loop (src/search_gpu.cu:525-570) and
// yields the same set; ties are resolved by id instead of by thread position.
//
// Nothing here traps or spins without bound: every mbarrier wait has a clock
// limit after which an error flag is raised; once it is up every later wait returns at once and
// no CTA (or cluster) takes another query.
#include "search_kernel.cuh"

#include <cstring>
#include <mutex>

namespace coral {

namespace {

constexpr int kScoutAhead = 64; // a scout step may start while fewer than this many ids are waiting
constexpr int kIdsPerLane = 4;  // neighbour ids examined per lane per scout step
constexpr int kMergeAhead = 4; // candidate passes whose keys are fetched together at the end of a round
constexpr int kProbeSlots = kIdsPerLane + 1;  // ids a lane probes per scout step: the new ones + one carried over
constexpr int kSmemProbes = 8;
constexpr int kGlobalProbes = 256;
constexpr uint32_t kEmpty32 = 0xFFFFFFFFu;
constexpr uint64_t kPadKey = 0xFFFFFFFFFFFFFFFFull;
constexpr long long kWaitClocks = 4000000000ll;  // ~2 s: far beyond any legitimate copy latency

// Self-checking build (-DCORAL_CHECKED): every index that addresses memory is tested first;
// the first failure is recorded (code, two values, query, CTA) and the access skipped, so a
// wrong index shows up as CORAL_ERR_KERNEL with its values instead of a device fault.
#ifdef CORAL_CHECKED
__device__ __noinline__ bool check_failed(long long* dbg, int code, long long v0, long long v1, int qid) {
    if (dbg && atomicCAS((unsigned long long*)&dbg[0], 0ull, (unsigned long long)code) == 0ull) {
        dbg[1] = v0;
        dbg[2] = v1;
        dbg[3] = qid;
        dbg[4] = blockIdx.x;
    }
    return false;
}
#define CORAL_CHECK(cond, code, v0, v1) ((cond) ? true : check_failed(a.dbg, (code), (long long)(v0), (long long)(v1), S.qid))
#else
#define CORAL_CHECK(cond, code, v0, v1) (true)
#endif

struct Control {
    int qid;
    int exp_count;
    int exp_next;
    int cand_count;
    int beam_cnt;
    int fill;
    int status;
    int abort;   // cluster mode: the leader saw the error flag; every CTA of the cluster stops after this query
    float worst;
    // per-query counters
    int n_dist, n_exp, n_scan, n_spill, hops, rounds, max_cand;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
// try_wait that lets the hardware park the thread for up to `ns` nanoseconds while the phase is
// pending, instead of returning at once.
__device__ __forceinline__ uint32_t mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok;
}
// Bounded wait: returns false (and raises *err) when the limit ran out.  Issuing a stage's 32 bulk
// copies already takes the warp about 2000 cycles, so the first try usually succeeds (measured:
// 0.0 retries per chunk on 10M x 512); when it does not, the retry parks the warp instead of
// polling, and the clock limit is only looked at every 64 wake-ups.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
    if (mbar_try_wait(bar, parity)) return true;
    // A wait that already ran out anywhere in the grid invalidates the launch: later waits give up
    // at once, so the kernel drains in the time of one limit instead of one limit per chunk.
    if (*(volatile int*)err != 0) return false;
    const long long t0 = clock64();
    for (uint32_t spins = 1; !mbar_try_wait_parked(bar, parity, 4000u); ++spins) {
        if ((spins & 63u) == 0u && clock64() - t0 > kWaitClocks) {
            atomicExch(err, 1);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Tensor copy that gathers one box (one row by chunk width) from each of four rows of a
// two-dimensional tensor map and lands them back to back at dst (128-byte aligned); the box bytes
// of all four rows, zero fill included, count on the mbarrier.
__device__ __forceinline__ void tensor_gather4(void* dst, const CUtensorMap* map, int col, int r0, int r1, int r2, int r3,
                                               uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_u32(bar))
        : "memory");
}
// 16-byte asynchronous copy global -> shared through the load/store path (L2 only, no L1
// allocation); completion is tracked per thread in commit groups.
__device__ __forceinline__ void ldgsts16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(__cvta_generic_to_global(src))
                 : "memory");
}
__device__ __forceinline__ void ldgsts_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most `younger` of this thread's commit groups are still pending.
__device__ __forceinline__ void ldgsts_wait(int younger) {
    switch (younger) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    }
}
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Thread-block cluster helpers (small-batch mode: one cluster per query).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_cta_count() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ int load_shared_int(const int* p) { return *(const volatile int*)p; }
__device__ __forceinline__ float load_shared_float(const float* p) { return *(const volatile float*)p; }

// "closer" == smaller key.  key = ord(dist):id:expanded-bit.
template <int METRIC>
__device__ __forceinline__ uint32_t ord_of(float d) {
    if (METRIC == 1) d = -d;
    uint32_t u = __float_as_uint(d);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
template <int METRIC>
__device__ __forceinline__ float dist_of(uint32_t o) {
    uint32_t u = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    float d = __uint_as_float(u);
    return METRIC == 1 ? -d : d;
}
template <int METRIC>
__device__ __forceinline__ uint64_t make_key(float d, int id, uint32_t expanded) {
    return ((uint64_t)ord_of<METRIC>(d) << 32) | ((uint64_t)(uint32_t)id << 1) | (uint64_t)expanded;
}
__device__ __forceinline__ int key_id(uint64_t k) { return (int)((uint32_t)(k & 0xffffffffu) >> 1); }

// include/utils.cuh:380-382 with d0 = worst: true when d is strictly closer.
template <int METRIC>
__device__ __forceinline__ bool closer_than(float worst, float d) {
    return METRIC == 0 ? worst > d : worst < d;
}

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

// Exact test-and-set.  0 = newly inserted, 1 = already present, 2 = tables full.
// A key lives in the shared table iff its probe window had a free slot when it
// first arrived; windows never lose entries within a query, so a later lookup
// takes the same route.
__device__ __forceinline__ int visited_insert(uint32_t* sh, int hs_bits, uint64_t* gh, uint32_t gmask,
                                              uint32_t epoch, int id, int& n_spill) {
    if (hs_bits > 0) {
        const uint32_t mask = (1u << hs_bits) - 1u;
        const uint32_t h = ((uint32_t)id * 0x9E3779B1u) >> (32 - hs_bits);
#pragma unroll 1
        for (int p = 0; p < kSmemProbes; ++p) {
            const uint32_t old = atomicCAS(&sh[(h + p) & mask], kEmpty32, (uint32_t)id);
            if (old == kEmpty32) return 0;
            if (old == (uint32_t)id) return 1;
        }
    }
    const uint64_t mine = ((uint64_t)epoch << 32) | (uint32_t)id;
    const uint32_t h = mix32((uint32_t)id) & ~1u;   // probe sequences start on an aligned slot pair (see the scout step)
#pragma unroll 1
    for (int p = 0; p < kGlobalProbes; ++p) {
        unsigned long long* slot = (unsigned long long*)&gh[(h + p) & gmask];
        unsigned long long cur = *(volatile unsigned long long*)slot;
        for (;;) {
            if ((uint32_t)(cur >> 32) == epoch) {
                if ((uint32_t)cur == (uint32_t)id) return 1;
                break;  // taken by another id of this query: next slot
            }
            const unsigned long long old = atomicCAS(slot, cur, (unsigned long long)mine);
            if (old == cur) {
                ++n_spill;
                return 0;
            }
            cur = old;
        }
    }
    return 2;
}

// CTA-wide bitonic sort of n (power of two) keys in shared memory, ascending.
__device__ void bitonic_sort(uint64_t* s, int n, int tid, int nthreads) {
    for (int k = 2; k <= n; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < n; i += nthreads) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const uint64_t a = s[i], b = s[ixj];
                    const bool asc = (i & k) == 0;
                    if ((a > b) == asc) {
                        s[i] = b;
                        s[ixj] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
}

__device__ __forceinline__ int lower_bound_u64(const uint64_t* a, int n, uint64_t x) {  // #{a[i] < x}
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (a[mid] < x)
            lo = mid + 1;
        else
            hi = mid;
    }
    return lo;
}
__device__ __forceinline__ int upper_bound_u64(const uint64_t* a, int n, uint64_t x) {  // #{a[i] <= x}
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (a[mid] <= x)
            lo = mid + 1;
        else
            hi = mid;
    }
    return lo;
}

// One sequential fused chain over a chunk: row and query both in shared memory.
template <int METRIC>
__device__ __forceinline__ float accumulate_chunk(float acc, const float4* __restrict__ row,
                                                  const float4* __restrict__ q, int n_vec) {
#pragma unroll 4
    for (int i = 0; i < n_vec; ++i) {
        const float4 a = row[i];
        const float4 b = q[i];
        if (METRIC == 0) {
            float d;
            d = a.x - b.x; acc = fmaf(d, d, acc);
            d = a.y - b.y; acc = fmaf(d, d, acc);
            d = a.z - b.z; acc = fmaf(d, d, acc);
            d = a.w - b.w; acc = fmaf(d, d, acc);
        } else {
            acc = fmaf(a.x, b.x, acc);
            acc = fmaf(a.y, b.y, acc);
            acc = fmaf(a.z, b.z, acc);
            acc = fmaf(a.w, b.w, acc);
        }
    }
    return acc;
}

// Seed distance in the order of src/search_gpu.cu:14-23: lane-strided fused
// chains, then sum += shfl_down(sum, off) for off = 16..1; lane 0 holds it.
template <int METRIC>
__device__ __forceinline__ float seed_distance(const float* __restrict__ row, const float* __restrict__ q,
                                               int dim, int lane) {
    float sum = 0.f;
    for (int d = lane; d < dim; d += 32) {
        const float b = __ldg(row + d);
        if (METRIC == 0) {
            const float diff = q[d] - b;
            sum = fmaf(diff, diff, sum);
        } else {
            sum = fmaf(q[d], b, sum);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum = sum + __shfl_down_sync(0xffffffffu, sum, off);
    return __shfl_sync(0xffffffffu, sum, 0);
}

// CLUSTER = false: one CTA per query.  CLUSTER = true (small batches): the CTAs of a thread-block
// cluster share one query -- the leader CTA (rank 0) owns the beam, builds the expansion list and
// merges; every CTA runs the scout/gather/distance pipeline against the shared global visited
// table, work counter and candidate buffer; two cluster barriers per round.
template <int METRIC, bool CLUSTER>
__global__ void __maxnreg__(96) beam_search_kernel(const SearchArgs a, const __grid_constant__ CUtensorMap row_map) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ Control S;

    const SearchPlan& P = a.plan;
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;

    float* sq = reinterpret_cast<float*>(smem + P.off_query);
    uint64_t* beam = reinterpret_cast<uint64_t*>(smem + P.off_beam0);
    uint64_t* beam_alt = reinterpret_cast<uint64_t*>(smem + P.off_beam1);
    int* exp_list = reinterpret_cast<int*>(smem + P.off_exp);
    uint32_t* shash = reinterpret_cast<uint32_t*>(smem + P.off_hash);
    // Direct-mapped cache of ids this CTA has already put through the visited set: a hit means
    // "seen" without touching the table (an entry is only written after the table answered).
    uint32_t* vcache = reinterpret_cast<uint32_t*>(smem + P.off_vcache);
    const uint32_t vc_mask = P.vc_bits > 0 ? (1u << P.vc_bits) - 1u : 0u;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P.off_bar) + warp * P.stages;
    int* pend = reinterpret_cast<int*>(smem + P.off_pend) + warp * kPendCap;
    int* bids = reinterpret_cast<int*>(smem + P.off_bids) + warp * 64;  // two batch slots of 32 ids
    unsigned char* stage0 = smem + P.off_stage + (size_t)warp * P.stages * P.stage_bytes;
    uint64_t* sortbuf = reinterpret_cast<uint64_t*>(smem + P.off_stage);  // aliases the staging rings

    int group = blockIdx.x, n_groups = gridDim.x;   // a group = the CTAs working on one query
    bool leader = true;
    if (CLUSTER) {
        const int csize = (int)cluster_cta_count();
        group = blockIdx.x / csize;
        n_groups = gridDim.x / csize;
        leader = cluster_cta_rank() == 0;
    }
    ClusterCtl* GC = CLUSTER ? a.cctl + group : nullptr;
    int32_t* gexp = CLUSTER ? a.gexp + (size_t)group * a.L : nullptr;
    uint64_t* ghash = a.ghash + (size_t)group * ((size_t)a.gh_mask + 1);
    uint64_t* gcand = a.gcand + (size_t)group * (size_t)a.cand_cap;
    int* p_exp_next = CLUSTER ? &GC->exp_next : &S.exp_next;
    int* p_cand_count = CLUSTER ? &GC->cand_count : &S.cand_count;

    if (tid == 0) S.abort = 0;
    if (lane == 0)
        for (int s = 0; s < P.stages; ++s) mbar_init(&bars[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
    __syncthreads();

    // This warp's stream of row chunks.  A batch (<= 32 rows) is n_chunks chunks; chunks go through
    // the ring's stages round-robin.  All bookkeeping is incremental (no divisions in the loop) and
    // lives for the whole kernel, so that the parity of the u-th use of a stage is u & 1.
    uint32_t formed = 0, issued = 0, done = 0;   // batches formed / completely issued / finalised
    int iss_c = 0, con_c = 0;                    // chunks of the current batch issued / consumed
    int iss_st = 0, con_st = 0;                  // ring stage the next issue / consume uses
    uint32_t con_par = 0;                        // parity the next consume waits for
    int inflight = 0;                            // chunks issued and not yet consumed
    const int n_chunks = P.n_chunks;
    const int chunk_vec = P.chunk_bytes >> 4;
    const int chunk_floats = P.chunk_bytes >> 2;
    // A scout step takes the next 32 * ids_per_lane neighbour slots of the round's expansion list
    // (slot = entry * deg_pad + column).  Large steps amortise the latency of a step when a CTA has
    // many entries to itself; small steps spread a short list over the many warps of a cluster.
    const int ipl = a.ids_per_lane < 1 ? kIdsPerLane : (a.ids_per_lane > kIdsPerLane ? kIdsPerLane : a.ids_per_lane);
    const int step_slots = 32 * ipl;
    const int row_bytes = a.dim * 4;
    // Unit-copy gather (P.gather == 1): a row chunk is chunk_vec 16-byte units; the warp's lanes
    // walk the (row, unit) pairs of a stage 32 at a time, so one instruction copies whole
    // contiguous runs (two 256-byte chunks, one 512-byte chunk, ...).
    const bool unit_gather = P.gather == 1;
    // Tensor gather (P.gather == 2): lane g < 8 copies the chunk of rows 4g..4g+3 with one
    // instruction; row r of the stage then sits at (r / 4) * group_stride + (r % 4) * chunk_bytes.
    const bool tensor_gather = P.gather == 2;
    const int lane_row_off = tensor_gather ? (lane >> 2) * P.group_stride + (lane & 3) * P.chunk_bytes : lane * P.row_stride;
    const int lane_r0 = lane / chunk_vec, lane_u0 = lane % chunk_vec;
    const int step_r = 32 / chunk_vec, step_u = 32 % chunk_vec;

    for (int turn = 0;; ++turn) {
        // ---------------------------------------------------------------- take a query
        __syncthreads();
        if (tid == 0) {
            int q = -1;
            if (CLUSTER)
                q = S.abort ? -1 : group + turn * n_groups;   // static: every CTA of the cluster must agree
            else if (*(volatile int*)a.err_flag == 0)
                q = atomicAdd(a.q_counter, 1);
            if (q < 0 || q >= a.Q) q = -1;
            else if (a.order) q = a.order[q];   // scheduled batches: the q-th query to run, results stay at its own row
            S.qid = q;
            S.status = 0;
            S.worst = METRIC == 0 ? 3.402823466e+38f : -3.402823466e+38f;
            S.n_dist = leader ? a.M : 0;
            S.n_exp = S.n_scan = S.n_spill = S.hops = S.rounds = S.max_cand = 0;
            S.beam_cnt = a.M;
        }
        __syncthreads();
        const int qid = S.qid;
        if (qid < 0) break;
        const uint32_t epoch = a.epoch_base + (uint32_t)qid + 1u;

        for (int d = tid; d < a.dim; d += nthreads) sq[d] = a.queries[(size_t)qid * a.dim + d];
        if (P.hs_bits > 0)
            for (int i = tid; i < (1 << P.hs_bits); i += nthreads) shash[i] = kEmpty32;
        if (P.vc_bits > 0)
            for (int i = tid; i < (1 << P.vc_bits); i += nthreads) vcache[i] = kEmpty32;
        for (int i = tid; i < P.LP; i += nthreads) beam[i] = kPadKey;
        __syncthreads();

        int n_spill = 0, n_scan = 0, n_exp = 0, n_dist = 0;  // per-thread tallies
        bool overflow = false;

        // ---------------------------------------------------------------- entry points
        for (int i = warp; leader && i < a.M; i += (nthreads >> 5)) {
            const int id = a.start_ids[i];
            if (id < 0 || (int64_t)id >= a.n) {   // never dereferenced: the slot stays padding, the query is flagged
                if (lane == 0) {
                    atomicSub(&S.beam_cnt, 1);
                    atomicSub(&S.n_dist, 1);
                    atomicMax(&S.status, 4);
                }
                continue;
            }
            if (lane == 0) {
                const int r = visited_insert(shash, P.hs_bits, ghash, a.gh_mask, epoch, id, n_spill);
                if (r == 2) overflow = true;  // duplicates are kept on purpose (src/search_gpu.cu:396-397)
            }
            const float d = seed_distance<METRIC>(a.vecs + (size_t)id * a.dim, sq, a.dim, lane);
            if (lane == 0) beam[i] = make_key<METRIC>(d, id, 0u);
        }
        __syncthreads();
        if (leader) bitonic_sort(beam, P.LP, tid, nthreads);

        // ---------------------------------------------------------------- rounds
        bool finished = false;   // leader's verdict on the previous round (cluster mode)
        for (;;) {
            // expansion list: every beam entry not yet expanded (src/search_gpu.cu:416-422)
            if (leader && !finished) {
                if (tid == 0) {
                    S.exp_count = 0;
                    S.exp_next = 0;
                    S.cand_count = 0;
                    S.rounds += 1;
                }
                __syncthreads();
                const int beam_cnt = S.beam_cnt;
                for (int i = tid; i < beam_cnt; i += nthreads) {
                    const uint64_t key = beam[i];
                    if ((key & 1ull) == 0ull) {
                        const int slot = atomicAdd(&S.exp_count, 1);
                        if (CORAL_CHECK(slot < a.L && key_id(key) >= 0 && (int64_t)key_id(key) < a.n, 1, slot, key)) {
                            if (CLUSTER) gexp[slot] = key_id(key); else exp_list[slot] = key_id(key);
                        }
                        beam[i] = key | 1ull;
                    }
                }
                __syncthreads();
            }
            if (CLUSTER) {
                if (leader && tid == 0) {   // publish the round to the other CTAs
                    GC->exp_count = S.exp_count;
                    GC->exp_next = 0;
                    GC->cand_count = 0;
                    GC->worst = S.worst;
                    GC->done = finished ? 1 : 0;
                }
                __threadfence();
                cluster_sync_all();
                if (load_shared_int(&GC->done)) break;
            }
            const int exp_count = CLUSTER ? load_shared_int(&GC->exp_count) : S.exp_count;
            const float worst = CLUSTER ? load_shared_float(&GC->worst) : S.worst;

            // ------------------------------------------------------------ warp pipeline
            {
                int pend_n = 0;
                int bcnt0 = 0, bcnt1 = 0;          // rows in batch slot 0 / 1
                // `more`: a step of the round's expansion list has been claimed for this warp and its
                // neighbour ids are on their way (or already) in nv[]: the adjacency rows of a step are
                // requested one step ahead, so their latency overlaps the visited-table probes of the
                // step before instead of preceding its own.
                bool more = false;
                int nv[kIdsPerLane];
                const int total_slots = exp_count << a.deg_shift;
                // The last steps of a round are claimed 32 slots at a time, so that the CTA's warps run out
                // of work within a quarter of a step of each other instead of a whole one.
                const int tail_slots = (nthreads >> 5) * step_slots;
                auto claim_step = [&]() {
                    int s0 = total_slots, want = step_slots;
                    if (lane == 0) {
                        if (!CLUSTER && total_slots - *(volatile int*)p_exp_next <= tail_slots) want = 32;
                        s0 = atomicAdd(p_exp_next, want);
                    }
                    s0 = __shfl_sync(0xffffffffu, s0, 0);
                    want = __shfl_sync(0xffffffffu, want, 0);
                    const int ipl = want >> 5;
                    more = s0 < total_slots;
                    if (more && lane == 0) {   // entries whose first slot falls into this step
                        const int s1 = s0 + want < total_slots ? s0 + want : total_slots;
                        n_exp += ((s1 + a.deg_pad - 1) >> a.deg_shift) - ((s0 + a.deg_pad - 1) >> a.deg_shift);
                    }
#pragma unroll
                    for (int t = 0; t < kIdsPerLane; ++t) {
                        const int slot = s0 + lane + 32 * t;
                        const int ent = slot >> a.deg_shift;
                        nv[t] = -1;
                        if (more && t < ipl && ent < exp_count) {
                            const int node = CLUSTER ? __ldcg(gexp + ent) : exp_list[ent];
                            if (CORAL_CHECK(ent < a.L && node >= 0 && (int64_t)node < a.n, 4, node, ent))
                                nv[t] = __ldg(a.adj + (size_t)node * a.deg_pad + (slot & (a.deg_pad - 1)));
                        }
                    }
                };
                if (exp_count > 0) claim_step();
                float acc = 0.f;
                // A scout step is split in two: its compare-and-swaps are issued and the warp goes back to
                // gathering and distances; their answers (which take microseconds under load) are only
                // looked at when the warp runs short of ids.
                // An id that its first pair of slots does not settle (both taken by other ids, or the
                // slot lost to another id) is carried into the lane's next step, which probes the next
                // pair for it, instead of walking the probe sequence with the warp waiting.
                bool sc_pending = false;
                uint32_t sc_cas = 0u;              // bit t: a compare-and-swap is in flight for sv[t]
                int sv[kProbeSlots];               // [kIdsPerLane] is the carried id
                unsigned long long scur[kProbeSlots], sold[kProbeSlots];
                int carry_att = 0;                 // pair of the probe sequence the carried id tries next
                bool has_carry = false;            // some lane of the warp carries an id
#pragma unroll
                for (int t = 0; t < kProbeSlots; ++t) {
                    sv[t] = -1;
                    scur[t] = sold[t] = 0ull;
                }
                for (;;) {
                    // form gather batches from pending ids
                    while (formed - done < 2u && (pend_n >= 32 || (!more && !sc_pending && !has_carry && pend_n > 0))) {
                        const int m = pend_n < 32 ? pend_n : 32;
                        const int slot = formed & 1u;
                        if (lane < m && CORAL_CHECK(pend_n - m + lane >= 0 && pend_n - m + lane < kPendCap, 2, pend_n, m))
                            bids[slot * 32 + lane] = pend[pend_n - m + lane];
                        if (slot) bcnt1 = m; else bcnt0 = m;
                        pend_n -= m;
                        ++formed;
                        __syncwarp();
                    }
                    // keep the ring full
                    while (issued < formed && inflight < P.stages) {
                        const uint32_t b = issued;
                        const int c = iss_c, st = iss_st;
                        const int cnt = (b & 1u) ? bcnt1 : bcnt0;
                        if (unit_gather) {
                            const int* ids = bids + (b & 1u) * 32;
                            unsigned char* dst0 = stage0 + (size_t)st * P.stage_bytes;
                            const unsigned char* src0 =
                                reinterpret_cast<const unsigned char*>(a.vecs) + (size_t)c * P.chunk_bytes;
                            int r = lane_r0, u = lane_u0;
                            while (r < cnt) {
                                int id = ids[r];
                                if (!CORAL_CHECK(id >= 0 && (int64_t)id < a.n && cnt <= 32 && (int)st < P.stages, 3, id, cnt)) id = 0;
                                ldgsts16(dst0 + r * P.row_stride + u * 16, src0 + (size_t)id * row_bytes + u * 16);
                                r += step_r;
                                u += step_u;
                                if (u >= chunk_vec) {
                                    u -= chunk_vec;
                                    ++r;
                                }
                            }
                            ldgsts_commit();
                        } else if (tensor_gather) {
                            const int groups = (cnt + 3) >> 2;
                            if (lane == 0) mbar_expect_tx(&bars[st], (uint32_t)groups * 4u * (uint32_t)P.chunk_bytes);
                            __syncwarp();
                            if (lane < groups) {
                                // a group the batch does not fill repeats its first row
                                const int* ids = bids + (b & 1u) * 32 + lane * 4;
                                int r[4];
#pragma unroll
                                for (int t = 0; t < 4; ++t) {
                                    r[t] = lane * 4 + t < cnt ? ids[t] : ids[0];
                                    if (!CORAL_CHECK(r[t] >= 0 && (int64_t)r[t] < a.n && cnt <= 32 && (int)st < P.stages, 3, r[t], cnt)) r[t] = 0;
                                }
                                tensor_gather4(stage0 + (size_t)st * P.stage_bytes + (size_t)lane * P.group_stride, &row_map,
                                               c * chunk_floats, r[0], r[1], r[2], r[3], &bars[st]);
                            }
                        } else {
                            if (lane == 0) mbar_expect_tx(&bars[st], (uint32_t)cnt * (uint32_t)P.chunk_bytes);
                            __syncwarp();
                            if (lane < cnt) {
                                int id = bids[(b & 1u) * 32 + lane];
                                if (!CORAL_CHECK(id >= 0 && (int64_t)id < a.n && cnt <= 32 && (int)st < P.stages, 3, id, cnt)) id = 0;
                                bulk_g2s(stage0 + (size_t)st * P.stage_bytes + (size_t)lane * P.row_stride,
                                         reinterpret_cast<const unsigned char*>(a.vecs) + (size_t)id * row_bytes +
                                             (size_t)c * P.chunk_bytes,
                                         (uint32_t)P.chunk_bytes, &bars[st]);
                            }
                        }
                        ++inflight;
                        iss_st = iss_st + 1 == P.stages ? 0 : iss_st + 1;
                        if (++iss_c == n_chunks) {
                            iss_c = 0;
                            ++issued;
                        }
                    }
                    if (sc_pending && pend_n < 32 && formed - done < 2u) {
                        // ---- scout, second half: read the answers; an id its pair did not settle is carried
                        bool isnew[kProbeSlots];
                        int carry_id = -1, carry_next = 0;
#pragma unroll
                        for (int tt = 0; tt < kProbeSlots; ++tt) {
                            const int t = tt == 0 ? kIdsPerLane : tt - 1;   // the carried id first: it may free the carry slot
                            isnew[t] = false;
                            // Keeps the comparison below from being scheduled next to the compare-and-swap
                            // (where it would wait for the answer the first half was written to not wait for).
                            asm volatile("" : "+l"(scur[t]));
                            if (sv[t] >= 0) {
                                int r = 3;   // 0 new, 1 seen, 2 table full, 3 = this pair did not settle it
                                bool pair_full = false;
                                if ((sc_cas >> t) & 1u) {
                                    if (sold[t] == scur[t]) {
                                        r = 0;
                                        ++n_spill;
                                    } else if (sold[t] == (((unsigned long long)epoch << 32) | (uint32_t)sv[t])) {
                                        r = 1;   // the same id won the slot first (another lane or warp)
                                    }            // else: lost to another id, the pair is looked at again
                                } else if ((uint32_t)scur[t] == (uint32_t)sv[t]) {
                                    r = 1;       // the slot held this id with this query's epoch
                                } else {
                                    pair_full = true;
                                }
                                if (r == 3) {
                                    const int att = (t == kIdsPerLane ? carry_att : 0) + (pair_full ? 1 : 0);
                                    if (P.carry && carry_id < 0 && att < kGlobalProbes / 2) {
                                        carry_id = sv[t];
                                        carry_next = att;
                                    } else {
                                        r = visited_insert(shash, 0, ghash, a.gh_mask, epoch, sv[t], n_spill);
                                    }
                                }
                                isnew[t] = r == 0;
                                if (r == 2) overflow = true;
                            }
                        }
#pragma unroll
                        for (int t = 0; t < kProbeSlots; ++t) {
                            const uint32_t m = __ballot_sync(0xffffffffu, isnew[t]);
                            if (isnew[t] && CORAL_CHECK(pend_n + __popc(m & lt_mask) < kPendCap, 5, pend_n, m))
                                pend[pend_n + __popc(m & lt_mask)] = sv[t];
                            pend_n += __popc(m);
                        }
                        sv[kIdsPerLane] = carry_id;
                        carry_att = carry_next;
                        has_carry = __any_sync(0xffffffffu, carry_id >= 0);
                        sc_pending = false;
                        __syncwarp();
                        continue;
                    }
                    if ((more || has_carry) && !sc_pending && pend_n < kScoutAhead) {
                        // ---- scout, first half: adjacency rows of the next slots, visited-table probes
                        int v[kIdsPerLane];
#pragma unroll
                        for (int t = 0; t < kIdsPerLane; ++t) v[t] = more ? nv[t] : -1;
                        if (more) claim_step();   // the next step's rows are requested before this step's probes
                        if (P.hs_bits == 0 && P.vc_bits == 0) {
                            // Visited set entirely in the global table.  The first probe slots of a lane's
                            // ids are loaded side by side; a slot of another query (or never used) is
                            // claimed by compare-and-swap, whose answer is read in the second half.
                            // The probe sequence of an id starts on an aligned pair of slots, read with
                            // one 16-byte load: only when both hold other ids of this query (rare at the
                            // table's load) is the id left to the full probe in the second half.
                            unsigned long long* slot[kProbeSlots];
                            ulonglong2 pair[kProbeSlots];
#pragma unroll
                            for (int t = 0; t < kProbeSlots; ++t) {
                                slot[t] = nullptr;
                                pair[t] = make_ulonglong2(0ull, 0ull);
                                int att = 0;
                                if (t < kIdsPerLane) {
                                    sv[t] = -1;
                                    if (v[t] >= 0 && (int64_t)v[t] < a.n) {
                                        ++n_scan;
                                        sv[t] = v[t];
                                    }
                                } else {
                                    att = carry_att;   // sv[t] still holds the carried id (or -1)
                                }
                                if (sv[t] >= 0) {
                                    slot[t] = (unsigned long long*)&ghash[((mix32((uint32_t)sv[t]) & ~1u) + 2u * (uint32_t)att) & a.gh_mask];
                                    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];"
                                                 : "=l"(pair[t].x), "=l"(pair[t].y)
                                                 : "l"(slot[t])
                                                 : "memory");
                                }
                            }
                            sc_cas = 0u;
#pragma unroll
                            for (int t = 0; t < kProbeSlots; ++t) {
                                scur[t] = ~0ull;   // "not settled by the pair": the full probe decides later
                                if (sv[t] >= 0) {
                                    const bool mine0 = (uint32_t)(pair[t].x >> 32) == epoch;
                                    const bool mine1 = (uint32_t)(pair[t].y >> 32) == epoch;
                                    if (mine0 && (uint32_t)pair[t].x == (uint32_t)sv[t]) {
                                        scur[t] = pair[t].x;                       // seen
                                    } else if (!mine0) {
                                        scur[t] = pair[t].x;                       // first slot is free: claim it
                                        sold[t] = atomicCAS(slot[t], scur[t], ((unsigned long long)epoch << 32) | (uint32_t)sv[t]);
                                        sc_cas |= 1u << t;
                                    } else if (mine1 && (uint32_t)pair[t].y == (uint32_t)sv[t]) {
                                        scur[t] = pair[t].y;                       // seen, in the second slot
                                    } else if (!mine1) {
                                        scur[t] = pair[t].y;                       // second slot is free: claim it
                                        sold[t] = atomicCAS(slot[t] + 1, scur[t], ((unsigned long long)epoch << 32) | (uint32_t)sv[t]);
                                        sc_cas |= 1u << t;
                                    }
                                }
                            }
                            sc_pending = true;
                            continue;
                        }
                        bool isnew[kIdsPerLane];
#pragma unroll
                        for (int t = 0; t < kIdsPerLane; ++t) {
                            isnew[t] = false;
                            if (v[t] >= 0 && (int64_t)v[t] < a.n) {
                                ++n_scan;
                                const uint32_t cslot = ((uint32_t)v[t] * 0x9E3779B1u >> 7) & vc_mask;
                                if (P.vc_bits > 0 && vcache[cslot] == (uint32_t)v[t]) continue;   // seen before
                                const int r =
                                    visited_insert(shash, P.hs_bits, ghash, a.gh_mask, epoch, v[t], n_spill);
                                isnew[t] = (r == 0);
                                if (r == 2) overflow = true;
                                else if (P.vc_bits > 0) vcache[cslot] = (uint32_t)v[t];
                            }
                        }
#pragma unroll
                        for (int t = 0; t < kIdsPerLane; ++t) {
                            const uint32_t m = __ballot_sync(0xffffffffu, isnew[t]);
                            if (isnew[t] && CORAL_CHECK(pend_n + __popc(m & lt_mask) < kPendCap, 5, pend_n, m))
                                pend[pend_n + __popc(m & lt_mask)] = v[t];
                            pend_n += __popc(m);
                        }
                        __syncwarp();
                        continue;
                    }
                    if (inflight > 0) {
                        // ---- distance: one chunk of the oldest batch in flight
                        const uint32_t b = done;
                        const int c = con_c, st = con_st;
                        const int cnt = (b & 1u) ? bcnt1 : bcnt0;
                        if (unit_gather) {
                            ldgsts_wait(inflight - 1);
                            __syncwarp();   // every lane's units have landed and are visible to the warp
                        } else {
                            mbar_wait(&bars[st], con_par, a.err_flag);
                        }
                        if (c == 0) acc = 0.f;
                        if (lane < cnt)
                            acc = accumulate_chunk<METRIC>(
                                acc,
                                reinterpret_cast<const float4*>(stage0 + (size_t)st * P.stage_bytes + (size_t)lane_row_off),
                                reinterpret_cast<const float4*>(sq + (size_t)c * chunk_floats),
                                c + 1 == n_chunks ? P.tail_vec : chunk_vec);
                        fence_async_smem();
                        __syncwarp();
                        --inflight;
                        if (++con_st == P.stages) {
                            con_st = 0;
                            con_par ^= 1u;
                        }
                        if (++con_c == n_chunks) {
                            con_c = 0;
                            // ---- filter and emit (src/search_gpu.cu:431-434)
                            const bool ok = lane < cnt && closer_than<METRIC>(worst, acc);
                            const uint32_t m = __ballot_sync(0xffffffffu, ok);
                            int base = 0;
                            if (lane == 0) {
                                n_dist += cnt;
                                if (m) base = atomicAdd(p_cand_count, __popc(m));
                            }
                            base = __shfl_sync(0xffffffffu, base, 0);
                            if (ok) {
                                const int pos = base + __popc(m & lt_mask);
                                if (pos < a.cand_cap)
                                    gcand[pos] = make_key<METRIC>(acc, bids[(b & 1u) * 32 + lane], 0u);
                            }
                            ++done;
                            __syncwarp();
                        }
                        continue;
                    }
                    if (!more && !has_carry && !sc_pending && pend_n == 0) break;
                }
            }
            if (CLUSTER) {
                __threadfence();   // candidates written by every CTA must be visible to the leader
                cluster_sync_all();
                if (!leader) continue;
            } else {
                __syncthreads();
            }

            // ------------------------------------------------------------ merge (leader CTA)
            int C = CLUSTER ? load_shared_int(&GC->cand_count) : S.cand_count;
            if (C > a.cand_cap) C = a.cand_cap;
            if (C == 0) {  // converged (src/search_gpu.cu:442)
                if (!CLUSTER) break;
                finished = true;
                continue;
            }
            int cnt = S.beam_cnt;
            const bool over = cnt + C > a.L;
            uint64_t bound = cnt >= a.L ? beam[a.L - 1] : kPadKey;
            int pos = 0;
            while (pos < C) {
                if (tid == 0) S.fill = 0;
                __syncthreads();
                int fill = 0;
                while (pos < C && fill + nthreads <= P.tile_max) {
                    // The keys of the next kMergeAhead passes are fetched together (one trip to L2
                    // for all of them); a pass that no longer fits the tile is fetched again later.
                    uint64_t ahead[kMergeAhead];
#pragma unroll
                    for (int j = 0; j < kMergeAhead; ++j) {
                        const int i = pos + j * nthreads + tid;
                        ahead[j] = i < C ? __ldcg(gcand + i) : kPadKey;
                    }
#pragma unroll
                    for (int j = 0; j < kMergeAhead; ++j) {
                        if (pos < C && fill + nthreads <= P.tile_max) {
                            int taken = 0;
                            const uint64_t key = ahead[j];
                            if (pos + tid < C && key < bound) {
                                const int slot = atomicAdd(&S.fill, 1);
                                if (CORAL_CHECK(slot < P.tile_max && key_id(key) >= 0 && (int64_t)key_id(key) < a.n, 6, slot, key))
                                    sortbuf[slot] = key;
                                taken = 1;
                            }
                            pos += nthreads;
                            // The tile's fill level must be the same number in every thread: it decides
                            // whether another pass runs.  Reading S.fill back after the barrier would
                            // race with the next pass's atomicAdd of faster threads; the barrier's own
                            // count cannot.
                            fill += __syncthreads_count(taken);
                        }
                    }
                }
                if (fill == 0) continue;
                int n2 = 32;
                while (n2 < fill) n2 <<= 1;
                for (int i = fill + tid; i < n2; i += nthreads) sortbuf[i] = kPadKey;
                __syncthreads();
                if (n2 == 32) {
                    // a tile of at most 32 keys (the usual case once the L-th key has tightened the
                    // filter): one warp sorts it in registers, no barrier per stage
                    if (warp == 0) {
                        uint64_t x = sortbuf[lane];
#pragma unroll
                        for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
                            for (int j = k >> 1; j > 0; j >>= 1) {
                                const uint64_t y = __shfl_xor_sync(0xffffffffu, x, j);
                                const bool keep_min = ((lane & j) == 0) == ((lane & k) == 0);
                                x = keep_min ? (x < y ? x : y) : (x < y ? y : x);
                            }
                        }
                        sortbuf[lane] = x;
                    }
                    __syncthreads();
                } else {
                    bitonic_sort(sortbuf, n2, tid, nthreads);
                }
                // merge by rank: beam[0..cnt) and sortbuf[0..fill), both ascending, keys distinct
                for (int i = tid; i < cnt; i += nthreads) {
                    const uint64_t x = beam[i];
                    const int p = i + lower_bound_u64(sortbuf, fill, x);
                    if (p < a.L && CORAL_CHECK(p >= 0 && p < P.LP, 7, p, i)) beam_alt[p] = x;
                }
                for (int j = tid; j < fill; j += nthreads) {
                    const uint64_t x = sortbuf[j];
                    const int p = j + upper_bound_u64(beam, cnt, x);
                    if (p < a.L && CORAL_CHECK(p >= 0 && p < P.LP, 8, p, j)) beam_alt[p] = x;
                }
                cnt = cnt + fill < a.L ? cnt + fill : a.L;
                for (int i = cnt + tid; i < P.LP; i += nthreads) beam_alt[i] = kPadKey;
                __syncthreads();
                uint64_t* t = beam;
                beam = beam_alt;
                beam_alt = t;
                if (cnt >= a.L) bound = beam[a.L - 1];
            }
            if (tid == 0) {
                S.hops += C;                          // src/search_gpu.cu:481,574
                if (C > S.max_cand) S.max_cand = C;
                S.beam_cnt = cnt;
                if (over) S.worst = dist_of<METRIC>((uint32_t)(beam[a.L - 1] >> 32));  // :573
                if (S.rounds >= a.max_rounds) S.status = 3;
            }
            // the sort tiles were written to the staging memory through the generic proxy; the
            // next round's bulk copies write the same bytes through the async proxy
            fence_async_smem();
            __syncthreads();
            if (S.status == 3) {
                if (!CLUSTER) break;
                finished = true;
            }
        }

        // ---------------------------------------------------------------- tallies
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            n_scan += __shfl_down_sync(0xffffffffu, n_scan, off);
            n_spill += __shfl_down_sync(0xffffffffu, n_spill, off);
        }
        if (lane == 0) {
            atomicAdd(&S.n_scan, n_scan);
            atomicAdd(&S.n_spill, n_spill);
            atomicAdd(&S.n_exp, n_exp);
            atomicAdd(&S.n_dist, n_dist);
        }
        if (__any_sync(0xffffffffu, overflow) && lane == 0) atomicMax(&S.status, 2);
        __syncthreads();
        if (CLUSTER) {   // fold the other CTAs' tallies into the leader's
            if (leader && tid == 0) GC->abort = *(volatile int*)a.err_flag;
            if (!leader && tid == 0) {
                atomicAdd(&GC->n_scan, S.n_scan);
                atomicAdd(&GC->n_spill, S.n_spill);
                atomicAdd(&GC->n_exp, S.n_exp);
                atomicAdd(&GC->n_dist, S.n_dist);
                if (S.status == 2) atomicMax(&GC->status, 2);
            }
            __threadfence();
            cluster_sync_all();
            if (leader && tid == 0) {
                S.n_scan += load_shared_int(&GC->n_scan);
                S.n_spill += load_shared_int(&GC->n_spill);
                S.n_exp += load_shared_int(&GC->n_exp);
                S.n_dist += load_shared_int(&GC->n_dist);
                if (load_shared_int(&GC->status) == 2 && S.status < 2) S.status = 2;
                GC->n_scan = GC->n_spill = GC->n_exp = GC->n_dist = GC->status = 0;
            }
            if (tid == 0) S.abort = load_shared_int(&GC->abort);
            __syncthreads();
        }

        // ---------------------------------------------------------------- top-k out (src/search_gpu.cu:447-472, :716)
        if (leader && warp == 0) {
            const int cnt = S.beam_cnt;
            const float far0 = METRIC == 0 ? 3.402823466e+38f : -3.402823466e+38f;
            int written = 0;
            for (int base = 0; base < cnt && written < a.k; base += 32) {
                const int i = base + lane;
                bool ok = i < cnt;
                uint64_t key = ok ? beam[i] : kPadKey;
                const int id = key_id(key);
                if (ok && a.deleted) ok = ((a.deleted[id >> 5] >> (id & 31)) & 1u) == 0u;
                const uint32_t m = __ballot_sync(0xffffffffu, ok);
                const int p = written + __popc(m & lt_mask);
                if (ok && p < a.k) {
                    a.ids_out[(size_t)qid * a.k + p] = id;
                    if (a.dists_out) a.dists_out[(size_t)qid * a.k + p] = dist_of<METRIC>((uint32_t)(key >> 32));
                }
                written += __popc(m);
            }
            for (int p = written + lane; p < a.k; p += 32) {
                a.ids_out[(size_t)qid * a.k + p] = -1;
                if (a.dists_out) a.dists_out[(size_t)qid * a.k + p] = far0;
            }
            if (lane == 0) {
                int st = S.status;
                if (st == 0 && cnt < a.L) st = 1;
                if (a.worst_status && st != 0) atomicMax(a.worst_status, st);
                if (a.stats_out) {
                    int32_t* o = a.stats_out + (size_t)qid * 8;
                    o[0] = st;
                    o[1] = S.n_dist;
                    o[2] = S.n_exp;
                    o[3] = S.rounds;
                    o[4] = S.hops;
                    o[5] = S.n_scan;
                    o[6] = S.max_cand;
                    o[7] = S.n_spill;
                }
                atomicAdd(a.hops_total, (unsigned long long)S.hops);
            }
        }
    }
}

}  // namespace

int* granted_slot(int* table, int device, int metric, bool cluster) {
    if (device < 0 || device >= kMaxGrantDevices || metric < 0 || metric > 1) return nullptr;   // uncached: always set
    return table + (device * 2 + metric) * 2 + (cluster ? 1 : 0);
}

namespace {
template <int METRIC, bool CLUSTER>
const void* kernel_ptr() {
    return (const void*)beam_search_kernel<METRIC, CLUSTER>;
}
const void* kernel_for(int metric, bool cluster) {
    if (metric == 0) return cluster ? kernel_ptr<0, true>() : kernel_ptr<0, false>();
    return cluster ? kernel_ptr<1, true>() : kernel_ptr<1, false>();
}
// The opt-in shared-memory limit of each instantiation only ever grows, so plans made for other
// beam capacities stay launchable.
// The attribute belongs to the current device's context, so the cache is kept per device; a
// mutex guards it because handles on different devices may be driven from different threads.
bool grant_smem(int metric, bool cluster, int bytes) {
    static std::mutex mu;
    static int granted[kMaxGrantDevices][2][2] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    std::lock_guard<std::mutex> lock(mu);
    int* slot = granted_slot(&granted[0][0][0], dev, metric, cluster);
    if (slot && bytes <= *slot) return true;
    if (cudaFuncSetAttribute(kernel_for(metric, cluster), cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) !=
        cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (slot) *slot = bytes;
    return true;
}
}  // namespace

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tensor_map_encoder() {
    static std::mutex mu;
    static EncodeTiledFn enc = nullptr;
    static bool asked = false;
    std::lock_guard<std::mutex> lock(mu);
    if (!asked) {
        asked = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            enc = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return enc;
}
}  // namespace

bool row_gather_available() { return tensor_map_encoder() != nullptr; }

bool make_row_gather_map(CUtensorMap* map, const float* vecs, int64_t n, int dim, int box_floats) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return false;
    if (!vecs || n <= 0 || dim <= 0 || dim % 4 != 0 || box_floats <= 0 || box_floats > 256 || box_floats % 4 != 0 ||
        ((uintptr_t)vecs & 15u) != 0)
        return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)dim, (cuuint64_t)n};
    const cuuint64_t gstride[1] = {(cuuint64_t)dim * 4};
    const cuuint32_t box[2] = {(cuuint32_t)box_floats, 1};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(vecs), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t launch_beam_search(const SearchArgs& a, int metric, int grid, cudaStream_t stream, int cluster_size,
                               const CUtensorMap* row_map) {
    const int threads = a.plan.warps * 32;
    if (a.plan.gather == 2 && !row_map) return cudaErrorInvalidValue;
    alignas(64) CUtensorMap map;
    if (row_map) map = *row_map;
    else memset(&map, 0, sizeof map);   // never dereferenced in the other gather modes
    if (cluster_size <= 1) {
        if (metric == 0)
            beam_search_kernel<0, false><<<grid, threads, a.plan.smem_bytes, stream>>>(a, map);
        else
            beam_search_kernel<1, false><<<grid, threads, a.plan.smem_bytes, stream>>>(a, map);
        return cudaGetLastError();
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = (size_t)a.plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (metric == 0) return cudaLaunchKernelEx(&cfg, beam_search_kernel<0, true>, a, map);
    return cudaLaunchKernelEx(&cfg, beam_search_kernel<1, true>, a, map);
}

int beam_search_occupancy(const SearchPlan& p, int metric) {
    if (!grant_smem(metric, false, p.smem_bytes)) return 0;
    int nb = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel_for(metric, false), p.warps * 32, p.smem_bytes) !=
        cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return nb;
}

int beam_search_max_clusters(const SearchPlan& p, int metric, int cluster_size) {
    if (cluster_size < 2 || !grant_smem(metric, true, p.smem_bytes)) return 0;
    const void* fn = kernel_for(metric, true);
    if (cluster_size > 8 &&
        cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster_size, 1, 1);
    cfg.blockDim = dim3((unsigned)(p.warps * 32), 1, 1);
    cfg.dynamicSmemBytes = (size_t)p.smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, fn, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

}  // namespace coral
