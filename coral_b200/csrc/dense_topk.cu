// Dense query-block x row-block scores on the tcgen05 tensor cores, fused with a per-query top-k'
// selection, plus the exact re-rank that makes the result exact nearest neighbours.
//
// Used for the contractions around the search path: the exact k_b-nearest base points of the
// training queries that the graph build starts from (the reference calls Faiss' flat GPU index,
// src/knn.cu:174-193, include/myfaiss.h:17-29), exact ground truth (tests/comp_gt.cpp:121-155), and
// the query x entry-point-neighbourhood scores that order a batch for locality.
//
// Scan kernel (dense_scan_kernel), one CTA of 6 warps per (query tile, column split):
//   warp 0    producer: TMA (cp.async.bulk.tensor.3d, 128-byte swizzle) brings one k-block (32
//             floats of every row) of the query tile and of the base tile into a 2-stage ring;
//   warp 1    one elected lane issues tcgen05.mma (kind::tf32, M = 128, N = 256, K = 8): per
//             k-block 4 k-slices x `passes` operand pairs accumulate into one of two 256-column
//             TMEM buffers; tcgen05.commit frees ring stages and publishes finished tiles;
//   warps 2-5 epilogue: thread t owns TMEM lane t = one query row, reads its 256 scores with
//             tcgen05.ld, and keeps what beats the row's running threshold.
// fp32 accuracy from tf32 tensor cores: every operand is split once into a tf32-exact high part and
// the remainder (hi = x with the 13 low mantissa bits cleared, lo = x - hi), and the product is
// formed as hi*hi + hi*lo + lo*hi in the fp32 accumulator (the dropped lo*lo term is 2^-22
// relative).  The scores only SELECT: the k' best per query are then re-ranked with the exact fp32
// distance in the reference's sequential order, and a query is "certified" when its exact k-th
// distance beats the best score an unselected row could have.
//
// Selection: every (query row, split) owns a buffer of kDenseRowCap keys in global memory.  A score
// that beats the row's threshold (the k'-th best so far) is appended; when fewer than one tile's
// worth of free slots is left the warp sorts that row's buffer in shared memory, keeps the k' best
// and tightens the threshold.  After the first few tiles almost nothing passes (about k' ln(N/k')
// appends per row in total).
//
// Every wait is bounded (clock limit -> error flag, the CTA drains and frees its TMEM).  Every CTA
// loads its own tiles; no clusters.
#include "dense_topk.cuh"

#include <cuda.h>

#include <mutex>

namespace coral {

namespace {

constexpr int kStages = 2;
constexpr int kTileABytes = kDenseTileM * kDenseTileK * 4;     // 16 KB
constexpr int kTileBBytes = kDenseTileN * kDenseTileK * 4;     // 32 KB
constexpr int kStageBytes = 2 * kTileABytes + 2 * kTileBBytes; // hi and lo of both operands: 96 KB
constexpr int kSortBytesPerWarp = kDenseRowCap * 8;            // 4 KB
constexpr int kOffSort = kStages * kStageBytes;
constexpr int kOffNorm = kOffSort + 4 * kSortBytesPerWarp;
constexpr int kOffBars = kOffNorm + 4 * kDenseTileN * 4;     // one copy of the tile's norms per epilogue warp
constexpr int kSmemBytes = kOffBars + 256 + 1024;              // + slack to align the base to 1024
constexpr int kThreads = 192;
constexpr long long kWaitClocks = 4000000000ll;                // ~2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)
        : "memory");
    return ok;
}
// Bounded wait.  Gives up when the clock limit runs out or another role of this CTA already gave
// up (*abort_flag, shared memory); on its own time-out it raises both flags.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spins = 1;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 15u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitClocks) {
                *abort_flag = 1;
                atomicExch(err, 1);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, stored with the
// 128-byte swizzle in groups of 8 rows (1024 bytes): start address, leading offset (unused for
// swizzled K-major layouts), stride between row groups, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulator, tf32 x tf32, both operands K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kDenseTileN >> 3) << 17) |
                                ((uint32_t)(kDenseTileM >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Larger score = better.  Keys sort ascending = best first: ~ord(score) in the high word, the
// column (global row id) in the low word, so equal scores order by id.
__device__ __forceinline__ uint32_t ord_f32(float d) {
    const uint32_t u = __float_as_uint(d);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unord_f32(uint32_t o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ uint64_t score_key(float s, uint32_t col) { return ((uint64_t)(~ord_f32(s)) << 32) | col; }
__device__ __forceinline__ float key_score(uint64_t k) { return unord_f32(~(uint32_t)(k >> 32)); }

// One warp sorts n <= kDenseRowCap keys of `row_keys` (global) ascending in its shared buffer,
// writes the first min(n, keep) back and returns how many it kept; *thr_out = score of the last kept
// key when `keep` keys were kept, else unchanged.
__device__ int warp_compact(uint64_t* row_keys, int n, int keep, uint64_t* sbuf, int lane, float* thr_out) {
    int n2 = 32;
    while (n2 < n) n2 <<= 1;
    for (int i = lane; i < n2; i += 32) sbuf[i] = i < n ? row_keys[i] : ~0ull;
    __syncwarp();
    for (int k = 2; k <= n2; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = lane; i < n2; i += 32) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const uint64_t a = sbuf[i], b = sbuf[ixj];
                    if ((a > b) == ((i & k) == 0)) {
                        sbuf[i] = b;
                        sbuf[ixj] = a;
                    }
                }
            }
            __syncwarp();
        }
    const int kept = n < keep ? n : keep;
    for (int i = lane; i < kept; i += 32) row_keys[i] = sbuf[i];
    if (kept == keep) *thr_out = key_score(sbuf[keep - 1]);
    __syncwarp();
    return kept;
}

struct ScanArgs {
    int Q, n_rows, dim, k_blocks, passes, metric, keep, n_split, tiles_total;
    uint32_t col_base;          // global id of the chunk's first row
    const float* b_norm;        // [n_rows] (L2)
    uint64_t* keys;
    int32_t* cnt;
    float* thr;
    int* err;
};

__global__ void __launch_bounds__(kThreads, 1)
dense_scan_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const ScanArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBars);
    uint64_t* full = bars;                 // [kStages] TMA bytes landed
    uint64_t* empty = bars + kStages;      // [kStages] the MMAs that read the stage have completed
    uint64_t* tfull = bars + 2 * kStages;  // [2] accumulator buffer complete
    uint64_t* tempty = tfull + 2;          // [2] accumulator buffer drained by the epilogue
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, qtile = blockIdx.y;
    const int t0 = (int)((long long)a.tiles_total * split / a.n_split);
    const int t1 = (int)((long long)a.tiles_total * (split + 1) / a.n_split);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull[b], 1);
            mbar_init(&tempty[b], 4);      // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {   // the whole tensor memory of the SM: two 256-column accumulator buffers
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t stage_bytes = (uint32_t)(a.passes == 1 ? kTileABytes + kTileBBytes : kStageBytes);

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0;
            uint32_t par = 0;
            bool ok = true;
            for (int t = t0; t < t1 && ok; ++t) {
                for (int kb = 0; kb < a.k_blocks; ++kb) {
                    if (!mbar_wait(&empty[s], par ^ 1u, abort_flag, a.err)) {
                        ok = false;
                        break;
                    }
                    unsigned char* st = smem + s * kStageBytes;
                    mbar_expect_tx(&full[s], stage_bytes);
                    tma_load_3d(st, &map_a, kb * kDenseTileK, qtile * kDenseTileM, 0, &full[s]);
                    tma_load_3d(st + 2 * kTileABytes, &map_b, kb * kDenseTileK, t * kDenseTileN, 0, &full[s]);
                    if (a.passes != 1) {
                        tma_load_3d(st + kTileABytes, &map_a, kb * kDenseTileK, qtile * kDenseTileM, 1, &full[s]);
                        tma_load_3d(st + 2 * kTileABytes + kTileBBytes, &map_b, kb * kDenseTileK, t * kDenseTileN, 1, &full[s]);
                    }
                    if (++s == kStages) {
                        s = 0;
                        par ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int s = 0;
            uint32_t par = 0;
            uint32_t tpar[2] = {0u, 0u};
            bool ok = true;
            for (int t = t0; t < t1 && ok; ++t) {
                const int b = (t - t0) & 1;
                if (!mbar_wait(&tempty[b], tpar[b] ^ 1u, abort_flag, a.err)) break;
                tpar[b] ^= 1u;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * kDenseTileN);
                for (int kb = 0; kb < a.k_blocks; ++kb) {
                    if (!mbar_wait(&full[s], par, abort_flag, a.err)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * kStageBytes);
                    const uint32_t a_hi = sa, a_lo = sa + kTileABytes;
                    const uint32_t b_hi = sa + 2 * kTileABytes, b_lo = b_hi + kTileBBytes;
#pragma unroll
                    for (int j = 0; j < kDenseTileK / 8; ++j) {       // K = 8 tf32 = 32 bytes per instruction
                        const uint32_t off = (uint32_t)j * 32u;
                        umma_tf32(tmem_d, smem_desc_sw128(a_hi + off), smem_desc_sw128(b_hi + off), (kb | j) != 0 ? 1u : 0u);
                        if (a.passes != 1) {
                            umma_tf32(tmem_d, smem_desc_sw128(a_hi + off), smem_desc_sw128(b_lo + off), 1u);
                            umma_tf32(tmem_d, smem_desc_sw128(a_lo + off), smem_desc_sw128(b_hi + off), 1u);
                        }
                    }
                    umma_commit(&empty[s]);      // the stage is free once these MMAs have read it
                    if (++s == kStages) {
                        s = 0;
                        par ^= 1u;
                    }
                }
                if (ok) umma_commit(&tfull[b]);  // the accumulator is complete once they have all finished
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int lane_group = warp & 3;                 // the 32 TMEM lanes this warp may read
        const int row = qtile * kDenseTileM + lane_group * 32 + lane;
        const bool row_ok = row < a.Q;
        const size_t slot = (size_t)(row_ok ? row : 0) * a.n_split + split;
        uint64_t* my_keys = a.keys + slot * kDenseRowCap;
        uint64_t* sbuf = reinterpret_cast<uint64_t*>(smem + kOffSort) + (size_t)(warp - 2) * kDenseRowCap;
        int cnt = row_ok ? a.cnt[slot] : 0;
        float thr = row_ok ? a.thr[slot] : 3.402823466e+38f;
        uint32_t tpar[2] = {0u, 0u};
        // squared norms of the current tile's rows, one private copy per warp (no CTA-wide barrier
        // in the epilogue: a warp that gives up on a wait must not leave the others waiting for it)
        float* snorm = reinterpret_cast<float*>(smem + kOffNorm) + (size_t)(warp - 2) * kDenseTileN;
        bool ok = true;
        // keep == 8 (the scheduling keys: few columns, a handful of survivors): the thread also tracks
        // the eight best scores of its row in registers and filters against the eighth, so the
        // threshold tightens with every accepted column instead of once per compaction -- about
        // 8 ln(columns / 8) keys reach the buffer and no compaction runs before the last one.  The
        // list starts as eight copies of the row's threshold, a lower bound of the keys already kept,
        // so the eighth entry never exceeds the true eighth best.
        const bool track8 = a.keep == 8;
        float top[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) top[i] = thr;
        for (int t = t0; t < t1 && ok; ++t) {
            const int b = (t - t0) & 1;
            const int col0 = t * kDenseTileN;
            // room for a whole tile of passing scores in every row of the warp
            for (;;) {
                const uint32_t need = __ballot_sync(0xffffffffu, cnt > kDenseRowCap - kDenseTileN);
                if (!need) break;
                const int src = __ffs(need) - 1;
                const int n = __shfl_sync(0xffffffffu, cnt, src);
                const unsigned long long p = __shfl_sync(0xffffffffu, (unsigned long long)my_keys, src);
                float new_thr = thr;
                const int kept = warp_compact(reinterpret_cast<uint64_t*>(p), n, a.keep, sbuf, lane, &new_thr);
                if (lane == src) {
                    cnt = kept;
                    thr = new_thr;
#pragma unroll
                    for (int i = 0; i < 8; ++i) top[i] = fmaxf(top[i], new_thr);
                }
            }
            if (a.metric == 0) {
                for (int i = lane; i < kDenseTileN; i += 32) snorm[i] = col0 + i < a.n_rows ? a.b_norm[col0 + i] : 0.f;
            }
            __syncwarp();
            if (!mbar_wait(&tfull[b], tpar[b], abort_flag, a.err)) {
                ok = false;
                break;
            }
            tpar[b] ^= 1u;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(b * kDenseTileN);
            const int valid = a.n_rows - col0;   // columns of this tile that exist
#pragma unroll 1
            for (int c = 0; c < kDenseTileN; c += 32) {
                uint32_t r[32];
                __syncwarp();
                tmem_ld32(taddr + (uint32_t)c, r);
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float s = __uint_as_float(r[j]);
                        if (a.metric == 0) s = fmaf(2.f, s, -snorm[c + j]);
                        if (s >= thr && c + j < valid) {
                            my_keys[cnt++] = score_key(s, a.col_base + (uint32_t)(col0 + c + j));
                            if (track8) {   // insert s into the descending list, drop its last entry
                                float v = s;
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    const float hi = fmaxf(top[i], v);
                                    v = fminf(top[i], v);
                                    top[i] = hi;
                                }
                                thr = top[7];
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[b]);
        }
        // leave at most `keep` keys per row behind and publish the state for the next chunk
        for (;;) {
            const uint32_t need = __ballot_sync(0xffffffffu, cnt > a.keep);
            if (!need) break;
            const int src = __ffs(need) - 1;
            const int n = __shfl_sync(0xffffffffu, cnt, src);
            const unsigned long long p = __shfl_sync(0xffffffffu, (unsigned long long)my_keys, src);
            float new_thr = thr;
            const int kept = warp_compact(reinterpret_cast<uint64_t*>(p), n, a.keep, sbuf, lane, &new_thr);
            if (lane == src) {
                cnt = kept;
                thr = new_thr;
            }
        }
        if (row_ok) {
            a.cnt[slot] = cnt;
            a.thr[slot] = thr;
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out: give copies and MMAs still in flight time to land before the shared
        // memory and the tensor memory go back (bounded: a fixed number of clocks).
        const long long t_end = clock64() + 20000000ll;
        while (clock64() < t_end) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// hi = x with the 13 low mantissa bits cleared (exactly representable in tf32), lo = x - hi.
__global__ void split_tf32_kernel(const float* __restrict__ x, long long n, float* __restrict__ hi, float* __restrict__ lo) {
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < n;
         i += (long long)gridDim.x * blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
        l.x = v.x - h.x;
        l.y = v.y - h.y;
        l.z = v.z - h.z;
        l.w = v.w - h.w;
        *reinterpret_cast<float4*>(hi + i) = h;
        *reinterpret_cast<float4*>(lo + i) = l;
    }
}

__global__ void row_norm_kernel(const float* __restrict__ x, int n_rows, int dim, float* __restrict__ out) {
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < n_rows; r += warps) {
        float s = 0.f;
        for (int d = lane; d < dim; d += 32) {
            const float v = x[(size_t)r * dim + d];
            s = fmaf(v, v, s);
        }
        for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
        if (lane == 0) out[r] = s;
    }
}

__global__ void reset_state_kernel(int32_t* cnt, float* thr, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        cnt[i] = 0;
        thr[i] = -3.402823466e+38f;
    }
}

// CTA-wide bitonic sort of n (power of two) keys in shared memory, ascending.
__device__ void block_sort(uint64_t* s, int n, int tid, int nthreads) {
    for (int k = 2; k <= n; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < n; i += nthreads) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const uint64_t a = s[i], b = s[ixj];
                    if ((a > b) == ((i & k) == 0)) {
                        s[i] = b;
                        s[ixj] = a;
                    }
                }
            }
            __syncthreads();
        }
}

// One CTA per query: merge the splits' keys, keep the `keep` best, re-rank them exactly.
// Exact distance = one sequential fp32 fused chain over d = 0..dim-1, the order of the
// reference's l2_distance / ip_distance (include/utils.cuh:254-275, :307-323).
__global__ void __launch_bounds__(128)
dense_finish_kernel(const float* __restrict__ queries, int Q, const float* __restrict__ vecs, int dim, int metric,
                    const uint64_t* __restrict__ keys, const int32_t* __restrict__ cnt, int n_split, int n2, int keep,
                    int k, float rel_eps, int32_t* __restrict__ ids_out, float* __restrict__ dists_out,
                    int32_t* __restrict__ certified_out, int* err) {
    extern __shared__ unsigned char fsm[];
    uint64_t* sk = reinterpret_cast<uint64_t*>(fsm);             // [n2]
    float* sq = reinterpret_cast<float*>(sk + n2);               // [dim]
    __shared__ uint64_t exact[kDenseMaxKeep];
    __shared__ int total;
    __shared__ float qnorm;
    const int q = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) total = 0;
    for (int d = tid; d < dim; d += 128) sq[d] = queries[(size_t)q * dim + d];
    for (int i = tid; i < n2; i += 128) sk[i] = ~0ull;
    __syncthreads();
    for (int s = 0; s < n_split; ++s) {
        const size_t slot = (size_t)q * n_split + s;
        const int n = cnt[slot];
        __shared__ int base;
        if (tid == 0) {
            base = total;
            total += n;
        }
        __syncthreads();
        for (int i = tid; i < n; i += 128)
            if (base + i < n2) sk[base + i] = keys[slot * kDenseRowCap + i];
        __syncthreads();
    }
    block_sort(sk, n2, tid, 128);
    const int have = total < keep ? total : keep;
    // best score any row outside the selection can have: the keep-th best selected score (nothing
    // was ever dropped when fewer than `keep` keys exist)
    const float outside = total >= keep ? key_score(sk[keep - 1]) : -3.402823466e+38f;
    if (tid == 0 && metric == 0) {
        float s = 0.f;
        for (int d = 0; d < dim; ++d) s = fmaf(sq[d], sq[d], s);
        qnorm = s;
    }
    for (int i = tid; i < kDenseMaxKeep; i += 128) exact[i] = ~0ull;
    __syncthreads();
    for (int i = tid; i < have; i += 128) {
        const uint32_t id = (uint32_t)sk[i];
        const float4* row = reinterpret_cast<const float4*>(vecs + (size_t)id * dim);
        const float4* qq = reinterpret_cast<const float4*>(sq);
        float acc = 0.f;
        for (int v = 0; v < dim / 4; ++v) {
            const float4 x = __ldg(row + v);
            const float4 y = qq[v];
            if (metric == 0) {
                float t;
                t = x.x - y.x; acc = fmaf(t, t, acc);
                t = x.y - y.y; acc = fmaf(t, t, acc);
                t = x.z - y.z; acc = fmaf(t, t, acc);
                t = x.w - y.w; acc = fmaf(t, t, acc);
            } else {
                acc = fmaf(x.x, y.x, acc);
                acc = fmaf(x.y, y.y, acc);
                acc = fmaf(x.z, y.z, acc);
                acc = fmaf(x.w, y.w, acc);
            }
        }
        // closest first: L2 ascending distance, IP descending product
        const uint32_t o = metric == 0 ? ord_f32(acc) : ~ord_f32(acc);
        exact[i] = ((uint64_t)o << 32) | id;
    }
    __syncthreads();
    block_sort(exact, kDenseMaxKeep, tid, 128);
    for (int i = tid; i < k; i += 128) {
        const uint64_t key = exact[i];
        if (key == ~0ull) {
            ids_out[(size_t)q * k + i] = -1;
            if (dists_out) dists_out[(size_t)q * k + i] = metric == 0 ? 3.402823466e+38f : -3.402823466e+38f;
        } else {
            const uint32_t o = (uint32_t)(key >> 32);
            ids_out[(size_t)q * k + i] = (int32_t)(uint32_t)key;
            if (dists_out) dists_out[(size_t)q * k + i] = metric == 0 ? unord_f32(o) : unord_f32(~o);
        }
    }
    if (tid == 0) {
        int ok = 1;
        if (total >= keep && have >= k) {
            const uint32_t o = (uint32_t)(exact[k - 1] >> 32);
            const float dk = metric == 0 ? unord_f32(o) : unord_f32(~o);
            // the exact k-th distance on the scale of the approximate scores (L2: 2 q.b - |b|^2 = |q|^2 - dist)
            const float s_exact = metric == 0 ? qnorm - dk : dk;
            const float scale = fabsf(s_exact) + fabsf(outside) + (metric == 0 ? qnorm : 0.f);
            ok = s_exact > outside + rel_eps * scale ? 1 : 0;
        }
        if (certified_out) certified_out[q] = ok;
        if (!ok) atomicAdd(err + 1, 1);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::mutex mu;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) != cudaSuccess ||
            res != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [2][rows_alloc][dim] split array seen as a 3-D tensor (k, row, part); loads of rows >= rows and
// of k >= dim read zeros.
bool make_map(CUtensorMap* map, const float* base, int rows, size_t rows_alloc, int dim, int box_rows) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t gdim[3] = {(cuuint64_t)dim, (cuuint64_t)rows, 2};
    const cuuint64_t gstride[2] = {(cuuint64_t)dim * 4, (cuuint64_t)rows_alloc * dim * 4};
    const cuuint32_t box[3] = {(cuuint32_t)kDenseTileK, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

size_t dense_workspace_bytes(int q_cap, int b_cap, int dim, int n_split) {
    size_t b = 0;
    b += align256((size_t)2 * q_cap * dim * 4);
    b += align256((size_t)2 * b_cap * dim * 4);
    b += align256((size_t)b_cap * 4);
    b += align256((size_t)q_cap * n_split * kDenseRowCap * 8);
    b += align256((size_t)q_cap * n_split * 4) * 2;
    b += 256;
    return b;
}

void dense_workspace_carve(void* base, int q_cap, int b_cap, int dim, int n_split, DenseWorkspace& w) {
    unsigned char* p = static_cast<unsigned char*>(base);
    w.a_split = reinterpret_cast<float*>(p);   p += align256((size_t)2 * q_cap * dim * 4);
    w.b_split = reinterpret_cast<float*>(p);   p += align256((size_t)2 * b_cap * dim * 4);
    w.b_norm = reinterpret_cast<float*>(p);    p += align256((size_t)b_cap * 4);
    w.keys = reinterpret_cast<uint64_t*>(p);   p += align256((size_t)q_cap * n_split * kDenseRowCap * 8);
    w.cnt = reinterpret_cast<int32_t*>(p);     p += align256((size_t)q_cap * n_split * 4);
    w.thr = reinterpret_cast<float*>(p);       p += align256((size_t)q_cap * n_split * 4);
    w.err = reinterpret_cast<int*>(p);
    w.q_cap = q_cap;
    w.b_cap = b_cap;
    w.n_split = n_split;
}

cudaError_t dense_begin(const DenseWorkspace& w, const float* d_queries, int Q, int dim, cudaStream_t stream,
                        int64_t* launches) {
    if (Q > w.q_cap) return cudaErrorInvalidValue;
    const long long n = (long long)Q * dim;
    const int blocks = (int)((n / 4 + 255) / 256 < 4096 ? (n / 4 + 255) / 256 : 4096);
    split_tf32_kernel<<<blocks, 256, 0, stream>>>(d_queries, n, w.a_split, w.a_split + (size_t)w.q_cap * dim);
    reset_state_kernel<<<256, 256, 0, stream>>>(w.cnt, w.thr, w.q_cap * w.n_split);
    cudaError_t e = cudaMemsetAsync(w.err, 0, 4 * sizeof(int), stream);
    if (launches) *launches += 2;
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t dense_scan_chunk(const DenseWorkspace& w, const float*, int Q, const float* d_vecs, int64_t row0, int n_rows,
                             int dim, int metric, int passes, int keep, int sm_count, cudaStream_t stream,
                             int64_t* launches) {
    if (Q > w.q_cap || n_rows > w.b_cap || keep > kDenseMaxKeep || keep < 1) return cudaErrorInvalidValue;
    static std::mutex mu;
    static bool granted[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !granted[dev]) {
            cudaError_t e = cudaFuncSetAttribute(dense_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) granted[dev] = true;
        }
    }
    const long long n = (long long)n_rows * dim;
    const int blocks = (int)((n / 4 + 255) / 256 < 8192 ? (n / 4 + 255) / 256 : 8192);
    split_tf32_kernel<<<blocks, 256, 0, stream>>>(d_vecs, n, w.b_split, w.b_split + (size_t)w.b_cap * dim);
    if (metric == 0) row_norm_kernel<<<sm_count * 8, 256, 0, stream>>>(d_vecs, n_rows, dim, w.b_norm);
    alignas(64) CUtensorMap map_a, map_b;
    if (!make_map(&map_a, w.a_split, Q, (size_t)w.q_cap, dim, kDenseTileM) ||
        !make_map(&map_b, w.b_split, n_rows, (size_t)w.b_cap, dim, kDenseTileN))
        return cudaErrorInvalidValue;
    ScanArgs a;
    a.Q = Q;
    a.n_rows = n_rows;
    a.dim = dim;
    a.k_blocks = (dim + kDenseTileK - 1) / kDenseTileK;
    a.passes = passes == 1 ? 1 : 3;
    a.metric = metric;
    a.keep = keep;
    a.n_split = w.n_split;
    a.tiles_total = (n_rows + kDenseTileN - 1) / kDenseTileN;
    a.col_base = (uint32_t)row0;
    a.b_norm = w.b_norm;
    a.keys = w.keys;
    a.cnt = w.cnt;
    a.thr = w.thr;
    a.err = w.err;
    dim3 grid((unsigned)w.n_split, (unsigned)((Q + kDenseTileM - 1) / kDenseTileM), 1);
    dense_scan_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, a);
    if (launches) *launches += metric == 0 ? 3 : 2;
    return cudaGetLastError();
}

cudaError_t dense_finish(const DenseWorkspace& w, const float* d_queries, int Q, const float* d_vecs, int dim, int metric,
                         int passes, int keep, int k, int32_t* d_ids_out, float* d_dists_out, int32_t* d_certified_out,
                         cudaStream_t stream, int64_t* launches) {
    if (k > keep || keep > kDenseMaxKeep || dim % 4 != 0) return cudaErrorInvalidValue;
    int n2 = 32;
    while (n2 < w.n_split * keep) n2 <<= 1;
    const size_t smem = (size_t)n2 * 8 + (size_t)dim * 4;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(dense_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    // relative slack between an approximate score and its exact value
    const float rel_eps = passes == 1 ? 2e-3f : 2e-5f;   // one truncated tf32 pass: 2^-10 per operand
    dense_finish_kernel<<<Q, 128, smem, stream>>>(d_queries, Q, d_vecs, dim, metric, w.keys, w.cnt, w.n_split, n2, keep, k,
                                                  rel_eps, d_ids_out, d_dists_out, d_certified_out, w.err);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

}  // namespace coral
