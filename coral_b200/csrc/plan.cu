// Shared-memory planning of the beam-search kernel (see plan.cuh).
#include "plan.cuh"

namespace coral {

namespace {
int next_pow2(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}
int align_up(int x, int a) { return (x + a - 1) / a * a; }
int imin(int a, int b) { return a < b ? a : b; }
int imax(int a, int b) { return a > b ? a : b; }
}  // namespace

// With warps = 0 the warp count per CTA is chosen to maximise resident warps per SM
// (CTAs per SM x warps), preferring more CTAs on a tie: on 10M x 512 the achieved bandwidth
// followed that product (16 warps/SM 0.83, 18 0.87, 20 0.90-0.94 of the measured peak).
bool make_plan(int dim, int smem_optin, const PlanOptions& o, int L, SearchPlan& p, const char** why) {
    if (o.warps > 0 || o.ctas_per_sm > 0)
        return make_plan_warps(dim, smem_optin, o, L, o.warps > 0 ? o.warps : 4, p, why);
    bool found = false;
    const int candidates[4] = {3, 4, 5, 6};
    for (int w : candidates) {
        SearchPlan q;
        const char* dummy = nullptr;
        if (!make_plan_warps(dim, smem_optin, o, L, w, q, &dummy)) continue;
        const int total = q.ctas_per_sm * q.warps, best = p.ctas_per_sm * p.warps;
        if (!found || total > best || (total == best && q.ctas_per_sm > p.ctas_per_sm)) p = q;
        found = true;
    }
    if (!found) return make_plan_warps(dim, smem_optin, o, L, 4, p, why);
    // Every bulk copy costs its warp about 54 cycles to issue whatever its size, so rows that do
    // not split into 256-byte chunks (dim 200: five chunks of 160 bytes) are better moved in chunks
    // of up to 512 bytes -- as long as five CTAs still fit an SM (measured on 1M x 200, L = 64:
    // 1.85M against 1.56M queries/s with 400-byte chunks; at L = 512, where only four CTAs fit,
    // 160-byte chunks stay ahead).
    if (o.chunk_bytes <= 0 && p.chunk_bytes < 256) {
        SearchPlan best{};
        bool have = false;
        for (int w : candidates) {
            SearchPlan q;
            const char* dummy = nullptr;
            if (!make_plan_warps(dim, smem_optin, o, L, w, q, &dummy, 512) || q.chunk_bytes <= p.chunk_bytes) continue;
            const int total = q.ctas_per_sm * q.warps, cur = best.ctas_per_sm * best.warps;
            if (!have || total > cur || (total == cur && q.ctas_per_sm > best.ctas_per_sm)) best = q;
            have = true;
        }
        if (have && best.ctas_per_sm >= 5) p = best;
    }
    return true;
}

bool make_plan_warps(int dim, int smem_optin, const PlanOptions& o, int L, int warps, SearchPlan& p,
                     const char** why, int chunk_target) {
    const int row_bytes = dim * 4;
    p = SearchPlan{};
    p.warps = imin(imax(warps, 1), 16);
    const bool auto_ctas = o.ctas_per_sm <= 0;
    p.ctas_per_sm = auto_ctas ? 1 : imin(o.ctas_per_sm, 8);
    int target = imax(16, chunk_target > 0 ? chunk_target : (o.chunk_bytes > 0 ? o.chunk_bytes : 256));
    int nc = (row_bytes + target - 1) / target;
    while (nc <= row_bytes / 16 && !(row_bytes % nc == 0 && (row_bytes / nc) % 16 == 0)) ++nc;
    if (nc > row_bytes / 16) {
        *why = "row size has no 16-byte chunking";
        return false;
    }
    p.n_chunks = nc;
    p.chunk_bytes = row_bytes / nc;
    p.row_stride = p.chunk_bytes + (((p.chunk_bytes / 16) % 2 == 0) ? 16 : 0);
    p.group_stride = 4 * p.row_stride;
    p.tail_vec = p.chunk_bytes / 16;
    p.stage_bytes = 32 * p.row_stride;
    if (o.gather == 2) {
        // One tensor copy lands the chunks of four rows back to back, and its destination has to be
        // 128-byte aligned, so the padding that keeps lane-per-row reads off the same banks goes
        // into the chunk width itself: an odd number of 16-byte units (rows r and r + 1 of a group
        // then start one bank group apart; lanes four apart still share one, a 2-way conflict).
        // The chunks need not tile the row: the last one runs past its end and reads zeros there.
        int units = imax(1, target / 16);
        if (units % 2 == 0) ++units;
        units = imin(units, 63);                 // a box is at most 256 elements wide
        p.chunk_bytes = units * 16;
        p.n_chunks = (row_bytes + p.chunk_bytes - 1) / p.chunk_bytes;
        p.row_stride = p.chunk_bytes;
        p.group_stride = align_up(4 * p.chunk_bytes, 128);
        p.tail_vec = (row_bytes - (p.n_chunks - 1) * p.chunk_bytes) / 16;
        p.stage_bytes = 8 * p.group_stride;
    }
    p.LP = next_pow2(imax(L, 32));
    p.hs_bits = imin(imax(o.smem_hash_bits, 0), 16);
    p.vc_bits = imin(imax(o.visit_cache_bits, 0), 14);
    p.gather = (o.gather == 1 || o.gather == 2) ? o.gather : 0;
    p.carry = o.probe_carry != 0 ? 1 : 0;

    const int budget = smem_optin / p.ctas_per_sm - 1024;  // the runtime keeps 1 KB per CTA
    for (;;) {
        int off = 0;
        p.off_query = off;  off = align_up(off + dim * 4, 16);
        p.off_beam0 = off;  off += p.LP * 8;
        p.off_beam1 = off;  off += p.LP * 8;
        p.off_exp = off;    off = align_up(off + L * 4, 16);
        p.off_hash = off;   off += p.hs_bits > 0 ? (4 << p.hs_bits) : 0;
        p.off_vcache = off; off += p.vc_bits > 0 ? (4 << p.vc_bits) : 0;
        p.off_bar = off;    off += p.warps * 8 * 8;  // room for up to 8 stages
        p.off_pend = off;   off += p.warps * kPendCap * 4;
        p.off_bids = off;   off += p.warps * 64 * 4;
        off = align_up(off, 128);
        p.off_stage = off;
        const int room = budget - off;
        int st = room / (p.warps * p.stage_bytes);
        if (o.stages > 0) st = imin(st, o.stages);
        else if (auto_ctas) st = imin(st, 1);
        st = imin(st, 6);
        if (st >= 1) {
            p.stages = st;
            p.smem_bytes = off + p.warps * st * p.stage_bytes;
            break;
        }
        if (p.hs_bits > 0) {  // shrink the shared hash before giving up
            p.hs_bits = p.hs_bits > 8 ? p.hs_bits - 1 : 0;
            continue;
        }
        *why = "shared memory budget too small for this dim/L/warps/ctas_per_sm";
        return false;
    }
    if (auto_ctas) p.ctas_per_sm = imin(imax(smem_optin / (p.smem_bytes + 1024), 1), 8);
    // Candidate sort tile.  Only the L best of a round's candidates survive, and after each tile is
    // merged the L-th key tightens the filter for the rest, so small tiles (about 2L) sort far
    // fewer keys in total than one big tile: a round with 1500 candidates and L = 64 sorts ~300
    // keys in 256-key tiles instead of 2048.  Bounded by the staging memory the tile lives in.
    int tile = 64;
    int cap = imin(p.warps * p.stages * p.stage_bytes / 8, 2048);
    const int want = o.sort_tile > 0 ? o.sort_tile : imax(2 * p.LP, next_pow2(p.warps * 32));
    cap = imin(cap, imax(want, p.warps * 32));
    while (tile * 2 <= cap) tile <<= 1;
    if (tile < p.warps * 32 && tile * 2 <= imin(p.warps * p.stages * p.stage_bytes / 8, 2048)) tile <<= 1;
    p.tile_max = tile;
    if (p.tile_max < p.warps * 32) {
        *why = "staging area too small to sort a candidate tile";
        return false;
    }
    return true;
}

}  // namespace coral
