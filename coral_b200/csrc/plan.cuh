// Shared-memory planning of the beam-search kernel: pure host arithmetic, no CUDA calls, no
// containers, no allocation -- every entry point (handle-based and allocation-free) uses it.
#pragma once
#include "search_kernel.cuh"

namespace coral {

// Tuning inputs of the planner; 0 = automatic unless noted.
struct PlanOptions {
    int ctas_per_sm = 0;   // resident CTAs per SM (at most 8)
    int warps = 0;         // warps per CTA
    int chunk_bytes = 0;   // bytes of a row moved by one bulk copy
    int stages = 0;        // stage buffers per warp
    int smem_hash_bits = 0;
    int visit_cache_bits = 0;
    int sort_tile = 0;
    int probe_carry = 1;
    int gather = 0;
};

// Plan for beam capacity L with exactly `warps` warps per CTA.  Returns false and sets *why (a
// string literal) when nothing fits `smem_optin` bytes of opt-in shared memory per CTA.
bool make_plan_warps(int dim, int smem_optin, const PlanOptions& o, int L, int warps, SearchPlan& p,
                     const char** why, int chunk_target = 0);

// The automatic plan: the warp count in 3..6 that keeps most warps resident per SM (more CTAs on a
// tie), and chunks of up to 512 bytes for rows that do not split into 256-byte chunks as long as
// five CTAs still fit an SM.  Explicit `warps`/`ctas_per_sm` options bypass the search.
bool make_plan(int dim, int smem_optin, const PlanOptions& o, int L, SearchPlan& p, const char** why);

}  // namespace coral
