// Stand-in for a Faiss header (Faiss is not installed here).  The reference's headers include it
// and name a few Faiss types in typedefs; the search path never uses them.  Test infrastructure.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
namespace faiss {
using idx_t = int64_t;
struct Index {};
struct IndexFlatL2 {};
struct IndexFlatIP {};
namespace gpu {
struct StandardGpuResources {};
struct GpuIndexIVFFlat {};
struct GpuIndexFlatL2 {};
struct GpuIndexFlatIP {};
}  // namespace gpu
}  // namespace faiss
