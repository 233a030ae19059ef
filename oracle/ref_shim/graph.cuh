// Stand-in for the reference's include/graph.cuh, which cannot be compiled here (it pulls in the
// CLOCK cache, LZ4 storage and OpenMP plumbing).  Declares only what src/search_gpu.cu uses of
// Graph: the two device pointers of the HBM tier (include/graph.cuh:485-494).  Test infrastructure.
#pragma once
#include <cuda_runtime.h>

#include "disk_graph.h"
#include "uni.h"

namespace efanna2e {
class Graph {
   public:
    Graph(Slot* slots, float* vecs) : gpu_slots(slots), gpu_vec_slots(vecs) {}
    inline Slot* get_gpu_slots() { return gpu_slots; }
    inline float* get_gpu_vec_slots() { return gpu_vec_slots; }

   private:
    Slot* gpu_slots = nullptr;
    float* gpu_vec_slots = nullptr;
};
}  // namespace efanna2e
