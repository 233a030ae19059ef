// Stand-in for the reference's include/gpufuncs.cuh, which cannot be compiled here (it includes a
// header the reference does not ship and the Faiss-based kNN code).  Declares only what
// src/search_gpu.cu uses of GPUFuncs -- member names and types as in include/gpufuncs.cuh:36-40,
// :547-564, :799, :822, :832 -- so that the reference's search_gpu launcher and its kernels compile
// unmodified from the reference tree.  Test infrastructure.
#pragma once
#include <cuda_runtime.h>
#include <thrust/device_vector.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "graph.cuh"
#include "uni.h"
#include "utils.cuh"

namespace efanna2e {

struct MyStream {
    cudaStream_t stream = nullptr;
};

template <typename BData>
struct Search_Data {
    int Q_ = 0, batch_ = 0;
    BCD* d_beams_ = nullptr;
    uint32_t* d_visited_ = nullptr;
};

class GPUFuncs {
   public:
    Test_Result search_gpu(const float* queries, int* ids_res, float* dists_res, int Q, int k,
                           std::vector<int>& start_node_ids, bool have_delete, cudaStream_t stream);
    void search_verify(const int* ids_res, const int* ids_gt, Test_Result& tr, int Q, int k,
                       cudaStream_t stream);

    BP bp;
    Graph* graph = nullptr;
    std::vector<Search_Data<Beam_Data>*> search_data;
    thrust::device_vector<uint32_t> d_deleted;
    std::unordered_map<std::string, MyStream> streams;
};

}  // namespace efanna2e
