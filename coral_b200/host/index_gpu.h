// Host-side mirror of the reference's search interface (reference
// include/index_gpu.h:46-76, include/efanna2e/parameters.h, include/uni.h:149,
// :411-437) over the C ABI in include/coral_b200.h.  Same names, argument meaning
// and units, so a caller of efanna2e::IndexGPU's search side compiles against
// this header unchanged.  Differences, all on purpose: errors are thrown as
// std::runtime_error instead of exiting the process; scratch is sized once and
// kept between searches; the build keeps no k-NN cache and runs NAP and CE in one
// pass on one GPU (no out-of-core tiers).
#pragma once
#include <cstddef>
#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/coral_b200.h"

namespace efanna2e {

enum Metric { L2 = 0, INNER_PRODUCT = 1, FAST_L2 = 2, PQ = 3, COSINE = 4 };  // include/efanna2e/distance.h:15
enum class DIST_METRIC { L2_ = 0, IP_ = 1 };
enum Mode { CONS, SEARCH, UPD, CE };  // include/uni.h:147

// String-typed parameter bag (include/efanna2e/parameters.h:15-58).
class Parameters {
   public:
    template <typename T>
    void Set(const std::string& name, const T& value) {
        std::ostringstream os;
        os << value;
        values_[name] = os.str();
    }
    template <typename T>
    T Get(const std::string& name) const {
        auto it = values_.find(name);
        if (it == values_.end()) throw std::invalid_argument("Invalid parameter name.");
        std::istringstream is(it->second);
        T v;
        if (!(is >> v) || !is.eof()) throw std::runtime_error("Failed to convert value '" + it->second + "'");
        return v;
    }
    template <typename T>
    T Get(const std::string& name, const T& fallback) const {
        return values_.count(name) ? Get<T>(name) : fallback;
    }

   private:
    std::unordered_map<std::string, std::string> values_;
};
template <>
inline std::string Parameters::Get<std::string>(const std::string& name) const {
    auto it = values_.find(name);
    if (it == values_.end()) throw std::invalid_argument("Invalid parameter name.");
    return it->second;
}

// include/uni.h:411-437.  `time` is in seconds and covers the kernel window
// (search kernel + counter copy), as in src/search_gpu.cu:861-877.
class Test_Result {
   public:
    Test_Result() = default;
    Test_Result(int hits_, size_t hops_, float time_) : time(time_), hits(hits_), hops(hops_) {}
    float get_recall() const { return recall; }
    size_t get_hops() const { return hops; }
    float get_time() const { return time; }
    float calc_recall(int total_num) { return recall = 100.0f * hits / total_num; }
    float avg_hops(int search_num) const { return 1.0f * hops / search_num; }
    void accumulate(const Test_Result& o) {
        hops += o.hops;
        time += o.time;
        hits += o.hits;
    }
    float recall = 0.f, time = 0.f;
    int hits = 0;
    size_t hops = 0;
};

// The keys of config.json the search path reads (include/uni.h:97-132).
struct ProConfig {
    int dim = 200, k = 100, max_degree = 32;
    int search_start_nodes_num = 16, test_beam_capacity = 512, search_in_cpu = 0;
    // build and update keys (config.json:5-8,36)
    int batch = 1024, enhance_nap_batch = 4096, enhance_search_batch = 524288, insert_batch = 2048;
};

class Index;  // the reference's base class is not needed by the search side

class IndexGPU {
   public:
    explicit IndexGPU(size_t dimension, size_t n, Metric m, Index* initializer);
    ~IndexGPU();
    IndexGPU(const IndexGPU&) = delete;
    IndexGPU& operator=(const IndexGPU&) = delete;

    // Reads the base vectors (.fbin), unit-normalising them for inner product
    // (src/index_gpu.cpp:625-650).  `sampled_query_file` may be "".
    void LoadSearchNeededData(const char* base_file, const char* sampled_query_file,
                              DIST_METRIC m = DIST_METRIC::L2_);
    // Reads config_file, the graph directory `graph_file` and its start ids, and
    // uploads everything (src/index_gpu.cpp:226-262).  Keys: dist, k, max_degree,
    // graph_file, base_file, config_file (optional: log_file, query_file, CE).
    // When n_bp > 0, `bp_data` (n_bp x dim floats) replaces the loaded base.
    void RunPrepare(Parameters& parameters, Mode mode, size_t n_bp = 0, float* bp_data = nullptr);
    // queries: host (or device) pointer to num*dim floats, already normalised for
    // inner product; ids_res: num*k ints.  M is ignored, as in the reference
    // (src/index_gpu.cpp:119): every id of graph.search_start_ids is an entry point.
    Test_Result Search(const float* queries, int num, int beam_capacity, int* ids_res, int M = 0);
    // gts: num*k ints (row stride k).  beam_capacity 0 = config test_beam_capacity.
    Test_Result Search_and_Verify(const float* queries, const int* gts, int num, int beam_capacity = 0);
    // Flat graph import; the file's entry point becomes the only start id
    // (src/graph.cu:709-743).
    void LoadRoarGraph(std::string filename);
    // Builds the graph over bp_data (n_bp x dim, already normalised for inner product) from the
    // n_sq training queries sq_data: exact k nearest base points per query, NAP, and -- CE = 1 -- the
    // connectivity enhancement; writes the graph directory `graph_file` and its entry points
    // (src/index_gpu.cpp:308-383).  Keys: dist, k, max_degree, CE, graph_file (optional config_file).
    // The handle stays searchable afterwards.
    void BuildGPU(size_t n_sq, float* sq_data, size_t n_bp, float* bp_data, Parameters& parameters);
    // Delete with topology repair / insert with neighbours from the search (src/index_gpu.cpp:138-224).
    // Mode::UPD in RunPrepare reserves room for as many inserted points as there are base points,
    // as the reference does (src/graph.cpp:141-142).
    void Delete(const std::vector<int> del_ids);
    void Insert(const float* ins_vectors, int ins_num);
    void RunFree();
    void load_config(const std::string& config_file);
    void SetParameters(Parameters& parameters) { parameters_ = parameters; }

    // Extensions used by the multi-GPU driver and the tests.
    void SetDevice(int device) { device_ = device; }
    void SetDeleted(const std::vector<int>& deleted_ids);
    Test_Result SearchWithDists(const float* queries, int num, int beam_capacity, int* ids_res, float* dists_res);
    coral_index_t* handle() const { return handle_; }
    const std::vector<int32_t>& start_ids() const { return start_ids_; }
    size_t size() const { return nd_; }
    ProConfig PC;
    bool need_normalize = false;

   private:
    void upload_graph(const std::vector<int32_t>& rows, int deg_pad);
    void ensure_prepared(int num, int beam_capacity);
    void check(int rc, const char* what) const;

    size_t dimension_, nd_;
    Metric metric_kind_;
    DIST_METRIC metric_ = DIST_METRIC::L2_;
    Parameters parameters_;
    int k_ = 1, max_degree_ = 32, device_ = 0;
    float* h_base_ = nullptr;
    bool own_base_ = false;
    coral_index_t* handle_ = nullptr;
    std::vector<int32_t> start_ids_;
    int prepared_q_ = 0, prepared_L_ = 0, prepared_k_ = 0;
    size_t capacity_ = 0;      // rows the handle was created for (>= nd_ in Mode::UPD)
    bool updating_ = false;
};

}  // namespace efanna2e
