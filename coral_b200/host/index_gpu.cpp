#include "index_gpu.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "formats.h"

namespace efanna2e {

IndexGPU::IndexGPU(size_t dimension, size_t n, Metric m, Index* /*initializer*/)
    : dimension_(dimension), nd_(n), metric_kind_(m) {
    if (m == COSINE) need_normalize = true;  // src/index_gpu.cpp:31-34
}

IndexGPU::~IndexGPU() {
    RunFree();
    if (own_base_) std::free(h_base_);
}

void IndexGPU::check(int rc, const char* what) const {
    if (rc == CORAL_OK) return;
    throw std::runtime_error(std::string(what) + ": " + coral_last_error(handle_));
}

void IndexGPU::load_config(const std::string& config_file) {
    const std::string path = config_file == "default" ? "../config.json" : config_file;  // src/index_gpu.cpp:42-47
    const auto j = coral_host::config_load(path);
    auto geti = [&](const char* key, int dflt) {
        auto it = j.find(key);
        return it == j.end() ? dflt : (int)it->second;
    };
    PC.dim = geti("dim", 200);
    PC.k = geti("k", 100);
    PC.max_degree = geti("max_degree", 32);
    PC.test_beam_capacity = geti("test_beam_capacity", 512);
    PC.search_start_nodes_num = geti("search_start_nodes_num", 16);
    PC.search_in_cpu = geti("search_in_cpu", 0);
    PC.batch = geti("batch", 1024);
    PC.enhance_nap_batch = geti("enhance_nap_batch", 4096);
    PC.enhance_search_batch = geti("enhance_search_batch", 524288);
    PC.insert_batch = geti("insert_batch", 2048);
}

void IndexGPU::LoadSearchNeededData(const char* base_file, const char* sampled_query_file, DIST_METRIC m) {
    coral_host::FbinMeta meta;
    if (sampled_query_file && std::strlen(sampled_query_file) != 0) {
        const coral_host::FbinMeta q = coral_host::fbin_meta(sampled_query_file);
        const coral_host::FbinMeta b = coral_host::fbin_meta(base_file);
        if (q.dim != b.dim) throw std::runtime_error("base and query dimension mismatch");
    }
    float* data = coral_host::fbin_load(base_file, meta);
    if ((size_t)meta.dim != dimension_) {
        std::free(data);
        throw std::runtime_error("base dimension does not match the index dimension");
    }
    if (m == DIST_METRIC::IP_) coral_host::normalize_rows(data, meta.n, (size_t)meta.dim);
    if (own_base_) std::free(h_base_);
    h_base_ = data;
    own_base_ = true;
    nd_ = meta.n;
    metric_ = m;
}

void IndexGPU::upload_graph(const std::vector<int32_t>& rows, int deg_pad) {
    check(coral_index_set_adjacency(handle_, rows.data(), deg_pad), "coral_index_set_adjacency");
}

void IndexGPU::BuildGPU(size_t n_sq, float* sq_data, size_t n_bp, float* bp_data, Parameters& parameters) {
    SetParameters(parameters);
    const std::string cfg = parameters.Get<std::string>("config_file", std::string(""));
    if (!cfg.empty()) load_config(cfg);
    const int CE = parameters.Get<int>("CE", 1);
    max_degree_ = parameters.Get<int>("max_degree");
    k_ = parameters.Get<int>("k");
    metric_ = parameters.Get<std::string>("dist") == "l2" ? DIST_METRIC::L2_ : DIST_METRIC::IP_;
    const std::string graph_dir = parameters.Get<std::string>("graph_file");
    if (own_base_) std::free(h_base_);
    h_base_ = bp_data;
    own_base_ = false;
    nd_ = n_bp;
    RunFree();
    int rc = coral_index_create(&handle_, device_, (int64_t)nd_, (int)dimension_, max_degree_,
                                metric_ == DIST_METRIC::L2_ ? CORAL_L2 : CORAL_IP);
    if (rc != CORAL_OK) throw std::runtime_error(std::string("coral_index_create: ") + coral_last_error(nullptr));
    capacity_ = nd_;
    check(coral_index_set_vectors(handle_, h_base_), "coral_index_set_vectors");
    std::vector<int32_t> knn(n_sq * (size_t)k_);
    const std::string train_gt = parameters.Get<std::string>("train_gt_file", std::string(""));
    if (!train_gt.empty() && train_gt != "None") {
        // the training queries' k-NN lists come from a file instead of the search (src/index_gpu.cpp:505-515)
        const coral_host::GroundTruth lists = coral_host::gt_load(train_gt);
        if (lists.k != k_) throw std::runtime_error("train_gt_file: its k differs from the build's k");
        if ((size_t)lists.nq < n_sq) throw std::runtime_error("train_gt_file: fewer lists than training queries");
        for (size_t i = 0; i < knn.size(); ++i) {
            knn[i] = lists.ids[i];
            if (knn[i] < 0 || (size_t)knn[i] >= nd_) throw std::runtime_error("train_gt_file: id out of range");
        }
    } else {
        check(coral_exact_knn(handle_, sq_data, (int)n_sq, k_, knn.data(), nullptr, nullptr), "coral_exact_knn");   // src/knn.cu:174-193
    }
    check(coral_build_begin(handle_), "coral_build_begin");
    check(coral_build_nap(handle_, knn.data(), (int)n_sq, k_, PC.batch), "coral_build_nap");
    int64_t n_iso = 0;
    if (CE)
        check(coral_build_connect_enhance(handle_, k_, 256, PC.enhance_search_batch, PC.enhance_nap_batch,
                                          PC.search_start_nodes_num, &n_iso),
              "coral_build_connect_enhance");
    coral_host::Adjacency g;
    g.n = (int64_t)nd_;
    int deg_pad = 0;
    check(coral_get_option(handle_, "deg_pad", &deg_pad), "coral_get_option");
    g.deg_pad = deg_pad;
    g.rows.resize(nd_ * (size_t)deg_pad);
    check(coral_index_get_adjacency(handle_, g.rows.data()), "coral_index_get_adjacency");
    if (!CE || n_iso == 0) {   // no enhancement ran: choose the entry points now
        int first = -1;
        for (int64_t i = 0; i < g.n && first < 0; ++i)
            if (g.rows[(size_t)i * g.deg_pad] >= 0) first = (int)i;
        if (first < 0) throw std::runtime_error("BuildGPU: the graph has no edges");
        check(coral_index_select_start_ids(handle_, first, PC.search_start_nodes_num, nullptr), "coral_index_select_start_ids");
    }
    start_ids_.resize((size_t)coral_index_get_start_ids(handle_, nullptr, 0));
    coral_index_get_start_ids(handle_, start_ids_.data(), (int)start_ids_.size());
    coral_host::graph_dir_write(graph_dir, g, start_ids_);          // Graph::save_build, include/graph.cuh:481-484
    check(coral_build_end(handle_), "coral_build_end");
}

void IndexGPU::Delete(const std::vector<int> del_ids) {
    if (!handle_) throw std::runtime_error("Delete: call RunPrepare first");
    if (!updating_) {
        check(coral_build_begin_from_graph(handle_), "coral_build_begin_from_graph");
        updating_ = true;
    }
    std::vector<int32_t> ids(del_ids.begin(), del_ids.end());
    check(coral_delete(handle_, ids.data(), (int)ids.size(), PC.search_start_nodes_num), "coral_delete");
    prepared_q_ = prepared_L_ = prepared_k_ = 0;
}

void IndexGPU::Insert(const float* ins_vectors, int ins_num) {
    if (!handle_) throw std::runtime_error("Insert: call RunPrepare first");
    if (nd_ + (size_t)ins_num > capacity_) throw std::runtime_error("Insert: no room left (RunPrepare with Mode::UPD reserves it)");
    if (!updating_) {
        check(coral_build_begin_from_graph(handle_), "coral_build_begin_from_graph");
        updating_ = true;
    }
    check(coral_index_write_vectors(handle_, (int64_t)nd_, ins_num, ins_vectors), "coral_index_write_vectors");
    check(coral_insert(handle_, (int64_t)nd_, ins_num, PC.k, PC.test_beam_capacity, PC.insert_batch,
                       PC.search_start_nodes_num),
          "coral_insert");
    nd_ += (size_t)ins_num;
    prepared_q_ = prepared_L_ = prepared_k_ = 0;     // coral_insert sized the search scratch for its own batches
}

void IndexGPU::RunPrepare(Parameters& parameters, Mode mode, size_t n_bp, float* bp_data) {
    if (mode != Mode::SEARCH && mode != Mode::UPD) throw std::runtime_error("RunPrepare: Mode::SEARCH or Mode::UPD (BuildGPU builds)");
    SetParameters(parameters);
    const std::string cfg = parameters.Get<std::string>("config_file", std::string(""));
    if (!cfg.empty()) load_config(cfg);
    k_ = parameters.Get<int>("k");
    max_degree_ = parameters.Get<int>("max_degree");
    metric_ = parameters.Get<std::string>("dist") == "l2" ? DIST_METRIC::L2_ : DIST_METRIC::IP_;
    const std::string graph_dir = parameters.Get<std::string>("graph_file");
    if (n_bp > 0) {
        if (own_base_) std::free(h_base_);
        h_base_ = bp_data;
        own_base_ = false;
        nd_ = n_bp;
    }
    if (!h_base_) throw std::runtime_error("RunPrepare: base vectors have not been loaded");

    RunFree();
    capacity_ = mode == Mode::UPD ? 2 * nd_ : nd_;
    int rc = coral_index_create(&handle_, device_, (int64_t)capacity_, (int)dimension_, max_degree_,
                                metric_ == DIST_METRIC::L2_ ? CORAL_L2 : CORAL_IP);
    if (rc != CORAL_OK) throw std::runtime_error(std::string("coral_index_create: ") + coral_last_error(nullptr));
    check(coral_index_write_vectors(handle_, 0, (int64_t)nd_, h_base_), "coral_index_write_vectors");
    check(coral_index_set_live(handle_, (int64_t)nd_), "coral_index_set_live");
    coral_host::Adjacency g = coral_host::graph_dir_load(graph_dir, (int64_t)nd_, max_degree_);
    if (capacity_ > nd_) g.rows.resize(capacity_ * (size_t)g.deg_pad, -1);   // rows of points still to be inserted
    upload_graph(g.rows, g.deg_pad);
    start_ids_ = coral_host::start_ids_load(graph_dir + "/graph.search_start_ids");
    if (start_ids_.empty()) {
        // No saved entry points: choose them as Graph::get_search_start_nodes_fps does
        // (src/graph.cpp:298-313 -> src/start.cu:72-145), starting from the lowest-numbered node that
        // has an out-edge instead of a random one, and save them where the reference does
        // (src/graph.cpp:315-327).
        int first = -1;
        for (int64_t i = 0; i < g.n && first < 0; ++i)
            if (g.rows[(size_t)i * g.deg_pad] >= 0) first = (int)i;
        if (first < 0) throw std::runtime_error("no entry points and no edges in " + graph_dir);
        const int M = std::max(1, PC.search_start_nodes_num);
        start_ids_.resize((size_t)M);
        check(coral_index_select_start_ids(handle_, first, M, start_ids_.data()), "coral_index_select_start_ids");
        try {
            coral_host::start_ids_write(graph_dir + "/graph.search_start_ids", start_ids_);
        } catch (const std::exception&) {
            // a read-only graph directory: the reference only logs the failed write (src/graph.cpp:317-319)
        }
        return;
    }
    check(coral_index_set_start_ids(handle_, start_ids_.data(), (int)start_ids_.size()), "coral_index_set_start_ids");
}

void IndexGPU::LoadRoarGraph(std::string filename) {
    if (!handle_) throw std::runtime_error("LoadRoarGraph: call RunPrepare first");
    int32_t ep = 0;
    const coral_host::Adjacency g = coral_host::flat_graph_load(filename, max_degree_, ep);
    if ((size_t)g.n != nd_) throw std::runtime_error("flat graph node count does not match the base");
    upload_graph(g.rows, g.deg_pad);
    start_ids_.assign(1, ep);  // src/graph.cu:741-742
    check(coral_index_set_start_ids(handle_, start_ids_.data(), 1), "coral_index_set_start_ids");
}

void IndexGPU::SetDeleted(const std::vector<int>& deleted_ids) {
    if (!handle_) throw std::runtime_error("SetDeleted: call RunPrepare first");
    if (deleted_ids.empty()) {
        check(coral_index_set_deleted(handle_, nullptr), "coral_index_set_deleted");
        return;
    }
    std::vector<uint32_t> bits((nd_ + 31) / 32, 0u);
    for (int id : deleted_ids)
        if (id >= 0 && (size_t)id < nd_) bits[(size_t)id >> 5] |= 1u << (id & 31);
    check(coral_index_set_deleted(handle_, bits.data()), "coral_index_set_deleted");
}

void IndexGPU::ensure_prepared(int num, int beam_capacity) {
    if (num <= prepared_q_ && beam_capacity <= prepared_L_ && k_ <= prepared_k_) return;
    prepared_q_ = std::max(prepared_q_, num);
    prepared_L_ = std::max(prepared_L_, beam_capacity);
    prepared_k_ = std::max(prepared_k_, k_);
    check(coral_search_prepare(handle_, prepared_q_, prepared_L_, prepared_k_), "coral_search_prepare");
}

Test_Result IndexGPU::SearchWithDists(const float* queries, int num, int beam_capacity, int* ids_res,
                                      float* dists_res) {
    if (!handle_) throw std::runtime_error("Search: call RunPrepare first");
    ensure_prepared(num, beam_capacity);
    int64_t hops = 0;
    check(coral_search(handle_, queries, num, beam_capacity, k_, ids_res, dists_res, nullptr, &hops), "coral_search");
    return Test_Result(-1, (size_t)hops, coral_last_kernel_ms(handle_) * 1e-3f);
}

Test_Result IndexGPU::Search(const float* queries, int num, int beam_capacity, int* ids_res, int /*M*/) {
    return SearchWithDists(queries, num, beam_capacity, ids_res, nullptr);
}

Test_Result IndexGPU::Search_and_Verify(const float* queries, const int* gts, int num, int beam_capacity) {
    if (beam_capacity <= 0) beam_capacity = PC.test_beam_capacity;
    std::vector<int> ids((size_t)num * k_);
    Test_Result tr = Search(queries, num, beam_capacity, ids.data());
    int64_t hits = 0;
    check(coral_count_hits(handle_, ids.data(), gts, num, k_, k_, &hits), "coral_count_hits");
    tr.hits = (int)hits;
    return tr;
}

void IndexGPU::RunFree() {
    if (handle_) coral_index_destroy(handle_);
    handle_ = nullptr;
    prepared_q_ = prepared_L_ = prepared_k_ = 0;
    updating_ = false;
}

}  // namespace efanna2e

// ---------------------------------------------------------------------------------------------
// C hooks over the loaders, so that they can be exercised without a GPU (ctypes).
extern "C" {

int coral_host_graph_dir_load(const char* dir, int64_t n, int max_degree, int32_t* rows_out, int* deg_pad_out) {
    try {
        const coral_host::Adjacency g = coral_host::graph_dir_load(dir, n, max_degree);
        if (deg_pad_out) *deg_pad_out = g.deg_pad;
        if (rows_out) std::memcpy(rows_out, g.rows.data(), g.rows.size() * 4);
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int coral_host_graph_dir_write(const char* dir, int64_t n, int deg_pad, const int32_t* rows, const int32_t* start, int m) {
    try {
        coral_host::Adjacency g;
        g.n = n;
        g.deg_pad = deg_pad;
        g.rows.assign(rows, rows + (size_t)n * deg_pad);
        coral_host::graph_dir_write(dir, g, std::vector<int32_t>(start, start + m));
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int coral_host_flat_graph_roundtrip(const char* path, int64_t n, int deg_pad, int max_degree, const int32_t* rows,
                                    int32_t ep, int32_t* rows_out, int32_t* ep_out) {
    try {
        coral_host::Adjacency g;
        g.n = n;
        g.deg_pad = deg_pad;
        g.rows.assign(rows, rows + (size_t)n * deg_pad);
        coral_host::flat_graph_write(path, g, ep);
        const coral_host::Adjacency r = coral_host::flat_graph_load(path, max_degree, *ep_out);
        std::memcpy(rows_out, r.rows.data(), r.rows.size() * 4);
        return r.deg_pad;
    } catch (const std::exception&) {
        return -1;
    }
}

int coral_host_start_ids_load(const char* path, int32_t* out, int cap) {
    try {
        const std::vector<int32_t> ids = coral_host::start_ids_load(path);
        for (size_t i = 0; i < ids.size() && (int)i < cap; ++i) out[i] = ids[i];
        return (int)ids.size();
    } catch (const std::exception&) {
        return -1;
    }
}

int coral_host_lz4_decode(const uint8_t* src, int src_len, uint8_t* dst, int cap) {
    return coral_host::lz4_block_decode(src, src_len, dst, cap);
}

int coral_host_fbin_load(const char* path, float* out, int64_t cap_floats, int64_t* n, int* dim, int normalize) {
    try {
        coral_host::FbinMeta m;
        float* p = coral_host::fbin_load(path, m);
        if (normalize) coral_host::normalize_rows(p, m.n, (size_t)m.dim);
        *n = (int64_t)m.n;
        *dim = m.dim;
        if (out && (int64_t)(m.n * m.dim) <= cap_floats) std::memcpy(out, p, m.n * (size_t)m.dim * 4);
        std::free(p);
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

int coral_host_config_get(const char* path, const char* key, double* value) {
    try {
        const auto m = coral_host::config_load(path);
        auto it = m.find(key);
        if (it == m.end()) return 1;
        *value = it->second;
        return 0;
    } catch (const std::exception&) {
        return -1;
    }
}

}  // extern "C"
