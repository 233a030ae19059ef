// Update driver with the reference's command line (reference tests/test_update.cpp:40-300): the
// index is built over the first half of the base file, then the second half slides in -- per round
// a batch of the oldest points is deleted (with topology repair) and/or a batch of new points is
// inserted -- and the search is verified against the exact neighbours among the points alive at
// that moment.  One line per verified round: round, recall (%), avg_hops, time, qps.
//
// Flags as in the reference: --dataset --base_data_path --sampled_query_data_path --query_path
// --dist --data_type --max_degree --k --L --upd_mode --config_file --update_gt_file
// --recall_thres --query_thres.  upd_mode (include/uni.h:53-56): 0 = delete + insert, verified every
// fourth round; 1 = delete only, half of the rounds; 2 = insert only; 4 = delete + insert, verified
// after each of the two.
// --update_gt_file is optional here: it is read when given (int32 rounds, then (rounds + 1) blocks
// of query_num x k int32 ids -- two blocks per round for upd_mode 4 -- as update_compute_gt writes
// them); without it --rounds N sets the number of rounds and the ground truth is computed by the
// library (coral_exact_knn over the live rows, deleted ids dropped).
// Additions: --graph_path DIR, --build 0|1 (default: build when the directory does not exist; the
// reference's config key upd_build), --csv FILE, --dump_graph DIR (final adjacency and entry points
// as a graph directory), --ids_out FILE (ids of the last verified search), --device N.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <numeric>
#include <string>
#include <sys/stat.h>
#include <vector>

#include "formats.h"
#include "index_gpu.h"

using namespace efanna2e;

namespace {

bool dir_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

// Exact k nearest among the rows that are alive: a wider exact list from the library, deleted ids
// dropped on the host.
std::vector<int> live_ground_truth(IndexGPU& index, const float* queries, int nq, int k, const std::vector<char>& dead) {
    const int wide = std::min<int>(228, (int)index.size());   // the exact search's widest list
    std::vector<int32_t> ids((size_t)nq * wide);
    int64_t uncertified = 0;
    const int rc = coral_exact_knn(index.handle(), queries, nq, wide, ids.data(), nullptr, &uncertified);
    if (rc != CORAL_OK) throw std::runtime_error(std::string("coral_exact_knn: ") + coral_last_error(index.handle()));
    std::vector<int> gt((size_t)nq * k);
    for (int q = 0; q < nq; ++q) {
        int w = 0;
        for (int j = 0; j < wide && w < k; ++j) {
            const int id = ids[(size_t)q * wide + j];
            if (id >= 0 && !dead[(size_t)id]) gt[(size_t)q * k + w++] = id;
        }
        if (w < k) throw std::runtime_error("ground truth: fewer than k live points among the 228 nearest");
    }
    return gt;
}

}  // namespace

int main(int argc, char** argv) {
    std::map<std::string, std::vector<std::string>> opt;
    std::string cur;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a.rfind("--", 0) == 0) {
            cur = a.substr(2);
            opt[cur];
        } else if (!cur.empty()) {
            opt[cur].push_back(a);
        }
    }
    auto has = [&](const char* k) { return opt.count(k) && !opt[k].empty(); };
    auto str = [&](const char* k, const std::string& d) { return has(k) ? opt[k][0] : d; };
    if (opt.count("help") || opt.count("h")) {
        std::cout << "see the header of test_update.cpp for the flags\n";
        return 0;
    }
    for (const char* req : {"dataset", "base_data_path", "sampled_query_data_path", "query_path", "upd_mode"})
        if (!has(req)) {
            std::cerr << "the option '--" << req << "' is required but missing\n";
            return -1;
        }
    const std::string dist = str("dist", "l2"), dataset = str("dataset", "");
    const int k = std::atoi(str("k", "1").c_str());
    const int L = std::atoi(str("L", "512").c_str());
    const int max_degree = std::atoi(str("max_degree", "2").c_str());
    const int upd_mode = std::atoi(str("upd_mode", "0").c_str());
    if (dist != "l2" && dist != "ip") {
        std::cout << "Unknown distance type: " << dist << std::endl;
        return -1;
    }
    if (upd_mode != 0 && upd_mode != 1 && upd_mode != 2 && upd_mode != 4) {
        std::cout << "Unknown update mode: " << upd_mode << std::endl;
        return -1;
    }
    if (k > L) {
        std::cout << "L must greater or equal than k" << std::endl;
        return 1;
    }
    std::cout << "Using " << (dist == "l2" ? "l2" : "inner product") << " as distance metric" << std::endl;
    const std::string graph_dir = str("graph_path", "../indexes/" + dataset + "_" + dist + "_" + std::to_string(max_degree) + "_upd");

    try {
        coral_host::FbinMeta bm, sm, qm;
        float* base = coral_host::fbin_load(str("base_data_path", ""), bm);
        float* train = coral_host::fbin_load(str("sampled_query_data_path", ""), sm);
        float* queries = coral_host::fbin_load(str("query_path", ""), qm);
        if (dist == "ip") {
            coral_host::normalize_rows(base, bm.n, (size_t)bm.dim);
            coral_host::normalize_rows(train, sm.n, (size_t)sm.dim);
            coral_host::normalize_rows(queries, qm.n, (size_t)qm.dim);
        }
        const size_t total_num = bm.n, base_num = total_num / 2, upd_num = base_num;   // tests/test_update.cpp:132
        const int query_num = (int)qm.n, dim = bm.dim;

        // ground truth from a file, when given
        int rounds = std::atoi(str("rounds", "4").c_str());
        std::vector<int> gts;
        const bool have_gt_file = has("update_gt_file");
        if (have_gt_file) {
            std::string path = str("update_gt_file", "");
            if (upd_mode == 1) path += ".del";          // :167-170
            else if (upd_mode == 2) path += ".ins";
            std::ifstream in(path, std::ios::binary);
            if (!in.is_open()) {
                std::cout << "Failed to open update_gt_file: " << path << std::endl;
                return -1;
            }
            in.read(reinterpret_cast<char*>(&rounds), sizeof(int));
            const size_t blocks = (size_t)(upd_mode == 4 ? 2 * rounds + 1 : rounds + 1);
            gts.resize((size_t)query_num * k * blocks);
            in.read(reinterpret_cast<char*>(gts.data()), (std::streamsize)(gts.size() * sizeof(int)));
            if (!in) throw std::runtime_error("update_gt_file is shorter than its header says");
        }
        if (rounds <= 0) throw std::runtime_error("need at least one round");

        Parameters parameters;
        parameters.Set<int>("max_degree", max_degree);
        parameters.Set<int>("k", k);
        parameters.Set<int>("CE", 1);
        parameters.Set<std::string>("base_file", str("base_data_path", ""));
        parameters.Set<std::string>("graph_file", graph_dir);
        parameters.Set<std::string>("config_file", str("config_file", ""));
        parameters.Set<std::string>("dist", dist);
        parameters.Set<std::string>("dataset", dataset);

        IndexGPU index((size_t)dim, base_num, dist == "l2" ? efanna2e::L2 : efanna2e::INNER_PRODUCT, nullptr);
        index.SetDevice(std::atoi(str("device", "0").c_str()));
        if (has("config_file")) index.load_config(str("config_file", ""));
        const bool build = has("build") ? std::atoi(str("build", "1").c_str()) != 0 : !dir_exists(graph_dir);
        if (build) {
            std::cout << "Building initial index..." << std::endl;
            Parameters bp = parameters;
            bp.Set<int>("k", index.PC.k);               // the build's list length is the config's k, not the search's
            index.BuildGPU(sm.n, train, base_num, base, bp);
        }
        index.RunPrepare(parameters, Mode::UPD, base_num, base);

        std::vector<char> dead(total_num, 0);
        std::ofstream csv;
        if (has("csv")) csv.open(str("csv", ""));
        std::cout << "round, recall, avg_hops, time, qps" << std::endl;
        if (csv.is_open()) csv << "round, recall, avg_hops, time, qps" << std::endl;
        std::vector<int> last_ids((size_t)query_num * k, -1);
        auto verify = [&](const std::string& label, size_t gt_block) {
            std::vector<int> computed;
            const int* gt = nullptr;
            if (have_gt_file) {
                gt = gts.data() + (size_t)query_num * k * gt_block;
            } else {
                computed = live_ground_truth(index, queries, query_num, k, dead);
                gt = computed.data();
            }
            Test_Result tr = index.Search_and_Verify(queries, gt, query_num, L);
            if (has("ids_out")) index.Search(queries, query_num, L, last_ids.data());
            const float recall = tr.calc_recall(query_num * k);
            std::cout << label << ", " << recall << ", " << tr.avg_hops(query_num) << ", " << tr.get_time() << ", "
                      << query_num / tr.get_time() << std::endl;
            if (csv.is_open())
                csv << label << ", " << recall << ", " << tr.avg_hops(query_num) << ", " << tr.get_time() << ", "
                    << query_num / tr.get_time() << std::endl;
        };
        verify("0", 0);

        const size_t batch = (upd_num + (size_t)rounds - 1) / (size_t)rounds;      // :221
        std::vector<int> del_ids;
        auto delete_batch = [&](int batch_i) {
            const size_t upd_n = std::min(batch, upd_num - (size_t)batch_i * batch);
            del_ids.resize(upd_n);
            std::iota(del_ids.begin(), del_ids.end(), (int)((size_t)batch_i * batch));
            index.Delete(del_ids);
            for (int id : del_ids) dead[(size_t)id] = 1;
        };
        auto insert_batch = [&](int batch_i) {
            const size_t upd_n = std::min(batch, upd_num - (size_t)batch_i * batch), first = base_num + (size_t)batch_i * batch;
            index.Insert(base + first * (size_t)dim, (int)upd_n);
        };
        if (upd_mode == 0) {                                   // :223-246
            for (int b = 0; b < rounds; ++b) {
                delete_batch(b);
                insert_batch(b);
                if ((b + 1) % 4 != 0 && b + 1 != rounds) continue;   // the reference verifies every fourth round; so does
                verify(std::to_string(b + 1), (size_t)b + 1);        // this driver, and the last round as well
            }
        } else if (upd_mode == 4) {                            // :247-275
            for (int b = 0; b < rounds; ++b) {
                delete_batch(b);
                verify(std::to_string(b + 1) + " after delete", (size_t)(b + 1) * 2 - 1);
                insert_batch(b);
                verify(std::to_string(b + 1), (size_t)(b + 1) * 2);
            }
        } else if (upd_mode == 1) {                            // :276-293
            for (int b = 0; b < rounds / 2; ++b) {
                delete_batch(b);
                verify(std::to_string(b + 1), (size_t)b + 1);
            }
        } else {                                               // :294-311
            for (int b = 0; b < rounds; ++b) {
                insert_batch(b);
                verify(std::to_string(b + 1), (size_t)b + 1);
            }
        }

        if (has("dump_graph")) {
            coral_host::Adjacency g;
            g.n = (int64_t)index.size();
            int deg_pad = 0;
            if (coral_get_option(index.handle(), "deg_pad", &deg_pad) != CORAL_OK) throw std::runtime_error("deg_pad");
            g.deg_pad = deg_pad;
            std::vector<int32_t> all((size_t)2 * base_num * (size_t)deg_pad);     // the handle holds room for every insert
            if (coral_index_get_adjacency(index.handle(), all.data()) != CORAL_OK)
                throw std::runtime_error(std::string("coral_index_get_adjacency: ") + coral_last_error(index.handle()));
            g.rows.assign(all.begin(), all.begin() + (std::ptrdiff_t)((size_t)g.n * (size_t)deg_pad));
            std::vector<int32_t> starts((size_t)coral_index_get_start_ids(index.handle(), nullptr, 0));
            coral_index_get_start_ids(index.handle(), starts.data(), (int)starts.size());
            coral_host::graph_dir_write(str("dump_graph", ""), g, starts);
        }
        if (has("ids_out")) {
            std::ofstream out(str("ids_out", ""), std::ios::binary);
            out.write(reinterpret_cast<const char*>(last_ids.data()), (std::streamsize)(last_ids.size() * sizeof(int)));
        }
        index.RunFree();
        std::free(base);
        std::free(train);
        std::free(queries);
        std::cout << "Finished\n";
    } catch (const std::exception& ex) {
        std::cerr << "error: " << ex.what() << std::endl;
        return 2;
    }
    return 0;
}
