// Build driver with the reference's command line (reference tests/test_build_pipeline.cpp:44-240):
// loads the base and the sampled (training) queries, unit-normalises both for inner product, and
// runs IndexGPU::BuildGPU -- exact k nearest base points of every training query, NAP, and with
// --CE 1 the connectivity enhancement -- which writes the graph directory
// ../indexes/<dataset>_<dist>_<M_pjbp>_<query_thres>_<CE> (or --graph_path DIR) with its entry
// points, the directory test_search_pipeline loads.
//
// Flags as in the reference: --data_type --dist --N --dataset --base_data_path
// --sampled_query_data_path --M_pjbp (maximum degree) --L_pjpq --CE --k (length of the k-NN lists)
// --query_thres --recall_thres --iso_thres --log_file --config_file --train_gt_file
// --query_test_file --gt_test_file, -T/--num_threads (accepted, unused).  --N > 0 keeps the first N
// base points.  --train_gt_file, when given, holds the training queries' k-NN lists (a
// ground-truth file: int32 nq, int32 k, ids) and replaces the exact search, as in the reference
// (src/index_gpu.cpp:350-352).  With --query_test_file and --gt_test_file the fresh index is
// searched once at L = test_beam_capacity and the recall printed.
// Additions: --graph_path DIR, --device N.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "formats.h"
#include "index_gpu.h"

using namespace efanna2e;

int main(int argc, char** argv) {
    std::map<std::string, std::vector<std::string>> opt;
    std::string cur;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "-T") a = "--num_threads";
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
        std::cout << "see the header of test_build_pipeline.cpp for the flags\n";
        return 0;
    }
    for (const char* req : {"data_type", "dist", "dataset", "base_data_path", "sampled_query_data_path"})
        if (!has(req)) {
            std::cerr << "the option '--" << req << "' is required but missing\n";
            return -1;
        }
    const std::string dist = str("dist", "l2"), dataset = str("dataset", "");
    const int max_degree = std::atoi(str("M_pjbp", "32").c_str());
    const int CE = std::atoi(str("CE", "1").c_str());
    const int k = std::atoi(str("k", "1").c_str());
    const size_t N = (size_t)std::atoll(str("N", "0").c_str());
    const float query_thres = (float)std::atof(str("query_thres", "100.0").c_str());
    std::cout << "sampled query: " << str("sampled_query_data_path", "") << std::endl;
    if (dist != "l2" && dist != "ip") {
        std::cout << "Unknown distance type: " << dist << std::endl;
        return -1;
    }
    std::cout << "Using " << (dist == "l2" ? "l2" : "inner product") << " as distance metric" << std::endl;
    char thres[32];
    std::snprintf(thres, sizeof thres, "%.1f", query_thres);
    const std::string graph_dir = str("graph_path", "../indexes/" + dataset + "_" + dist + "_" + std::to_string(max_degree) + "_" +
                                                        thres + "_" + std::to_string(CE ? 1 : 0));
    try {
        coral_host::FbinMeta bm, sm;
        float* base = coral_host::fbin_load(str("base_data_path", ""), bm);
        float* train = coral_host::fbin_load(str("sampled_query_data_path", ""), sm);
        if (bm.dim != sm.dim) throw std::runtime_error("base and sampled-query dimension mismatch");
        size_t base_num = bm.n;
        if (N > 0 && N < base_num) base_num = N;
        if (dist == "ip") {                                      // tests/test_build_pipeline.cpp:169-172
            coral_host::normalize_rows(base, base_num, (size_t)bm.dim);
            coral_host::normalize_rows(train, sm.n, (size_t)sm.dim);
        }
        Parameters parameters;
        parameters.Set<int>("max_degree", max_degree);
        parameters.Set<int>("L_pjpq", std::atoi(str("L_pjpq", "32").c_str()));
        parameters.Set<int>("CE", CE);
        parameters.Set<int>("k", k);
        parameters.Set<std::string>("base_file", str("base_data_path", ""));
        parameters.Set<std::string>("graph_file", graph_dir);
        parameters.Set<std::string>("train_gt_file", str("train_gt_file", ""));
        parameters.Set<std::string>("log_file", str("log_file", ""));
        parameters.Set<std::string>("config_file", str("config_file", ""));
        parameters.Set<std::string>("dist", dist);
        parameters.Set<std::string>("dataset", dataset);

        IndexGPU index((size_t)bm.dim, base_num, dist == "l2" ? efanna2e::L2 : efanna2e::INNER_PRODUCT, nullptr);
        index.SetDevice(std::atoi(str("device", "0").c_str()));
        const auto t0 = std::chrono::steady_clock::now();
        index.BuildGPU(sm.n, train, base_num, base, parameters);
        const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        std::cout << "Build " << base_num << " points, " << sm.n << " training queries, k=" << k << ", max_degree=" << max_degree
                  << ", CE=" << CE << ": " << secs << " s -> " << graph_dir << std::endl;

        if (has("query_test_file") && has("gt_test_file")) {
            coral_host::FbinMeta qm;
            float* q = coral_host::fbin_load(str("query_test_file", ""), qm);
            if (dist == "ip") coral_host::normalize_rows(q, qm.n, (size_t)qm.dim);
            const coral_host::GroundTruth gt = coral_host::gt_load(str("gt_test_file", ""));
            const int kk = std::min(gt.k, 10), nq = std::min<int>((int)qm.n, gt.nq);
            Parameters sp = parameters;
            sp.Set<int>("k", kk);
            index.RunPrepare(sp, Mode::SEARCH, base_num, base);
            std::vector<int> res((size_t)nq * kk);
            const Test_Result tr = index.Search(q, nq, index.PC.test_beam_capacity, res.data());
            long hits = 0;
            for (int i = 0; i < nq; ++i)
                for (int j = 0; j < kk; ++j) {
                    const int p = gt.ids[(size_t)i * gt.k + j];
                    if (std::find(res.begin() + (size_t)i * kk, res.begin() + (size_t)(i + 1) * kk, p) != res.begin() + (size_t)(i + 1) * kk)
                        ++hits;
                }
            std::cout << "Search result: recall@" << kk << "=" << (float)hits / (float)((long)nq * kk) << ", avg_hops=" << tr.avg_hops(nq)
                      << ", time=" << tr.get_time() << "s, qps=" << nq / tr.get_time() << std::endl;
            std::free(q);
        }
        index.RunFree();
        std::free(base);
        std::free(train);
    } catch (const std::exception& ex) {
        std::cerr << "error: " << ex.what() << std::endl;
        return 2;
    }
    return 0;
}
