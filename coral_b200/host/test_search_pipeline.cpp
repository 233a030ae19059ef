// Search driver with the reference's command line (reference
// tests/test_search_pipeline.cpp:88-128): loads an .fbin base and query set, a
// ground-truth file and a graph directory, sweeps the beam capacities given by
// --L and prints L, QPS, time, recall@k and average hops per sweep point.
//
// Flags accepted as in the reference: --data_type --dist --base_data_path
// --dataset --recall_thres --query_path --gt_path --L a b c --max_recall
// --max_hop --k --max_degree --query_thres --log_file --res_file --config_file
// --CE --index_type, plus -T (accepted, unused, like the reference).
// Additions: --graph_path DIR (instead of ../indexes/<dataset>_<dist>_<deg>_<thres>_<CE>),
// --roar_graph FILE (flat graph import), --csv FILE, --device N, --ids_out FILE,
// --deleted_ids FILE (text list of ids hidden from the results, IndexGPU::SetDeleted),
// --verify (count hits on the device with IndexGPU::Search_and_Verify, needs a
// ground truth exactly k wide; prints "hits <n>" per sweep point).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "formats.h"
#include "index_gpu.h"

using namespace efanna2e;

// tests/test_search_pipeline.cpp:25-39
static float ComputeRecall(int q_num, int k, int gt_dim, const int* res, const int* gt) {
    long total = 0;
    for (int i = 0; i < q_num; i++)
        for (int j = 0; j < k; j++) {
            const int p = gt[(size_t)i * gt_dim + j];
            if (std::find(res + (size_t)i * k, res + (size_t)i * k + k, p) != res + (size_t)i * k + k) ++total;
        }
    return (float)total / (float)((long)k * q_num);
}

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
        std::cout << "see the header of test_search_pipeline.cpp for the flags\n";
        return 0;
    }
    for (const char* req : {"data_type", "dist", "base_data_path", "dataset", "query_path", "gt_path"})
        if (!has(req)) {
            std::cerr << "the option '--" << req << "' is required but missing\n";
            return -1;
        }
    const std::string dist = str("dist", "l2"), dataset = str("dataset", "");
    const int k = std::atoi(str("k", "1").c_str());
    const int max_degree = std::atoi(str("max_degree", "32").c_str());
    const int CE = std::atoi(str("CE", "1").c_str());
    const double max_recall = std::atof(str("max_recall", "0").c_str());
    const float query_thres = (float)std::atof(str("query_thres", "1.0").c_str());
    std::vector<int> L_vec;
    if (opt.count("L"))
        for (const auto& s : opt["L"]) L_vec.push_back(std::atoi(s.c_str()));
    if (dist != "l2" && dist != "ip") {
        std::cout << "Unknown distance type: " << dist << std::endl;
        return -1;
    }
    char thres[32];
    std::snprintf(thres, sizeof thres, "%.1f", query_thres);
    const std::string dataset_dist = dataset + "_" + dist + "_" + std::to_string(max_degree);
    const std::string graph_dir =
        str("graph_path", "../indexes/" + dataset_dist + "_" + thres + "_" + std::to_string(CE ? 1 : 0));

    try {
        coral_host::FbinMeta qm;
        float* query_data = coral_host::fbin_load(str("query_path", ""), qm);
        if (dist == "ip") coral_host::normalize_rows(query_data, qm.n, (size_t)qm.dim);  // :193
        const coral_host::GroundTruth gt = coral_host::gt_load(str("gt_path", ""));
        std::cout << "Using " << (dist == "l2" ? "l2" : "inner product") << " as distance metric" << std::endl;

        Parameters parameters;
        parameters.Set<std::string>("dist", dist);
        parameters.Set<int>("k", k);
        parameters.Set<int>("max_degree", max_degree);
        parameters.Set<int>("CE", CE);
        parameters.Set<std::string>("graph_file", graph_dir);
        parameters.Set<std::string>("base_file", str("base_data_path", ""));
        parameters.Set<std::string>("log_file", str("log_file", ""));
        parameters.Set<std::string>("config_file", str("config_file", ""));

        IndexGPU index((size_t)qm.dim, 0, dist == "l2" ? efanna2e::L2 : efanna2e::INNER_PRODUCT, nullptr);
        index.SetDevice(std::atoi(str("device", "0").c_str()));
        index.LoadSearchNeededData(str("base_data_path", "").c_str(), "",
                                   dist == "l2" ? DIST_METRIC::L2_ : DIST_METRIC::IP_);
        std::cout << "Load graph index: " << graph_dir << std::endl;
        index.RunPrepare(parameters, Mode::SEARCH);
        if (has("roar_graph")) index.LoadRoarGraph(str("roar_graph", ""));
        if (has("deleted_ids")) {
            std::ifstream in(str("deleted_ids", ""));
            if (!in.is_open()) throw std::runtime_error("cannot open " + str("deleted_ids", ""));
            std::vector<int> dead;
            for (long long v; in >> v;) dead.push_back((int)v);
            index.SetDeleted(dead);
        }

        std::cout << "k: " << k << std::endl;
        std::vector<int> res(qm.n * (size_t)k, 0);
        std::ofstream csv;
        if (has("csv")) {
            csv.open(str("csv", ""));
            csv << "L, QPS, time, recall@" << k << ", avg_hops" << std::endl;
        }
        std::cout << "L\t\tQPS\t\tavg_time\t\trecall@" << k << "\t\tavg_hops" << std::endl;
        if (L_vec.empty() && max_recall > 0.5) L_vec.push_back(128);
        for (size_t i = 0; i < L_vec.size(); ++i) {
            const int L = L_vec[i];
            if (k > L) {
                std::cout << "L must greater or equal than k" << std::endl;
                return 1;
            }
            Test_Result tr = index.Search(query_data, (int)qm.n, L, res.data());
            const float time = tr.get_time(), qps = (float)qm.n / time;
            const int nq = std::min<int>((int)qm.n, gt.nq);
            const float recall = ComputeRecall(nq, k, gt.k, res.data(), gt.ids.data());
            const float avg_hops = tr.avg_hops((int)qm.n);
            std::cout << L << "\t\t" << qps << "\t\t" << time << "\t\t" << recall << "\t\t" << avg_hops << std::endl;
            if (csv.is_open()) csv << L << "," << qps << "," << time << "," << recall << "," << avg_hops << std::endl;
            if (opt.count("verify")) {   // src/index_gpu.cpp:89-115: search + hit count on the device
                if (gt.k != k) throw std::runtime_error("--verify needs a ground truth exactly k wide");
                const Test_Result tv = index.Search_and_Verify(query_data, gt.ids.data(), nq, L);
                std::cout << "hits " << tv.hits << std::endl;
            }
            if (max_recall > 0.5 && recall < max_recall) L_vec.push_back(128 + L_vec.back());  // :308-310
            if (i > 50) break;
        }
        if (has("ids_out")) {
            std::ofstream out(str("ids_out", ""), std::ios::binary);
            out.write(reinterpret_cast<const char*>(res.data()), (std::streamsize)(res.size() * sizeof(int)));
        }
        std::free(query_data);
    } catch (const std::exception& ex) {
        std::cerr << ex.what() << '\n';
        return -1;
    }
    return 0;
}
