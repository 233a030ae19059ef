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
// Multi-GPU (one host thread and one handle per GPU, devices 0..N-1):
//   --gpus N              the index is replicated and the batch split into N contiguous parts;
//   --shards G --seed S   the base is split into G shards by a seeded balanced random partition,
//                         one graph per shard under <graph_path>/shard<g> (built from
//                         --train_path FILE with IndexGPU::BuildGPU when the directory is missing),
//                         every shard searches every query and the per-shard top-k are merged
//                         through one NCCL all-gather (coral_search_sharded).
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <numeric>
#include <random>
#include <string>
#include <sys/stat.h>
#include <thread>
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

// Balanced random partition of n ids into G shards: shard_of[id], seeded.
static std::vector<int> random_partition(size_t n, int G, unsigned seed) {
    std::vector<size_t> perm(n);
    std::iota(perm.begin(), perm.end(), (size_t)0);
    std::mt19937_64 gen(seed);
    std::shuffle(perm.begin(), perm.end(), gen);
    std::vector<int> shard_of(n);
    for (size_t i = 0; i < n; ++i) shard_of[perm[i]] = (int)(i * (size_t)G / n);
    return shard_of;
}

static bool dir_exists(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}

// --shards: returns 0 on success.  Prints the same table as the single-GPU sweep.
static int run_sharded(int G, unsigned seed, const std::string& dist, int k, int max_degree, const std::string& graph_dir,
                       const std::string& base_path, const std::string& train_path, const std::string& config_file,
                       const float* query_data, const coral_host::FbinMeta& qm, const coral_host::GroundTruth& gt,
                       const std::vector<int>& L_vec) {
    coral_host::FbinMeta bm;
    float* base = coral_host::fbin_load(base_path, bm);
    if (dist == "ip") coral_host::normalize_rows(base, bm.n, (size_t)bm.dim);
    const std::vector<int> shard_of = random_partition(bm.n, G, seed);
    std::vector<std::vector<int32_t>> ids_of((size_t)G);
    for (size_t i = 0; i < bm.n; ++i) ids_of[(size_t)shard_of[i]].push_back((int32_t)i);
    std::vector<std::vector<float>> vecs((size_t)G);
    for (int g = 0; g < G; ++g) {
        vecs[(size_t)g].resize(ids_of[(size_t)g].size() * (size_t)bm.dim);
        for (size_t r = 0; r < ids_of[(size_t)g].size(); ++r)
            std::memcpy(&vecs[(size_t)g][r * (size_t)bm.dim], base + (size_t)ids_of[(size_t)g][r] * bm.dim, (size_t)bm.dim * 4);
    }
    std::free(base);
    coral_host::FbinMeta tm;
    float* train = nullptr;
    std::vector<IndexGPU*> shards((size_t)G, nullptr);
    for (int g = 0; g < G; ++g) {
        Parameters p;
        p.Set<std::string>("dist", dist);
        p.Set<int>("k", 100);
        p.Set<int>("max_degree", max_degree);
        p.Set<int>("CE", 1);
        const std::string dir = graph_dir + "/shard" + std::to_string(g);
        p.Set<std::string>("graph_file", dir);
        p.Set<std::string>("config_file", config_file);
        IndexGPU* ix = new IndexGPU((size_t)bm.dim, ids_of[(size_t)g].size(), dist == "l2" ? efanna2e::L2 : efanna2e::INNER_PRODUCT, nullptr);
        ix->SetDevice(g);
        if (dir_exists(dir)) {
            p.Set<int>("k", k);
            ix->RunPrepare(p, Mode::SEARCH, ids_of[(size_t)g].size(), vecs[(size_t)g].data());
        } else {
            if (train_path.empty()) throw std::runtime_error("no graph under " + dir + " and no --train_path to build it from");
            if (!train) {
                train = coral_host::fbin_load(train_path, tm);
                if (dist == "ip") coral_host::normalize_rows(train, tm.n, (size_t)tm.dim);
            }
            std::cout << "Build shard " << g << ": " << ids_of[(size_t)g].size() << " points" << std::endl;
            ix->BuildGPU(tm.n, train, ids_of[(size_t)g].size(), vecs[(size_t)g].data(), p);
        }
        shards[(size_t)g] = ix;
    }
    std::free(train);
    std::vector<int> devices((size_t)G);
    std::iota(devices.begin(), devices.end(), 0);
    std::vector<coral_comm_t*> comms((size_t)G, nullptr);
    if (coral_comm_create_all(comms.data(), devices.data(), G) != CORAL_OK)
        throw std::runtime_error(std::string("coral_comm_create_all: ") + coral_comm_last_error(nullptr));
    for (int g = 0; g < G; ++g)
        if (coral_comm_set_id_map(comms[(size_t)g], ids_of[(size_t)g].data(), (int64_t)ids_of[(size_t)g].size()) != CORAL_OK)
            throw std::runtime_error(std::string("coral_comm_set_id_map: ") + coral_comm_last_error(comms[(size_t)g]));
    std::vector<int> res(qm.n * (size_t)k, -1);
    const int Q = (int)qm.n;
    std::cout << "L\t\tQPS\t\tavg_time\t\trecall@" << k << std::endl;
    for (int L : L_vec) {
        for (int g = 0; g < G; ++g)
            if (coral_search_prepare(shards[(size_t)g]->handle(), Q, L, k) != CORAL_OK)
                throw std::runtime_error(std::string("coral_search_prepare: ") + coral_last_error(shards[(size_t)g]->handle()));
        double best = 0.0;
        for (int rep = 0; rep < 2; ++rep) {                  // the first pass also sizes the exchange buffers
            std::vector<std::string> errors((size_t)G);
            std::vector<std::thread> th;
            const auto t0 = std::chrono::steady_clock::now();
            for (int g = 0; g < G; ++g)
                th.emplace_back([&, g]() {
                    int lo = 0, hi = 0;
                    coral_query_slice(Q, G, g, &lo, &hi);
                    const int rc = coral_search_sharded(shards[(size_t)g]->handle(), comms[(size_t)g], nullptr, query_data, Q, L, k,
                                                        res.data() + (size_t)lo * k, nullptr, nullptr);
                    if (rc != CORAL_OK) errors[(size_t)g] = coral_comm_last_error(comms[(size_t)g]);
                });
            for (auto& t : th) t.join();
            best = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            for (const auto& e : errors)
                if (!e.empty()) throw std::runtime_error("coral_search_sharded: " + e);
        }
        const int nq = std::min<int>(Q, gt.nq);
        const float recall = ComputeRecall(nq, k, gt.k, res.data(), gt.ids.data());
        std::cout << L << "\t\t" << Q / best << "\t\t" << best << "\t\t" << recall << std::endl;
    }
    for (auto* c : comms) coral_comm_destroy(c);
    for (auto* ix : shards) delete ix;
    return 0;
}

// --gpus N: N replicas, the batch split into contiguous parts, one host thread per GPU.
static int run_replicated(int N, Parameters& parameters, const std::string& dist, int k, const std::string& base_path,
                          const float* query_data, const coral_host::FbinMeta& qm, const coral_host::GroundTruth& gt,
                          const std::vector<int>& L_vec) {
    std::vector<IndexGPU*> reps((size_t)N, nullptr);
    for (int g = 0; g < N; ++g) {
        reps[(size_t)g] = new IndexGPU((size_t)qm.dim, 0, dist == "l2" ? efanna2e::L2 : efanna2e::INNER_PRODUCT, nullptr);
        reps[(size_t)g]->SetDevice(g);
        reps[(size_t)g]->LoadSearchNeededData(base_path.c_str(), "", dist == "l2" ? DIST_METRIC::L2_ : DIST_METRIC::IP_);
        reps[(size_t)g]->RunPrepare(parameters, Mode::SEARCH);
    }
    const int Q = (int)qm.n;
    std::vector<int> res((size_t)Q * k, -1);
    std::cout << "L\t\tQPS\t\tavg_time\t\trecall@" << k << "\t\tavg_hops" << std::endl;
    for (int L : L_vec) {
        std::vector<float> secs((size_t)N, 0.f);
        std::vector<size_t> hops((size_t)N, 0);
        std::vector<std::string> errors((size_t)N);
        for (int rep = 0; rep < 2; ++rep) {                  // the first pass sizes the scratch
            std::vector<std::thread> th;
            for (int g = 0; g < N; ++g)
                th.emplace_back([&, g]() {
                    try {
                        int lo = 0, hi = 0;
                        coral_query_slice(Q, N, g, &lo, &hi);
                        const Test_Result tr = reps[(size_t)g]->Search(query_data + (size_t)lo * qm.dim, hi - lo, L,
                                                                       res.data() + (size_t)lo * k);
                        secs[(size_t)g] = tr.get_time();
                        hops[(size_t)g] = tr.get_hops();
                    } catch (const std::exception& ex) {
                        errors[(size_t)g] = ex.what();
                    }
                });
            for (auto& t : th) t.join();
            for (const auto& e : errors)
                if (!e.empty()) throw std::runtime_error(e);
        }
        const float time = *std::max_element(secs.begin(), secs.end());      // the slowest GPU's kernel window
        const size_t total_hops = std::accumulate(hops.begin(), hops.end(), (size_t)0);
        const int nq = std::min<int>(Q, gt.nq);
        const float recall = ComputeRecall(nq, k, gt.k, res.data(), gt.ids.data());
        std::cout << L << "\t\t" << Q / time << "\t\t" << time << "\t\t" << recall << "\t\t" << (float)total_hops / Q << std::endl;
    }
    for (auto* ix : reps) delete ix;
    return 0;
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

        if (L_vec.empty() && max_recall > 0.5) L_vec.push_back(128);   // :279-281
        const int n_shards = std::atoi(str("shards", "0").c_str()), n_gpus = std::atoi(str("gpus", "1").c_str());
        if (n_shards > 0) {
            for (int L : L_vec)
                if (k > L) {
                    std::cout << "L must greater or equal than k" << std::endl;
                    return 1;
                }
            const int rc = run_sharded(n_shards, (unsigned)std::atol(str("seed", "20260004").c_str()), dist, k, max_degree, graph_dir,
                                       str("base_data_path", ""), str("train_path", ""), str("config_file", ""), query_data, qm,
                                       gt, L_vec);
            std::free(query_data);
            return rc;
        }
        if (n_gpus > 1) {
            const int rc = run_replicated(n_gpus, parameters, dist, k, str("base_data_path", ""), query_data, qm, gt, L_vec);
            std::free(query_data);
            return rc;
        }

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
