// Ground-truth tool with the reference's command line (reference tests/comp_gt.cpp:48-176): the exact
// k nearest base points of every query, written as int32 nq, int32 k, nq x k int32 ids -- the file
// test_search_pipeline reads with --gt_path and test_build_pipeline with --train_gt_file.
// The reference runs a Faiss flat index; here the lists come from the library's exact search
// (tensor-core scan, exact fp32 re-rank, ties by id).
//
// Flags as in the reference: --data_type --dist --base_data_path --query_data_path --gt_save_file
// --k --nq (0 = every query of the file).  Inner product: base and queries are unit-normalised
// first, as the drivers do.  Addition: --device N.
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "../../include/coral_b200.h"
#include "formats.h"

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
        std::cout << "see the header of comp_gt.cpp for the flags\n";
        return 0;
    }
    for (const char* req : {"base_data_path", "query_data_path", "gt_save_file"})
        if (!has(req)) {
            std::cerr << "the option '--" << req << "' is required but missing\n";
            return -1;
        }
    const std::string dist = str("dist", "l2");
    const int k = std::atoi(str("k", "10").c_str());
    int nq = std::atoi(str("nq", "0").c_str());
    if (dist != "l2" && dist != "ip") {
        std::cout << "Unknown distance type: " << dist << std::endl;
        return -1;
    }
    coral_index_t* h = nullptr;
    float *base = nullptr, *queries = nullptr;
    int rc = 0;
    try {
        coral_host::FbinMeta bm, qm;
        base = coral_host::fbin_load(str("base_data_path", ""), bm);
        queries = coral_host::fbin_load(str("query_data_path", ""), qm);
        if (bm.dim != qm.dim) throw std::runtime_error("base and query dimension mismatch");
        if (nq <= 0 || (size_t)nq > qm.n) nq = (int)qm.n;
        if (k <= 0 || (size_t)k > bm.n) throw std::runtime_error("need 0 < k <= number of base points");
        if (dist == "ip") {
            coral_host::normalize_rows(base, bm.n, (size_t)bm.dim);
            coral_host::normalize_rows(queries, (size_t)nq, (size_t)qm.dim);
        }
        std::cout << "base " << bm.n << " x " << bm.dim << ", queries " << nq << ", k " << k << ", " << dist << std::endl;
        if (coral_index_create(&h, std::atoi(str("device", "0").c_str()), (int64_t)bm.n, bm.dim, 32,
                               dist == "l2" ? CORAL_L2 : CORAL_IP) != CORAL_OK)
            throw std::runtime_error(std::string("coral_index_create: ") + coral_last_error(nullptr));
        if (coral_index_set_vectors(h, base) != CORAL_OK) throw std::runtime_error(coral_last_error(h));
        std::vector<int32_t> ids((size_t)nq * k);
        int64_t uncertified = 0;
        if (coral_exact_knn(h, queries, nq, k, ids.data(), nullptr, &uncertified) != CORAL_OK)
            throw std::runtime_error(std::string("coral_exact_knn: ") + coral_last_error(h));
        coral_host::gt_write(str("gt_save_file", ""), ids.data(), nq, k);
        std::cout << "wrote " << str("gt_save_file", "") << " (" << coral_last_dense_flops(h) / (coral_last_dense_ms(h) * 1e9)
                  << " TFLOP/s of 3-pass tf32 arithmetic, " << uncertified << " lists not certified exact)" << std::endl;
    } catch (const std::exception& ex) {
        std::cerr << "error: " << ex.what() << std::endl;
        rc = 2;
    }
    if (h) coral_index_destroy(h);
    std::free(base);
    std::free(queries);
    return rc;
}
