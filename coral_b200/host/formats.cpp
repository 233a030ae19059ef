#include "formats.h"

#include <sys/stat.h>

#include <algorithm>
#include <cctype>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

namespace coral_host {

namespace {

constexpr int64_t kNodesPerPartition = 100000000;  // reference CPU_N, include/uni.h:71

[[noreturn]] void die(const std::string& what) { throw std::runtime_error(what); }

size_t file_size(const std::string& path) {
    struct stat st;
    if (stat(path.c_str(), &st) != 0) die("cannot stat " + path);
    return (size_t)st.st_size;
}

struct File {
    FILE* f = nullptr;
    File(const std::string& path, const char* mode) : f(std::fopen(path.c_str(), mode)) {
        if (!f) die("cannot open " + path);
    }
    ~File() {
        if (f) std::fclose(f);
    }
    void read(void* dst, size_t bytes, const std::string& what) {
        if (bytes && std::fread(dst, 1, bytes, f) != bytes) die("short read: " + what);
    }
    void write(const void* src, size_t bytes) {
        if (bytes && std::fwrite(src, 1, bytes, f) != bytes) die("short write");
    }
};

#pragma pack(push, 1)
struct IdxEntry {  // reference NodeDiskIndex, include/disk_graph.h:78-84
    uint64_t offset;
    uint32_t size;
    int32_t pos;  // 0 = .data, 1 = .append
};
#pragma pack(pop)
static_assert(sizeof(IdxEntry) == 16, "index entry is 16 bytes on disk");

void append_row(Adjacency& g, int64_t node, const int32_t* nbrs, int deg, int max_degree) {
    int32_t* row = g.rows.data() + (size_t)node * g.deg_pad;
    int w = 0;
    for (int j = 0; j < deg && w < max_degree; ++j)
        if (nbrs[j] >= 0 && (int64_t)nbrs[j] < g.n) row[w++] = nbrs[j];
    g.avg_degree += w;
    if (w == 0) ++g.isolated;
}

Adjacency empty_graph(int64_t n, int max_degree) {
    Adjacency g;
    g.n = n;
    g.deg_pad = padded_degree(max_degree);
    g.rows.assign((size_t)n * g.deg_pad, -1);
    return g;
}

}  // namespace

int padded_degree(int max_degree) { return max_degree <= 32 ? 32 : (max_degree <= 64 ? 64 : 128); }

// ------------------------------------------------------------------ vectors

FbinMeta fbin_meta(const std::string& path) {
    File f(path, "rb");
    int32_t n = 0, dim = 0;
    f.read(&n, 4, path);
    f.read(&dim, 4, path);
    if (n < 0 || dim <= 0) die("bad .fbin header in " + path);
    const size_t have = (file_size(path) - 8) / (size_t)dim / sizeof(float);
    if ((size_t)n > have) die("Data file size wrong! " + path);  // util.h:121-125
    FbinMeta m;
    m.n = (size_t)n;
    m.dim = dim;
    return m;
}

float* fbin_load(const std::string& path, FbinMeta& meta) {
    meta = fbin_meta(path);
    const size_t count = meta.n * (size_t)meta.dim;
    void* p = nullptr;
    if (posix_memalign(&p, 64, std::max<size_t>(count * sizeof(float), 64)) != 0) die("out of memory loading " + path);
    File f(path, "rb");
    std::fseek(f.f, 8, SEEK_SET);
    if (count && std::fread(p, sizeof(float), count, f.f) != count) {
        std::free(p);
        die("Data file size wrong! " + path);  // util.h:211-214
    }
    return static_cast<float*>(p);
}

void fbin_write(const std::string& path, const float* data, size_t n, int dim) {
    File f(path, "wb");
    const int32_t hdr[2] = {(int32_t)n, dim};
    f.write(hdr, 8);
    f.write(data, n * (size_t)dim * sizeof(float));
}

GroundTruth gt_load(const std::string& path) {
    File f(path, "rb");
    GroundTruth g;
    f.read(&g.nq, 4, path);
    f.read(&g.k, 4, path);
    if (g.nq < 0 || g.k <= 0) die("bad ground-truth header in " + path);
    g.ids.resize((size_t)g.nq * g.k);
    f.read(g.ids.data(), g.ids.size() * 4, path);  // the reference ignores trailing distances
    return g;
}

void gt_write(const std::string& path, const int32_t* ids, int nq, int k) {
    File f(path, "wb");
    const int32_t hdr[2] = {nq, k};
    f.write(hdr, 8);
    f.write(ids, (size_t)nq * k * 4);
}

void normalize_rows(float* x, size_t n, size_t dim) {
#pragma omp parallel for
    for (long long i = 0; i < (long long)n; ++i) {
        float* row = x + (size_t)i * dim;
        float norm2 = 0.0f;
        for (size_t j = 0; j < dim; ++j) norm2 += row[j] * row[j];
        const float norm = std::sqrt(norm2);
        if (norm > 0.0f) {
            const float inv = 1.0f / norm;
            for (size_t j = 0; j < dim; ++j) row[j] *= inv;
        }
    }
}

// ------------------------------------------------------------------ LZ4 block format

int lz4_block_decode(const uint8_t* src, int src_len, uint8_t* dst, int cap) {
    int ip = 0, op = 0;
    while (ip < src_len) {
        const unsigned token = src[ip++];
        int lit = (int)(token >> 4);
        if (lit == 15) {
            for (;;) {
                if (ip >= src_len) return -1;
                const int b = src[ip++];
                lit += b;
                if (b != 255) break;
            }
        }
        if (lit > src_len - ip || lit > cap - op) return -1;
        std::memcpy(dst + op, src + ip, (size_t)lit);
        ip += lit;
        op += lit;
        if (ip >= src_len) break;  // the last sequence has literals only
        if (src_len - ip < 2) return -1;
        const int offset = src[ip] | (src[ip + 1] << 8);
        ip += 2;
        if (offset == 0 || offset > op) return -1;
        int mlen = (int)(token & 15u);
        if (mlen == 15) {
            for (;;) {
                if (ip >= src_len) return -1;
                const int b = src[ip++];
                mlen += b;
                if (b != 255) break;
            }
        }
        mlen += 4;
        if (mlen > cap - op) return -1;
        for (int i = 0; i < mlen; ++i, ++op) dst[op] = dst[op - offset];  // may overlap by design
    }
    return op;
}

std::vector<uint8_t> lz4_block_store(const uint8_t* src, int len) {
    std::vector<uint8_t> out;
    out.reserve((size_t)len + len / 255 + 16);
    if (len < 15) {
        out.push_back((uint8_t)(len << 4));
    } else {
        out.push_back(0xF0);
        int rest = len - 15;
        while (rest >= 255) {
            out.push_back(255);
            rest -= 255;
        }
        out.push_back((uint8_t)rest);
    }
    out.insert(out.end(), src, src + len);
    return out;
}

// ------------------------------------------------------------------ graph directory

std::vector<int32_t> start_ids_load(const std::string& path) {
    std::ifstream in(path);
    std::vector<int32_t> ids;
    if (!in.is_open()) return ids;  // the reference only logs this (src/graph.cpp:332-335)
    int m = -1;
    in >> m;
    for (int i = 0; i < m; ++i) {
        long long v;
        if (!(in >> v)) return {};  // a truncated list is dropped as a whole (:341-345)
        ids.push_back((int32_t)v);
    }
    return ids;
}

void start_ids_write(const std::string& path, const std::vector<int32_t>& ids) {
    std::ofstream out(path);
    if (!out.is_open()) die("cannot write " + path);
    out << ids.size() << " ";
    for (int32_t v : ids) out << v << " ";
}

Adjacency graph_dir_load(const std::string& dir, int64_t n, int max_degree) {
    if (n <= 0) die("graph_dir_load: n must be positive");
    Adjacency g = empty_graph(n, max_degree);
    const int64_t parts = (n + kNodesPerPartition - 1) / kNodesPerPartition;  // src/disk.cpp:102-103
    const int64_t per_part = (n + parts - 1) / parts;
    std::vector<uint8_t> comp, raw;
    for (int64_t p = 0; p < parts; ++p) {
        const int64_t first = p * per_part, count = std::min(per_part, n - first);
        const std::string stem = dir + "/graph.part" + std::to_string(p);
        std::vector<IdxEntry> idx((size_t)count);
        {
            const size_t have = file_size(stem + ".idx");
            if (have < (size_t)count * sizeof(IdxEntry)) die("index table too short: " + stem + ".idx");
            File f(stem + ".idx", "rb");
            f.read(idx.data(), (size_t)count * sizeof(IdxEntry), stem + ".idx");
        }
        FILE* files[2] = {std::fopen((stem + ".data").c_str(), "rb"), std::fopen((stem + ".append").c_str(), "rb")};
        auto close_all = [&]() {
            for (FILE* f : files)
                if (f) std::fclose(f);
        };
        try {
            for (int64_t i = 0; i < count; ++i) {
                const IdxEntry& e = idx[(size_t)i];
                const int64_t node = first + i;
                if (e.size == 0) {  // no record: degree 0 (src/disk.cpp:342-346)
                    ++g.isolated;
                    continue;
                }
                if (e.size < 8) die("corrupted block for node " + std::to_string(node));
                FILE* f = files[e.pos == 1 ? 1 : 0];
                if (!f) die("missing data file for node " + std::to_string(node));
                comp.resize(e.size);
                if (fseeko(f, (off_t)e.offset, SEEK_SET) != 0 || std::fread(comp.data(), 1, e.size, f) != e.size)
                    die("read block fail node " + std::to_string(node));
                int32_t raw_size = 0;
                std::memcpy(&raw_size, comp.data() + 4, 4);  // [node_id][raw_size][LZ4 block]
                if (raw_size < 4 || raw_size > 4 + 8 * 4096) die("bad record size for node " + std::to_string(node));
                raw.resize((size_t)raw_size);
                const int clen = (int)e.size - 8;
                int got = clen > 0 ? lz4_block_decode(comp.data() + 8, clen, raw.data(), raw_size) : -1;
                if (got != raw_size) {
                    // the reference stores the record uncompressed when LZ4 refuses it (src/disk.cpp:410-412)
                    if (clen == raw_size)
                        std::memcpy(raw.data(), comp.data() + 8, (size_t)raw_size);
                    else
                        die("LZ4 decompress failed node " + std::to_string(node));
                }
                int32_t deg = 0;
                std::memcpy(&deg, raw.data(), 4);  // [deg][nbrs[deg]][dists[deg]] (src/disk.cpp:22-37)
                if (deg < 0 || 4 + 8 * (int64_t)deg > raw_size) die("bad degree for node " + std::to_string(node));
                append_row(g, node, reinterpret_cast<const int32_t*>(raw.data() + 4), deg, max_degree);
            }
        } catch (...) {
            close_all();
            throw;
        }
        close_all();
    }
    g.avg_degree /= (double)n;
    return g;
}

void graph_dir_write(const std::string& dir, const Adjacency& g, const std::vector<int32_t>& start_ids) {
    mkdir(dir.c_str(), 0755);
    const int64_t parts = (g.n + kNodesPerPartition - 1) / kNodesPerPartition;
    const int64_t per_part = (g.n + parts - 1) / parts;
    for (int64_t p = 0; p < parts; ++p) {
        const int64_t first = p * per_part, count = std::min(per_part, g.n - first);
        const std::string stem = dir + "/graph.part" + std::to_string(p);
        std::vector<IdxEntry> idx((size_t)count);
        File data(stem + ".data", "wb");
        File append(stem + ".append", "wb");
        uint64_t off = 0;
        std::vector<uint8_t> raw;
        for (int64_t i = 0; i < count; ++i) {
            const int32_t* row = g.rows.data() + (size_t)(first + i) * g.deg_pad;
            int32_t deg = 0;
            while (deg < g.deg_pad && row[deg] >= 0) ++deg;
            if (deg == 0) {
                idx[(size_t)i] = IdxEntry{0, 0, 0};
                continue;
            }
            raw.assign(4 + 8 * (size_t)deg, 0);  // distances are not kept by the search path: zeros
            std::memcpy(raw.data(), &deg, 4);
            std::memcpy(raw.data() + 4, row, 4 * (size_t)deg);
            const std::vector<uint8_t> block = lz4_block_store(raw.data(), (int)raw.size());
            const int32_t node = (int32_t)(first + i), raw_size = (int32_t)raw.size();
            data.write(&node, 4);
            data.write(&raw_size, 4);
            data.write(block.data(), block.size());
            idx[(size_t)i] = IdxEntry{off, (uint32_t)(8 + block.size()), 0};
            off += 8 + block.size();
        }
        File f(stem + ".idx", "wb");
        f.write(idx.data(), idx.size() * sizeof(IdxEntry));
    }
    start_ids_write(dir + "/graph.search_start_ids", start_ids);
}

// ------------------------------------------------------------------ flat graph

Adjacency flat_graph_load(const std::string& path, int max_degree, int32_t& entry_point) {
    File f(path, "rb");
    uint32_t ep = 0, npts = 0;
    f.read(&ep, 4, path);
    f.read(&npts, 4, path);
    if (npts == 0) die("empty flat graph " + path);
    Adjacency g = empty_graph(npts, max_degree);
    std::vector<uint32_t> nbrs;
    for (uint32_t i = 0; i < npts; ++i) {
        uint32_t deg = 0;
        f.read(&deg, 4, path);
        if (deg > (1u << 20)) die("implausible degree in " + path);
        nbrs.resize(deg);
        f.read(nbrs.data(), 4 * (size_t)deg, path);
        append_row(g, i, reinterpret_cast<const int32_t*>(nbrs.data()), (int)deg, max_degree);  // cut at max_degree (:723-727)
    }
    g.avg_degree /= (double)npts;
    entry_point = (int32_t)ep;
    return g;
}

void flat_graph_write(const std::string& path, const Adjacency& g, int32_t entry_point) {
    File f(path, "wb");
    const uint32_t hdr[2] = {(uint32_t)entry_point, (uint32_t)g.n};
    f.write(hdr, 8);
    for (int64_t i = 0; i < g.n; ++i) {
        const int32_t* row = g.rows.data() + (size_t)i * g.deg_pad;
        uint32_t deg = 0;
        while ((int)deg < g.deg_pad && row[deg] >= 0) ++deg;
        f.write(&deg, 4);
        f.write(row, 4 * (size_t)deg);
    }
}

// ------------------------------------------------------------------ config.json

std::map<std::string, double> config_load(const std::string& path) {
    std::ifstream in(path);
    if (!in.is_open()) die("Cannot open config file " + path);
    std::stringstream ss;
    ss << in.rdbuf();
    const std::string s = ss.str();
    std::map<std::string, double> out;
    size_t i = 0;
    auto skip = [&]() {
        while (i < s.size() && std::isspace((unsigned char)s[i])) ++i;
    };
    skip();
    if (i >= s.size() || s[i] != '{') die("config: expected '{' in " + path);
    ++i;
    for (;;) {
        skip();
        if (i < s.size() && s[i] == '}') break;
        if (i >= s.size() || s[i] != '"') die("config: expected a key in " + path);
        const size_t e = s.find('"', i + 1);
        if (e == std::string::npos) die("config: unterminated key in " + path);
        const std::string key = s.substr(i + 1, e - i - 1);
        i = e + 1;
        skip();
        if (i >= s.size() || s[i] != ':') die("config: expected ':' after " + key);
        ++i;
        skip();
        char* endp = nullptr;
        const double v = std::strtod(s.c_str() + i, &endp);
        if (endp == s.c_str() + i) die("config: value of " + key + " is not a number");
        i = (size_t)(endp - s.c_str());
        out[key] = v;
        skip();
        if (i < s.size() && s[i] == ',') ++i;
    }
    return out;
}

}  // namespace coral_host
