// Readers (and the two writers used for interchange) of the file formats the
// reference's search path consumes.  Everything throws std::runtime_error with a
// message instead of exiting the process.
//
//   .fbin vectors        uint32 n, uint32 dim, float32[n][dim]
//                        (reference include/efanna2e/util.h:105-128, :183-218)
//   ground truth .bin    int32 nq, int32 k, int32[nq][k]
//                        (reference include/efanna2e/util.h:82-103, :160-180)
//   graph directory      graph.part<p>.idx / .data / .append, graph.search_start_ids
//                        (reference include/disk_graph.h:78-84, src/disk.cpp:22-37,
//                         :102-103, :336-378, src/graph.cpp:316-351)
//   flat graph           uint32 ep, uint32 npts, {uint32 deg, uint32 nbrs[deg]} x npts
//                        (reference src/graph.cu:709-743)
//   config.json          one flat JSON object of numbers (reference config.json)
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace coral_host {

struct FbinMeta {
    size_t n = 0;
    int dim = 0;
};

// Header of an .fbin file; throws when the file is shorter than its header claims.
FbinMeta fbin_meta(const std::string& path);
// All vectors, row-major, into a 64-byte aligned buffer the caller frees with free().
float* fbin_load(const std::string& path, FbinMeta& meta);
void fbin_write(const std::string& path, const float* data, size_t n, int dim);

struct GroundTruth {
    int nq = 0, k = 0;
    std::vector<int32_t> ids;  // [nq][k]
};
GroundTruth gt_load(const std::string& path);
void gt_write(const std::string& path, const int32_t* ids, int nq, int k);

// x[i] /= |x[i]| for every row with a non-zero norm (reference src/uni.cpp:38-54).
void normalize_rows(float* x, size_t n, size_t dim);

// Decodes one LZ4 block (the raw block format, no frame).  Returns the number of
// bytes written, or -1 when the input is malformed or does not fit `cap`.
int lz4_block_decode(const uint8_t* src, int src_len, uint8_t* dst, int cap);
// Encodes `src` as an LZ4 block made of literals only (valid for every decoder).
std::vector<uint8_t> lz4_block_store(const uint8_t* src, int len);

struct Adjacency {
    int64_t n = 0;
    int deg_pad = 0;            // 32, 64 or 128
    std::vector<int32_t> rows;  // [n][deg_pad], valid ids first, -1 padding
    double avg_degree = 0.0;
    int64_t isolated = 0;
};

int padded_degree(int max_degree);

// Reads every node's slot from a CORAL graph directory.  Degrees above
// max_degree are cut, like the reference's flat import does.
Adjacency graph_dir_load(const std::string& dir, int64_t n, int max_degree);
// Writes the same layout (one partition per 100M nodes, records in .data, LZ4
// blocks stored as literals) so that an index made here loads in the reference.
void graph_dir_write(const std::string& dir, const Adjacency& g, const std::vector<int32_t>& start_ids);

std::vector<int32_t> start_ids_load(const std::string& path);  // "M id0 id1 ..."
void start_ids_write(const std::string& path, const std::vector<int32_t>& ids);

// Flat graph: returns the adjacency and the entry point stored in the file.
Adjacency flat_graph_load(const std::string& path, int max_degree, int32_t& entry_point);
void flat_graph_write(const std::string& path, const Adjacency& g, int32_t entry_point);

// Flat JSON object of numbers -> map; unknown syntax throws.
std::map<std::string, double> config_load(const std::string& path);

}  // namespace coral_host
