// Stand-in for lz4.h (only the runtime library is installed here): declarations the reference's
// disk_graph.h needs to parse; the search path never calls them.
#pragma once
extern "C" {
int LZ4_compress_default(const char* src, char* dst, int srcSize, int dstCapacity);
int LZ4_decompress_safe(const char* src, char* dst, int compressedSize, int dstCapacity);
int LZ4_compressBound(int inputSize);
}
