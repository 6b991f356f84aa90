// Reader/writer of cccc's weight container (the INIReaderBin format that
// scripts/convert_weights.py:54-83 writes and cccc/Net.cpp:1324-1527 loads): a 32-byte magic
// "CFG_BIN INI", a little-endian uint64 index length, a text index of "key = offset,length" lines,
// then the blobs.  Named weights are "weight_<dtype>_<name>" (suffixes of Net.cpp:222-248) with
// optional "scale_<name>" (one float32 dequant multiplier) and "blockscale_<name>" (E4M3 bytes, one
// per 16 elements; a legacy float32 form is re-encoded on load, Net.cpp:1466-1477).
//
// Unlike the reference, which reads whole blobs, a tensor-parallel rank reads ONLY the byte ranges of
// its shard: one range for a column shard, one run per output row for a row shard.
#pragma once

#include "cccc_host.h"

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace cccc
{

struct BinEntry
{
    uint64_t offset = 0;    // from the start of the blob area
    uint64_t length = 0;
};

class BinFile
{
public:
    BinFile() = default;
    ~BinFile() { close(); }
    BinFile(const BinFile&) = delete;
    BinFile& operator=(const BinFile&) = delete;

    bool open(const std::string& path);    // false: missing file, bad magic, truncated or malformed index
    void close();
    bool has(const std::string& key) const { return entries_.count(key) != 0; }
    BinEntry entry(const std::string& key) const;
    size_t size() const { return entries_.size(); }
    // Reads [off, off+len) of the blob `key` into dst; false if out of range or short read.
    bool read(const std::string& key, uint64_t off, uint64_t len, void* dst) const;
    std::string text(const std::string& key) const;    // small values such as "data_type"
    // The first "weight_<suffix>_<name>" present, in the reference's order of suffixes.
    bool findTypedWeight(const std::string& name, std::string* key, DataType* dt) const;
    uint64_t bytesRead() const { return bytes_read_; }

private:
    int fd_ = -1;
    uint64_t data_base_ = 0, file_size_ = 0;
    std::map<std::string, BinEntry> entries_;
    mutable uint64_t bytes_read_ = 0;
};

struct WeightShard;

class BinWriter
{
public:
    void add(const std::string& key, const void* data, size_t len);
    // A quantised tensor under the keys the loaders look up: "weight_<suffix>_<name>" (suffix of
    // cccc/Net.cpp:222-248 for the shard's type), "scale_<name>" (float32 dequant multiplier, FP8) and
    // "blockscale_<name>" (E4M3 bytes, FP4).
    void addQuantised(const std::string& name, const WeightShard& shard);
    bool save(const std::string& path) const;

private:
    std::vector<std::pair<std::string, std::vector<uint8_t>>> entries_;
};

// What a rank holds of one quantised linear after loading.
struct WeightShard
{
    DataType dtype = FLOAT;
    int n = 0, k = 0;                    // shard shape: n output features x k input features
    float quant_scale = 1.0f;            // per-tensor dequant multiplier, shared by all shards
    std::vector<uint8_t> weights;        // compact [n, k]
    std::vector<uint8_t> block_scales;   // FP4 only: compact [n, k/16] E4M3 bytes
};

// kind 'c': column-parallel (split the N output features), 'r': row-parallel (split K).
// Returns false with *err set when the tensor is missing, the sizes do not match N*K, or the split
// is not allowed (N % world, or K not a multiple of world * 64 (FP8) / world * 256 (FP4)).
bool loadWeightShard(const BinFile& f, const std::string& name, int N, int K, char kind, int world, int rank, WeightShard* out,
    std::string* err);

// Truncating float -> E4M3 of the reference's host codec (cccc/types.h:92-126).
uint8_t floatToE4M3Trunc(float f);

}    // namespace cccc
