#include "bin_file.h"

#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace cccc
{

static const char kMagic[] = "CFG_BIN INI";

bool BinFile::open(const std::string& path)
{
    close();
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) { return false; }
    struct stat st;
    if (fstat(fd_, &st) != 0)
    {
        close();
        return false;
    }
    file_size_ = (uint64_t)st.st_size;
    unsigned char head[40];
    if (file_size_ < sizeof(head) || pread(fd_, head, sizeof(head), 0) != (ssize_t)sizeof(head)
        || std::memcmp(head, kMagic, sizeof(kMagic) - 1) != 0)
    {
        close();
        return false;
    }
    uint64_t index_len = 0;
    std::memcpy(&index_len, head + 32, 8);
    if (index_len > file_size_ - 40)
    {
        close();
        return false;
    }
    std::string index(index_len, '\0');
    if (index_len && pread(fd_, &index[0], index_len, 40) != (ssize_t)index_len)
    {
        close();
        return false;
    }
    data_base_ = 40 + index_len;
    size_t pos = 0;
    while (pos < index.size())
    {
        size_t eol = index.find('\n', pos);
        if (eol == std::string::npos) { eol = index.size(); }
        const std::string line = index.substr(pos, eol - pos);
        pos = eol + 1;
        if (line.empty()) { continue; }
        const size_t eq = line.find(" = ");
        const size_t comma = line.rfind(',');
        if (eq == std::string::npos || comma == std::string::npos || comma < eq)
        {
            close();
            return false;
        }
        BinEntry e;
        char* endp = nullptr;
        e.offset = std::strtoull(line.c_str() + eq + 3, &endp, 10);
        if (endp != line.c_str() + comma)
        {
            close();
            return false;
        }
        e.length = std::strtoull(line.c_str() + comma + 1, &endp, 10);
        if (*endp != '\0' || e.offset > file_size_ - data_base_ || e.length > file_size_ - data_base_ - e.offset)
        {
            close();
            return false;    // an entry that points past the end of the file: truncated container
        }
        entries_[line.substr(0, eq)] = e;
    }
    return true;
}

void BinFile::close()
{
    if (fd_ >= 0) { ::close(fd_); }
    fd_ = -1;
    entries_.clear();
    data_base_ = file_size_ = 0;
}

BinEntry BinFile::entry(const std::string& key) const
{
    auto it = entries_.find(key);
    return it == entries_.end() ? BinEntry() : it->second;
}

bool BinFile::read(const std::string& key, uint64_t off, uint64_t len, void* dst) const
{
    auto it = entries_.find(key);
    if (it == entries_.end() || off > it->second.length || len > it->second.length - off) { return false; }
    uint64_t done = 0;
    while (done < len)
    {
        const ssize_t r = pread(fd_, (char*)dst + done, len - done, (off_t)(data_base_ + it->second.offset + off + done));
        if (r <= 0) { return false; }
        done += (uint64_t)r;
    }
    bytes_read_ += len;
    return true;
}

std::string BinFile::text(const std::string& key) const
{
    const BinEntry e = entry(key);
    std::string s(e.length, '\0');
    if (e.length && !read(key, 0, e.length, &s[0])) { return std::string(); }
    return s;
}

bool BinFile::findTypedWeight(const std::string& name, std::string* key, DataType* dt) const
{
    static const std::pair<const char*, DataType> suffixes[] = {
        { "fp8_e4m3", FP8_E4M3 }, { "fp8e4m3", FP8_E4M3 }, { "fp8", FP8_E4M3 }, { "bf16", BFLOAT16 }, { "bfloat16", BFLOAT16 },
        { "float", FLOAT }, { "half", HALF }, { "fp8_e5m2", FP8_E5M2 }, { "fp4_e2m1", FP4_E2M1 },
    };
    for (auto& s : suffixes)
    {
        const std::string k = std::string("weight_") + s.first + "_" + name;
        if (has(k))
        {
            *key = k;
            *dt = s.second;
            return true;
        }
    }
    return false;
}

void BinWriter::add(const std::string& key, const void* data, size_t len)
{
    entries_.emplace_back(key, std::vector<uint8_t>((const uint8_t*)data, (const uint8_t*)data + len));
}

void BinWriter::addQuantised(const std::string& name, const WeightShard& shard)
{
    const char* suffix = shard.dtype == FP8_E4M3 ? "fp8_e4m3" : shard.dtype == FP8_E5M2 ? "fp8_e5m2" : "fp4_e2m1";
    add(std::string("weight_") + suffix + "_" + name, shard.weights.data(), shard.weights.size());
    if (shard.dtype != FP4_E2M1) { add("scale_" + name, &shard.quant_scale, sizeof(float)); }
    if (!shard.block_scales.empty()) { add("blockscale_" + name, shard.block_scales.data(), shard.block_scales.size()); }
}

bool BinWriter::save(const std::string& path) const
{
    std::string index;
    uint64_t off = 0;
    for (auto& e : entries_)
    {
        index += e.first + " = " + std::to_string(off) + "," + std::to_string(e.second.size()) + "\n";
        off += e.second.size();
    }
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) { return false; }
    unsigned char head[32] = { 0 };
    std::memcpy(head, kMagic, sizeof(kMagic) - 1);
    const uint64_t n = index.size();
    bool ok = std::fwrite(head, 1, 32, f) == 32 && std::fwrite(&n, 8, 1, f) == 1 && std::fwrite(index.data(), 1, n, f) == n;
    for (auto& e : entries_) { ok = ok && std::fwrite(e.second.data(), 1, e.second.size(), f) == e.second.size(); }
    return std::fclose(f) == 0 && ok;
}

uint8_t floatToE4M3Trunc(float f)
{
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) { return 0x7Fu; }
    const uint32_t s = u >> 31;
    const int fe = (int)((u >> 23) & 0xFFu) - 127;
    const uint32_t fm = u & 0x7FFFFFu;
    if (fe > 8 || (fe == 8 && fm >= 0xC00000u)) { return (uint8_t)((s << 7) | 0x7Eu); }
    const int e8 = fe + 7;
    if (e8 <= 0)
    {
        const int shift = 14 - fe;
        if (shift >= 32) { return (uint8_t)(s << 7); }
        return (uint8_t)((s << 7) | (((fm | 0x800000u) >> shift) & 0x7u));
    }
    uint32_t m8 = fm >> 20;
    if (e8 == 15 && m8 == 7u) { m8 = 6u; }
    return (uint8_t)((s << 7) | ((uint32_t)(e8 & 0xF) << 3) | m8);
}

bool loadWeightShard(const BinFile& f, const std::string& name, int N, int K, char kind, int world, int rank, WeightShard* out,
    std::string* err)
{
    auto fail = [&](const std::string& m) {
        if (err) { *err = m; }
        return false;
    };
    std::string key;
    DataType dt;
    if (!f.findTypedWeight(name, &key, &dt)) { return fail("weight '" + name + "' not found"); }
    if (world < 1 || rank < 0 || rank >= world) { return fail("bad rank"); }
    const uint64_t total = (uint64_t)N * (uint64_t)K;
    if (dt == BFLOAT16 || dt == HALF || dt == FLOAT)
    {
        // An unquantised tensor (the reference's BF16 / float checkpoints): the shard's raw elements, which the
        // caller quantises on the GPU (Net::quantizeWeights, cccc/Net.cpp:1142-1233).
        const uint64_t eb = dt == FLOAT ? 4 : 2;
        if (f.entry(key).length != total * eb) { return fail("weight '" + name + "' does not hold N*K elements"); }
        int n0 = 0, n1 = N, k0 = 0, k1 = K;
        if (kind == 'c')
        {
            if (N % world) { return fail("N does not divide over the ranks"); }
            n0 = rank * (N / world);
            n1 = n0 + N / world;
        }
        else if (kind == 'r')
        {
            if (K % (world * 256)) { return fail("K does not divide over the ranks in whole k steps"); }
            k0 = rank * (K / world);
            k1 = k0 + K / world;
        }
        else { return fail("kind must be 'c' or 'r'"); }
        out->dtype = dt;
        out->n = n1 - n0;
        out->k = k1 - k0;
        out->quant_scale = 1.0f;
        out->block_scales.clear();
        const uint64_t row_bytes = (uint64_t)out->k * eb;
        out->weights.resize((uint64_t)out->n * row_bytes);
        if (kind == 'c')
        {
            if (!f.read(key, (uint64_t)n0 * K * eb, out->weights.size(), out->weights.data())) { return fail("short read"); }
            return true;
        }
        for (int n = 0; n < N; n++)
        {
            if (!f.read(key, ((uint64_t)n * K + k0) * eb, row_bytes, out->weights.data() + (uint64_t)n * row_bytes)) { return fail("short read"); }
        }
        return true;
    }
    if (dt != FP8_E4M3 && dt != FP8_E5M2 && dt != FP4_E2M1) { return fail("weight '" + name + "' has a type this loader does not take"); }
    const uint64_t per = dt == FP4_E2M1 ? 2 : 1;    // elements per byte
    if (f.entry(key).length != total / per) { return fail("weight '" + name + "' does not hold N*K elements"); }
    const bool fp4 = dt == FP4_E2M1;
    const std::string skey = "blockscale_" + name;
    bool legacy_float_scales = false;
    if (fp4)
    {
        if (!f.has(skey)) { return fail("block scales of '" + name + "' not found"); }
        const uint64_t sl = f.entry(skey).length;
        if (sl == total / 16 * 4) { legacy_float_scales = true; }
        else if (sl != total / 16) { return fail("block scales of '" + name + "' do not hold N*K/16 entries"); }
    }
    int n0 = 0, n1 = N, k0 = 0, k1 = K;
    if (kind == 'c')
    {
        if (N % world) { return fail("N does not divide over the ranks"); }
        n0 = rank * (N / world);
        n1 = n0 + N / world;
    }
    else if (kind == 'r')
    {
        const int align = fp4 ? 256 : 64;
        if (K % (world * align)) { return fail("K does not divide over the ranks in whole k steps"); }
        k0 = rank * (K / world);
        k1 = k0 + K / world;
    }
    else { return fail("kind must be 'c' or 'r'"); }
    out->dtype = dt;
    out->n = n1 - n0;
    out->k = k1 - k0;
    out->quant_scale = 1.0f;
    if (f.has("scale_" + name) && f.entry("scale_" + name).length >= 4)
    {
        if (!f.read("scale_" + name, 0, 4, &out->quant_scale)) { return fail("cannot read the scale of '" + name + "'"); }
    }
    const uint64_t row_bytes = (uint64_t)out->k / per;
    out->weights.resize((uint64_t)out->n * row_bytes);
    const uint64_t srow = (uint64_t)out->k / 16;
    out->block_scales.assign(fp4 ? (uint64_t)out->n * srow : 0, 0);
    std::vector<float> tmp;
    auto read_scales = [&](uint64_t first_block, uint64_t count, uint8_t* dst) {
        if (!legacy_float_scales) { return f.read(skey, first_block, count, dst); }
        tmp.resize(count);
        if (!f.read(skey, first_block * 4, count * 4, tmp.data())) { return false; }
        for (uint64_t i = 0; i < count; i++) { dst[i] = floatToE4M3Trunc(tmp[i]); }
        return true;
    };
    if (kind == 'c')
    {
        // one contiguous range of the blob (and of its block scales)
        if (!f.read(key, (uint64_t)n0 * K / per, out->weights.size(), out->weights.data())) { return fail("short read"); }
        if (fp4 && !read_scales((uint64_t)n0 * K / 16, out->block_scales.size(), out->block_scales.data())) { return fail("short read"); }
        return true;
    }
    for (int n = 0; n < N; n++)
    {
        const uint64_t e = (uint64_t)n * K + k0;
        if (!f.read(key, e / per, row_bytes, out->weights.data() + (uint64_t)n * row_bytes)) { return fail("short read"); }
        if (fp4 && !read_scales(e / 16, srow, out->block_scales.data() + (uint64_t)n * srow)) { return fail("short read"); }
    }
    return true;
}

}    // namespace cccc
