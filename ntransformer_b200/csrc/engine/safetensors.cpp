// safetensors.cpp — see safetensors.h.
#include "safetensors.h"
#include "json.h"
#include <cstdio>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace nt { namespace b200 {

SafeTensorsFile::~SafeTensorsFile() { if (fd_ >= 0) close(fd_); }

bool SafeTensorsFile::open(const std::string& path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) { fprintf(stderr, "safetensors: cannot open %s\n", path.c_str()); return false; }
    struct stat st;
    if (fstat(fd_, &st) != 0 || st.st_size < 8) { fprintf(stderr, "safetensors: %s is too short\n", path.c_str()); return false; }
    size_ = (size_t)st.st_size;
    unsigned char lenb[8];
    if (pread(fd_, lenb, 8, 0) != 8) return false;
    uint64_t hlen = 0;
    for (int i = 7; i >= 0; i--) hlen = (hlen << 8) | lenb[i];
    if (hlen > size_ - 8 || hlen > ((uint64_t)1 << 30)) { fprintf(stderr, "safetensors: header length %llu exceeds the file\n", (unsigned long long)hlen); return false; }
    std::string header((size_t)hlen, '\0');
    size_t got = 0;
    while (got < header.size()) {
        ssize_t n = pread(fd_, &header[got], header.size() - got, (off_t)(8 + got));
        if (n <= 0) { fprintf(stderr, "safetensors: short read of the header\n"); return false; }
        got += (size_t)n;
    }
    data_offset_ = 8 + (size_t)hlen;
    Json root;
    std::string err;
    if (!Json::parse(header, root, &err) || !root.is_object()) { fprintf(stderr, "safetensors: %s\n", err.c_str()); return false; }
    for (const auto& kv : root.obj) {
        if (kv.first == "__metadata__") continue;
        const Json& t = kv.second;
        SafeTensorInfo ti;
        ti.name = kv.first;
        const std::string dt = t.at("dtype").string_or("");
        if (dt == "F32") ti.dtype = DType::F32; else if (dt == "F16") ti.dtype = DType::F16; else if (dt == "BF16") ti.dtype = DType::BF16;
        else if (dt == "I32") ti.dtype = DType::I32;
        else { fprintf(stderr, "safetensors: tensor %s has unsupported dtype %s\n", ti.name.c_str(), dt.c_str()); return false; }
        int64_t count = 1;
        for (const Json& d : t.at("shape").arr) { ti.shape.push_back((int64_t)d.int_or(0)); count *= ti.shape.back(); }
        const Json& off = t.at("data_offsets");
        if (!off.is_array() || off.arr.size() != 2) { fprintf(stderr, "safetensors: tensor %s has no data_offsets\n", ti.name.c_str()); return false; }
        ti.begin = (uint64_t)off.arr[0].int_or(0); ti.end = (uint64_t)off.arr[1].int_or(0);
        if (ti.end < ti.begin || data_offset_ + ti.end > size_ || count < 0 || (uint64_t)count * dtype_size(ti.dtype) != ti.end - ti.begin) {
            fprintf(stderr, "safetensors: tensor %s: byte range does not match its shape or the file\n", ti.name.c_str());
            return false;
        }
        index_[ti.name] = tensors_.size();
        tensors_.push_back(std::move(ti));
    }
    return true;
}

const SafeTensorInfo* SafeTensorsFile::find(const std::string& name) const {
    auto it = index_.find(name);
    return it == index_.end() ? nullptr : &tensors_[it->second];
}

bool SafeTensorsFile::read(const SafeTensorInfo& t, void* dst) const {
    size_t got = 0, bytes = (size_t)(t.end - t.begin);
    while (got < bytes) {
        ssize_t n = pread(fd_, static_cast<char*>(dst) + got, bytes - got, (off_t)(data_offset_ + t.begin + got));
        if (n <= 0) return false;
        got += (size_t)n;
    }
    return true;
}

}}  // namespace nt::b200
