// safetensors.h — reader of a .safetensors checkpoint: an 8-byte little-endian header length, that many bytes of JSON
// (tensor name -> {dtype, shape, data_offsets}), then the raw row-major tensor data.  The file is opened for pread; nothing
// is mapped.  Dense dtypes only (F32, F16, BF16, I32): this is the loader of the layer-spec model families, the quantised
// GGUF families keep engine/gguf.h.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>
#include "../nt_types.h"

namespace nt { namespace b200 {

struct SafeTensorInfo {
    std::string name;
    DType dtype = DType::F32;
    std::vector<int64_t> shape;            // outermost first (row-major), as stored
    uint64_t begin = 0, end = 0;           // byte range inside the data section
    int64_t rows() const { return shape.size() >= 2 ? shape[0] : 1; }
    int64_t cols() const { int64_t c = 1; for (size_t d = shape.size() >= 2 ? 1 : 0; d < shape.size(); d++) c *= shape[d]; return c; }
};

class SafeTensorsFile {
public:
    SafeTensorsFile() = default;
    ~SafeTensorsFile();
    SafeTensorsFile(const SafeTensorsFile&) = delete;
    SafeTensorsFile& operator=(const SafeTensorsFile&) = delete;
    bool open(const std::string& path);                 // false (+ message on stderr) on a malformed or truncated file
    const SafeTensorInfo* find(const std::string& name) const;
    const std::vector<SafeTensorInfo>& tensors() const { return tensors_; }
    bool read(const SafeTensorInfo& t, void* dst) const;   // the tensor's bytes, host destination
    size_t data_offset() const { return data_offset_; }
    int fd() const { return fd_; }

private:
    int fd_ = -1;
    size_t size_ = 0, data_offset_ = 0;
    std::vector<SafeTensorInfo> tensors_;
    std::unordered_map<std::string, size_t> index_;
};

}}  // namespace nt::b200
