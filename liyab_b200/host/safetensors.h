// Reading and writing the safetensors container.
//
// The format: eight bytes of little-endian header length, a JSON object mapping
// each tensor's name to {"dtype", "shape", "data_offsets": [begin, end)} (offsets
// relative to the end of the header), then the raw little-endian data.  The
// header is parsed and checked before any data is touched, as the reference
// describes a model from metadata and tensor shapes alone
// (src/compat/architecture.h:30-32) and rejects malformed files with the tensor
// named (src/core/transformer.cpp:1052-1072).  A model folder holds either
// `model.safetensors` or shards listed by `model.safetensors.index.json`
// ({"weight_map": {tensor: file}}).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "device.h"
#include "json.h"

namespace liyab {

struct TensorEntry {
    std::string name;
    DType dtype = DType::F32;
    std::vector<int64_t> shape;
    uint64_t begin = 0, end = 0;        // absolute byte offsets in the file
};

const char* safetensors_tag(DType t);                      // "F32", "BF16", ...
DType dtype_from_safetensors_tag(const std::string& tag, bool* known);

// A file opened for reading: header checked, data mapped on demand.
class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path);
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;

    const std::string& path() const { return path_; }
    const std::vector<TensorEntry>& entries() const { return entries_; }      // in header order
    const TensorEntry* find(const std::string& name) const;
    const Json& metadata() const { return metadata_; }
    const void* data(const TensorEntry& e);                                   // mapped bytes of the tensor

private:
    std::string path_;
    int fd_ = -1;
    uint64_t size_ = 0;
    void* map_ = nullptr;
    std::vector<TensorEntry> entries_;
    std::map<std::string, size_t> index_;
    Json metadata_ = Json::object();
};

// The tensors of a model folder, whichever way they are spread over files.
class ModelFiles {
public:
    explicit ModelFiles(const std::string& model_dir);
    std::string shown_path() const { return shown_; }
    std::vector<std::string> names() const;
    const TensorEntry* find(const std::string& name) const;
    const void* data(const std::string& name);

private:
    std::string shown_;
    std::vector<std::unique_ptr<SafetensorsFile>> files_;
    std::map<std::string, std::pair<size_t, const TensorEntry*>> index_;
};

struct TensorToWrite {
    std::string name;
    DType dtype = DType::F32;
    std::vector<int64_t> shape;
    const void* data = nullptr;
};
// Writes tensors in the order given; data starts 8-byte aligned.
void write_safetensors(const std::string& path, const std::vector<TensorToWrite>& tensors, const Json& metadata = Json::object());

}  // namespace liyab
