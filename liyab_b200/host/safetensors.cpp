#include "safetensors.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <fstream>

#include "arch.h"

namespace liyab {
namespace {
struct Tag { const char* tag; DType dtype; };
const Tag kTags[] = {{"F64", DType::F64}, {"F32", DType::F32}, {"F16", DType::F16}, {"BF16", DType::BF16}, {"I64", DType::I64},
                     {"I32", DType::I32}, {"I16", DType::I16}, {"I8", DType::I8},   {"U8", DType::U8},     {"BOOL", DType::Bool}};
}  // namespace

const char* safetensors_tag(DType t) {
    for (const auto& k : kTags)
        if (k.dtype == t) return k.tag;
    return "?";
}

DType dtype_from_safetensors_tag(const std::string& tag, bool* known) {
    for (const auto& k : kTags)
        if (tag == k.tag) { *known = true; return k.dtype; }
    *known = false;
    return DType::F32;
}

SafetensorsFile::SafetensorsFile(const std::string& path) : path_(path) {
    fd_ = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd_ < 0) throw make_error(Code::Io, "cannot open {}: {}", path, std::strerror(errno));
    struct stat st {};
    if (fstat(fd_, &st) != 0) { ::close(fd_); throw make_error(Code::Io, "cannot stat {}: {}", path, std::strerror(errno)); }
    size_ = static_cast<uint64_t>(st.st_size);
    try {
        if (size_ < 8) throw invalid_model("{}: file of {} bytes is too short for a safetensors header", path, size_);
        uint8_t len8[8];
        if (pread(fd_, len8, 8, 0) != 8) throw make_error(Code::Io, "cannot read {}", path);
        uint64_t hlen = 0;
        for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | len8[i];
        if (hlen < 2 || hlen > size_ - 8) throw invalid_model("{}: header length {} does not fit a file of {} bytes", path, hlen, size_);
        std::string text(hlen, '\0');
        if (pread(fd_, text.data(), hlen, 8) != static_cast<ssize_t>(hlen)) throw make_error(Code::Io, "cannot read the header of {}", path);
        Json header;
        try {
            header = Json::parse(text, path + ": header");
        } catch (const Error& e) {
            std::string msg = e.message();
            const auto twice = msg.find("appears twice");
            if (twice != std::string::npos) throw invalid_model("{}: tensor {}", path, msg.substr(msg.find('\'')));
            throw invalid_model("{}", msg);
        }
        if (!header.is_object()) throw invalid_model("{}: header is not a JSON object", path);
        const uint64_t base = 8 + hlen, data_size = size_ - base;
        struct Span { uint64_t b, e; std::string name; };
        std::vector<Span> spans;
        for (const auto& [name, info] : header.members()) {
            if (name == "__metadata__") {
                if (info.is_object()) metadata_ = info;
                continue;
            }
            TensorEntry t;
            t.name = name;
            std::string tag;
            int64_t b = 0, e = 0;
            try {
                tag = info.at("dtype").as_string();
                t.shape = info.at("shape").int_list();
                const auto& off = info.at("data_offsets").items();
                if (off.size() != 2) throw invalid_argument("offsets");
                b = off[0].as_int();
                e = off[1].as_int();
            } catch (const Error&) {
                throw invalid_model("{}: malformed header entry for tensor '{}'", path, name);
            }
            bool known = false;
            t.dtype = dtype_from_safetensors_tag(tag, &known);
            if (!known) throw invalid_model("{}: tensor '{}' has unsupported dtype {}", path, name, tag);
            int64_t count = 1;
            bool negative = false;
            for (const int64_t s : t.shape) { negative = negative || s < 0; count *= s; }
            const int64_t need = count * static_cast<int64_t>(dtype_size(t.dtype));
            if (negative || b < 0 || e < b || e - b != need)
                throw invalid_model("{}: tensor '{}' has the wrong size: shape {} of {} needs {} bytes, offsets give {}", path, name,
                                    shape_text(t.shape), tag, need, e - b);
            if (static_cast<uint64_t>(e) > data_size)
                throw invalid_model("{}: tensor '{}' ends at byte {} but the file holds {} bytes of data (truncated file)", path, name,
                                    e, data_size);
            t.begin = base + static_cast<uint64_t>(b);
            t.end = base + static_cast<uint64_t>(e);
            if (e > b) spans.push_back({static_cast<uint64_t>(b), static_cast<uint64_t>(e), name});
            index_[name] = entries_.size();
            entries_.push_back(std::move(t));
        }
        std::sort(spans.begin(), spans.end(), [](const Span& x, const Span& y) { return x.b < y.b; });
        for (size_t i = 1; i < spans.size(); ++i)
            if (spans[i].b < spans[i - 1].e)
                throw invalid_model("{}: tensors '{}' and '{}' overlap in the file", path, spans[i - 1].name, spans[i].name);
    } catch (...) {
        ::close(fd_);
        fd_ = -1;
        throw;
    }
}

SafetensorsFile::~SafetensorsFile() {
    if (map_ != nullptr) munmap(map_, size_);
    if (fd_ >= 0) ::close(fd_);
}

const TensorEntry* SafetensorsFile::find(const std::string& name) const {
    const auto it = index_.find(name);
    return it == index_.end() ? nullptr : &entries_[it->second];
}

const void* SafetensorsFile::data(const TensorEntry& e) {
    if (map_ == nullptr) {
        void* p = mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (p == MAP_FAILED) throw make_error(Code::Io, "cannot map {}: {}", path_, std::strerror(errno));
        map_ = p;
    }
    return static_cast<const char*>(map_) + e.begin;
}

ModelFiles::ModelFiles(const std::string& model_dir) {
    const std::string single = model_dir + "/model.safetensors", index = single + ".index.json";
    std::vector<std::string> paths;
    if (access(single.c_str(), F_OK) == 0 || access(index.c_str(), F_OK) != 0) {
        paths.push_back(single);
        shown_ = single;
    } else {
        shown_ = index;
        Json j;
        try {
            j = Json::parse(read_text_file(index), index);
        } catch (const Error& e) {
            if (e.code() == Code::Io) throw;
            throw invalid_model("{}", e.message());
        }
        const Json* map = j.find("weight_map");
        if (map == nullptr || !map->is_object()) throw invalid_model("{} has no weight_map", index);
        for (const auto& m : map->members()) {
            if (!m.second.is_string()) throw invalid_model("{}: weight_map entry '{}' is not a file name", index, m.first);
            const std::string p = model_dir + "/" + m.second.as_string();
            if (std::find(paths.begin(), paths.end(), p) == paths.end()) paths.push_back(p);
        }
        if (paths.empty()) throw invalid_model("{} lists no files", index);
    }
    for (const auto& p : paths) {
        files_.push_back(std::make_unique<SafetensorsFile>(p));
        for (const auto& e : files_.back()->entries()) {
            if (index_.count(e.name)) throw invalid_model("tensor '{}' appears in {} and in another shard", e.name, p);
            index_[e.name] = {files_.size() - 1, &e};
        }
    }
}

std::vector<std::string> ModelFiles::names() const {
    std::vector<std::string> out;
    for (const auto& kv : index_) out.push_back(kv.first);
    return out;
}

const TensorEntry* ModelFiles::find(const std::string& name) const {
    const auto it = index_.find(name);
    return it == index_.end() ? nullptr : it->second.second;
}

const void* ModelFiles::data(const std::string& name) {
    const auto& [file, entry] = index_.at(name);
    return files_[file]->data(*entry);
}

void write_safetensors(const std::string& path, const std::vector<TensorToWrite>& tensors, const Json& metadata) {
    Json header = Json::object();
    if (metadata.size()) header.set("__metadata__", metadata);
    uint64_t offset = 0;
    for (const auto& t : tensors) {
        const uint64_t bytes = static_cast<uint64_t>(shape_numel(t.shape)) * dtype_size(t.dtype);
        header.set(t.name, Json::object().set("dtype", safetensors_tag(t.dtype)).set("shape", Json::array_of(t.shape))
                               .set("data_offsets", Json::array().push(offset).push(offset + bytes)));
        offset += bytes;
    }
    std::string text = header.dump();
    text.append((8 - text.size() % 8) % 8, ' ');
    const std::string tmp = path + ".tmp";
    std::FILE* f = std::fopen(tmp.c_str(), "wb");
    if (f == nullptr) throw make_error(Code::Io, "cannot write {}: {}", tmp, std::strerror(errno));
    uint8_t len8[8];
    for (int i = 0; i < 8; ++i) len8[i] = static_cast<uint8_t>(text.size() >> (8 * i));
    bool ok = std::fwrite(len8, 1, 8, f) == 8 && std::fwrite(text.data(), 1, text.size(), f) == text.size();
    for (const auto& t : tensors) {
        const size_t bytes = static_cast<size_t>(shape_numel(t.shape)) * dtype_size(t.dtype);
        if (ok && bytes) ok = std::fwrite(t.data, 1, bytes, f) == bytes;
    }
    ok = std::fclose(f) == 0 && ok;
    if (!ok || std::rename(tmp.c_str(), path.c_str()) != 0) throw make_error(Code::Io, "cannot write {}", path);
}

}  // namespace liyab
