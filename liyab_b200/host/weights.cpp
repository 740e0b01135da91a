#include "weights.h"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <regex>
#include <set>
#include <thread>

#include "log.h"
#include "safetensors.h"

namespace liyab {

uint16_t float_to_bf16(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);      // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}

float bf16_to_float(uint16_t v) {
    const uint32_t u = static_cast<uint32_t>(v) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

namespace {

float half_to_float(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while ((m & 0x400u) == 0);
            u = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (m & 0x3ffu) << 13;
        }
    } else if (exp == 31) u = sign | 0x7f800000u | man << 13;
    else u = sign | (exp + 112) << 23 | man << 13;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

uint16_t float_to_half(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const int32_t exp = static_cast<int32_t>((u >> 23) & 0xff) - 127 + 15;
    uint32_t man = u & 0x7fffffu;
    if (((u >> 23) & 0xff) == 0xff) return static_cast<uint16_t>(sign | 0x7c00u | (man ? 0x200u : 0));
    if (exp >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
    if (exp <= 0) {
        if (exp < -10) return static_cast<uint16_t>(sign);
        man |= 0x800000u;
        const int shift = 14 - exp;
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1))) ++h;
        return static_cast<uint16_t>(sign | h);
    }
    uint32_t h = static_cast<uint32_t>(exp) << 10 | man >> 13;
    const uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
}

bool is_float(DType t) { return t == DType::F32 || t == DType::F16 || t == DType::BF16 || t == DType::F64; }

DType storage_dtype(ParamKind kind, DType stored, DType compute) {
    if (!is_float(stored)) return DType::I32;
    if (compute == DType::F32 || kind == ParamKind::Vector) return DType::F32;
    return compute;
}

// Element-wise conversion of `count` elements into `to` (float32, bfloat16 or int32).
void convert(const void* src, DType from, void* dst, DType to, int64_t count) {
    if (from == to) { std::memcpy(dst, src, static_cast<size_t>(count) * dtype_size(to)); return; }
    if (to == DType::I32) {
        auto* out = static_cast<int32_t*>(dst);
        for (int64_t i = 0; i < count; ++i) {
            int64_t v = 0;
            switch (from) {
                case DType::I64: v = static_cast<const int64_t*>(src)[i]; break;
                case DType::I16: v = static_cast<const int16_t*>(src)[i]; break;
                case DType::I8: v = static_cast<const int8_t*>(src)[i]; break;
                case DType::U8: case DType::Bool: v = static_cast<const uint8_t*>(src)[i]; break;
                default: v = 0;
            }
            out[i] = static_cast<int32_t>(v);
        }
        return;
    }
    auto load = [&](int64_t i) -> float {
        switch (from) {
            case DType::F32: return static_cast<const float*>(src)[i];
            case DType::F64: return static_cast<float>(static_cast<const double*>(src)[i]);
            case DType::BF16: return bf16_to_float(static_cast<const uint16_t*>(src)[i]);
            case DType::F16: return half_to_float(static_cast<const uint16_t*>(src)[i]);
            default: return 0.0f;
        }
    };
    if (to == DType::F32) {
        auto* out = static_cast<float*>(dst);
        for (int64_t i = 0; i < count; ++i) out[i] = load(i);
    } else {
        auto* out = static_cast<uint16_t*>(dst);
        for (int64_t i = 0; i < count; ++i) out[i] = float_to_bf16(load(i));
    }
}

template <class T>
void transpose2d(const T* src, T* dst, int64_t rows, int64_t cols) {
    constexpr int64_t B = 32;
    for (int64_t r0 = 0; r0 < rows; r0 += B)
        for (int64_t c0 = 0; c0 < cols; c0 += B)
            for (int64_t r = r0; r < std::min(r0 + B, rows); ++r)
                for (int64_t c = c0; c < std::min(c0 + B, cols); ++c) dst[c * rows + r] = src[r * cols + c];
}

// One parameter from its sources: convert, transform, join, cut.
HostTensor assemble(ModelFiles& files, const std::string& prefix, const CheckpointTensor& spec, DType compute) {
    std::vector<HostTensor> parts;
    for (const auto& src : spec.sources) {
        const TensorEntry* e = files.find(prefix + src.name);
        HostTensor t;
        t.dtype = storage_dtype(spec.kind, e->dtype, compute);
        t.shape = e->shape;
        const int64_t n = shape_numel(e->shape);
        t.bytes.resize(static_cast<size_t>(n) * dtype_size(t.dtype));
        convert(files.data(prefix + src.name), e->dtype, t.bytes.data(), t.dtype, n);
        if (spec.transform == "transpose") {
            if (t.shape.size() != 2) throw invalid_model("tensor '{}' cannot be transposed: it has shape {}", src.name, shape_text(t.shape));
            std::vector<uint8_t> out(t.bytes.size());
            if (dtype_size(t.dtype) == 2) transpose2d(reinterpret_cast<const uint16_t*>(t.bytes.data()), reinterpret_cast<uint16_t*>(out.data()), t.shape[0], t.shape[1]);
            else transpose2d(reinterpret_cast<const uint32_t*>(t.bytes.data()), reinterpret_cast<uint32_t*>(out.data()), t.shape[0], t.shape[1]);
            t.bytes = std::move(out);
            std::swap(t.shape[0], t.shape[1]);
        } else if (spec.transform != "none") {
            throw invalid_model("unknown transform '{}' for tensor '{}'", spec.transform, src.name);
        }
        parts.push_back(std::move(t));
    }
    HostTensor out = std::move(parts[0]);
    if (parts.size() > 1) {
        // Join along concat_axis: view every part as [outer, axis * inner].
        const size_t ax = static_cast<size_t>(spec.concat_axis);
        if (ax >= out.shape.size()) throw invalid_model("concat axis {} is outside shape {}", spec.concat_axis, shape_text(out.shape));
        int64_t outer = 1, inner = 1, total = out.shape[ax];
        for (size_t i = 0; i < ax; ++i) outer *= out.shape[i];
        for (size_t i = ax + 1; i < out.shape.size(); ++i) inner *= out.shape[i];
        for (size_t p = 1; p < parts.size(); ++p) {
            auto s = parts[p].shape;
            if (s.size() != out.shape.size() || parts[p].dtype != out.dtype) throw invalid_model("tensors to join differ in rank or type");
            for (size_t i = 0; i < s.size(); ++i)
                if (i != ax && s[i] != out.shape[i]) throw invalid_model("tensors to join differ outside axis {}", spec.concat_axis);
            total += s[ax];
        }
        const size_t es = dtype_size(out.dtype);
        std::vector<uint8_t> joined(static_cast<size_t>(outer * total * inner) * es);
        parts[0] = std::move(out);
        int64_t at = 0;
        for (const auto& p : parts) {
            const int64_t width = p.shape[ax] * inner;
            for (int64_t o = 0; o < outer; ++o)
                std::memcpy(joined.data() + static_cast<size_t>((o * total * inner) + at) * es, p.bytes.data() + static_cast<size_t>(o * width) * es,
                            static_cast<size_t>(width) * es);
            at += width;
        }
        out = HostTensor{parts[0].dtype, parts[0].shape, std::move(joined)};
        out.shape[ax] = total;
    }
    if (spec.slice_axis >= 0) {
        const size_t ax = static_cast<size_t>(spec.slice_axis);
        if (ax >= out.shape.size() || spec.slice_begin < 0 || spec.slice_end > out.shape[ax] || spec.slice_begin >= spec.slice_end)
            throw invalid_model("slice [{}, {}) of axis {} is outside shape {}", spec.slice_begin, spec.slice_end, spec.slice_axis, shape_text(out.shape));
        int64_t outer = 1, inner = 1;
        for (size_t i = 0; i < ax; ++i) outer *= out.shape[i];
        for (size_t i = ax + 1; i < out.shape.size(); ++i) inner *= out.shape[i];
        const size_t es = dtype_size(out.dtype);
        const int64_t keep = spec.slice_end - spec.slice_begin, full = out.shape[ax];
        std::vector<uint8_t> cut(static_cast<size_t>(outer * keep * inner) * es);
        for (int64_t o = 0; o < outer; ++o)
            std::memcpy(cut.data() + static_cast<size_t>(o * keep * inner) * es,
                        out.bytes.data() + static_cast<size_t>((o * full + spec.slice_begin) * inner) * es, static_cast<size_t>(keep * inner) * es);
        out.bytes = std::move(cut);
        out.shape[ax] = keep;
    }
    return out;
}

template <class Fn>
void parallel_for(size_t n, Fn&& fn) {
    const size_t workers = std::min<size_t>(n, std::max(1u, std::min(16u, std::thread::hardware_concurrency())));
    if (workers <= 1) { for (size_t i = 0; i < n; ++i) fn(i); return; }
    std::atomic<size_t> next{0};
    std::vector<std::thread> threads;
    std::exception_ptr failure;
    std::mutex mutex;
    for (size_t w = 0; w < workers; ++w)
        threads.emplace_back([&] {
            try {
                for (size_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
            } catch (...) {
                std::lock_guard<std::mutex> lock(mutex);
                if (!failure) failure = std::current_exception();
            }
        });
    for (auto& t : threads) t.join();
    if (failure) std::rethrow_exception(failure);
}

}  // namespace

std::map<std::string, HostTensor> load_parameters(const std::string& model_dir, const ArchitectureConfig& config, DType compute) {
    ModelFiles files(model_dir);
    const CheckpointMap wanted = config.checkpoint_map();
    const auto names = files.names();
    const std::set<std::string> have(names.begin(), names.end());
    // The prefix under which most of the wanted tensors are found.
    std::string prefix;
    size_t best = 0;
    bool first = true;
    for (const auto& p : config.name_prefixes()) {
        size_t hits = 0;
        for (const auto& kv : wanted)
            for (const auto& s : kv.second.sources) hits += have.count(p + s.name);
        if (first || hits > best) { prefix = p; best = hits; first = false; }
    }
    std::vector<std::string> missing, wrong;
    std::set<std::string> used;
    for (const auto& [dest, spec] : wanted)
        for (const auto& src : spec.sources) {
            const std::string full = prefix + src.name;
            const TensorEntry* e = files.find(full);
            if (e == nullptr) { missing.push_back(std::format("missing tensor '{}'", full)); continue; }
            used.insert(full);
            if (e->shape != src.shape)
                wrong.push_back(std::format("tensor '{}' has shape {}, expected {}", full, shape_text(e->shape), shape_text(src.shape)));
            else if (!is_float(e->dtype) && spec.kind != ParamKind::Index)
                wrong.push_back(std::format("tensor '{}' has dtype {}, expected a floating type", full, dtype_name(e->dtype)));
        }
    // A tensor that carries no weights may sit under the file's prefix or outside it (a stored copy of a
    // tied head usually does not carry the body's prefix).
    std::vector<std::regex> ignored;
    std::string escaped;
    for (const char c : prefix) { if (std::strchr(".^$|()[]{}*+?\\", c)) escaped += '\\'; escaped += c; }
    for (const auto& pat : config.ignored_tensors()) ignored.emplace_back("^(?:" + escaped + ")?" + pat + "$");
    std::vector<std::string> unexpected;
    for (const auto& n : names) {
        if (used.count(n)) continue;
        if (std::any_of(ignored.begin(), ignored.end(), [&](const std::regex& r) { return std::regex_match(n, r); })) {
            log(LogLevel::Info, "{}: tensor '{}' carries no weights for this engine and is ignored", files.shown_path(), n);
            continue;
        }
        unexpected.push_back(n);
    }
    if (!missing.empty() || !wrong.empty() || !unexpected.empty()) {
        auto join = [](const std::vector<std::string>& v) {
            std::string s;
            for (const auto& x : v) s += (s.empty() ? "" : "; ") + x;
            return s;
        };
        std::vector<std::string> parts;
        if (!missing.empty()) parts.push_back(std::format("{} missing: {}", missing.size(), join(missing)));
        if (!unexpected.empty()) {
            std::vector<std::string> u;
            for (const auto& n : unexpected) u.push_back(std::format("unexpected tensor '{}'", n));
            parts.push_back(std::format("{} unexpected: {}", u.size(), join(u)));
        }
        if (!wrong.empty()) parts.push_back(std::format("{} of the wrong shape: {}", wrong.size(), join(wrong)));
        std::string all;
        for (const auto& p : parts) all += (all.empty() ? "" : " | ") + p;
        throw invalid_model("{} does not fit the configuration. {}", files.shown_path(), all);
    }
    for (const auto& n : names) files.data(n);      // map every file before the workers start
    std::vector<HostTensor> built(wanted.size());
    parallel_for(wanted.size(), [&](size_t i) { built[i] = assemble(files, prefix, wanted[i].second, compute); });
    std::map<std::string, HostTensor> out;
    for (size_t i = 0; i < wanted.size(); ++i) out[wanted[i].first] = std::move(built[i]);
    return out;
}

WeightStore::WeightStore(const std::map<std::string, HostTensor>& host) {
    size_t total = 0;
    for (const auto& kv : host) total += (kv.second.bytes.size() + 255) / 256 * 256;
    arena_ = DeviceBuffer(std::max<size_t>(total, 256));
    size_t at = 0;
    for (const auto& [name, t] : host) {
        char* dst = static_cast<char*>(arena_.data()) + at;
        if (!t.bytes.empty()) LIYAB_CUDA(cudaMemcpy(dst, t.bytes.data(), t.bytes.size(), cudaMemcpyHostToDevice));
        params_.add(name, Tensor{dst, t.dtype, t.shape});
        at += (t.bytes.size() + 255) / 256 * 256;
    }
}

namespace {
uint64_t fnv1a64(const std::string& text) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (const unsigned char b : text) h = (h ^ b) * 0x100000001B3ull;
    return h;
}
uint64_t splitmix64(uint64_t x) {
    uint64_t z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
}  // namespace

void normal_values(uint64_t seed, const std::string& name, int64_t first, int64_t count, double mean, double std, double* out) {
    const uint64_t key = fnv1a64(name) ^ (seed * 0x9E3779B97F4A7C15ull);
    constexpr double two_pi = 6.283185307179586476925286766559;
    for (int64_t i = 0; i < count; ++i) {
        const uint64_t bits = splitmix64(static_cast<uint64_t>(first + i) + key);
        const double u1 = (static_cast<double>(bits >> 32) + 1.0) / 4294967296.0;      // (0, 1]
        const double u2 = static_cast<double>(bits & 0xFFFFFFFFull) / 4294967296.0;     // [0, 1)
        out[i] = mean + std * (std::sqrt(-2.0 * std::log(u1)) * std::cos(two_pi * u2));
    }
}

void write_random_model(const std::string& model_dir, const ArchitectureConfig& config, uint64_t seed, const std::string& dtype) {
    DType store;
    if (dtype == "float32") store = DType::F32;
    else if (dtype == "bfloat16") store = DType::BF16;
    else if (dtype == "float16") store = DType::F16;
    else throw invalid_argument("cannot store weights as '{}'; choose one of float32, bfloat16, float16", dtype);
    if (mkdir(model_dir.c_str(), 0777) != 0 && errno != EEXIST) {
        // parents may be missing
        std::string partial;
        for (size_t i = 0; i <= model_dir.size(); ++i)
            if (i == model_dir.size() || model_dir[i] == '/') {
                partial = model_dir.substr(0, i);
                if (!partial.empty()) mkdir(partial.c_str(), 0777);
            }
    }
    Json raw = config.to_json();
    raw.set("torch_dtype", dtype);
    {
        std::ofstream f(model_dir + "/config.json");
        if (!f) throw make_error(Code::Io, "cannot write {}/config.json", model_dir);
        f << raw.dump(1) << "\n";
    }
    struct Item { std::string name; std::vector<int64_t> shape; double mean, std; std::vector<uint8_t> bytes; };
    std::vector<Item> items;
    for (const auto& [dest, spec] : config.checkpoint_map())
        for (const auto& src : spec.sources) items.push_back({src.name, src.shape, spec.init_mean, spec.init_std, {}});
    const size_t es = dtype_size(store);
    // Large tensors are cut into pieces so that every core has work.
    struct Piece { size_t item; int64_t first, count; };
    std::vector<Piece> pieces;
    for (size_t i = 0; i < items.size(); ++i) {
        const int64_t n = shape_numel(items[i].shape);
        items[i].bytes.resize(static_cast<size_t>(n) * es);
        for (int64_t at = 0; at < n; at += int64_t{1} << 20) pieces.push_back({i, at, std::min<int64_t>(int64_t{1} << 20, n - at)});
    }
    parallel_for(pieces.size(), [&](size_t p) {
        const Piece& pc = pieces[p];
        Item& it = items[pc.item];
        std::vector<double> v(static_cast<size_t>(pc.count));
        normal_values(seed, it.name, pc.first, pc.count, it.mean, it.std, v.data());
        uint8_t* dst = it.bytes.data() + static_cast<size_t>(pc.first) * es;
        for (int64_t i = 0; i < pc.count; ++i) {
            const float f = static_cast<float>(v[static_cast<size_t>(i)]);
            if (store == DType::F32) std::memcpy(dst + 4 * i, &f, 4);
            else {
                const uint16_t h = store == DType::BF16 ? float_to_bf16(f) : float_to_half(f);
                std::memcpy(dst + 2 * i, &h, 2);
            }
        }
    });
    std::vector<TensorToWrite> out;
    for (const auto& it : items) out.push_back({it.name, store, it.shape, it.bytes.data()});
    write_safetensors(model_dir + "/model.safetensors", out, Json::object().set("format", "pt").set("seed", std::to_string(seed)));
}

}  // namespace liyab
