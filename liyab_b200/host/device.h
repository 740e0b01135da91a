// Device memory, streams and scratch buffers of the host runtime.
//
// Everything on the GPU is owned here through plain CUDA runtime calls: weights
// and cache pages in `DeviceBuffer`s, staging in pinned host memory, one stream
// per engine.  Nothing in the host library depends on a tensor framework.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "status.h"

namespace liyab {

// Element types; F32 and BF16 carry the numbers of the kernel interface (LB_F32, LB_BF16).
enum class DType : int { F32 = 0, BF16 = 1, I32 = 2, F16 = 3, F64 = 4, I64 = 5, I16 = 6, I8 = 7, U8 = 8, Bool = 9 };
size_t dtype_size(DType t);
const char* dtype_name(DType t);
DType compute_dtype_from_name(const std::string& name);      // bfloat16/bf16, float32/fp32/f32; else INVALID_ARGUMENT

void cuda_check(cudaError_t err, const char* what);
#define LIYAB_CUDA(expr) ::liyab::cuda_check((expr), #expr)

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes, bool zero = false);
    ~DeviceBuffer();
    DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    void* data() const { return ptr_; }
    size_t bytes() const { return bytes_; }

private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

class PinnedBuffer {
public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(size_t bytes);
    ~PinnedBuffer();
    PinnedBuffer(PinnedBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) { o.ptr_ = nullptr; o.bytes_ = 0; }
    PinnedBuffer& operator=(PinnedBuffer&& o) noexcept;
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    void* data() const { return ptr_; }
    size_t bytes() const { return bytes_; }

private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

class Event {
public:
    explicit Event(bool timing = false);
    ~Event();
    Event(const Event&) = delete;
    Event& operator=(const Event&) = delete;
    void record(cudaStream_t stream);
    void synchronize();
    cudaEvent_t get() const { return event_; }

private:
    cudaEvent_t event_ = nullptr;
    bool recorded_ = false;
};

// A view of a parameter or buffer: device (or, for loaded-but-not-uploaded weights, host) memory.
struct Tensor {
    void* data = nullptr;
    DType dtype = DType::F32;
    std::vector<int64_t> shape;

    int64_t numel() const;
    size_t bytes() const { return static_cast<size_t>(numel()) * dtype_size(dtype); }
    int64_t dim(int i) const { return shape.at(static_cast<size_t>(i)); }
    explicit operator bool() const { return data != nullptr; }
};

// Rows of activations: `cols` dense elements per row, rows `stride` elements apart.
struct Rows {
    void* data = nullptr;
    DType dtype = DType::F32;
    int64_t rows = 0, cols = 0, stride = 0;

    Rows columns(int64_t first, int64_t count) const {
        return Rows{static_cast<char*>(data) + static_cast<size_t>(first) * dtype_size(dtype), dtype, rows, count, stride};
    }
    float* f32() const { return static_cast<float*>(data); }
};

// Element type of activations and matrices, the device and the stream every launch goes to.
struct Runtime {
    DType dtype = DType::BF16;
    int device = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 148;

    bool reduced() const { return dtype != DType::F32; }
};

// Named scratch buffers that persist across steps.  A buffer is created at first
// use and grows when a step needs more rows, so a steady state allocates nothing;
// `reserve_rows` sizes the per-token buffers up front, which keeps addresses fixed
// for captured CUDA graphs (`generation` grows whenever a buffer is created or moved).
class Workspace {
public:
    void reserve_rows(int64_t rows) { if (rows > min_rows_) min_rows_ = rows; }
    int64_t min_rows() const { return min_rows_; }
    // [rows, cols] of `dtype`; at least min_rows() rows unless `per_token` is false (buffers sized by
    // the number of logit rows, not by the step's tokens).
    Rows get(const std::string& name, int64_t rows, int64_t cols, DType dtype, bool per_token = true);
    // A one-dimensional buffer of at least `count` elements; `zero`: cleared when created
    // (counters that kernels leave at zero).
    void* flat(const std::string& name, int64_t count, DType dtype, bool zero = false);
    uint64_t generation() const { return generation_; }
    size_t bytes() const;

private:
    struct Entry {
        DeviceBuffer buffer;
        int64_t rows = 0;
    };
    std::map<std::tuple<std::string, int64_t, int>, Entry> buffers_;
    int64_t min_rows_ = 0;
    uint64_t generation_ = 0;
};

}  // namespace liyab
