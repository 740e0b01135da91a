#include "device.h"

#include <algorithm>

namespace liyab {

size_t dtype_size(DType t) {
    switch (t) {
        case DType::F64: case DType::I64: return 8;
        case DType::F32: case DType::I32: return 4;
        case DType::BF16: case DType::F16: case DType::I16: return 2;
        case DType::I8: case DType::U8: case DType::Bool: return 1;
    }
    return 0;
}

const char* dtype_name(DType t) {
    switch (t) {
        case DType::F32: return "float32";
        case DType::BF16: return "bfloat16";
        case DType::I32: return "int32";
        case DType::F16: return "float16";
        case DType::F64: return "float64";
        case DType::I64: return "int64";
        case DType::I16: return "int16";
        case DType::I8: return "int8";
        case DType::U8: return "uint8";
        case DType::Bool: return "bool";
    }
    return "?";
}

DType compute_dtype_from_name(const std::string& name) {
    if (name == "bfloat16" || name == "bf16") return DType::BF16;
    if (name == "float32" || name == "fp32" || name == "f32") return DType::F32;
    throw invalid_argument("unknown dtype '{}'; choose bfloat16 or float32", name);
}

void cuda_check(cudaError_t err, const char* what) {
    if (err == cudaSuccess) return;
    const Code code = err == cudaErrorMemoryAllocation ? Code::OutOfMemory : Code::Backend;
    throw Error(code, std::format("{} failed: {}", what, cudaGetErrorString(err)));
}

DeviceBuffer::DeviceBuffer(size_t bytes, bool zero) : bytes_(bytes) {
    if (bytes == 0) return;
    LIYAB_CUDA(cudaMalloc(&ptr_, bytes));
    if (zero) LIYAB_CUDA(cudaMemset(ptr_, 0, bytes));
}
DeviceBuffer::~DeviceBuffer() {
    if (ptr_ != nullptr) cudaFree(ptr_);
}
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
        if (ptr_ != nullptr) cudaFree(ptr_);
        ptr_ = o.ptr_; bytes_ = o.bytes_;
        o.ptr_ = nullptr; o.bytes_ = 0;
    }
    return *this;
}

PinnedBuffer::PinnedBuffer(size_t bytes) : bytes_(bytes) {
    if (bytes) LIYAB_CUDA(cudaMallocHost(&ptr_, bytes));
}
PinnedBuffer::~PinnedBuffer() {
    if (ptr_ != nullptr) cudaFreeHost(ptr_);
}
PinnedBuffer& PinnedBuffer::operator=(PinnedBuffer&& o) noexcept {
    if (this != &o) {
        if (ptr_ != nullptr) cudaFreeHost(ptr_);
        ptr_ = o.ptr_; bytes_ = o.bytes_;
        o.ptr_ = nullptr; o.bytes_ = 0;
    }
    return *this;
}

Event::Event(bool timing) { LIYAB_CUDA(cudaEventCreateWithFlags(&event_, timing ? cudaEventDefault : cudaEventDisableTiming)); }
Event::~Event() {
    if (event_ != nullptr) cudaEventDestroy(event_);
}
void Event::record(cudaStream_t stream) {
    LIYAB_CUDA(cudaEventRecord(event_, stream));
    recorded_ = true;
}
void Event::synchronize() {
    if (recorded_) LIYAB_CUDA(cudaEventSynchronize(event_));
}

int64_t Tensor::numel() const {
    int64_t n = 1;
    for (const int64_t d : shape) n *= d;
    return n;
}

Rows Workspace::get(const std::string& name, int64_t rows, int64_t cols, DType dtype, bool per_token) {
    // layers of different sizes get buffers of their own
    auto& e = buffers_[{name, cols, static_cast<int>(dtype)}];
    if (e.buffer.data() == nullptr || e.rows < rows) {
        const int64_t cap = std::max<int64_t>({rows, per_token ? min_rows_ : 0, 1});
        e.buffer = DeviceBuffer(static_cast<size_t>(cap) * static_cast<size_t>(cols) * dtype_size(dtype));
        e.rows = cap;
        ++generation_;
    }
    return Rows{e.buffer.data(), dtype, rows, cols, cols};
}

void* Workspace::flat(const std::string& name, int64_t count, DType dtype, bool zero) {
    auto& e = buffers_[{name, -1, static_cast<int>(dtype)}];
    if (e.buffer.data() == nullptr || e.rows < count) {
        int64_t cap = 1024;
        while (cap < count) cap *= 2;
        e.buffer = DeviceBuffer(static_cast<size_t>(cap) * dtype_size(dtype), zero);
        e.rows = cap;
        ++generation_;
    }
    return e.buffer.data();
}

size_t Workspace::bytes() const {
    size_t n = 0;
    for (const auto& kv : buffers_) n += kv.second.buffer.bytes();
    return n;
}

}  // namespace liyab
