// Weights by tensor name, checked as a whole before any is used; and the
// random-weights mode.
//
// Every parameter the configuration asks for is looked up by its name in the
// model file; a file that lacks a tensor, holds one nobody asked for, or has one
// of the wrong shape is refused with ONE error that lists all three kinds, in the
// words of the reference's loader ("missing tensor 'X'", "tensor 'X' has shape
// [..], expected [..]": src/core/transformer.cpp:1052-1072).
//
// Storage types.  In the 32-bit mode every floating tensor is widened to float32.
// In the bfloat16 mode matrices and embedding tables (the operands of matrix
// products) are kept in bfloat16, while vectors (norm gains, biases) stay or
// become float32, which the kernels add in 32-bit anyway; integer tensors become
// int32.
//
// Random-weights mode: a model folder (config.json, model.safetensors in the
// architecture's own tensor names and layouts) from a configuration and a seed;
// the reference's tests write tiny models on the fly the same way
// (tests/test_model.h:64-318).  Values come from a counter-based generator
// (SplitMix64 of a key made of the seed and the tensor's name, plus the element's
// index, then Box-Muller in 64-bit), so a tensor's values depend on nothing but
// (seed, name, index).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "arch.h"
#include "device.h"
#include "parts.h"

namespace liyab {

struct HostTensor {
    DType dtype = DType::F32;
    std::vector<int64_t> shape;
    std::vector<uint8_t> bytes;
};

// Reads the model file(s) of `model_dir` into {parameter path: tensor} on the host, transformed and in
// their storage types for `compute`.
std::map<std::string, HostTensor> load_parameters(const std::string& model_dir, const ArchitectureConfig& config, DType compute);

// The parameters of a model on the device: one arena, every tensor 256-byte aligned.
class WeightStore {
public:
    WeightStore() = default;
    explicit WeightStore(const std::map<std::string, HostTensor>& host);
    const Params& params() const { return params_; }
    size_t bytes() const { return arena_.bytes(); }

private:
    DeviceBuffer arena_;
    Params params_;
};

// `count` draws of N(mean, std) for the tensor `name` under `seed`, from index `first` on.
void normal_values(uint64_t seed, const std::string& name, int64_t first, int64_t count, double mean, double std, double* out);
// Writes `model_dir`/config.json and model.safetensors; dtype float32, bfloat16 or float16.
void write_random_model(const std::string& model_dir, const ArchitectureConfig& config, uint64_t seed, const std::string& dtype);

uint16_t float_to_bf16(float v);      // round to nearest even
float bf16_to_float(uint16_t v);

}  // namespace liyab
