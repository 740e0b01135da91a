// The fused decode step: a stack of pre-norm blocks run by one persistent kernel.
//
// A decode step of a few requests is bound by launch count and memory round
// trips, not by bytes or flops.  Where a model is made of nothing but the standard
// parts (LayerNorm, attention with a fused projection, dense feed-forward,
// pre-norm arrangement, learned or no positions) in bfloat16, its decode steps of
// up to 16 tokens are handed to csrc/decode_stack.cu, which runs the whole step
// as one cooperative kernel.  Anything else (another mixer, another arrangement,
// float32, more tokens, prompt portions, a head with a scale or a cap) takes the
// part-by-part path; the results agree to bfloat16 rounding, which the tests check.
//
// It is an option (off by default): with one-launch products, launches that overlap the kernel before and the rows
// normalised inside the projections, the part-by-part path in a captured graph has become as fast or faster at
// every size measured (8 tokens: GPT-2 small 379 against 417 us, medium 820 against 820 us, GPT-2 large 1.47
// against 3.38 ms, whose slices no longer fit the registers this kernel sets aside for a phase's weights).
//
// This class only describes the model to the kernel: it packs one record per
// run-order entry from the parts' own parameters and owns the step's buffers.
#pragma once

#include <memory>
#include <vector>

#include "decoder.h"

namespace liyab {

class FusedDecodeStack {
public:
    static constexpr int kMaxTokens = 16;
    // Null when the model or the cache is not of the shape the kernel takes.
    static std::unique_ptr<FusedDecodeStack> try_build(const DecoderModel& model, const CacheManager& cache);

    // Up to 16 tokens, and no more (token, key/value head) pairs than the GPU has SMs: beyond that the attention phase
    // takes two rounds (measured: GPT-2 small at 14 tokens 537 us against 486 us part by part).
    bool accepts(int n_tokens) const;
    // Computes the logits of a decode step ([n_tokens, vocab] float32, valid until the next run).
    Rows run(StepContext& ctx);
    // Time stamps from inside the kernel (a measuring aid): once switched on, every launch has block 0 write the
    // global timer after each grid barrier (entry = barrier number) and at the marks inside the phases, and every
    // block its arrival at the five barriers of one middle layer; `stamps` copies the last launch's out.
    static constexpr size_t kStamps = 2048;
    void record_stamps(bool on);
    std::vector<uint64_t> stamps() const;

private:
    FusedDecodeStack() = default;
    void splits(int n_tokens, int* n_splits, int* unit_warps) const;

    const DecoderModel* model_ = nullptr;
    const CacheManager* cache_ = nullptr;
    int head_dim_ = 0, n_layers_ = 0, max_k_ = 0, max_qd_ = 0, max_inner_ = 0, max_heads_ = 0, max_kv_heads_ = 0;
    const void* pos_table_ = nullptr;
    const float* lnf_w_ = nullptr;
    const float* lnf_b_ = nullptr;
    float lnf_eps_ = 0.0f;
    DeviceBuffer layers_, x_, q_, att_, inner_, logits_, partial_, counters_, barrier_, stamps_;
    uint64_t launches_ = 0;
};

}  // namespace liyab
