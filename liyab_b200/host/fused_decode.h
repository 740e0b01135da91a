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
    // takes two rounds and the part-by-part path with its overlapped launches is faster (measured: GPT-2 small at 14
    // tokens 537 us against 486 us, medium at 12 tokens 1,042 us against 1,005 us).  And only for layers heavy enough:
    // the one kernel streams a layer's matrices better (it asks for them while blocks wait at its barriers: about 1.7 us
    // more a layer from GPT-2 small's 14 MB to medium's 25 MB, against 4.2 us part by part), the part-by-part path has
    // the shorter chain per layer (small: 28.8 against 29.5 us a layer, 8 tokens: 396 against 417 us a step; medium: 33.0
    // against 31.2 us, 864 against 803 us), so the one kernel is taken from 18 MB of matrices a layer on.
    bool accepts(int n_tokens) const;
    static constexpr int64_t kMinLayerBytes = 18 << 20;
    // Lifts that last condition (tests of the kernel with tiny models; measurements).
    void take_light_layers() { light_layers_too_ = true; }
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
    int64_t min_layer_bytes_ = 0;    // the lightest layer's matrices
    bool light_layers_too_ = false;
    uint64_t launches_ = 0;
};

}  // namespace liyab
