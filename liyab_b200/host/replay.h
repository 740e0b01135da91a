// Trace replay: given token ids go through the model step by step and the
// logits at the wanted places are written out.  Nothing is sampled.
//
// It drives the framework's own model, step function, cache manager and kernels:
// the ones that generation uses.  The reference's counterparts are its schedule
// harness (Plan / Trace / run_batched: tests/test_sequences.cpp:87-252) and the
// teacher-forced passes of liyab-kl (tools/liyab_kl.cpp:45-47).
//
// Input, one JSON object per line:
//     {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
// For a step in which something is wanted, OUT/<step>.f32 receives the logits at
// the wanted places, in the order of the entries and of `want`, as little-endian
// float32 [wanted, vocab].  After every step a line `done <step>` is printed.
#pragma once

#include <cstdio>
#include <memory>
#include <string>

#include "engine.h"

namespace liyab {

struct ReplayerOptions {
    int device = 0;
    int page_size = 16;
    int max_requests = 16;
    int num_pages = 0;              // 0: from max_tokens
    bool cuda_graphs = false;
    bool fused_decode = false;
    int max_step_tokens = 0;        // scratch sized up front for this many tokens (what lets steps with portions be captured)
};

// A model, a cache sized for `max_tokens` live tokens and the step function over them.
class Replayer {
public:
    Replayer(const std::string& model_dir, const std::string& dtype, int64_t max_tokens, const ReplayerOptions& options);

    std::unique_ptr<LoadedModel> loaded;
    std::unique_ptr<CacheManager> cache;
    std::unique_ptr<Stepper> stepper;

    // Runs one step; the logits at the wanted places are copied to `host` (resized to rows * vocab).
    StepOutput step(const std::vector<StepEntry>& entries, std::vector<float>* host);
};

// Reads steps from `in` until it ends; returns the process's exit code.
int replay_stream(const std::string& model_dir, const std::string& dtype, const std::string& out_dir, int64_t max_tokens,
                  const ReplayerOptions& options, std::FILE* in, std::FILE* done);

}  // namespace liyab
