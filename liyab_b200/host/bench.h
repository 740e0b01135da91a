// Measurements on the engine's own step function, timed on the device.
//
// The reference ships its benchmarks as programs of the engine (synthetic token
// ids through the stock code path: tools/liyab_bench.cpp:21-30; decode tokens per
// second for 1..N sequences: tools/liyab_seq_bench.cpp:1-35).  These are the same
// for this engine; bench.py calls them through the C interface.
#pragma once

#include <cstdint>

#include "replay.h"

namespace liyab {

struct BenchResult {
    double ms_total = 0, ms_per_step = 0, wall_ms_per_step = 0, mean_context = 0;
    uint64_t kernel_launches = 0, graph_steps = 0, fused_steps = 0, eager_steps = 0;
    uint64_t h2d_bytes_per_step = 0, d2h_bytes_per_step = 0, checksum = 0;
};

BenchResult bench_decode(Replayer& r, int batch, int prompt_len, int steps, int warmup, uint64_t seed);
BenchResult bench_prefill(Replayer& r, int n_seq, int seq_len, int repeats, uint64_t seed);

}  // namespace liyab
