// Runs the reference's own forward pass (andrei-borcea/liyab, built on the CPU)
// over a GGUF model and writes the logits of every position as raw float32.
// Usage: reference_forward MODEL.gguf OUT.f32 N_WHOLE tok0 tok1 ...
// The first N_WHOLE tokens go through one forward(Logits::All); the rest one by
// one (Logits::Last), so the file holds one row per token either way.
// Built and run by make_golden.py against the reference's build tree; it is not
// part of the engine and nothing in the engine or its tests needs it to exist.
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "core/thread_pool.h"
#include "core/transformer.h"
#include "liyab/backend.h"
#include "liyab/mmap_loader.h"

int main(int argc, char** argv) {
    if (argc < 5) return 2;
    using namespace liyab;
    auto file = MmapLoader::open(argv[1]);
    if (!file) { std::fprintf(stderr, "open: %s\n", file.status().to_string().c_str()); return 1; }
    TransformerOptions opt;
    opt.kv_type = KvCacheType::F16;
    auto model = Transformer::load(std::move(file.value()), opt);
    if (!model) { std::fprintf(stderr, "load: %s\n", model.status().to_string().c_str()); return 1; }
    ThreadPool pool(1);
    auto cpu = make_cpu_backend(pool);
    Route route{cpu.get(), cpu.get(), cpu.get()};
    const int whole = std::atoi(argv[3]);
    std::vector<int32_t> tokens;
    for (int i = 4; i < argc; ++i) tokens.push_back(std::atoi(argv[i]));
    std::FILE* out = std::fopen(argv[2], "wb");
    if (out == nullptr) return 1;
    auto& t = *model.value();
    auto rows = t.forward(std::span<const int32_t>(tokens.data(), static_cast<size_t>(whole)),
                          Transformer::Logits::All, route, pool);
    if (!rows) { std::fprintf(stderr, "forward: %s\n", rows.status().to_string().c_str()); return 1; }
    std::fwrite(rows.value().data(), sizeof(float), rows.value().size(), out);
    for (size_t i = static_cast<size_t>(whole); i < tokens.size(); ++i) {
        auto row = t.forward(std::span<const int32_t>(&tokens[i], 1), Transformer::Logits::Last, route, pool);
        if (!row) { std::fprintf(stderr, "step: %s\n", row.status().to_string().c_str()); return 1; }
        std::fwrite(row.value().data(), sizeof(float), row.value().size(), out);
    }
    std::fclose(out);
    return 0;
}
