#include "replay.h"

#include <sys/stat.h>

#include <unordered_map>

namespace liyab {

Replayer::Replayer(const std::string& model_dir, const std::string& dtype, int64_t max_tokens, const ReplayerOptions& o) {
    loaded = std::make_unique<LoadedModel>(model_dir, dtype, o.device);
    DecoderModel& model = *loaded->model;
    const int num_pages = o.num_pages > 0 ? o.num_pages : static_cast<int>(std::max<int64_t>(1, (max_tokens + o.page_size - 1) / o.page_size));
    cache = std::make_unique<CacheManager>(model.kv_needs(), model.state_needs(), o.page_size, num_pages, o.max_requests, model.runtime.dtype, true);
    StepperOptions so;
    so.cuda_graphs = o.cuda_graphs;
    so.fused_decode = o.fused_decode;
    so.max_step_tokens = o.max_step_tokens;
    so.max_logit_rows = o.max_step_tokens;
    stepper = std::make_unique<Stepper>(model, *cache, so);
}

StepOutput Replayer::step(const std::vector<StepEntry>& entries, std::vector<float>* host) {
    LIYAB_CUDA(cudaSetDevice(loaded->runtime.device));
    StepOutput out = stepper->step(entries);
    const size_t rows = out.rows.size(), vocab = static_cast<size_t>(loaded->model->spec.vocab_size());
    if (host != nullptr) {
        host->resize(rows * vocab);
        if (rows > 0)
            LIYAB_CUDA(cudaMemcpy2DAsync(host->data(), vocab * 4, out.logits.data, static_cast<size_t>(out.logits.stride) * 4, vocab * 4, rows,
                                         cudaMemcpyDeviceToHost, loaded->runtime.stream));
    }
    LIYAB_CUDA(cudaStreamSynchronize(loaded->runtime.stream));
    return out;
}

int replay_stream(const std::string& model_dir, const std::string& dtype, const std::string& out_dir, int64_t max_tokens,
                  const ReplayerOptions& options, std::FILE* in, std::FILE* done) {
    mkdir(out_dir.c_str(), 0777);
    Replayer replayer(model_dir, dtype, max_tokens, options);
    std::unordered_map<std::string, RequestId> ids;
    RequestId next_id = 0;
    auto id_of = [&](const Json& j) {
        const std::string key = j.dump();
        const auto it = ids.find(key);
        if (it != ids.end()) return it->second;
        return ids[key] = next_id++;
    };
    std::string line;
    std::vector<float> logits;
    char buf[1 << 16];
    while (true) {
        line.clear();
        bool eof = false;
        while (true) {
            if (std::fgets(buf, sizeof buf, in) == nullptr) { eof = true; break; }
            line += buf;
            if (!line.empty() && line.back() == '\n') break;
        }
        if (line.find_first_not_of(" \t\r\n") != std::string::npos) {
            const Json record = Json::parse(line, "a replay step");
            const Json& step_id = record.at("step");
            const std::string step_name = step_id.is_string() ? step_id.as_string() : step_id.dump();
            std::vector<std::vector<int32_t>> tokens, wants;
            std::vector<StepEntry> entries;
            if (const Json* es = record.find("entries")) {
                tokens.reserve(es->size());
                wants.reserve(es->size());
                for (const auto& e : es->items()) {
                    const RequestId id = id_of(e.at("id"));
                    if (!replayer.cache->is_open(id)) replayer.cache->open(id);
                    tokens.emplace_back();
                    for (const int64_t t : e.at("tokens").int_list()) tokens.back().push_back(static_cast<int32_t>(t));
                    wants.emplace_back();
                    if (const Json* w = e.find("want"))
                        for (const int64_t v : w->int_list()) wants.back().push_back(static_cast<int32_t>(v));
                    entries.push_back({id, tokens.back().data(), static_cast<int>(tokens.back().size()), wants.back().data(),
                                       static_cast<int>(wants.back().size())});
                }
            }
            if (!entries.empty()) {
                const StepOutput out = replayer.step(entries, &logits);
                if (!out.rows.empty()) {
                    const std::string tmp = out_dir + "/." + step_name + ".f32.tmp", path = out_dir + "/" + step_name + ".f32";
                    std::FILE* f = std::fopen(tmp.c_str(), "wb");
                    if (f == nullptr) throw make_error(Code::Io, "cannot write {}", tmp);
                    const bool ok = std::fwrite(logits.data(), 4, logits.size(), f) == logits.size();
                    if (std::fclose(f) != 0 || !ok || std::rename(tmp.c_str(), path.c_str()) != 0) throw make_error(Code::Io, "cannot write {}", path);
                }
            }
            if (const Json* end = record.find("end"))
                for (const auto& e : end->items()) {
                    const RequestId id = id_of(e);
                    if (replayer.cache->is_open(id)) replayer.cache->close(id);
                }
            std::fprintf(done, "done %s\n", step_name.c_str());
            std::fflush(done);
        }
        if (eof) break;
    }
    return 0;
}

}  // namespace liyab
