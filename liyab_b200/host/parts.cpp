#include "parts.h"

#include <dlfcn.h>

#include <mutex>
#include <set>

#include "log.h"

namespace liyab {

const Tensor& Params::at(const std::string& name) const {
    const auto it = tensors_.find(name);
    if (it == tensors_.end()) throw invalid_model("missing parameter '{}'", name);
    return it->second;
}

const Tensor* Params::find(const std::string& name) const {
    const auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : &it->second;
}

Params Params::sub(const std::string& prefix) const {
    Params out;
    for (const auto& [name, t] : tensors_)
        if (name.compare(0, prefix.size(), prefix) == 0) out.add(name.substr(prefix.size()), t);
    return out;
}

void* StepContext::kv(int unit, const GroupView** view) const {
    const auto it = cache->group_of_unit.find(unit);
    if (it == cache->group_of_unit.end()) throw internal_error("run-order entry {} keeps no keys and values", unit);
    const GroupView& v = groups.at(static_cast<size_t>(it->second));
    if (view != nullptr) *view = &v;
    return v.group->unit_storage(unit);
}

void* StepContext::state(int unit, size_t* slot_bytes) const {
    const auto it = cache->states.storage.find(unit);
    if (it == cache->states.storage.end()) throw internal_error("run-order entry {} keeps no state", unit);
    if (slot_bytes != nullptr) *slot_bytes = cache->states.needs.at(unit).bytes();
    return it->second.data();
}

const char* phase_name(Phase p) {
    static const char* names[] = {"embed", "norm", "mixer", "feed_forward", "head"};
    return names[static_cast<int>(p) % 5];
}

void PhaseTimer::mark(cudaStream_t stream, Phase phase) {
    if (used_ == events_.size()) events_.push_back(std::make_unique<Event>(true));
    events_[used_++]->record(stream);
    marks_.push_back(static_cast<int>(phase));
}

void PhaseTimer::end_step(cudaStream_t stream, double* totals) {
    if (used_ == 0) return;
    if (used_ == events_.size()) events_.push_back(std::make_unique<Event>(true));
    events_[used_]->record(stream);
    events_[used_]->synchronize();
    for (size_t i = 0; i < used_; ++i) {
        float ms = 0.0f;
        LIYAB_CUDA(cudaEventElapsedTime(&ms, events_[i]->get(), events_[i + 1]->get()));
        totals[marks_[i]] += ms;
    }
    used_ = 0;
    marks_.clear();
}

Registry<PartFactory<Norm>>& norms() {
    static Registry<PartFactory<Norm>> r("norm");
    return r;
}
Registry<PartFactory<PositionEncoding>>& positions() {
    static Registry<PartFactory<PositionEncoding>> r("position encoding");
    return r;
}
Registry<PartFactory<Mixer>>& mixers() {
    static Registry<PartFactory<Mixer>> r("mixer");
    return r;
}
Registry<PartFactory<FeedForward>>& feed_forwards() {
    static Registry<PartFactory<FeedForward>> r("feed-forward");
    return r;
}
Registry<ArrangementFactory>& arrangements() {
    static Registry<ArrangementFactory> r("block arrangement");
    return r;
}

void load_plugin(const std::string& path) {
    static std::mutex mutex;
    static std::set<std::string> loaded;
    std::lock_guard<std::mutex> lock(mutex);
    if (loaded.count(path)) return;
    register_builtin_parts();
    void* handle = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) throw make_error(Code::Io, "cannot load plug-in {}: {}", path, dlerror());
    using Init = int (*)();
    auto init = reinterpret_cast<Init>(dlsym(handle, "liyab_b200_plugin_init"));
    if (init == nullptr) throw invalid_argument("plug-in {} has no liyab_b200_plugin_init", path);
    const int rc = init();
    if (rc != 0) throw make_error(Code::Internal, "plug-in {}: liyab_b200_plugin_init returned {}", path, rc);
    loaded.insert(path);
    log(LogLevel::Info, "loaded plug-in {}", path);
}

}  // namespace liyab
