// The interfaces of a model's parts and the registries that map a part's `kind`
// to its implementation.
//
// One registry per role: norms, position encodings, mixers, feed-forwards and
// block arrangements.  The model builder (decoder.h) looks every part of every
// layer up here by the `kind` in its spec, so a new kind is added by registering a
// factory (from this library or from a plug-in loaded at run time), with no
// change to the model, the step function or the cache manager.
//
// What a part sees of a step is the `StepContext`: a flat batch of T tokens from
// S requests.  Request i contributes q_len[i] consecutive tokens starting at row
// q_start[i]; its first token sits at position n_past[i] of its sequence.  The
// reference resolves the same facts per segment (`Segment{first, n, kv, n_past}`
// with `pos_of` and `row_of`: src/core/transformer.h:890-916); here they are
// arrays on the device, built once per step, that every kernel indexes.
//
// Capture.  A step whose shape repeats may be captured into a CUDA graph and
// replayed with new contents in the same device arrays.  Only the device arrays
// change between replays: a part whose forward reads the host copies of the
// layout (host_q_start, host_n_past, max_kv_len), copies from the device, or
// keeps host-side state between steps must leave `capturable()` false (the
// default); a model with one such part is never captured.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <string_view>
#include <vector>

#include "cache.h"
#include "device.h"
#include "spec.h"

namespace liyab {

// A part's own parameters by their names inside the part ("qkv.weight").
class Params {
public:
    void add(std::string name, Tensor t) { tensors_[std::move(name)] = std::move(t); }
    const Tensor& at(const std::string& name) const;                  // INVALID_MODEL when absent
    const Tensor* find(const std::string& name) const;
    Params sub(const std::string& prefix) const;                      // members under `prefix`, prefix removed
    const std::map<std::string, Tensor>& all() const { return tensors_; }

private:
    std::map<std::string, Tensor> tensors_;
};

// Which cache unit a run of a layer reads, and whether it writes it.
struct CacheUnit {
    int read = 0;
    bool write = true;
};

// One cache group as a step sees it.
struct GroupView {
    const KvGroup* group = nullptr;
    const int32_t* block_table = nullptr;        // device int32 [S, table_width]
    int table_width = 0;
    const int32_t* slot_mapping = nullptr;       // device int32 [T]
};

using TapFn = std::function<void(std::string_view name, const Rows& rows)>;

// Where a step's time goes, by phase, measured with events on the step's stream when asked for (the
// reference's PhaseTimer and its "decode phases (ms/token)": src/core/transformer.cpp:464-482).
enum class Phase : int { Embed = 0, Norm = 1, Mixer = 2, FeedForward = 3, Head = 4, Count = 5 };
const char* phase_name(Phase p);

class PhaseTimer {
public:
    void begin_step() { used_ = 0; marks_.clear(); }
    // From here on the stream's time belongs to `phase`.
    void mark(cudaStream_t stream, Phase phase);
    // Ends the step: waits for it and adds each phase's milliseconds to `totals` (Phase::Count entries).
    void end_step(cudaStream_t stream, double* totals);

private:
    std::vector<std::unique_ptr<Event>> events_;
    std::vector<int> marks_;
    size_t used_ = 0;
};

struct StepContext {
    Runtime runtime;
    Workspace* workspace = nullptr;
    CacheManager* cache = nullptr;
    int n_tokens = 0;
    int n_seq = 0;
    // device, int32
    const int32_t* tokens = nullptr;             // [T]
    const int32_t* positions = nullptr;          // [T] absolute position of each token
    const int32_t* tok_seq = nullptr;            // [T] row of the token's request in this step
    const int32_t* q_start = nullptr;            // [S + 1] first row of each request
    const int32_t* n_past = nullptr;             // [S] tokens each request held before the step
    const int32_t* state_slots = nullptr;        // [S] the requests' state slots
    const int32_t* logit_rows = nullptr;         // [R] rows whose logits are wanted
    int n_logit_rows = 0;
    std::vector<GroupView> groups;
    // host copies of the same layout (not for capturable parts)
    std::vector<int32_t> host_q_start, host_n_past, host_state_slots;
    int max_q_len = 0;
    int max_kv_len = 0;
    bool decode_only = false;
    int max_positions = 0;          // the longest sequence the engine serves (fixes split counts and table widths)
    const TapFn* tap_fn = nullptr;  // when set, parts' outputs are shown to it (tests)
    PhaseTimer* phases = nullptr;   // when set, phase boundaries are recorded

    cudaStream_t stream() const { return runtime.stream; }
    // The unit's pages [page, K|V, kv_head, slot, head_dim] and its group's view.
    void* kv(int unit, const GroupView** view) const;
    // The unit's state storage [slot, ...]; index it with `state_slots`.
    void* state(int unit, size_t* slot_bytes = nullptr) const;
    void tap(std::string_view name, const Rows& rows) const {
        if (tap_fn != nullptr) (*tap_fn)(name, rows);
    }
    void phase(Phase p) const {
        if (phases != nullptr) phases->mark(runtime.stream, p);
    }
};

class Part {
public:
    virtual ~Part() = default;
    // Whether this part's launches may be captured into a CUDA graph (see the header comment).
    virtual bool capturable() const { return false; }
};

// What a norm may hand to the part after it instead of its output: the recipe of a LayerNorm with 32-bit two-pass
// statistics, y = (x - mean) / sqrt(var + eps) * gain + offset (gain and offset may be null).  A part that can apply
// it while it reads its input (a projection of a few tokens normalises the rows inside its kernel) saves the launch.
struct NormRecipe {
    const float* gain = nullptr;
    const float* offset = nullptr;
    float eps = 0.0f;
};

class Norm : public Part {
public:
    // out[r] = norm(x[rows ? rows[r] : r]) for r < n_rows; x is the float32 residual stream,
    // `rows` a device array or null.
    virtual void forward(StepContext& ctx, const Rows& x, const Rows& out, int n_rows, const int32_t* rows) = 0;
    // The recipe, where the norm is of that kind; an arrangement may then offer the un-normalised rows and the recipe
    // to the part after the norm (forward_from) and only runs the norm itself where that part declines.
    virtual std::optional<NormRecipe> recipe() const { return std::nullopt; }
};

class PositionEncoding : public Part {
public:
    // x[t] = table[token t] * scale (+ its encoding) for the step's tokens.
    virtual void embed(StepContext& ctx, const Tensor& table, float scale, const Rows& x) = 0;
    virtual int64_t max_positions() const = 0;
};

class Mixer : public Part {
public:
    virtual std::optional<KvNeed> kv_need() const { return std::nullopt; }
    virtual std::optional<StateNeed> state_need() const { return std::nullopt; }
    // Adds the mixer's output for the step's tokens to the residual stream x; `h` is its normalised input.
    virtual void forward(StepContext& ctx, const Rows& h, const Rows& x, CacheUnit unit) = 0;
    // The same from the un-normalised rows `x_in` (float32) and the norm's recipe; false (and nothing done) where the
    // mixer cannot apply the recipe itself for this step.
    virtual bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x, CacheUnit unit) { return false; }
};

class FeedForward : public Part {
public:
    virtual void forward(StepContext& ctx, const Rows& h, const Rows& x) = 0;
    // As Mixer::forward_from.
    virtual bool forward_from(StepContext& ctx, const Rows& x_in, const NormRecipe& norm, const Rows& x) { return false; }
};

// The built parts of one layer, by slot name.
struct LayerParts {
    std::map<std::string, std::shared_ptr<Part>> by_name;

    template <class T>
    T& get(const std::string& name) const {
        const auto it = by_name.find(name);
        T* p = it == by_name.end() ? nullptr : dynamic_cast<T*>(it->second.get());
        if (p == nullptr) throw invalid_model("the arrangement needs a slot '{}' of another role", name);
        return *p;
    }
};

class Arrangement : public Part {
public:
    // Runs norms, mixer and feed-forward around the residual stream.
    virtual void forward(StepContext& ctx, const Rows& x, CacheUnit unit) = 0;
    // The mixers of the layer, for the cache manager's needs (usually one).
    virtual std::vector<Mixer*> mixers() const = 0;
};

// -- registries ---------------------------------------------------------------------------------

template <class T>
struct PartFactory {
    std::function<std::vector<ParamDecl>(const PartSpec&)> parameters;
    std::function<std::shared_ptr<T>(const PartSpec&, const Params&, const Runtime&)> build;
};

struct ArrangementFactory {
    // The arrangement checks that the layer has the slots it needs.
    std::function<std::shared_ptr<Arrangement>(const LayerSpec&, const LayerParts&, const Runtime&)> build;
};

template <class F>
class Registry {
public:
    explicit Registry(std::string role) : role_(std::move(role)) {}
    void add(const std::string& kind, F factory) { kinds_[kind] = std::move(factory); }
    const F& get(const std::string& kind) const {
        const auto it = kinds_.find(kind);
        if (it == kinds_.end()) {
            std::string known;
            for (const auto& kv : kinds_) known += (known.empty() ? "" : ", ") + kv.first;
            throw unsupported("no {} of kind '{}' is registered; registered: {}", role_, kind, known.empty() ? "none" : known);
        }
        return it->second;
    }
    std::vector<std::string> kinds() const {
        std::vector<std::string> out;
        for (const auto& kv : kinds_) out.push_back(kv.first);
        return out;
    }

private:
    std::string role_;
    std::map<std::string, F> kinds_;
};

Registry<PartFactory<Norm>>& norms();
Registry<PartFactory<PositionEncoding>>& positions();
Registry<PartFactory<Mixer>>& mixers();
Registry<PartFactory<FeedForward>>& feed_forwards();
Registry<ArrangementFactory>& arrangements();

// Registers the library's own parts (idempotent; called before any model is built).
void register_builtin_parts();

// Loads a shared object and calls its `extern "C" int liyab_b200_plugin_init(void)`, which registers
// parts and architectures through the functions above.  A path already loaded is not loaded again.
void load_plugin(const std::string& path);

}  // namespace liyab
