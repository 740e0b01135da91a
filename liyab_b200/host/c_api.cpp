// The C interface (include/liyab_b200.h) over the host classes.  Every function is
// wrapped by guarded(), which turns any exception into a status and a thread-local
// message (the reference's pattern: src/c_api/liyab_c_api.cpp:34-58).
#include "../include/liyab_b200.h"

#include <cstring>
#include <map>
#include <unordered_map>

#include "../csrc/api.h"
#include "arch.h"
#include "bench.h"
#include "kernels.h"
#include "engine.h"
#include "log.h"
#include "replay.h"
#include "safetensors.h"
#include "weights.h"

extern "C" void lb_set_last_error(const char* message);      // csrc/elementwise.cu keeps the thread's message

using namespace liyab;

struct lb_engine { std::unique_ptr<Engine> engine; };
struct lb_weights { std::map<std::string, HostTensor> tensors; };
struct lb_cache {
    std::unique_ptr<CacheManager> owned;
    CacheManager* cache = nullptr;
};
struct lb_scheduler {
    std::unique_ptr<Scheduler> scheduler;
    std::unordered_map<int64_t, std::unique_ptr<Request>> requests;
    std::map<int64_t, StepPlan> plans;          // planned and not yet finished (two at most when the host runs a step ahead)
    int64_t next_plan = 0;
};
struct lb_replayer {
    std::unique_ptr<Replayer> replayer;
    lb_cache cache_handle;
    std::unique_ptr<Event> t0, t1;
    std::vector<float> host_logits;
};

namespace {

int32_t fail(Code code, const std::string& message) {
    lb_set_last_error(message.c_str());
    return static_cast<int32_t>(code);
}

template <class Fn>
int32_t guarded(Fn&& fn) noexcept {
    try {
        fn();
        return LB_STATUS_OK;
    } catch (const Error& e) {
        return fail(e.code(), e.message());
    } catch (const std::bad_alloc&) {
        return fail(Code::OutOfMemory, "out of memory");
    } catch (const std::exception& e) {
        return fail(Code::Internal, std::string("internal error: ") + e.what());
    } catch (...) {
        return fail(Code::Internal, "internal error");
    }
}

void need(const void* p, const char* what) {
    if (p == nullptr) throw invalid_argument("{} is NULL", what);
}

void copy_out(const std::string& text, char* buffer, size_t size, size_t* needed) {
    if (buffer != nullptr && size > 0) {
        const size_t n = std::min(size - 1, text.size());
        std::memcpy(buffer, text.data(), n);
        buffer[n] = '\0';
    }
    if (needed != nullptr) *needed = text.size();
}

SamplingParams to_cpp(const lb_sampling_params* p) {
    SamplingParams s;
    if (p != nullptr) {
        s.temperature = p->temperature;
        s.top_k = p->top_k;
        s.top_p = p->top_p;
        s.seed = p->seed;
        s.max_tokens = p->max_tokens;
        s.ignore_eos = p->ignore_eos != 0;
    }
    return s;
}

void to_c(const GenerationResult& r, lb_generation_stats* out) {
    if (out == nullptr) return;
    const GenerationStats& s = r.stats;
    *out = lb_generation_stats{};
    out->prompt_tokens = s.prompt_tokens;
    out->generated_tokens = s.generated_tokens;
    out->prefill_ms = s.prefill_ms;
    out->decode_ms = s.decode_ms;
    out->tokens_per_second = s.tokens_per_second;
    out->cancelled = s.cancelled ? 1 : 0;
    out->kv_cache_bytes = s.kv_cache_bytes;
    out->ttft_ms = s.ttft_ms;
    out->preemptions = s.preemptions;
    out->finish_reason = static_cast<int32_t>(r.finish_reason);
    out->decode_steps = s.decode_steps;
    out->embed_ms = s.phase_ms[static_cast<int>(Phase::Embed)];
    out->norm_ms = s.phase_ms[static_cast<int>(Phase::Norm)];
    out->attention_ms = s.phase_ms[static_cast<int>(Phase::Mixer)];
    out->dense_ffn_ms = s.phase_ms[static_cast<int>(Phase::FeedForward)];
    out->lm_head_ms = s.phase_ms[static_cast<int>(Phase::Head)];
}

void fill_scheduler_stats(const SchedulerStats& s, lb_scheduler_stats* out) {
    out->steps = s.steps;
    out->batched_tokens = s.batched_tokens;
    out->prefill_tokens = s.prefill_tokens;
    out->decode_tokens = s.decode_tokens;
    out->preemptions = s.preemptions;
    out->finished = s.finished;
    out->peak_running = s.peak_running;
    for (int i = 0; i < 7; ++i) out->histogram[i] = s.histogram[i];
}

Json describe_config(const ArchitectureConfig& cfg) {
    Json out = Json::object();
    const ModelSpec spec = cfg.model_spec();
    out.set("architecture", spec.architecture);
    out.set("config", cfg.to_json());
    out.set("spec", spec.to_json());
    Json ck = Json::object();
    for (const auto& [dest, t] : cfg.checkpoint_map()) ck.set(dest, t.to_json());
    out.set("checkpoint", ck);
    out.set("ignored_tensors", Json::array_of(cfg.ignored_tensors()));
    out.set("name_prefixes", Json::array_of(cfg.name_prefixes()));
    return out;
}

Json ids_json(const std::vector<Request*>& rs) {
    Json a = Json::array();
    for (const Request* r : rs) a.push(r->id);
    return a;
}

const char* state_name(RequestState s) {
    return s == RequestState::Waiting ? "waiting" : s == RequestState::Running ? "running" : "finished";
}

}  // namespace

extern "C" {

const char* lb_version(void) { return "liyab_b200 0.2"; }

void lb_set_log_level(int32_t level) { set_log_level(level); }
void lb_set_log_callback(lb_log_callback callback, void* user_data) { set_log_sink(callback, user_data); }

void lb_engine_config_default(lb_engine_config* c) {
    if (c == nullptr) return;
    const EngineConfig d;
    *c = lb_engine_config{};
    c->model_path = nullptr;
    c->dtype = "bfloat16";
    c->device = d.device;
    c->context_length = d.context_length;
    c->max_batched_tokens = d.max_batched_tokens;
    c->max_sequences = d.max_requests;
    c->page_size = d.page_size;
    c->num_pages = d.num_pages;
    c->kv_memory_fraction = static_cast<float>(d.kv_memory_fraction);
    c->cuda_graphs = d.cuda_graphs;
    c->fused_decode = d.fused_decode;
    c->pipeline = d.pipeline;
    c->profile_phases = d.profile_phases;
}

void lb_sampling_params_default(lb_sampling_params* p) {
    if (p == nullptr) return;
    const SamplingParams d;
    *p = lb_sampling_params{d.temperature, d.top_k, d.top_p, d.seed, d.max_tokens, d.ignore_eos ? 1 : 0};
}

int32_t lb_engine_create(const lb_engine_config* c, lb_engine** out) {
    return guarded([&] {
        need(c, "config");
        need(out, "out_engine");
        *out = nullptr;
        if (c->model_path == nullptr || c->model_path[0] == '\0') throw invalid_argument("lb_engine_config.model_path is required");
        EngineConfig e;
        e.model = c->model_path;
        if (c->dtype != nullptr && c->dtype[0] != '\0') e.dtype = c->dtype;
        e.device = c->device;
        e.context_length = c->context_length;
        if (c->max_batched_tokens > 0) e.max_batched_tokens = c->max_batched_tokens;
        if (c->max_sequences > 0) e.max_requests = c->max_sequences;
        if (c->page_size > 0) e.page_size = c->page_size;
        e.num_pages = c->num_pages;
        if (c->kv_memory_fraction > 0) e.kv_memory_fraction = c->kv_memory_fraction;
        e.cuda_graphs = c->cuda_graphs != 0;
        e.fused_decode = c->fused_decode != 0;
        e.pipeline = c->pipeline != 0;
        e.profile_phases = c->profile_phases != 0;
        auto handle = std::make_unique<lb_engine>();
        handle->engine = std::make_unique<Engine>(e);
        *out = handle.release();
    });
}

void lb_engine_destroy(lb_engine* engine) { delete engine; }

int32_t lb_engine_generate_batch(lb_engine* engine, lb_request* requests, size_t n) {
    return guarded([&] {
        need(engine, "engine");
        if (n > 0) need(requests, "requests");
        std::vector<GenerationRequest> batch;
        for (size_t i = 0; i < n; ++i) {
            lb_request& q = requests[i];
            if (q.n_tokens > 0) need(q.tokens, "a request's tokens");
            GenerationRequest g;
            g.prompt.assign(q.tokens, q.tokens + q.n_tokens);
            g.params = to_cpp(&q.params);
            if (q.callback != nullptr) {
                const lb_token_callback cb = q.callback;
                void* user = q.user_data;
                g.callback = [cb, user](int32_t token) { return cb(token, user) != 0; };
            }
            batch.push_back(std::move(g));
        }
        const auto results = engine->engine->generate_batch(batch);
        for (size_t i = 0; i < n; ++i) {
            lb_request& q = requests[i];
            const GenerationResult& r = results[i];
            q.n_out = r.tokens.size();
            if (q.out_tokens != nullptr) std::memcpy(q.out_tokens, r.tokens.data(), std::min(q.out_capacity, r.tokens.size()) * 4);
            q.status = r.error ? static_cast<int32_t>(r.error->code()) : LB_STATUS_OK;
            std::snprintf(q.error, sizeof q.error, "%s", r.error ? r.error->message().c_str() : "");
            to_c(r, &q.stats);
        }
    });
}

int32_t lb_engine_generate_tokens(lb_engine* engine, const int32_t* tokens, size_t n_tokens, const lb_sampling_params* params,
                                  lb_token_callback callback, void* user_data, int32_t* out_tokens, size_t out_capacity, size_t* n_out,
                                  lb_generation_stats* stats) {
    lb_request q{};
    q.tokens = tokens;
    q.n_tokens = n_tokens;
    if (params != nullptr) q.params = *params;
    else lb_sampling_params_default(&q.params);
    q.callback = callback;
    q.user_data = user_data;
    q.out_tokens = out_tokens;
    q.out_capacity = out_capacity;
    const int32_t rc = lb_engine_generate_batch(engine, &q, 1);
    if (rc != LB_STATUS_OK) return rc;
    if (n_out != nullptr) *n_out = q.n_out;
    if (stats != nullptr) *stats = q.stats;
    if (q.status != LB_STATUS_OK) return fail(static_cast<Code>(q.status), q.error);
    return LB_STATUS_OK;
}

void lb_engine_cancel(lb_engine* engine) {
    if (engine != nullptr) engine->engine->cancel();
}

size_t lb_engine_describe(const lb_engine* engine, char* buffer, size_t size) {
    if (engine == nullptr) return 0;
    size_t needed = 0;
    copy_out(engine->engine->describe(), buffer, size, &needed);
    return needed;
}

int32_t lb_engine_scheduler_stats(const lb_engine* engine, lb_scheduler_stats* out) {
    return guarded([&] {
        need(engine, "engine");
        need(out, "out");
        const EngineCounters c = engine->engine->counters();
        *out = lb_scheduler_stats{};
        fill_scheduler_stats(c.scheduler, out);
        out->graph_steps = c.graph_steps;
        out->fused_steps = c.fused_steps;
        out->eager_steps = c.eager_steps;
        out->graphs_captured = c.graphs_captured;
        out->kernel_launches = c.kernel_launches;
        out->pages_in_use = c.pages_in_use;
        out->pages_total = c.pages_total;
        out->h2d_bytes = c.h2d_bytes;
        out->d2h_bytes = c.d2h_bytes;
        out->device_faults = c.device_faults;
    });
}

int32_t lb_engine_context_length(const lb_engine* e) { return e == nullptr ? 0 : static_cast<int32_t>(e->engine->max_positions); }
int32_t lb_engine_vocab_size(const lb_engine* e) { return e == nullptr ? 0 : static_cast<int32_t>(e->engine->loaded().model->spec.vocab_size()); }
double lb_engine_load_ms(const lb_engine* e) { return e == nullptr ? 0.0 : e->engine->load_ms; }
uint64_t lb_engine_weight_bytes(const lb_engine* e) { return e == nullptr ? 0 : e->engine->loaded().model->weight_bytes(); }

// ---- layers one by one -------------------------------------------------------------------------------

int32_t lb_load_plugin(const char* path) {
    return guarded([&] {
        need(path, "path");
        load_plugin(path);
    });
}

int32_t lb_supported_architectures(char* buffer, size_t size, size_t* needed) {
    return guarded([&] { copy_out(Json::array_of(supported_architectures()).dump(), buffer, size, needed); });
}

int32_t lb_config_describe(const char* config_json, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(config_json, "config_json");
        Json raw;
        try {
            raw = Json::parse(config_json, "the configuration");
        } catch (const Error& e) {
            throw invalid_model("{}", e.message());
        }
        copy_out(describe_config(*parse_config(raw)).dump(), buffer, size, needed);
    });
}

int32_t lb_config_describe_folder(const char* model_dir, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(model_dir, "model_dir");
        copy_out(describe_config(*read_config(model_dir)).dump(), buffer, size, needed);
    });
}

int32_t lb_write_random_model(const char* config_json, uint64_t seed, const char* dtype, const char* model_dir) {
    return guarded([&] {
        need(config_json, "config_json");
        need(model_dir, "model_dir");
        const auto cfg = parse_config(Json::parse(config_json, "the configuration"));
        write_random_model(model_dir, *cfg, seed, dtype != nullptr ? dtype : "float32");
    });
}

int32_t lb_normal_values(uint64_t seed, const char* name, int64_t first, int64_t count, double mean, double std, double* out) {
    return guarded([&] {
        need(name, "name");
        need(out, "out");
        normal_values(seed, name, first, count, mean, std, out);
    });
}

double lb_uniform_draw(uint64_t seed, uint64_t stream, uint64_t counter) { return uniform_draw(seed, stream, counter); }

int32_t lb_safetensors_describe(const char* path, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(path, "path");
        SafetensorsFile f(path);
        Json tensors = Json::object();
        for (const auto& e : f.entries())
            tensors.set(e.name, Json::object().set("dtype", safetensors_tag(e.dtype)).set("shape", Json::array_of(e.shape))
                                    .set("bytes", static_cast<int64_t>(e.end - e.begin)));
        copy_out(Json::object().set("metadata", f.metadata()).set("tensors", tensors).dump(), buffer, size, needed);
    });
}

int32_t lb_safetensors_read(const char* path, const char* name, void* out, size_t out_bytes) {
    return guarded([&] {
        need(path, "path");
        need(name, "name");
        SafetensorsFile f(path);
        const TensorEntry* e = f.find(name);
        if (e == nullptr) throw invalid_argument("{} holds no tensor '{}'", path, name);
        if (out_bytes != e->end - e->begin) throw invalid_argument("tensor '{}' has {} bytes, the buffer {}", name, e->end - e->begin, out_bytes);
        if (out_bytes) std::memcpy(out, f.data(*e), out_bytes);
    });
}

int32_t lb_safetensors_write(const char* path, size_t n, const char* const* names, const char* const* dtypes, const int32_t* ranks,
                             const int64_t* shapes, const void* const* data, const char* metadata_json) {
    return guarded([&] {
        need(path, "path");
        std::vector<TensorToWrite> ts;
        size_t at = 0;
        for (size_t i = 0; i < n; ++i) {
            bool known = false;
            const DType dt = dtype_from_safetensors_tag(dtypes[i], &known);
            if (!known) throw invalid_argument("tensor '{}' has dtype {}, which cannot be stored", names[i], dtypes[i]);
            TensorToWrite t{names[i], dt, std::vector<int64_t>(shapes + at, shapes + at + ranks[i]), data[i]};
            at += static_cast<size_t>(ranks[i]);
            ts.push_back(std::move(t));
        }
        write_safetensors(path, ts, metadata_json != nullptr ? Json::parse(metadata_json, "metadata") : Json::object());
    });
}

int32_t lb_weights_load(const char* model_dir, const char* dtype, lb_weights** out) {
    return guarded([&] {
        need(model_dir, "model_dir");
        need(out, "out");
        *out = nullptr;
        const DType compute = compute_dtype_from_name(dtype != nullptr ? dtype : "bfloat16");
        const auto cfg = read_config(model_dir);
        auto w = std::make_unique<lb_weights>();
        w->tensors = load_parameters(model_dir, *cfg, compute);
        *out = w.release();
    });
}

void lb_weights_free(lb_weights* w) { delete w; }

int32_t lb_weights_describe(const lb_weights* w, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(w, "weights");
        Json j = Json::object();
        for (const auto& [name, t] : w->tensors) j.set(name, Json::object().set("dtype", dtype_name(t.dtype)).set("shape", Json::array_of(t.shape)));
        copy_out(j.dump(), buffer, size, needed);
    });
}

int32_t lb_weights_data(const lb_weights* w, const char* name, const void** data, size_t* bytes) {
    return guarded([&] {
        need(w, "weights");
        need(name, "name");
        const auto it = w->tensors.find(name);
        if (it == w->tensors.end()) throw invalid_argument("no parameter '{}'", name);
        *data = it->second.bytes.data();
        *bytes = it->second.bytes.size();
    });
}

// ---- cache manager

int32_t lb_cache_create(const char* needs_json, int32_t page_size, int32_t num_pages, int32_t max_requests, lb_cache** out) {
    return guarded([&] {
        need(needs_json, "needs_json");
        need(out, "out");
        *out = nullptr;
        const Json j = Json::parse(needs_json, "the cache's needs");
        std::map<int, KvNeed> kv;
        std::map<int, StateNeed> state;
        std::map<KvNeed, int> per_group;
        if (const Json* k = j.find("kv"))
            for (const auto& m : k->members()) {
                const auto v = m.second.int_list();
                kv[std::stoi(m.first)] = KvNeed{static_cast<int>(v.at(0)), static_cast<int>(v.at(1)), static_cast<int>(v.at(2))};
            }
        if (const Json* s = j.find("state"))
            for (const auto& m : s->members()) {
                StateNeed need_;
                need_.shape = m.second.at("shape").int_list();
                need_.dtype = m.second.get_string("dtype", "float32") == "float32" ? DType::F32 : DType::BF16;
                state[std::stoi(m.first)] = need_;
            }
        if (const Json* p = j.find("pages_per_group"))
            for (const auto& e : p->items()) {
                const auto v = e.int_list();
                per_group[KvNeed{static_cast<int>(v.at(0)), static_cast<int>(v.at(1)), static_cast<int>(v.at(2))}] = static_cast<int>(v.at(3));
            }
        auto h = std::make_unique<lb_cache>();
        h->owned = std::make_unique<CacheManager>(kv, state, page_size, num_pages, max_requests, DType::F32, false, per_group);
        h->cache = h->owned.get();
        *out = h.release();
    });
}

void lb_cache_destroy(lb_cache* cache) {
    if (cache != nullptr && cache->owned) delete cache;
}

int32_t lb_cache_describe(const lb_cache* c, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(c, "cache");
        Json groups = Json::array();
        for (const auto& g : c->cache->groups)
            groups.push(Json::object().set("units", Json::array_of(g.units)).set("n_kv_head", g.need.n_kv_head).set("head_dim", g.need.head_dim)
                            .set("window", g.need.window).set("num_pages", g.pool.num_pages()).set("page_size", g.page_size));
        Json unit_groups = Json::object();
        for (const auto& [u, g] : c->cache->group_of_unit) unit_groups.set(std::to_string(u), g);
        Json open = Json::object();
        for (const auto& [id, row] : c->cache->states.slot_of) open.set(std::to_string(id), c->cache->length_of_row[static_cast<size_t>(row)]);
        copy_out(Json::object().set("groups", groups).set("group_of_unit", unit_groups).set("page_size", c->cache->page_size)
                     .set("max_requests", c->cache->max_requests).set("lengths", open)
                     .set("bytes_per_token", static_cast<int64_t>(c->cache->bytes_per_token())).dump(), buffer, size, needed);
    });
}

int32_t lb_cache_open(lb_cache* c, int64_t request) { return guarded([&] { need(c, "cache"); c->cache->open(request); }); }
int32_t lb_cache_close(lb_cache* c, int64_t request) { return guarded([&] { need(c, "cache"); c->cache->close(request); }); }
int32_t lb_cache_is_open(const lb_cache* c, int64_t request) { return c != nullptr && c->cache->is_open(request) ? 1 : 0; }
int64_t lb_cache_length(const lb_cache* c, int64_t request) {
    int64_t out = -1;
    guarded([&] { need(c, "cache"); out = c->cache->length(request); });
    return out;
}
int32_t lb_cache_reserve(lb_cache* c, int64_t request, int64_t n_new) { return guarded([&] { need(c, "cache"); c->cache->reserve(request, n_new); }); }
int32_t lb_cache_commit(lb_cache* c, int64_t request, int64_t n_new) { return guarded([&] { need(c, "cache"); c->cache->commit(request, n_new); }); }
int32_t lb_cache_truncate(lb_cache* c, int64_t request, int64_t length) { return guarded([&] { need(c, "cache"); c->cache->truncate(request, length); }); }

int32_t lb_cache_can_reserve(const lb_cache* c, size_t n, const int64_t* requests, const int64_t* n_new, int32_t* out) {
    return guarded([&] {
        need(c, "cache");
        std::vector<int> rows;
        std::vector<int64_t> counts;
        for (size_t i = 0; i < n; ++i) {
            rows.push_back(c->cache->row_of(requests[i]));
            counts.push_back(n_new[i]);
        }
        *out = c->cache->can_reserve_rows(rows, counts) ? 1 : 0;
    });
}

int32_t lb_cache_state_slot(const lb_cache* c, int64_t request, int32_t* out) {
    return guarded([&] { need(c, "cache"); *out = c->cache->row_of(request); });
}

int32_t lb_cache_block_table(const lb_cache* c, int32_t group, size_t n, const int64_t* requests, int32_t* width, int32_t* out, size_t cap) {
    return guarded([&] {
        need(c, "cache");
        need(width, "width");
        std::vector<int> rows;
        for (size_t i = 0; i < n; ++i) rows.push_back(c->cache->row_of(requests[i]));
        int w = *width;
        const auto t = c->cache->table_rows(group, rows, &w);
        *width = w;
        if (out != nullptr) {
            if (cap < t.size()) throw invalid_argument("the block table needs {} entries, the buffer holds {}", t.size(), cap);
            std::memcpy(out, t.data(), t.size() * 4);
        }
    });
}

int32_t lb_cache_slot_mapping(const lb_cache* c, int32_t group, int64_t request, int64_t start, int64_t n, int32_t* out) {
    return guarded([&] {
        need(c, "cache");
        const int row = c->cache->row_of(request);
        for (int64_t i = 0; i < n; ++i) out[i] = c->cache->slot_of(group, row, start + i);
    });
}

int32_t lb_cache_pages(const lb_cache* c, int32_t* in_use, int32_t* free_pages, size_t capacity) {
    return guarded([&] {
        need(c, "cache");
        const auto u = c->cache->pages_in_use(), f = c->cache->free_pages();
        if (capacity < u.size()) throw invalid_argument("the cache has {} groups, the buffers hold {}", u.size(), capacity);
        for (size_t i = 0; i < u.size(); ++i) {
            if (in_use != nullptr) in_use[i] = u[i];
            if (free_pages != nullptr) free_pages[i] = f[i];
        }
    });
}

int32_t lb_cache_state_slots_free(const lb_cache* c) { return c == nullptr ? -1 : c->cache->states.pool.free_count(); }
int32_t lb_cache_check(const lb_cache* c) { return guarded([&] { need(c, "cache"); c->cache->check(); }); }

// ---- scheduler

int32_t lb_scheduler_create(lb_cache* cache, int64_t max_positions, int32_t max_batched_tokens, int32_t max_requests, int64_t eos,
                            lb_scheduler** out) {
    return guarded([&] {
        need(cache, "cache");
        need(out, "out");
        *out = nullptr;
        auto s = std::make_unique<lb_scheduler>();
        s->scheduler = std::make_unique<Scheduler>(*cache->cache, max_positions, max_batched_tokens, max_requests,
                                                   eos >= 0 ? std::optional<int64_t>(eos) : std::nullopt);
        *out = s.release();
    });
}

void lb_scheduler_destroy(lb_scheduler* s) { delete s; }

int32_t lb_scheduler_add(lb_scheduler* s, int64_t request, const int32_t* prompt, size_t n, const lb_sampling_params* params,
                         lb_token_callback callback, void* user_data) {
    return guarded([&] {
        need(s, "scheduler");
        if (s->requests.count(request)) throw invalid_argument("request {} was added before", request);
        auto r = std::make_unique<Request>();
        r->id = request;
        if (n > 0) r->prompt.assign(prompt, prompt + n);
        r->params = to_cpp(params);
        if (callback != nullptr) r->callback = [callback, user_data](int32_t t) { return callback(t, user_data) != 0; };
        s->scheduler->add(r.get());
        s->requests[request] = std::move(r);
    });
}

int32_t lb_scheduler_cancel(lb_scheduler* s, int64_t request) { return guarded([&] { need(s, "scheduler"); s->scheduler->cancel(request); }); }
int32_t lb_scheduler_has_work(const lb_scheduler* s) { return s != nullptr && s->scheduler->has_work() ? 1 : 0; }

int32_t lb_scheduler_plan(lb_scheduler* s, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(s, "scheduler");
        std::vector<Request*> finished;
        const int64_t id = s->next_plan++;
        StepPlan& plan = s->plans[id];
        plan = s->scheduler->plan(&finished);
        while (s->plans.size() > 4) s->plans.erase(s->plans.begin());       // plans that were never stepped
        Json entries = Json::array();
        for (const auto& e : plan.entries) {
            Json toks = Json::array();
            for (int64_t i = e.start; i < e.start + e.count; ++i) toks.push(e.request->tokens[static_cast<size_t>(i)]);
            entries.push(Json::object().set("request", e.request->id).set("start", e.start).set("count", e.count).set("sample", e.sample).set("tokens", toks));
        }
        copy_out(Json::object().set("plan", id).set("entries", entries).set("preempted", ids_json(plan.preempted)).set("finished", ids_json(finished)).dump(),
                 buffer, size, needed);
    });
}

int32_t lb_scheduler_begin_step(lb_scheduler* s, int64_t plan) {
    return guarded([&] {
        need(s, "scheduler");
        const auto it = s->plans.find(plan);
        if (it == s->plans.end()) throw invalid_argument("plan {} is unknown or finished", plan);
        s->scheduler->begin_step(it->second);
    });
}

int32_t lb_scheduler_finish_step(lb_scheduler* s, int64_t plan, const int32_t* sampled, size_t n, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(s, "scheduler");
        const auto it = s->plans.find(plan);
        if (it == s->plans.end()) throw invalid_argument("plan {} is unknown or finished", plan);
        const std::vector<int32_t> ids(sampled, sampled + n);
        const std::string done = ids_json(s->scheduler->finish_step(it->second, ids)).dump();
        s->plans.erase(it);
        copy_out(done, buffer, size, needed);
    });
}

int32_t lb_scheduler_request(const lb_scheduler* s, int64_t request, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(s, "scheduler");
        const auto it = s->requests.find(request);
        if (it == s->requests.end()) throw invalid_argument("request {} is unknown", request);
        const Request& r = *it->second;
        Json j = Json::object();
        j.set("state", state_name(r.state)).set("tokens", Json::array_of(r.tokens)).set("n_prompt", static_cast<int64_t>(r.prompt.size()));
        j.set("n_computed", r.n_computed).set("finish_reason", r.finish_reason == FinishReason::None ? Json(nullptr) : Json(finish_reason_name(r.finish_reason)));
        j.set("error_code", r.error ? static_cast<int>(r.error->code()) : 0).set("error", r.error ? r.error->message() : "");
        j.set("preemptions", r.preemptions).set("seed", r.seed).set("stream", r.stream);
        copy_out(j.dump(), buffer, size, needed);
    });
}

int32_t lb_scheduler_stats_get(const lb_scheduler* s, lb_scheduler_stats* out) {
    return guarded([&] {
        need(s, "scheduler");
        need(out, "out");
        *out = lb_scheduler_stats{};
        fill_scheduler_stats(s->scheduler->stats, out);
    });
}

// ---- replayer

void lb_replayer_options_default(lb_replayer_options* o) {
    if (o == nullptr) return;
    const ReplayerOptions d;
    *o = lb_replayer_options{d.device, d.page_size, d.max_requests, d.num_pages, d.cuda_graphs, d.fused_decode, d.max_step_tokens};
}

int32_t lb_replayer_create(const char* model_dir, const char* dtype, int64_t max_tokens, const lb_replayer_options* options, lb_replayer** out) {
    return guarded([&] {
        need(model_dir, "model_dir");
        need(out, "out");
        *out = nullptr;
        ReplayerOptions o;
        if (options != nullptr) {
            o.device = options->device;
            if (options->page_size > 0) o.page_size = options->page_size;
            if (options->max_requests > 0) o.max_requests = options->max_requests;
            o.num_pages = options->num_pages;
            o.cuda_graphs = options->cuda_graphs != 0;
            o.fused_decode = options->fused_decode != 0;
            o.max_step_tokens = options->max_step_tokens;
        }
        auto h = std::make_unique<lb_replayer>();
        h->replayer = std::make_unique<Replayer>(model_dir, dtype != nullptr ? dtype : "bfloat16", max_tokens, o);
        h->cache_handle.cache = h->replayer->cache.get();
        *out = h.release();
    });
}

void lb_replayer_destroy(lb_replayer* r) { delete r; }
lb_cache* lb_replayer_cache(lb_replayer* r) { return r == nullptr ? nullptr : &r->cache_handle; }

int32_t lb_replayer_describe(const lb_replayer* r, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(r, "replayer");
        const DecoderModel& m = *r->replayer->loaded->model;
        Json kv = Json::array(), st = Json::array(), groups = Json::array();
        for (const auto& kvp : m.kv_needs()) kv.push(kvp.first);
        for (const auto& sp : m.state_needs()) st.push(sp.first);
        for (const auto& g : r->replayer->cache->groups)
            groups.push(Json::object().set("units", Json::array_of(g.units)).set("window", g.need.window).set("num_pages", g.pool.num_pages()));
        copy_out(Json::object().set("spec", m.spec.to_json()).set("kv_units", kv).set("state_units", st).set("max_positions", m.max_positions())
                     .set("vocab_size", m.spec.vocab_size()).set("weight_bytes", static_cast<int64_t>(m.weight_bytes()))
                     .set("fused", r->replayer->stepper->has_fused()).set("capturable", m.capturable()).set("groups", groups).dump(),
                 buffer, size, needed);
    });
}

int32_t lb_replayer_step(lb_replayer* r, size_t n_entries, const int64_t* requests, const int32_t* n_tokens, const int32_t* tokens,
                         const int32_t* n_want, const int32_t* want, float* logits, size_t logits_capacity, int32_t* n_rows) {
    return guarded([&] {
        need(r, "replayer");
        std::vector<StepEntry> entries;
        size_t t_at = 0, w_at = 0;
        for (size_t i = 0; i < n_entries; ++i) {
            entries.push_back({requests[i], tokens + t_at, n_tokens[i], want + w_at, n_want[i]});
            t_at += static_cast<size_t>(n_tokens[i]);
            w_at += static_cast<size_t>(n_want[i]);
        }
        const StepOutput out = r->replayer->step(entries, logits != nullptr ? &r->host_logits : nullptr);
        if (n_rows != nullptr) *n_rows = static_cast<int32_t>(out.rows.size());
        if (logits != nullptr) {
            if (logits_capacity < r->host_logits.size())
                throw invalid_argument("the step's logits need {} floats, the buffer holds {}", r->host_logits.size(), logits_capacity);
            std::memcpy(logits, r->host_logits.data(), r->host_logits.size() * 4);
        }
    });
}

int32_t lb_replayer_set(lb_replayer* r, const char* option, int32_t value) {
    return guarded([&] {
        need(r, "replayer");
        need(option, "option");
        const std::string o = option;
        if (o == "cuda_graphs") r->replayer->stepper->cuda_graphs = value != 0;
        else if (o == "fused_decode" && value == 0) r->replayer->stepper->disable_fused();
        else if (o == "reserve_rows") r->replayer->stepper->workspace.reserve_rows(value);
        else if (o == "fused_stamps") {
            if (r->replayer->stepper->fused() == nullptr) throw invalid_argument("this replayer has no one-kernel decode step to take stamps from");
            r->replayer->stepper->fused()->record_stamps(value != 0);
        }
        else throw invalid_argument("unknown replayer option '{}'", o);
    });
}

int32_t lb_replayer_fused_stamps(lb_replayer* r, uint64_t* out, int32_t capacity, int32_t* n) {
    return guarded([&] {
        need(r, "replayer");
        need(n, "n");
        std::vector<uint64_t> stamps;
        if (r->replayer->stepper->fused() != nullptr) stamps = r->replayer->stepper->fused()->stamps();
        *n = static_cast<int32_t>(stamps.size());
        if (out != nullptr)
            for (int32_t i = 0; i < std::min<int32_t>(capacity, *n); ++i) out[i] = stamps[static_cast<size_t>(i)];
    });
}

int32_t lb_replayer_counters(const lb_replayer* r, char* buffer, size_t size, size_t* needed) {
    return guarded([&] {
        need(r, "replayer");
        const Stepper& s = *r->replayer->stepper;
        copy_out(Json::object().set("steps", s.steps).set("graph_steps", s.graph_steps).set("fused_steps", s.fused_steps).set("eager_steps", s.eager_steps)
                     .set("graphs_captured", s.graphs_captured).set("tokens_run", s.tokens_run).set("kernel_launches", kernels::launches.load()).dump(),
                 buffer, size, needed);
    });
}

int32_t lb_replayer_set_tap(lb_replayer* r, lb_tap_callback tap, void* user_data) {
    return guarded([&] {
        need(r, "replayer");
        if (tap == nullptr) {
            r->replayer->stepper->set_tap({});
            return;
        }
        cudaStream_t stream = r->replayer->loaded->runtime.stream;
        r->replayer->stepper->set_tap([tap, user_data, stream](std::string_view name, const Rows& rows) {
            // The rows as float32 on the host, whatever their type and stride on the device.
            const size_t es = dtype_size(rows.dtype), n = static_cast<size_t>(rows.rows), c = static_cast<size_t>(rows.cols);
            std::vector<uint8_t> raw(n * c * es);
            LIYAB_CUDA(cudaMemcpy2DAsync(raw.data(), c * es, rows.data, static_cast<size_t>(rows.stride) * es, c * es, n, cudaMemcpyDeviceToHost, stream));
            LIYAB_CUDA(cudaStreamSynchronize(stream));
            std::vector<float> f(n * c);
            if (rows.dtype == DType::F32) std::memcpy(f.data(), raw.data(), raw.size());
            else
                for (size_t i = 0; i < n * c; ++i) f[i] = bf16_to_float(reinterpret_cast<const uint16_t*>(raw.data())[i]);
            const std::string nm(name);
            tap(nm.c_str(), f.data(), static_cast<int32_t>(n), static_cast<int32_t>(c), user_data);
        });
    });
}

int32_t lb_replayer_timer_start(lb_replayer* r) {
    return guarded([&] {
        need(r, "replayer");
        cudaStream_t stream = r->replayer->loaded->runtime.stream;
        if (!r->t0) { r->t0 = std::make_unique<Event>(true); r->t1 = std::make_unique<Event>(true); }
        LIYAB_CUDA(cudaStreamSynchronize(stream));
        r->t0->record(stream);
    });
}

int32_t lb_replayer_timer_stop(lb_replayer* r, double* ms) {
    return guarded([&] {
        need(r, "replayer");
        need(ms, "ms");
        if (!r->t0) throw invalid_argument("the timer was not started");
        r->t1->record(r->replayer->loaded->runtime.stream);
        r->t1->synchronize();
        float f = 0;
        LIYAB_CUDA(cudaEventElapsedTime(&f, r->t0->get(), r->t1->get()));
        *ms = f;
    });
}

int32_t lb_device_status(int32_t* words2) {
    return guarded([&] {
        need(words2, "words2");
        int a = 0, b = 0;
        kernels::check(lb_gemm_tcgen05_status(&a), "device_status");
        kernels::check(lb_decode_stack_status(&b), "device_status");
        words2[0] = a;
        words2[1] = b;
    });
}

int32_t lb_debug_set_device_status(int32_t which, int32_t value) {
    return guarded([&] {
        if (which == 0) kernels::check(lb_gemm_tcgen05_status_set(value), "set_device_status");
        else if (which == 1) kernels::check(lb_decode_stack_status_set(value), "set_device_status");
        else throw invalid_argument("status word {} does not exist (0: tcgen05/TMA waits, 1: the fused step's barrier)", which);
    });
}

int32_t lb_debug_withhold_next(int32_t which, int32_t on) {
    return guarded([&] {
        if (which == 0) kernels::check(lb_gemm_tcgen05_withhold_next(on), "withhold_next");
        else if (which == 1) kernels::check(lb_decode_stack_withhold_next(on), "withhold_next");
        else throw invalid_argument("wait {} does not exist (0: the tcgen05 product's accumulator barrier, 1: the fused step's grid barrier)", which);
    });
}

static void to_c_bench(const BenchResult& b, lb_bench_result* out) {
    *out = lb_bench_result{b.ms_total, b.ms_per_step, b.wall_ms_per_step, b.mean_context, b.kernel_launches, b.graph_steps, b.fused_steps,
                           b.eager_steps, b.h2d_bytes_per_step, b.d2h_bytes_per_step, b.checksum};
}

int32_t lb_replayer_bench_decode(lb_replayer* r, int32_t batch, int32_t prompt_len, int32_t steps, int32_t warmup, uint64_t seed, lb_bench_result* out) {
    return guarded([&] {
        need(r, "replayer");
        need(out, "out");
        to_c_bench(bench_decode(*r->replayer, batch, prompt_len, steps, warmup, seed), out);
    });
}

int32_t lb_replayer_bench_prefill(lb_replayer* r, int32_t n_seq, int32_t seq_len, int32_t repeats, uint64_t seed, lb_bench_result* out) {
    return guarded([&] {
        need(r, "replayer");
        need(out, "out");
        to_c_bench(bench_prefill(*r->replayer, n_seq, seq_len, repeats, seed), out);
    });
}

int32_t lb_trace_run_main(int32_t argc, const char* const* argv) {
    std::string model, dtype, out_dir;
    int64_t max_tokens = 0;
    ReplayerOptions options;
    auto usage = [] {
        std::fprintf(stderr, "usage: trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--device D] [--page-size 16|32|64]\n"
                             "Replays given token ids through the engine (steps as JSON lines on standard input) and writes logits.\n");
    };
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&]() -> std::string {
            if (i + 1 >= argc) { usage(); throw invalid_argument("option {} needs a value", a); }
            return argv[++i];
        };
        try {
            if (a == "--model") model = value();
            else if (a == "--dtype") dtype = value();
            else if (a == "--out") out_dir = value();
            else if (a == "--max-tokens") max_tokens = std::stoll(value());
            else if (a == "--device") { std::string d = value(); if (d.rfind("cuda:", 0) == 0) d = d.substr(5); options.device = std::stoi(d); }
            else if (a == "--page-size") options.page_size = std::stoi(value());
            else if (a == "-h" || a == "--help") { usage(); return 0; }
            else { usage(); std::fprintf(stderr, "trace_run: unknown option %s\n", a.c_str()); return 2; }
        } catch (const std::exception& e) {
            std::fprintf(stderr, "trace_run: %s\n", e.what());
            return 2;
        }
    }
    if (model.empty() || dtype.empty() || out_dir.empty() || max_tokens <= 0 || (dtype != "bfloat16" && dtype != "float32") ||
        (options.page_size != 16 && options.page_size != 32 && options.page_size != 64)) {
        usage();
        return 2;
    }
    int rc = 1;
    const int32_t status = guarded([&] { rc = replay_stream(model, dtype, out_dir, max_tokens, options, stdin, stdout); });
    if (status != LB_STATUS_OK) {
        std::fprintf(stderr, "trace_run: %s: %s\n", code_name(static_cast<Code>(status)), lb_last_error());
        return 1;
    }
    return rc;
}

}  // extern "C"
