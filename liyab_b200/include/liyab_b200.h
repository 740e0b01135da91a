/*
 * liyab_b200: the engine's C interface.
 *
 * The surface follows the reference's (include/liyab/liyab_c_api.h): an opaque
 * engine handle, structs initialised by their *_default() function before use (so
 * fields can be appended without breaking callers), one status per call in the
 * reference's numbering, and the description of the most recent failure on the
 * calling thread from lb_last_error().  No C++ exception crosses this boundary.
 * A NULL handle fails with LB_ERR_INVALID_ARGUMENT.  Strings passed in are UTF-8
 * and only borrowed for the call's duration.  Token ids go in and come out; the
 * engine has no tokenizer.
 *
 * Three layers are exported:
 *   1. the engine: create, generate (one prompt or a batch), cancel, describe,
 *      statistics, logging;
 *   2. the engine's layers one by one, for tools and tests: configuration and
 *      registry, model files and random weights, the cache manager, the
 *      scheduler, the step function (a "replayer": model + cache + step);
 *   3. the kernels (csrc/api.h), on raw device pointers.
 */
#ifndef LIYAB_B200_H
#define LIYAB_B200_H

#include <stddef.h>
#include <stdint.h>

#define LB_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

typedef enum lb_status_code {
    LB_STATUS_OK = 0,
    LB_STATUS_INVALID_ARGUMENT = 1,
    LB_STATUS_IO = 2,
    LB_STATUS_INVALID_MODEL = 3,
    LB_STATUS_UNSUPPORTED = 4,
    LB_STATUS_OUT_OF_MEMORY = 5,
    LB_STATUS_CONTEXT_FULL = 6,
    LB_STATUS_CANCELLED = 7,
    LB_STATUS_BACKEND = 8,
    LB_STATUS_BUSY = 9,
    LB_STATUS_INTERNAL = 10
} lb_status_code;

typedef struct lb_engine lb_engine;

typedef struct lb_engine_config {
    const char* model_path;        /* required: folder with config.json and model.safetensors (or its shards) */
    const char* dtype;             /* "bfloat16" (default) or "float32": compute and cache type */
    int32_t device;                /* CUDA device (default 0) */
    int32_t context_length;        /* 0: the model's positions */
    int32_t max_batched_tokens;    /* token budget of one step (default 2048) */
    int32_t max_sequences;         /* requests served together (default 64) */
    int32_t page_size;             /* positions per cache page (default 16) */
    int32_t num_pages;             /* 0: enough for max_sequences full contexts, within kv_memory_fraction */
    float kv_memory_fraction;      /* of the free device memory, at most, for the cache when num_pages is 0 (default 0.5) */
    int32_t cuda_graphs;           /* nonzero (default): replay captured graphs for steps whose shape repeats */
    int32_t fused_decode;          /* nonzero: decode steps of up to 16 requests run as one persistent kernel where that
                                      kernel takes the model.  Default 0: the part-by-part path (one-launch products,
                                      launches that overlap the kernel before, a captured graph) is faster at every
                                      size measured */
    int32_t pipeline;              /* nonzero (default): plan and launch step n+1 while step n runs */
    int32_t profile_phases;        /* nonzero: time every step's phases (slower: part by part, one step at a time) */
} lb_engine_config;

typedef struct lb_sampling_params {
    float temperature;             /* <= 0: greedy (default 0.8) */
    int32_t top_k;                 /* <= 0: disabled (default 40) */
    float top_p;                   /* >= 1: disabled (default 0.95) */
    uint64_t seed;                 /* 0: random */
    int32_t max_tokens;            /* default 256 */
    int32_t ignore_eos;            /* nonzero: do not stop at the end-of-sequence token */
} lb_sampling_params;

enum { LB_FINISH_NONE = 0, LB_FINISH_EOS = 1, LB_FINISH_LENGTH = 2, LB_FINISH_CONTEXT = 3, LB_FINISH_STOPPED = 4,
       LB_FINISH_CANCELLED = 5, LB_FINISH_ERROR = 6 };

typedef struct lb_generation_stats {
    int32_t prompt_tokens;
    int32_t generated_tokens;
    double prefill_ms;
    double decode_ms;
    double tokens_per_second;
    int32_t cancelled;
    uint64_t kv_cache_bytes;
    double ttft_ms;
    int32_t preemptions;
    int32_t finish_reason;         /* LB_FINISH_* */
    /* Decode time by phase, ms (decode steps only; filled when the engine profiles phases) */
    int32_t decode_steps;
    double embed_ms;
    double norm_ms;
    double attention_ms;           /* the mixers */
    double dense_ffn_ms;           /* the feed-forwards */
    double lm_head_ms;             /* final norm and output projection */
} lb_generation_stats;

/* Called with each new token on the thread that called generate; return nonzero to continue, 0 to stop. */
typedef int32_t (*lb_token_callback)(int32_t token, void* user_data);

/* One request of a batch.  `out_tokens` (capacity `out_capacity`) receives the generated ids, `n_out` their
 * number (the number generated, even when larger than the capacity); `status` and `error` the request's own
 * outcome (a request that ran out of cache pages fails alone). */
typedef struct lb_request {
    const int32_t* tokens;
    size_t n_tokens;
    lb_sampling_params params;
    lb_token_callback callback;    /* may be NULL */
    void* user_data;
    int32_t* out_tokens;           /* may be NULL */
    size_t out_capacity;
    size_t n_out;
    int32_t status;                /* lb_status_code */
    char error[256];
    lb_generation_stats stats;
} lb_request;

/* How the scheduler batched since the engine was created (the reference's SchedulerStats, engine.h:1036-1045). */
typedef struct lb_scheduler_stats {
    uint64_t steps;
    uint64_t batched_tokens;
    uint64_t prefill_tokens;
    uint64_t decode_tokens;
    uint64_t preemptions;
    uint64_t finished;
    int32_t peak_running;
    uint64_t histogram[7];         /* steps by batched tokens: 1, 2-8, 9-32, 33-128, 129-512, 513-2048, more */
    uint64_t graph_steps;          /* steps replayed from a captured CUDA graph */
    uint64_t fused_steps;          /* steps run by the one-kernel decode step */
    uint64_t eager_steps;          /* steps launched part by part */
    uint64_t graphs_captured;
    uint64_t kernel_launches;      /* launches of this library's kernels by this process */
    int32_t pages_in_use;
    int32_t pages_total;
    uint64_t h2d_bytes;            /* copied by steps, host to device */
    uint64_t d2h_bytes;
    int32_t device_faults;         /* steps whose kernels reported a bounded wait that ran out */
} lb_scheduler_stats;

LB_API const char* lb_version(void);
LB_API const char* lb_last_error(void);

/* Diagnostics. Levels: 0 debug, 1 info, 2 warn (default), 3 error, 4 off. The callback receives every
 * message at or above the level; NULL removes it (messages then go to stderr). */
typedef void (*lb_log_callback)(int32_t level, const char* message, void* user_data);
LB_API void lb_set_log_level(int32_t level);
LB_API void lb_set_log_callback(lb_log_callback callback, void* user_data);

LB_API void lb_engine_config_default(lb_engine_config* config);
LB_API void lb_sampling_params_default(lb_sampling_params* params);

/* Loads the model and sizes the cache. *out_engine is set on success. */
LB_API int32_t lb_engine_create(const lb_engine_config* config, lb_engine** out_engine);
LB_API void lb_engine_destroy(lb_engine* engine);

/* Blocking generation after the prompt `tokens`; generated ids arrive through `callback` (may be NULL) and in
 * `out_tokens` (may be NULL; *n_out receives their number). `stats` may be NULL. Cancellation is not an error:
 * LB_STATUS_OK with stats->cancelled = 1. One call at a time per engine (LB_STATUS_BUSY otherwise). */
LB_API int32_t lb_engine_generate_tokens(lb_engine* engine, const int32_t* tokens, size_t n_tokens,
                                         const lb_sampling_params* params, lb_token_callback callback, void* user_data,
                                         int32_t* out_tokens, size_t out_capacity, size_t* n_out, lb_generation_stats* stats);
/* The same for several prompts served together, each with its own options and outcome. */
LB_API int32_t lb_engine_generate_batch(lb_engine* engine, lb_request* requests, size_t n_requests);
/* Thread-safe; stops the running call's requests at their next token. */
LB_API void lb_engine_cancel(lb_engine* engine);
/* Writes a NUL-terminated summary of the model into `buffer` (truncated to `size`); returns the length the
 * full text needs, excluding NUL. */
LB_API size_t lb_engine_describe(const lb_engine* engine, char* buffer, size_t size);
LB_API int32_t lb_engine_scheduler_stats(const lb_engine* engine, lb_scheduler_stats* out);
LB_API int32_t lb_engine_context_length(const lb_engine* engine);
LB_API int32_t lb_engine_vocab_size(const lb_engine* engine);
LB_API double lb_engine_load_ms(const lb_engine* engine);
LB_API uint64_t lb_engine_weight_bytes(const lb_engine* engine);

/* ---- the engine's layers one by one (tools and tests) --------------------------------------------------
 * Functions that return text write a NUL-terminated string into `buffer` (truncated to `size`) and store the
 * length the full text needs in *needed. */

/* Registers the parts and architectures of a shared object (its `liyab_b200_plugin_init`). */
LB_API int32_t lb_load_plugin(const char* path);
LB_API int32_t lb_supported_architectures(char* buffer, size_t size, size_t* needed);      /* JSON array */
/* {"architecture", "config": typed configuration, "spec": model description, "checkpoint": parameter -> file tensors}
 * from the text of a config.json, or from a model folder. */
LB_API int32_t lb_config_describe(const char* config_json, char* buffer, size_t size, size_t* needed);
LB_API int32_t lb_config_describe_folder(const char* model_dir, char* buffer, size_t size, size_t* needed);
LB_API int32_t lb_write_random_model(const char* config_json, uint64_t seed, const char* dtype, const char* model_dir);
LB_API int32_t lb_normal_values(uint64_t seed, const char* name, int64_t first, int64_t count, double mean, double std, double* out);
LB_API double lb_uniform_draw(uint64_t seed, uint64_t stream, uint64_t counter);

/* A safetensors file: header as JSON {"metadata", "tensors": {name: {dtype, shape}}}; one tensor's bytes. */
LB_API int32_t lb_safetensors_describe(const char* path, char* buffer, size_t size, size_t* needed);
LB_API int32_t lb_safetensors_read(const char* path, const char* name, void* out, size_t out_bytes);
/* dtypes as safetensors tags ("F32", "BF16", ...); shapes flattened, `ranks[i]` dims each. */
LB_API int32_t lb_safetensors_write(const char* path, size_t n, const char* const* names, const char* const* dtypes,
                                    const int32_t* ranks, const int64_t* shapes, const void* const* data, const char* metadata_json);

/* The parameters of a model folder on the host, transformed and in their storage types for `dtype`. */
typedef struct lb_weights lb_weights;
LB_API int32_t lb_weights_load(const char* model_dir, const char* dtype, lb_weights** out);
LB_API void lb_weights_free(lb_weights* w);
LB_API int32_t lb_weights_describe(const lb_weights* w, char* buffer, size_t size, size_t* needed);   /* {name: {dtype, shape}} */
LB_API int32_t lb_weights_data(const lb_weights* w, const char* name, const void** data, size_t* bytes);

/* The cache manager (host bookkeeping only, no device storage).  `needs_json`:
 * {"kv": {"<unit>": [n_kv_head, head_dim, window]}, "state": {"<unit>": {"shape": [...], "dtype": "float32"}},
 *  "pages_per_group": [[n_kv_head, head_dim, window, pages]]}. */
typedef struct lb_cache lb_cache;
LB_API int32_t lb_cache_create(const char* needs_json, int32_t page_size, int32_t num_pages, int32_t max_requests, lb_cache** out);
LB_API void lb_cache_destroy(lb_cache* cache);
LB_API int32_t lb_cache_describe(const lb_cache* cache, char* buffer, size_t size, size_t* needed);
LB_API int32_t lb_cache_open(lb_cache* cache, int64_t request);
LB_API int32_t lb_cache_close(lb_cache* cache, int64_t request);
LB_API int32_t lb_cache_is_open(const lb_cache* cache, int64_t request);
LB_API int64_t lb_cache_length(const lb_cache* cache, int64_t request);                      /* -1 on error */
LB_API int32_t lb_cache_reserve(lb_cache* cache, int64_t request, int64_t n_new);
LB_API int32_t lb_cache_commit(lb_cache* cache, int64_t request, int64_t n_new);
LB_API int32_t lb_cache_truncate(lb_cache* cache, int64_t request, int64_t length);
LB_API int32_t lb_cache_can_reserve(const lb_cache* cache, size_t n, const int64_t* requests, const int64_t* n_new, int32_t* out);
LB_API int32_t lb_cache_state_slot(const lb_cache* cache, int64_t request, int32_t* out);
/* Block tables of `requests` in `group`, row-major [n, *width]; *width 0 on entry: the widest of them. */
LB_API int32_t lb_cache_block_table(const lb_cache* cache, int32_t group, size_t n, const int64_t* requests, int32_t* width,
                                    int32_t* out, size_t out_capacity);
LB_API int32_t lb_cache_slot_mapping(const lb_cache* cache, int32_t group, int64_t request, int64_t start, int64_t n, int32_t* out);
LB_API int32_t lb_cache_pages(const lb_cache* cache, int32_t* in_use, int32_t* free_pages, size_t capacity);   /* per group */
LB_API int32_t lb_cache_state_slots_free(const lb_cache* cache);
LB_API int32_t lb_cache_check(const lb_cache* cache);

/* The scheduler over a cache manager (the caller plays the step function). */
typedef struct lb_scheduler lb_scheduler;
LB_API int32_t lb_scheduler_create(lb_cache* cache, int64_t max_positions, int32_t max_batched_tokens, int32_t max_requests,
                                   int64_t eos_token_id /* -1: none */, lb_scheduler** out);
LB_API void lb_scheduler_destroy(lb_scheduler* s);
LB_API int32_t lb_scheduler_add(lb_scheduler* s, int64_t request, const int32_t* prompt, size_t n, const lb_sampling_params* params,
                                lb_token_callback callback, void* user_data);
LB_API int32_t lb_scheduler_cancel(lb_scheduler* s, int64_t request);
LB_API int32_t lb_scheduler_has_work(const lb_scheduler* s);
/* Plans the next step; a JSON object {"plan": id, "entries": [{"request", "start", "count", "sample", "tokens"}],
 * "preempted": [ids], "finished": [ids]}.  A plan lives until its lb_scheduler_finish_step (a host that runs one
 * step ahead holds two). */
LB_API int32_t lb_scheduler_plan(lb_scheduler* s, char* buffer, size_t size, size_t* needed);
LB_API int32_t lb_scheduler_begin_step(lb_scheduler* s, int64_t plan);
/* `sampled`: one id per planned entry with "sample", in the plan's order; the finished requests' ids as JSON. */
LB_API int32_t lb_scheduler_finish_step(lb_scheduler* s, int64_t plan, const int32_t* sampled, size_t n, char* buffer, size_t size,
                                        size_t* needed);
/* {"state", "tokens", "n_prompt", "n_computed", "finish_reason", "error_code", "error", "preemptions", "seed", "stream"} */
LB_API int32_t lb_scheduler_request(const lb_scheduler* s, int64_t request, char* buffer, size_t size, size_t* needed);
LB_API int32_t lb_scheduler_stats_get(const lb_scheduler* s, lb_scheduler_stats* out);

/* A replayer: a model, a cache for `max_tokens` live tokens and the step function. */
typedef struct lb_replayer lb_replayer;
typedef struct lb_replayer_options {
    int32_t device;
    int32_t page_size;             /* default 16 */
    int32_t max_requests;          /* default 16 */
    int32_t num_pages;             /* 0: from max_tokens */
    int32_t cuda_graphs;           /* default 0 */
    int32_t fused_decode;          /* default 0; as lb_engine_config */
    int32_t max_step_tokens;       /* scratch sized up front (0: grows on demand; steps with portions are captured only within it) */
} lb_replayer_options;
LB_API void lb_replayer_options_default(lb_replayer_options* options);
LB_API int32_t lb_replayer_create(const char* model_dir, const char* dtype, int64_t max_tokens, const lb_replayer_options* options,
                                  lb_replayer** out);
LB_API void lb_replayer_destroy(lb_replayer* r);
LB_API lb_cache* lb_replayer_cache(lb_replayer* r);                                           /* borrowed */
/* {"spec", "kv_units", "state_units", "max_positions", "vocab_size", "weight_bytes", "fused", "capturable", "groups"} */
LB_API int32_t lb_replayer_describe(const lb_replayer* r, char* buffer, size_t size, size_t* needed);
/* One step: entry i brings n_tokens[i] tokens (flattened in `tokens`) and wants n_want[i] places (flattened in `want`).
 * The logits at the wanted places, [*n_rows, vocab] float32, are copied to `logits` (host; may be NULL). */
LB_API int32_t lb_replayer_step(lb_replayer* r, size_t n_entries, const int64_t* requests, const int32_t* n_tokens,
                                const int32_t* tokens, const int32_t* n_want, const int32_t* want, float* logits,
                                size_t logits_capacity, int32_t* n_rows);
/* Options at run time: "cuda_graphs" 0/1, "fused_decode" 0 (cannot be switched back on). */
LB_API int32_t lb_replayer_set(lb_replayer* r, const char* option, int32_t value);
/* {"steps", "graph_steps", "fused_steps", "eager_steps", "graphs_captured", "tokens_run", "kernel_launches"} */
/* Time stamps from inside the one-kernel decode step (a measuring aid): after lb_replayer_set(r, "fused_stamps", 1)
 * every such step has block 0 write the device's global timer (ns) after each grid barrier (entry = the barrier's
 * number, from 1), at marks inside the phases (entries 128 + 8 * layer + mark) and every block its arrival at the five
 * barriers of layer 5 (entries 256 + 160 * barrier + block).  Copies the last step's stamps out; *n = how many exist. */
LB_API int32_t lb_replayer_fused_stamps(lb_replayer* r, uint64_t* out, int32_t capacity, int32_t* n);
LB_API int32_t lb_replayer_counters(const lb_replayer* r, char* buffer, size_t size, size_t* needed);
/* Every part's output of the following steps is handed to `tap` as float32 rows on the host (NULL removes it). */
typedef void (*lb_tap_callback)(const char* name, const float* rows, int32_t n_rows, int32_t n_cols, void* user_data);
LB_API int32_t lb_replayer_set_tap(lb_replayer* r, lb_tap_callback tap, void* user_data);
/* Device-timed work on the replayer's stream: lb_replayer_timer_start, steps, lb_replayer_timer_stop -> milliseconds. */
LB_API int32_t lb_replayer_timer_start(lb_replayer* r);
LB_API int32_t lb_replayer_timer_stop(lb_replayer* r, double* ms);
/* Reads and clears the two device status words (tcgen05/TMA waits, the fused step's barrier); synchronises. */
LB_API int32_t lb_device_status(int32_t* words2);
/* Writes status word `which` (0 or 1) as a kernel whose bounded wait ran out would: for tests of what the engine does
 * when a step reports one (its requests end with LB_STATUS_INTERNAL, the words are cleared, a failing fused step is
 * switched off, the engine goes on). */
LB_API int32_t lb_debug_set_device_status(int32_t which, int32_t value);
/* With `on`, the next launch of kernel family `which` (0: the one-tile tcgen05 product, 1: the one-kernel decode
 * step) meets a wait that nothing ends, once.  Its bounded wait runs to its limit (about two seconds), sets the
 * status word and the kernel returns; the context stays usable.  Without `on`, takes an order back that no launch
 * has used yet.  For tests of that path. */
LB_API int32_t lb_debug_withhold_next(int32_t which, int32_t on);

/* Measurements on a replayer, timed on the device with events around exactly the stated work (the reference's
 * liyab-bench and liyab-seq-bench are programs of the engine too: tools/liyab_bench.cpp, tools/liyab_seq_bench.cpp).
 * Decode: `batch` requests get `prompt_len`-token prompts (uniform ids from `seed`), then `warmup` untimed and
 * `steps` timed decode steps run the way the engine runs them: greedy sampling on the device, the sampled ids
 * feeding the next step without leaving the device, their copy to the host overlapped with it.  A request that
 * reaches the model's last position is cut back to its prompt, so any number of steps can be timed. */
typedef struct lb_bench_result {
    double ms_total;               /* device time of the timed region */
    double ms_per_step;
    double wall_ms_per_step;
    double mean_context;           /* positions attended per request and step, averaged over the timed steps */
    uint64_t kernel_launches;      /* inside the timed region */
    uint64_t graph_steps, fused_steps, eager_steps;
    uint64_t h2d_bytes_per_step, d2h_bytes_per_step;
    uint64_t checksum;             /* of the ids sampled in the timed region (equal runs give equal sums) */
} lb_bench_result;
LB_API int32_t lb_replayer_bench_decode(lb_replayer* r, int32_t batch, int32_t prompt_len, int32_t steps, int32_t warmup,
                                        uint64_t seed, lb_bench_result* out);
/* Prefill: `n_seq` prompts of `seq_len` tokens in one step, logits at each last token; `repeats` timed runs after
 * two untimed ones; ms_per_step is the best, wall_ms_per_step the median. */
LB_API int32_t lb_replayer_bench_prefill(lb_replayer* r, int32_t n_seq, int32_t seq_len, int32_t repeats, uint64_t seed,
                                         lb_bench_result* out);

/* The body of bin/trace_run (arguments as its --help says; steps from standard input). */
LB_API int32_t lb_trace_run_main(int32_t argc, const char* const* argv);

#ifdef __cplusplus
}
#endif

#endif /* LIYAB_B200_H */
