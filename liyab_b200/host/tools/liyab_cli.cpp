// The command line, in the manner of the reference's liyab-cli, over the C interface only.
//
// Options keep the reference's names and meanings where it has them
// (tools/liyab_cli.cpp:242-334: -m, -p, -n, --temp, --top-k, --top-p, --seed, --ctx,
// --json, --tokenize, --then) with their defaults (-n 128, --temp 0.8, --top-k 40,
// --top-p 0.95, random seed).  The engine has no tokenizer, so a prompt is a list
// of token ids ("-p 464,3290,318") or `--prompt-len N` random ids; `--kv` becomes
// `--dtype` (the cache has the compute type).  The summary on stderr and the JSON
// lines follow tools/liyab_cli.cpp:145-240.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/liyab_b200.h"

namespace {

void usage() {
    std::fputs(
        "usage: liyab-cli -m MODEL_DIR (-p IDS | --prompt-len N) [options]\n"
        "Generate token ids with the liyab_b200 engine.\n"
        "  -m, --model DIR          model folder (config.json + model.safetensors)\n"
        "  --random-weights CONFIG  no model folder: write one with random weights from this config.json first\n"
        "  --weights-seed N         seed of --random-weights (default 0)\n"
        "  -p, --prompt IDS         prompt token ids, comma separated (repeatable: prompts are served together)\n"
        "  --prompt-len N           instead of -p: this many uniform random token ids\n"
        "  --prompt-seed N          (default 0)\n"
        "  --batch B                with --prompt-len: this many prompts served together (default 1)\n"
        "  --tokenize               print the prompt's token ids and exit\n"
        "  -n N                     max new tokens per turn (default 128)\n"
        "  --then IDS               a follow-up turn (repeatable): the previous prompt, the reply and these ids\n"
        "  --json                   stdout: one JSON line after loading and one per request and turn\n"
        "  --temp T                 temperature, 0 = greedy (default 0.8)\n"
        "  --top-k K                (default 40)\n"
        "  --top-p P                (default 0.95)\n"
        "  --seed N                 RNG seed (default random)\n"
        "  --ignore-eos             do not stop at the end-of-sequence token\n"
        "  --ctx N                  context length (default: the model's)\n"
        "  --dtype T                bfloat16 (default) or float32: compute and cache type\n"
        "  --max-batched-tokens N   token budget of one step (default 2048)\n"
        "  --max-requests N         requests served together (default 64)\n"
        "  --page-size N            positions per cache page (default 16)\n"
        "  --num-pages N            cache pages (default: sized from free memory)\n"
        "  --no-graphs              do not replay captured CUDA graphs\n"
        "  --phases                 time the decode phases (slower) and print them per token\n"
        "  --log-level N            0 debug, 1 info, 2 warn (default), 3 error, 4 off\n",
        stderr);
}

bool parse_ids(const std::string& text, std::vector<int32_t>* out) {
    std::string tok;
    auto flush = [&]() -> bool {
        if (tok.empty()) return true;
        char* end = nullptr;
        const long v = std::strtol(tok.c_str(), &end, 10);
        if (*end != '\0') return false;
        out->push_back(static_cast<int32_t>(v));
        tok.clear();
        return true;
    };
    for (const char c : text) {
        if (c == ',' || c == ' ') {
            if (!flush()) return false;
        } else {
            tok.push_back(c);
        }
    }
    return flush();
}

std::string ids_text(const std::vector<int32_t>& ids, const char* sep) {
    std::string s;
    for (size_t i = 0; i < ids.size(); ++i) s += (i ? sep : "") + std::to_string(ids[i]);
    return s;
}

uint64_t mix(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

const char* finish_name(int r) {
    static const char* names[] = {"unfinished", "eos", "length", "context", "stopped", "cancelled", "error"};
    return r >= 0 && r <= 6 ? names[r] : "?";
}

void print_stats(const lb_generation_stats& s, bool phases) {
    std::fprintf(stderr,
                 "\n=== Generation ===\n"
                 "prompt: %d tokens (0 reused), %.1f ms, TTFT %.1f ms\n"
                 "decode: %d tokens, %.1f ms, %.2f tok/s%s\n"
                 "memory: KV %.1f MiB\n",
                 s.prompt_tokens, s.prefill_ms, s.ttft_ms, s.generated_tokens, s.decode_ms, s.tokens_per_second,
                 s.cancelled ? ", cancelled" : "", static_cast<double>(s.kv_cache_bytes) / 1048576.0);
    if (phases && s.decode_steps > 0) {
        const double n = s.decode_steps;
        std::fprintf(stderr, "decode phases (ms/token): embed %.3f, norms %.3f, attention %.3f, dense ffn %.3f, lm head %.3f\n", s.embed_ms / n,
                     s.norm_ms / n, s.attention_ms / n, s.dense_ffn_ms / n, s.lm_head_ms / n);
    }
}

}  // namespace

int main(int argc, char** argv) {
    std::string model, random_config, dtype = "bfloat16";
    std::vector<std::vector<int32_t>> prompts, then;
    int prompt_len = 0, batch = 1, max_tokens = 128, ctx = 0, max_batched = 2048, max_requests = 64, page_size = 16, num_pages = 0;
    uint64_t prompt_seed = 0, weights_seed = 0, seed = 0;
    float temp = 0.8f, top_p = 0.95f;
    int top_k = 40;
    bool tokenize = false, json = false, ignore_eos = false, graphs = true, phases = false;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&]() -> const char* {
            if (i + 1 >= argc) {
                std::fprintf(stderr, "liyab-cli: option %s needs a value\n", a.c_str());
                std::exit(2);
            }
            return argv[++i];
        };
        if (a == "-m" || a == "--model") model = value();
        else if (a == "--random-weights") random_config = value();
        else if (a == "--weights-seed") weights_seed = std::strtoull(value(), nullptr, 10);
        else if (a == "-p" || a == "--prompt" || a == "--then") {
            std::vector<int32_t> ids;
            const char* v = value();
            if (!parse_ids(v, &ids)) {
                std::fprintf(stderr, "liyab-cli: a prompt is a list of token ids, e.g. 464,3290,318 (got '%s')\n", v);
                return 2;
            }
            (a == "--then" ? then : prompts).push_back(ids);
        } else if (a == "--prompt-len") prompt_len = std::atoi(value());
        else if (a == "--prompt-seed") prompt_seed = std::strtoull(value(), nullptr, 10);
        else if (a == "--batch") batch = std::atoi(value());
        else if (a == "--tokenize") tokenize = true;
        else if (a == "-n") max_tokens = std::atoi(value());
        else if (a == "--json") json = true;
        else if (a == "--temp") temp = static_cast<float>(std::atof(value()));
        else if (a == "--top-k") top_k = std::atoi(value());
        else if (a == "--top-p") top_p = static_cast<float>(std::atof(value()));
        else if (a == "--seed") seed = std::strtoull(value(), nullptr, 10);
        else if (a == "--ignore-eos") ignore_eos = true;
        else if (a == "--ctx") ctx = std::atoi(value());
        else if (a == "--dtype") dtype = value();
        else if (a == "--max-batched-tokens") max_batched = std::atoi(value());
        else if (a == "--max-requests") max_requests = std::atoi(value());
        else if (a == "--page-size") page_size = std::atoi(value());
        else if (a == "--num-pages") num_pages = std::atoi(value());
        else if (a == "--no-graphs") graphs = false;
        else if (a == "--phases") phases = true;
        else if (a == "--log-level") lb_set_log_level(std::atoi(value()));
        else if (a == "-h" || a == "--help") { usage(); return 0; }
        else {
            usage();
            std::fprintf(stderr, "liyab-cli: unknown option %s\n", a.c_str());
            return 2;
        }
    }
    if (dtype == "bf16") dtype = "bfloat16";
    if (dtype == "fp32") dtype = "float32";
    std::string tmp_dir;
    if (!random_config.empty()) {
        std::ifstream f(random_config);
        if (!f) {
            std::fprintf(stderr, "liyab-cli: cannot read %s\n", random_config.c_str());
            return 1;
        }
        std::ostringstream text;
        text << f.rdbuf();
        char templ[] = "/tmp/liyab_b200_model_XXXXXX";
        if (mkdtemp(templ) == nullptr) {
            std::fprintf(stderr, "liyab-cli: cannot make a temporary folder\n");
            return 1;
        }
        tmp_dir = templ;
        if (lb_write_random_model(text.str().c_str(), weights_seed, dtype.c_str(), tmp_dir.c_str()) != LB_STATUS_OK) {
            std::fprintf(stderr, "liyab-cli: %s\n", lb_last_error());
            return 1;
        }
        model = tmp_dir;
    }
    auto cleanup = [&] {
        if (!tmp_dir.empty()) {
            std::remove((tmp_dir + "/config.json").c_str());
            std::remove((tmp_dir + "/model.safetensors").c_str());
            std::remove(tmp_dir.c_str());
        }
    };
    if (model.empty()) {
        std::fprintf(stderr, "liyab-cli: -m MODEL (or --random-weights CONFIG.json) is required\n");
        return 2;
    }
    if (prompts.empty() && prompt_len <= 0) {
        std::fprintf(stderr, "liyab-cli: a prompt is required (-p IDS or --prompt-len N)\n");
        cleanup();
        return 2;
    }
    if (tokenize && prompt_len <= 0) {
        for (const auto& p : prompts) std::printf("%s\n", ids_text(p, " ").c_str());
        cleanup();
        return 0;
    }
    lb_engine_config cfg;
    lb_engine_config_default(&cfg);
    cfg.model_path = model.c_str();
    cfg.dtype = dtype.c_str();
    cfg.context_length = ctx;
    cfg.max_batched_tokens = max_batched;
    cfg.max_sequences = max_requests;
    cfg.page_size = page_size;
    cfg.num_pages = num_pages;
    cfg.cuda_graphs = graphs;
    cfg.profile_phases = phases;
    lb_engine* engine = nullptr;
    if (lb_engine_create(&cfg, &engine) != LB_STATUS_OK) {
        std::fprintf(stderr, "liyab-cli: %s\n", lb_last_error());
        cleanup();
        return 1;
    }
    char text[1024];
    lb_engine_describe(engine, text, sizeof text);
    if (json) {
        std::string escaped;
        for (const char* c = text; *c; ++c) {
            if (*c == '"' || *c == '\\') escaped.push_back('\\');
            escaped.push_back(*c);
        }
        std::printf("{\"load_ms\": %.1f, \"context\": %d, \"describe\": \"%s\"}\n", lb_engine_load_ms(engine), lb_engine_context_length(engine),
                    escaped.c_str());
        std::fflush(stdout);
    } else {
        std::fprintf(stderr, "%s\n", text);
    }
    if (prompt_len > 0) {
        const uint64_t vocab = static_cast<uint64_t>(lb_engine_vocab_size(engine));
        for (int b = 0; b < (batch > 0 ? batch : 1); ++b) {
            std::vector<int32_t> p;
            for (int i = 0; i < prompt_len; ++i)
                p.push_back(static_cast<int32_t>(mix(prompt_seed * 0x632BE59BD9B4E019ull + static_cast<uint64_t>(b) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(i)) % vocab));
            prompts.push_back(std::move(p));
        }
        if (tokenize) {
            for (const auto& p : prompts) std::printf("%s\n", ids_text(p, " ").c_str());
            lb_engine_destroy(engine);
            cleanup();
            return 0;
        }
    }
    lb_sampling_params params;
    lb_sampling_params_default(&params);
    params.temperature = temp;
    params.top_k = top_k;
    params.top_p = top_p;
    params.seed = seed;
    params.max_tokens = max_tokens;
    params.ignore_eos = ignore_eos;
    int rc = 0;
    std::vector<std::vector<int32_t>> replies(prompts.size());
    for (size_t turn = 0; turn <= then.size(); ++turn) {
        if (turn > 0)
            for (size_t i = 0; i < prompts.size(); ++i) {
                prompts[i].insert(prompts[i].end(), replies[i].begin(), replies[i].end());
                prompts[i].insert(prompts[i].end(), then[turn - 1].begin(), then[turn - 1].end());
            }
        std::vector<lb_request> requests(prompts.size());
        for (size_t i = 0; i < prompts.size(); ++i) {
            requests[i] = lb_request{};
            requests[i].tokens = prompts[i].data();
            requests[i].n_tokens = prompts[i].size();
            requests[i].params = params;
            replies[i].assign(static_cast<size_t>(max_tokens > 0 ? max_tokens : 1), 0);
            requests[i].out_tokens = replies[i].data();
            requests[i].out_capacity = replies[i].size();
        }
        if (lb_engine_generate_batch(engine, requests.data(), requests.size()) != LB_STATUS_OK) {
            std::fprintf(stderr, "liyab-cli: %s\n", lb_last_error());
            rc = 1;
            break;
        }
        for (size_t i = 0; i < requests.size(); ++i) {
            const lb_request& q = requests[i];
            replies[i].resize(std::min(q.n_out, replies[i].size()));
            if (q.status != LB_STATUS_OK) std::fprintf(stderr, "liyab-cli: %s\n", q.error);
            const lb_generation_stats& s = q.stats;
            if (json) {
                std::printf("{\"prompt_tokens\": %d, \"generated_tokens\": %d, \"prefill_ms\": %.3f, \"decode_ms\": %.3f, \"ttft_ms\": %.3f, "
                            "\"tokens_per_second\": %.2f, \"kv_cache_bytes\": %llu, \"finish_reason\": \"%s\", \"tokens\": [%s]}\n",
                            s.prompt_tokens, s.generated_tokens, s.prefill_ms, s.decode_ms, s.ttft_ms, s.tokens_per_second,
                            static_cast<unsigned long long>(s.kv_cache_bytes), finish_name(s.finish_reason), ids_text(replies[i], ", ").c_str());
                std::fflush(stdout);
            } else {
                std::printf("%s\n", ids_text(replies[i], " ").c_str());
                std::fflush(stdout);
                print_stats(s, phases);
            }
        }
    }
    lb_scheduler_stats st;
    if (lb_engine_scheduler_stats(engine, &st) == LB_STATUS_OK && !json)
        std::fprintf(stderr,
                     "scheduler: %llu steps (%llu fused, %llu graph, %llu part by part), %llu tokens batched (%llu prompt, %llu decode), "
                     "%llu preemptions, peak %d running\n",
                     static_cast<unsigned long long>(st.steps), static_cast<unsigned long long>(st.fused_steps),
                     static_cast<unsigned long long>(st.graph_steps), static_cast<unsigned long long>(st.eager_steps),
                     static_cast<unsigned long long>(st.batched_tokens), static_cast<unsigned long long>(st.prefill_tokens),
                     static_cast<unsigned long long>(st.decode_tokens), static_cast<unsigned long long>(st.preemptions), st.peak_running);
    lb_engine_destroy(engine);
    cleanup();
    return rc;
}
