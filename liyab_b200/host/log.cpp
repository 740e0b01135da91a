#include "log.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace liyab {
namespace {
std::atomic<int> g_level{[] {
    const char* env = std::getenv("LIYAB_B200_LOG");
    return env != nullptr ? std::atoi(env) : static_cast<int>(LogLevel::Warn);
}()};
std::mutex g_mutex;
LogSink g_sink = nullptr;
void* g_user = nullptr;
}  // namespace

void set_log_level(int level) { g_level.store(level < 0 ? 0 : (level > 4 ? 4 : level)); }
int log_level() { return g_level.load(std::memory_order_relaxed); }

void set_log_sink(LogSink sink, void* user) {
    std::lock_guard<std::mutex> lock(g_mutex);
    g_sink = sink;
    g_user = user;
}

void log_message(LogLevel level, const std::string& message) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_sink != nullptr) {
        g_sink(static_cast<int>(level), message.c_str(), g_user);
        return;
    }
    static const char* names[] = {"debug", "info", "warn", "error"};
    std::fprintf(stderr, "[liyab_b200 %s] %s\n", names[static_cast<int>(level) & 3], message.c_str());
    std::fflush(stderr);
}

}  // namespace liyab
