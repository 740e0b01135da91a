// Leveled diagnostics with an optional sink, after the reference's logger
// (src/core/log.h:14-35; C face include/liyab/liyab_c_api.h:200-221): levels
// 0 debug, 1 info, 2 warn (default), 3 error, 4 off.  Messages at or above the
// level go to the callback when one is set, else to stderr.
#pragma once

#include <format>
#include <string>

namespace liyab {

enum class LogLevel : int { Debug = 0, Info = 1, Warn = 2, Error = 3, Off = 4 };
using LogSink = void (*)(int level, const char* message, void* user);

void set_log_level(int level);
int log_level();
void set_log_sink(LogSink sink, void* user);
void log_message(LogLevel level, const std::string& message);

template <class... Args>
void log(LogLevel level, std::format_string<Args...> fmt, Args&&... args) {
    if (static_cast<int>(level) >= log_level()) log_message(level, std::format(fmt, std::forward<Args>(args)...));
}

}  // namespace liyab
