// Status codes and the one exception type the host raises.
//
// The codes and their numbers are the reference's (include/liyab/types.h:36-48,
// mirrored by the C enum at include/liyab/liyab_c_api.h:41-53), so a caller that
// already switches on liyab's status values keeps working.  Inside the library
// failures travel as `Error`; the C interface turns them into a status and a
// thread-local message (the reference's guarded(): src/c_api/liyab_c_api.cpp:34-58).
#pragma once

#include <exception>
#include <format>
#include <string>
#include <utility>

namespace liyab {

enum class Code : int {
    Ok = 0,
    InvalidArgument = 1,
    Io = 2,
    InvalidModel = 3,
    Unsupported = 4,
    OutOfMemory = 5,
    ContextFull = 6,
    Cancelled = 7,
    Backend = 8,
    Busy = 9,
    Internal = 10,
};

inline const char* code_name(Code c) {
    switch (c) {
        case Code::Ok: return "OK";
        case Code::InvalidArgument: return "INVALID_ARGUMENT";
        case Code::Io: return "IO_ERROR";
        case Code::InvalidModel: return "INVALID_MODEL";
        case Code::Unsupported: return "UNSUPPORTED";
        case Code::OutOfMemory: return "OUT_OF_MEMORY";
        case Code::ContextFull: return "CONTEXT_FULL";
        case Code::Cancelled: return "CANCELLED";
        case Code::Backend: return "BACKEND_ERROR";
        case Code::Busy: return "BUSY";
        case Code::Internal: return "INTERNAL";
    }
    return "INTERNAL";
}

// A failure with a reference status code and a message that names the key,
// tensor or request at fault.
class Error : public std::exception {
public:
    Error(Code code, std::string message)
        : code_(code), message_(std::move(message)), what_(std::string(code_name(code)) + ": " + message_) {}
    Code code() const noexcept { return code_; }
    const std::string& message() const noexcept { return message_; }
    const char* what() const noexcept override { return what_.c_str(); }

private:
    Code code_;
    std::string message_;
    std::string what_;
};

template <class... Args>
Error make_error(Code code, std::format_string<Args...> fmt, Args&&... args) {
    return Error(code, std::format(fmt, std::forward<Args>(args)...));
}
template <class... Args>
Error invalid_argument(std::format_string<Args...> fmt, Args&&... args) {
    return Error(Code::InvalidArgument, std::format(fmt, std::forward<Args>(args)...));
}
template <class... Args>
Error invalid_model(std::format_string<Args...> fmt, Args&&... args) {
    return Error(Code::InvalidModel, std::format(fmt, std::forward<Args>(args)...));
}
template <class... Args>
Error unsupported(std::format_string<Args...> fmt, Args&&... args) {
    return Error(Code::Unsupported, std::format(fmt, std::forward<Args>(args)...));
}
template <class... Args>
Error internal_error(std::format_string<Args...> fmt, Args&&... args) {
    return Error(Code::Internal, std::format(fmt, std::forward<Args>(args)...));
}
template <class... Args>
Error backend_error(std::format_string<Args...> fmt, Args&&... args) {
    return Error(Code::Backend, std::format(fmt, std::forward<Args>(args)...));
}

// A reservation that the free pages cannot cover; nothing was taken.
class OutOfPages : public Error {
public:
    explicit OutOfPages(std::string message) : Error(Code::OutOfMemory, std::move(message)) {}
};

}  // namespace liyab
