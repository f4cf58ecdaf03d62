// Status codes of the engine's C interface and the exception that carries them inside the host.
//
// Every exported function returns one of these integers; the message of the last failure of the
// calling thread is read with fg_last_error().  The reference reports failures by printing a line
// and returning NULL / -1 (missing tensor: fastgguf.c:4154-4164; bad config: :4215-4218; load
// errors exit 2: :5224-5228); here the line is kept for the caller instead of printed.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <stdexcept>
#include <string>

#include "../fastgguf_engine.h"

namespace fg {

struct Error : std::runtime_error {
    int code;
    Error(int code_, const std::string &msg) : std::runtime_error(msg), code(code_) {}
};

inline std::string format(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    va_list ap2;
    va_copy(ap2, ap);
    int n = vsnprintf(nullptr, 0, fmt, ap);
    va_end(ap);
    std::string s((size_t)(n > 0 ? n : 0), '\0');
    if (n > 0) vsnprintf(&s[0], (size_t)n + 1, fmt, ap2);
    va_end(ap2);
    return s;
}

[[noreturn]] inline void fail(int code, const std::string &msg) { throw Error(code, msg); }

}  // namespace fg
