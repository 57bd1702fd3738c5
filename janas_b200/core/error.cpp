#include "error.h"

#include <cstdio>
#include <new>
#include <vector>

#include "json.h"

namespace jb {

std::string fmt(const char *f, ...) {
    va_list ap;
    va_start(ap, f);
    va_list ap2;
    va_copy(ap2, ap);
    int n = vsnprintf(nullptr, 0, f, ap);
    va_end(ap);
    std::vector<char> buf((size_t)(n < 0 ? 0 : n) + 1);
    vsnprintf(buf.data(), buf.size(), f, ap2);
    va_end(ap2);
    return std::string(buf.data());
}

static thread_local std::string t_last_error;

const char *last_error() { return t_last_error.c_str(); }
void set_last_error(const std::string &m) { t_last_error = m; }

int32_t guard(const std::function<void()> &f) noexcept {
    try {
        f();
        return JB_LLM_OK;
    } catch (const Error &e) {
        try { t_last_error = e.what(); } catch (...) {}
        return e.code;
    } catch (const JsonError &e) {
        try { t_last_error = std::string("not JSON: ") + e.what(); } catch (...) {}
        return JB_LLM_EINVAL;
    } catch (const std::bad_alloc &) {
        try { t_last_error = "out of memory"; } catch (...) {}
        return JB_LLM_ENOMEM;
    } catch (const std::exception &e) {
        try { t_last_error = e.what(); } catch (...) {}
        return JB_LLM_EFAIL;
    } catch (...) {
        try { t_last_error = "unknown failure"; } catch (...) {}
        return JB_LLM_EFAIL;
    }
}

}  // namespace jb
