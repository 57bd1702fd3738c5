// Error codes of the C interface and the one exception type that carries them.
//
// The codes and their meanings are the reference's (include/janas/llm.h:43-53):
// every call of the C interface returns one of them and leaves a text for the
// calling thread (jb_llm_last_error, as janas_llm_last_error :74).  Inside the
// library a failure is a jb::Error thrown where it is found; the C interface
// catches it at the boundary (core/error.cpp: guard).
#pragma once

#include <cstdarg>
#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>

#define JB_LLM_OK 0
#define JB_LLM_DONE 1
#define JB_LLM_EINVAL (-1)  /* invalid argument */
#define JB_LLM_ENOMEM (-2)  /* out of memory (host or device) */
#define JB_LLM_EOPEN (-3)   /* model folder missing, unreadable, invalid */
#define JB_LLM_EMODEL (-4)  /* model not supported (architecture) */
#define JB_LLM_EFULL (-5)   /* the context or the cache is full */
#define JB_LLM_EBUSY (-6)   /* the object is in use */
#define JB_LLM_ESMALL (-7)  /* buffer too small */
#define JB_LLM_EFAIL (-8)   /* internal failure (a CUDA call, a kernel's bounded wait) */
#define JB_LLM_ELIMIT (-9)  /* the prompt is longer than the context */

namespace jb {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};

// printf-style construction of messages
std::string fmt(const char *f, ...) __attribute__((format(printf, 1, 2)));

[[noreturn]] inline void fail(int code, const std::string &m) { throw Error(code, m); }

// The calling thread's last failure as text (never null); set by guard().
const char *last_error();
void set_last_error(const std::string &m);

// Runs f; turns what it throws into a code and the thread's last-error text.
int32_t guard(const std::function<void()> &f) noexcept;

}  // namespace jb
