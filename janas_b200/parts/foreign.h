// Registration of parts whose code lies outside the library (see foreign.cpp).
#pragma once

#include <string>

#include "part.h"

namespace jb {

// The callback: method and arguments as JSON text in, JSON text out (valid until
// the callback's next call), null for a failure.
typedef const char *(*ForeignCall)(void *user, const char *method, const char *args_json);

struct ForeignPartHost {
    ForeignCall fn = nullptr;
    void *user = nullptr;
};

void register_foreign_part(const std::string &role, const std::string &kind, ForeignPartHost host);

}  // namespace jb
