// What the files of the C interface share.
#pragma once

#include <memory>

#include "../engine/engine.h"
#include "../engine/generate.h"
#include "../include/janas_b200/llm.h"
#include "../parts/foreign.h"

struct jb_llm {
    jb_llm_params params;
    std::unique_ptr<jb::Engine> engine;     // null for a handle that stands in for an engine
    std::unique_ptr<jb::Driver> driver;
};

struct jb_llm_session {
    jb_llm *llm = nullptr;
    std::unique_ptr<jb::Session> session;
};

namespace jb {

// {name: {"ptr", "dtype", "shape"}} (device addresses) -> copies on `dev`, in the
// dtype the model keeps each tensor in (compute dtype float32 widens everything).
TensorMap tensors_from_json(Device &dev, const Json &tensors, const TensorList &expected, DType compute);

// A driver whose engine is a callback (api/call.cpp: "llm.open_foreign").
std::unique_ptr<Driver> foreign_driver(ForeignCall fn, void *user);

}  // namespace jb
