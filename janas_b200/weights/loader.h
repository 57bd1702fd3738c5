// Weights from a model folder by tensor name.
//
// The model says which tensors it expects (name -> TensorSpec, in its own
// order); the folder is checked against that list as a whole, and ONE error
// lists every missing tensor, every unexpected one, every wrong shape and every
// wrong type.  The reference checks tensor by tensor and stops at the first
// ("tensor %s missing", "tensor %s: unexpected type or shape":
// src/llm/model_load.c:53-77); a tied head is an absent output matrix
// (src/llm/model_load.c:1004-1007).
//
// Resident dtypes: with compute dtype bfloat16 a tensor stored as BF16 or F16 is
// kept in bfloat16, a tensor stored in 32-bit floats stays in 32-bit floats, and
// a table of integers becomes int32.  With compute dtype float32 every float
// tensor is widened to float32 (exactly; nothing is rounded).
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "../core/json.h"
#include "../engine/device.h"
#include "safetensors.h"

namespace jb {

// kinds of tensors; they decide the resident dtype and the random distribution
enum TensorKind { MATRIX, EMBEDDING, NORM, INT_TABLE };
const char *kind_name(TensorKind k);
TensorKind parse_kind(const std::string &s);

struct TensorSpec {
    std::vector<long long> shape;
    TensorKind kind = MATRIX;
    bool optional = false;          // absent is allowed (a tied head)
};

// name -> spec, in the order the model names them
using TensorList = std::vector<std::pair<std::string, TensorSpec>>;
Json tensor_list_json(const TensorList &l);
TensorList tensor_list_from_json(const Json &j);

// The folder's tensors do not match what the model needs.
struct WeightMismatch : Error {
    std::vector<std::string> missing, unexpected;
    struct Shape { std::string name; std::vector<long long> want, got; };
    std::vector<Shape> wrong_shape;
    std::vector<std::pair<std::string, std::string>> wrong_type;     // name, stored dtype
    WeightMismatch(const std::string &msg) : Error(JB_LLM_EOPEN, msg) {}
    Json to_json() const;
};

// The dtype a tensor is kept in on the device.
DType resident_dtype(const std::string &stored, TensorKind kind, DType compute);

// Throws WeightMismatch when the checkpoint and the list disagree.
void check_weights(const Checkpoint &ckpt, const TensorList &expected);

// One tensor from the file to the device in its resident dtype (converted on
// the way where the stored type differs).  Synchronous.
DevTensor upload_tensor(Device &dev, const TensorInfo &info, DType resident);
// The same conversion into host memory (dst holds count * dtype_size(resident) bytes).
void convert_tensor(const TensorInfo &info, DType resident, void *dst);

// Random weights, made on the device: every linear and embedding weight
// N(0, 0.02), every norm weight 1 + N(0, 0.1), from a counter-based generator
// seeded by `seed` and the tensor's name, so a tensor's values do not depend on
// which other tensors exist.  (The folder writer of the Python package draws on
// the host with another generator; a model made here has no twin on the host.)
DevTensor random_tensor(Device &dev, const std::string &name, const TensorSpec &spec,
                        unsigned long long seed, DType dt);

}  // namespace jb

// weights/random_init.cu
extern "C" int jb_fill_normal(void *out, int dt, long long n, unsigned long long seed, float mean,
                              float std, cudaStream_t st);
