// Reading and writing safetensors files, without a library.
//
// The format: an 8-byte little-endian header length, a JSON header that gives
// each tensor's dtype, shape and byte range relative to the end of the header,
// then the bytes.  Every field is checked against the file before it is used, as
// the reference's reader does (src/common/hf_safetensors.h:1-52,
// tools/hf2gguf.c:117-164).  A folder may hold one model.safetensors or the
// shards named by model.safetensors.index.json.  Files are memory-mapped; a
// tensor's bytes are read where they lie.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../core/error.h"

namespace jb {

struct TensorInfo {
    std::string name;
    std::string dtype;                 // "F32", "F16", "BF16", "I32", "I64"
    std::vector<long long> shape;
    size_t begin = 0, end = 0;         // byte range in the file
    std::string path;
    const uint8_t *data = nullptr;     // the bytes, valid while the checkpoint is open

    long long count() const { long long n = 1; for (auto s : shape) n *= s; return n; }
};

// bytes per element of a stored dtype name; 0 for one that is not read
int stored_size(const std::string &dtype);

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string &path);     // Error(JB_LLM_EOPEN)
    ~SafetensorsFile();
    SafetensorsFile(const SafetensorsFile &) = delete;
    SafetensorsFile &operator=(const SafetensorsFile &) = delete;

    std::string path;
    std::vector<TensorInfo> tensors;       // in the header's order

private:
    int fd_ = -1;
    void *map_ = nullptr;
    size_t size_ = 0;
};

// All tensors of a model folder by name, whichever file holds them.
class Checkpoint {
public:
    explicit Checkpoint(const std::string &model_dir);     // Error(JB_LLM_EOPEN)

    std::string model_dir;
    std::vector<std::string> names;                        // in file order
    std::map<std::string, TensorInfo> tensors;

private:
    std::vector<std::unique_ptr<SafetensorsFile>> files_;
    void open_file(const std::string &path);
};

}  // namespace jb
