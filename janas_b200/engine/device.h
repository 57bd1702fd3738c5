// One GPU as the engine sees it: a stream, owned allocations, a pool of
// temporaries, and a ring of pinned host buffers for the small index arrays
// that every step copies to the device.
//
// Temporaries (activations, partial sums, scratch) come from the pool and go
// back to it when their handle dies.  All work of an engine runs on one stream,
// so a buffer that went back can be handed out again at once: whatever used it
// before is ahead in the stream.  The pool never gives memory back to the driver
// while the engine lives (trim() is for the owner, who must first drop every
// captured graph): a captured decode step has the addresses of its temporaries
// baked in, and replaying it is only safe while those addresses stay this
// pool's.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../core/error.h"

namespace jb {

// element types; F32 and BF16 have the values the kernels' C interface uses
enum DType : int { F32 = 0, BF16 = 1, I32 = 2, I64 = 3, F16 = 4 };
size_t dtype_size(DType dt);
const char *dtype_name(DType dt);
DType parse_compute_dtype(const std::string &name);     // "bfloat16"/"bf16"/"float32"/"fp32"

// Throws Error (JB_LLM_ENOMEM for an allocation, else JB_LLM_EFAIL) when e is not success.
void cuda_check(cudaError_t e, const char *what);
// Whether a CUDA device can be used at all, and why not (for error messages).
bool cuda_available(std::string *why);

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    DeviceBuffer(size_t bytes, bool zero);
    ~DeviceBuffer();
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    void *ptr = nullptr;
    size_t bytes = 0;
};

class Pool;

// A temporary from the pool; move-only, returns to the pool when destroyed.
class Buf {
public:
    Buf() = default;
    Buf(void *p, size_t b, size_t c, Pool *pool) : ptr(p), bytes(b), cap_(c), pool_(pool) {}
    Buf(Buf &&o) noexcept { *this = std::move(o); }
    Buf &operator=(Buf &&o) noexcept;
    Buf(const Buf &) = delete;
    Buf &operator=(const Buf &) = delete;
    ~Buf() { reset(); }
    void reset();
    explicit operator bool() const { return ptr != nullptr; }
    template <class T> T *as() const { return (T *)ptr; }
    void *ptr = nullptr;
    size_t bytes = 0;

private:
    size_t cap_ = 0;
    Pool *pool_ = nullptr;
};

class Pool {
public:
    ~Pool();
    Buf get(size_t bytes);
    void put(void *p, size_t cap);
    void trim();                    // frees what is idle; the caller has synchronized
    // called at the start of trim(): whoever holds addresses of pool buffers beyond a
    // step (captured graphs) drops them here
    std::function<void()> before_trim;
    size_t reserved() const { return reserved_; }
    long long allocations() const { return allocations_; }   // cudaMalloc calls so far

private:
    std::map<size_t, std::vector<void *>> free_;
    size_t reserved_ = 0;
    long long allocations_ = 0;
};

// A weight (or any long-lived tensor) on the device.  Several tensors may share
// one allocation (a tied head is the embedding table).
struct DevTensor {
    std::shared_ptr<DeviceBuffer> buf;
    void *ptr = nullptr;
    DType dt = F32;
    std::vector<long long> shape;
    long long numel() const { long long n = 1; for (auto s : shape) n *= s; return n; }
    size_t bytes() const { return (size_t)numel() * dtype_size(dt); }
    explicit operator bool() const { return ptr != nullptr; }
};

class Device {
public:
    explicit Device(int index);     // Error(JB_LLM_EFAIL) without a usable GPU
    ~Device();
    Device(const Device &) = delete;
    Device &operator=(const Device &) = delete;

    void make_current() const;
    void sync() const;
    DevTensor tensor(DType dt, std::vector<long long> shape, bool zero = false);

    // Copies host bytes to device memory behind what the stream holds, through
    // the pinned ring; returns at once.  For the small arrays of a step.
    void upload(void *dst, const void *src, size_t bytes);
    // A pinned host buffer of the ring, free to write (its last copy is over);
    // the caller fills it and calls upload_pinned with the same pointer.
    void *pinned(size_t bytes);
    void upload_pinned(void *dst, const void *pinned_src, size_t bytes);

    int index = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    Pool pool;
    long long h2d_bytes = 0;        // bytes of step inputs copied to the device so far

private:
    struct Stage { void *host = nullptr; size_t cap = 0; cudaEvent_t done = nullptr; bool used = false; };
    std::vector<Stage> ring_;
    size_t turn_ = 0;
    int last_ = -1;
};

}  // namespace jb
