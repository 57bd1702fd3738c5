#include "device.h"

#include <cstring>

namespace jb {

size_t dtype_size(DType dt) {
    switch (dt) {
        case F32: case I32: return 4;
        case BF16: case F16: return 2;
        case I64: return 8;
    }
    return 0;
}

const char *dtype_name(DType dt) {
    switch (dt) {
        case F32: return "float32";
        case BF16: return "bfloat16";
        case I32: return "int32";
        case I64: return "int64";
        case F16: return "float16";
    }
    return "?";
}

DType parse_compute_dtype(const std::string &n) {
    if (n == "bfloat16" || n == "bf16") return BF16;
    if (n == "float32" || n == "fp32") return F32;
    fail(JB_LLM_EINVAL, "dtype '" + n + "': bfloat16 or float32");
}

void cuda_check(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return;
    cudaGetLastError();     // a sticky "last error" must not fail the next, unrelated call
    int code = e == cudaErrorMemoryAllocation ? JB_LLM_ENOMEM : JB_LLM_EFAIL;
    fail(code, std::string(what) + ": " + cudaGetErrorString(e));
}

bool cuda_available(std::string *why) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (why) *why = cudaGetErrorString(e);
        return false;
    }
    if (n <= 0) {
        if (why) *why = "no CUDA device";
        return false;
    }
    return true;
}

DeviceBuffer::DeviceBuffer(size_t b, bool zero) : bytes(b) {
    cuda_check(cudaMalloc(&ptr, b ? b : 1), "device allocation");
    if (zero && b) {
        cudaError_t e = cudaMemset(ptr, 0, b);
        if (e != cudaSuccess) {
            cudaFree(ptr);
            ptr = nullptr;
            cuda_check(e, "clearing device memory");
        }
    }
}

DeviceBuffer::~DeviceBuffer() {
    if (ptr) cudaFree(ptr);
}

Buf &Buf::operator=(Buf &&o) noexcept {
    if (this != &o) {
        reset();
        ptr = o.ptr; bytes = o.bytes; cap_ = o.cap_; pool_ = o.pool_;
        o.ptr = nullptr; o.bytes = 0; o.cap_ = 0; o.pool_ = nullptr;
    }
    return *this;
}

void Buf::reset() {
    if (ptr && pool_) pool_->put(ptr, cap_);
    ptr = nullptr;
    bytes = 0;
    pool_ = nullptr;
}

// Sizes are rounded up to 512 bytes below 1 MiB and to 1/8 of their leading power of
// two above it, so that steps of slightly different row counts share buffers.
static size_t size_class(size_t b) {
    if (b <= 512) return 512;
    if (b <= (1u << 20)) return (b + 511) & ~(size_t)511;
    size_t p = 1;
    while (p * 2 <= b) p *= 2;
    size_t step = p / 8;
    return (b + step - 1) / step * step;
}

Buf Pool::get(size_t bytes) {
    size_t cap = size_class(bytes);
    auto it = free_.find(cap);
    if (it != free_.end() && !it->second.empty()) {
        void *p = it->second.back();
        it->second.pop_back();
        return Buf(p, bytes, cap, this);
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, cap);
    if (e == cudaErrorMemoryAllocation) {
        // what lies idle in other size classes may make room (the stream is drained
        // first: idle buffers may still be read by kernels that are under way)
        cudaGetLastError();
        cudaDeviceSynchronize();
        trim();
        e = cudaMalloc(&p, cap);
    }
    cuda_check(e, "device allocation (temporaries)");
    reserved_ += cap;
    allocations_++;
    return Buf(p, bytes, cap, this);
}

void Pool::put(void *p, size_t cap) { free_[cap].push_back(p); }

void Pool::trim() {
    if (before_trim) before_trim();
    for (auto &kv : free_) {
        for (void *p : kv.second) {
            cudaFree(p);
            reserved_ -= kv.first;
        }
        kv.second.clear();
    }
}

Pool::~Pool() {
    before_trim = nullptr;
    trim();
}

Device::Device(int idx) : index(idx) {
    std::string why;
    if (!cuda_available(&why))
        fail(JB_LLM_EFAIL, "janas_b200 needs a CUDA device; none can be used (" + why +
                           "); there is no CPU path");
    int n = 0;
    cudaGetDeviceCount(&n);
    if (idx < 0 || idx >= n) fail(JB_LLM_EINVAL, fmt("device %d: this machine has %d", idx, n));
    cuda_check(cudaSetDevice(idx), "cudaSetDevice");
    cudaDeviceProp prop;
    cuda_check(cudaGetDeviceProperties(&prop, idx), "cudaGetDeviceProperties");
    sm_count = prop.multiProcessorCount;
    if (prop.major != 10)
        fail(JB_LLM_EFAIL, fmt("device %d is %s (compute capability %d.%d); the kernels are built "
                               "for sm_100a only", idx, prop.name, prop.major, prop.minor));
    cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
    ring_.resize(6);
}

Device::~Device() {
    if (stream) cudaStreamSynchronize(stream);
    for (auto &s : ring_) {
        if (s.done) cudaEventDestroy(s.done);
        if (s.host) cudaFreeHost(s.host);
    }
    pool.trim();
    if (stream) cudaStreamDestroy(stream);
}

void Device::make_current() const { cuda_check(cudaSetDevice(index), "cudaSetDevice"); }

void Device::sync() const { cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize"); }

DevTensor Device::tensor(DType dt, std::vector<long long> shape, bool zero) {
    DevTensor t;
    t.dt = dt;
    t.shape = std::move(shape);
    t.buf = std::make_shared<DeviceBuffer>(t.bytes(), zero);
    t.ptr = t.buf->ptr;
    return t;
}

void *Device::pinned(size_t bytes) {
    Stage &s = ring_[turn_];
    last_ = (int)turn_;
    turn_ = (turn_ + 1) % ring_.size();
    if (s.used) cuda_check(cudaEventSynchronize(s.done), "cudaEventSynchronize");
    s.used = false;
    if (s.cap < bytes) {
        if (s.host) cudaFreeHost(s.host);
        s.host = nullptr;
        s.cap = 0;
        size_t cap = 4096;
        while (cap < bytes) cap *= 2;
        cuda_check(cudaMallocHost(&s.host, cap), "pinned host allocation");
        s.cap = cap;
    }
    if (!s.done) cuda_check(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming), "cudaEventCreate");
    return s.host;
}

void Device::upload_pinned(void *dst, const void *src, size_t bytes) {
    Stage *s = nullptr;
    if (last_ >= 0 && ring_[(size_t)last_].host == src) s = &ring_[(size_t)last_];
    if (!s) fail(JB_LLM_EFAIL, "upload_pinned: not the buffer that pinned() gave last");
    if (bytes) cuda_check(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream), "copy to the device");
    cuda_check(cudaEventRecord(s->done, stream), "cudaEventRecord");
    s->used = true;
    h2d_bytes += (long long)bytes;
}

void Device::upload(void *dst, const void *src, size_t bytes) {
    void *h = pinned(bytes);
    if (bytes) memcpy(h, src, bytes);
    upload_pinned(dst, h, bytes);
}

}  // namespace jb
