// Host-side plumbing shared by the C-ABI translation units: RAII device buffers,
// host/device pointer classification, the thread-local error slot and the tq_array
// handle that travels through the `void*` slots of the C interface.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "tq_common.cuh"

namespace tq {

// ---- error slot (one per thread) -----------------------------------------------------
std::string& last_error_slot();
inline void set_last_error(const std::string& m) { last_error_slot() = m; }

// Run `body`, translating exceptions into the error slot.  Returns `ok` or `fail`.
template <typename R, typename F>
R guarded(R ok_unused, R fail, F&& body) {
    (void)ok_unused;
    try {
        return body();
    } catch (const std::exception& e) {
        set_last_error(e.what());
    } catch (...) {
        set_last_error("unknown error");
    }
    return fail;
}

// ---- device selection -------------------------------------------------------------------
int current_device();
int sm_count(int device);

// ---- pointers ---------------------------------------------------------------------------
// True when the CUDA driver knows `p` as device (or managed) memory.
inline bool is_device_pointer(const void* p) {
    if (!p) return false;
    cudaPointerAttributes attr{};
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear the sticky-free error for unregistered host memory on old drivers
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

// For page-locked host memory (cudaHostAlloc / cudaHostRegister, mapped as usual under unified
// addressing) returns the address a kernel can use for it, else NULL.
inline void* pinned_host_device_alias(const void* p) {
    if (!p) return nullptr;
    cudaPointerAttributes attr{};
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? attr.devicePointer : nullptr;
}

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes) { resize(bytes); }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { release(); p_ = o.p_; n_ = o.n_; o.p_ = nullptr; o.n_ = 0; }
        return *this;
    }
    ~DeviceBuffer() { release(); }

    // Grow-only: keeps the allocation when it is already large enough (contents kept
    // only in that case).
    void reserve(size_t bytes) {
        if (bytes <= n_) return;
        release();
        if (bytes) TQ_CUDA(cudaMalloc(&p_, bytes));
        n_ = bytes;
    }
    void resize(size_t bytes) { reserve(bytes); }
    void release() {
        if (p_) cudaFree(p_);
        p_ = nullptr;
        n_ = 0;
    }
    template <typename T = void> T* as() const { return static_cast<T*>(p_); }
    size_t bytes() const { return n_; }

private:
    void* p_ = nullptr;
    size_t n_ = 0;
};

// A read-only view of caller data on the device: device pointers are used in place,
// host pointers are copied into `staging` on `stream`.
template <typename T>
const T* device_view(const T* p, size_t count, DeviceBuffer& staging, cudaStream_t stream) {
    if (count == 0) return p;
    if (is_device_pointer(p)) return p;
    staging.reserve(count * sizeof(T));
    TQ_CUDA(cudaMemcpyAsync(staging.as<void>(), p, count * sizeof(T), cudaMemcpyHostToDevice, stream));
    return staging.as<T>();
}

}  // namespace tq

// ---- tensor handle ------------------------------------------------------------------------
struct tq_array_s {
    void* data = nullptr;   // device pointer
    int dtype = 0;          // TQ_F32 / TQ_F16 / TQ_U8 / TQ_U32
    int ndim = 0;
    int shape[8] = {0};
    int device = 0;
    bool owns = false;

    size_t count() const {
        size_t n = 1;
        for (int i = 0; i < ndim; ++i) n *= static_cast<size_t>(shape[i]);
        return n;
    }
    static size_t elem_size(int dt) { return dt == 0 || dt == 3 ? 4 : (dt == 1 ? 2 : 1); }
    size_t nbytes() const { return count() * elem_size(dtype); }
};
