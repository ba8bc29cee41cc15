// Device-memory helpers: a grow-only buffer and a per-index scratch workspace, so that steady-
// state searches allocate nothing (the analogue of the reference's per-index resource pool,
// AscendIndexConfig::resourceSize, FR/ascend/AscendIndex.h:41-58).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

namespace b200 {

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { release(); }

    void release() {
        if (ptr_) cudaFree(ptr_);
        ptr_ = nullptr;
        bytes_ = 0;
    }
    // Scratch semantics: contents are not preserved when the buffer grows.
    void* ensure(size_t bytes) {
        if (bytes > bytes_) {
            release();
            size_t want = bytes + bytes / 4;
            want = (want + 255) & ~size_t(255);
            B200_CUDA_CHECK(cudaMalloc(&ptr_, want));
            bytes_ = want;
        }
        return ptr_;
    }
    // Storage semantics: grows geometrically and keeps the first keep_bytes bytes.
    void* grow_keep(size_t bytes, size_t keep_bytes, cudaStream_t stream) {
        if (bytes > bytes_) {
            size_t want = bytes_ + bytes_ / 2;
            if (want < bytes) want = bytes;
            want = (want + 255) & ~size_t(255);
            void* np = nullptr;
            B200_CUDA_CHECK(cudaMalloc(&np, want));
            if (ptr_ && keep_bytes) {
                B200_CUDA_CHECK(cudaMemcpyAsync(np, ptr_, keep_bytes, cudaMemcpyDeviceToDevice, stream));
                B200_CUDA_CHECK(cudaStreamSynchronize(stream));
            }
            if (ptr_) cudaFree(ptr_);
            ptr_ = np;
            bytes_ = want;
        }
        return ptr_;
    }
    void swap(DeviceBuffer& o) {
        void* p = ptr_; ptr_ = o.ptr_; o.ptr_ = p;
        size_t b = bytes_; bytes_ = o.bytes_; o.bytes_ = b;
    }
    template <typename T>
    T* as() const { return static_cast<T*>(ptr_); }
    void* get() const { return ptr_; }
    size_t bytes() const { return bytes_; }

private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

class PinnedBuffer {
public:
    PinnedBuffer() = default;
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    ~PinnedBuffer() {
        if (ptr_) cudaFreeHost(ptr_);
    }
    void* ensure(size_t bytes) {
        if (bytes > bytes_) {
            if (ptr_) cudaFreeHost(ptr_);
            ptr_ = nullptr;
            size_t want = (bytes + bytes / 4 + 255) & ~size_t(255);
            B200_CUDA_CHECK(cudaMallocHost(&ptr_, want));
            bytes_ = want;
        }
        return ptr_;
    }
    template <typename T>
    T* as() const { return static_cast<T*>(ptr_); }

private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

struct DeviceGuard {
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev_);
        if (prev_ != dev) cudaSetDevice(dev);
        dev_ = dev;
    }
    ~DeviceGuard() {
        if (prev_ != dev_) cudaSetDevice(prev_);
    }
    int prev_ = 0, dev_ = 0;
};

}  // namespace b200
