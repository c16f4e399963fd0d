// Error types, CUDA call checking and a grow-only device array shared by the host-side code.
#pragma once

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

namespace smx {

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct ArgError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

#define SMX_CUDA(expr)                                                                              \
    do {                                                                                            \
        cudaError_t err__ = (expr);                                                                 \
        if (err__ != cudaSuccess)                                                                   \
            throw ::smx::CudaError(std::string(#expr) + ": " + cudaGetErrorString(err__));          \
    } while (0)

// Grow-only device array. `n` is the logical length, `cap` the allocated one.
template <typename T>
struct DevBuf {
    T* p = nullptr;
    size_t cap = 0, n = 0;
    ~DevBuf() { if (p) cudaFree(p); }
    DevBuf() = default;
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    // Set the logical length to `count`, reallocating if needed; contents survive only if `keep`.
    void resize(size_t count, cudaStream_t s, bool keep = false) {
        if (count > cap) {
            T* q = nullptr;
            const size_t newcap = count + count / 8 + 16;
            SMX_CUDA(cudaMalloc(&q, newcap * sizeof(T)));
            if (keep && p && n) SMX_CUDA(cudaMemcpyAsync(q, p, n * sizeof(T), cudaMemcpyDeviceToDevice, s));
            if (p) { SMX_CUDA(cudaStreamSynchronize(s)); cudaFree(p); }
            p = q;
            cap = newcap;
        }
        n = count;
    }
    void upload(const std::vector<T>& h, cudaStream_t s) {
        resize(h.size(), s);
        if (!h.empty()) SMX_CUDA(cudaMemcpyAsync(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice, s));
    }
    void zero(cudaStream_t s) { if (n) SMX_CUDA(cudaMemsetAsync(p, 0, n * sizeof(T), s)); }
};

}  // namespace smx
