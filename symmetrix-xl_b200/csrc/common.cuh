// Shared host/device helpers of the sm_100a force-path library.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>

namespace sxb {

struct CudaError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

inline void cuda_check(cudaError_t status, const char* what, const char* file, int line)
{
    if (status != cudaSuccess) {
        char buffer[512];
        std::snprintf(buffer, sizeof(buffer), "CUDA error %d (%s) at %s:%d: %s", static_cast<int>(status),
                      cudaGetErrorString(status), file, line, what);
        throw CudaError(buffer);
    }
}
#define SXB_CUDA(expr) ::sxb::cuda_check((expr), #expr, __FILE__, __LINE__)

// Owning device buffer; grows only when asked for more than it holds.
template <typename T>
struct DeviceBuffer {
    T* ptr = nullptr;
    std::size_t capacity = 0;

    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& other) noexcept : ptr(other.ptr), capacity(other.capacity)
    {
        other.ptr = nullptr;
        other.capacity = 0;
    }
    ~DeviceBuffer() { release(); }

    void release()
    {
        if (ptr != nullptr) cudaFree(ptr);
        ptr = nullptr;
        capacity = 0;
    }
    void reserve(std::size_t count)
    {
        if (count <= capacity) return;
        release();
        SXB_CUDA(cudaMalloc(reinterpret_cast<void**>(&ptr), (count > 0 ? count : 1) * sizeof(T)));
        capacity = count;
    }
    // reserve with ~3 % head room: for arrays whose extent fluctuates from one neighbor-list rebuild to
    // the next (edges), so that a rebuild does not free and reallocate gigabytes
    void reserve_with_slack(std::size_t count)
    {
        if (count > capacity) reserve(count + count / 32 + 1024);
    }
    std::size_t bytes() const { return capacity * sizeof(T); }
};

// Per-edge geometry record written once per step and read by every edge kernel:
// unit direction in float and the length rounded once from double, which is the
// precision the reference evaluates its splines and harmonics in.
struct alignas(16) EdgeGeom {
    float ux, uy, uz, r;
};

// Radial spline grid in the precision the kernels evaluate it in.
struct SplineGrid {
    float x0, h, r_cut;
    int intervals;     // points - 1
};

// Coupling coefficients of the layer-1 tensor product, indexed by compiled term.
struct CouplingConstants {
    float cg[256];
};

constexpr int kVirialSlots = 64;   // spread the 9-component virial atomics over this many slots

}  // namespace sxb
