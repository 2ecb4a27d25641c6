// Stand-alone reduction of directed edge forces to atom forces and stress:
//   F_j += f_ij,  F_i -= f_ij,  sigma = -(1/V) sum_ij f_ij (x) xyz_ij
// for callers that hold per-edge forces and explicit edge lists (the graph-less mode of the
// reference's _reduce_atom_forces / _reduce_stress, symmetrix/source/cpp/mace_kokkos.cpp:2103-2154;
// kernels reduce_node_forces and reduce_stress, libsymmetrix/source/mace_kokkos_evaluate.cpp:92-106
// and 157-186).  Atom forces use FP64 atomics; the virial is reduced deterministically in two
// stages through a scratch array of per-block partial sums.
#include "../../include/symmetrix_b200.h"

#include <cmath>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>
#include <stdexcept>
#include <string>

#include "common.cuh"

namespace sxb {

constexpr int kReduceThreads = 256;

// One thread per edge.  partials[block][9] receives the block's sum of f (x) xyz.
__global__ void __launch_bounds__(kReduceThreads)
reduce_edge_forces_kernel(long num_edges, int num_nodes, const int* __restrict__ receivers, const int* __restrict__ sources,
                          const double* __restrict__ edge_forces, const double* __restrict__ xyz,
                          double* __restrict__ atom_forces, double* __restrict__ partials, int* __restrict__ error_flag)
{
    __shared__ double warp_sums[kReduceThreads / 32][9];
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    double v[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (e < num_edges) {
        const int i = receivers[e], j = sources[e];
        if (i < 0 || i >= num_nodes || j < 0 || j >= num_nodes) {
            atomicOr(error_flag, 1);
        } else {
            const double fx = edge_forces[3 * e], fy = edge_forces[3 * e + 1], fz = edge_forces[3 * e + 2];
            atomicAdd(atom_forces + 3 * static_cast<long>(j), fx);
            atomicAdd(atom_forces + 3 * static_cast<long>(j) + 1, fy);
            atomicAdd(atom_forces + 3 * static_cast<long>(j) + 2, fz);
            atomicAdd(atom_forces + 3 * static_cast<long>(i), -fx);
            atomicAdd(atom_forces + 3 * static_cast<long>(i) + 1, -fy);
            atomicAdd(atom_forces + 3 * static_cast<long>(i) + 2, -fz);
            const double rx = xyz[3 * e], ry = xyz[3 * e + 1], rz = xyz[3 * e + 2];
            v[0] = fx * rx; v[1] = fx * ry; v[2] = fx * rz;
            v[3] = fy * rx; v[4] = fy * ry; v[5] = fy * rz;
            v[6] = fz * rx; v[7] = fz * ry; v[8] = fz * rz;
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
#pragma unroll
        for (int q = 0; q < 9; ++q) v[q] += __shfl_xor_sync(0xffffffffu, v[q], offset);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
#pragma unroll
        for (int q = 0; q < 9; ++q) warp_sums[warp][q] = v[q];
    __syncthreads();
    if (threadIdx.x < 9) {
        double s = 0.0;
        for (int w = 0; w < kReduceThreads / 32; ++w) s += warp_sums[w][threadIdx.x];
        partials[static_cast<long>(blockIdx.x) * 9 + threadIdx.x] = s;
    }
}

// One block: stress[q] = -(1/volume) * sum over blocks of partials[block][q], summed in a fixed order.
__global__ void __launch_bounds__(kReduceThreads)
finish_stress_kernel(int num_blocks, const double* __restrict__ partials, double volume, double* __restrict__ stress)
{
    __shared__ double sums[kReduceThreads / 32][9];
    double v[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = threadIdx.x; b < num_blocks; b += blockDim.x)
#pragma unroll
        for (int q = 0; q < 9; ++q) v[q] += partials[static_cast<long>(b) * 9 + q];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
#pragma unroll
        for (int q = 0; q < 9; ++q) v[q] += __shfl_xor_sync(0xffffffffu, v[q], offset);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
#pragma unroll
        for (int q = 0; q < 9; ++q) sums[warp][q] = v[q];
    __syncthreads();
    if (threadIdx.x < 9) {
        double s = 0.0;
        for (int w = 0; w < kReduceThreads / 32; ++w) s += sums[w][threadIdx.x];
        stress[threadIdx.x] = -s / volume;
    }
}

// Enqueues the whole reduction on `stream`; every pointer is a device pointer.
// scratch: at least blocks*9 doubles; error_flag: one int, zeroed here.
void launch_reduce_edge_forces(long num_edges, int num_nodes, const int* receivers, const int* sources, const double* edge_forces,
                               const double* xyz, double volume, double* atom_forces, double* stress, double* scratch,
                               int* error_flag, cudaStream_t stream)
{
    const int blocks = static_cast<int>((num_edges + kReduceThreads - 1) / kReduceThreads);
    SXB_CUDA(cudaMemsetAsync(atom_forces, 0, sizeof(double) * 3 * static_cast<size_t>(num_nodes), stream));
    SXB_CUDA(cudaMemsetAsync(error_flag, 0, sizeof(int), stream));
    if (blocks > 0)
        reduce_edge_forces_kernel<<<blocks, kReduceThreads, 0, stream>>>(num_edges, num_nodes, receivers, sources, edge_forces, xyz,
                                                                         atom_forces, scratch, error_flag);
    finish_stress_kernel<<<1, kReduceThreads, 0, stream>>>(blocks, scratch, volume, stress);
    SXB_CUDA(cudaGetLastError());
}

void set_last_error(const std::string& message);   // c_api.cu

}  // namespace sxb

extern "C" int sxb_reduce_edge_forces(int32_t num_nodes, int64_t num_edges, const int32_t* edge_receivers,
                                      const int32_t* edge_sources, const double* edge_forces, const double* xyz, double volume,
                                      double* atom_forces, double* stress9)
{
    using namespace sxb;
    try {
        if (num_nodes <= 0 || num_edges < 0) throw std::invalid_argument("Force reduction extents must be positive.");
        if (!std::isfinite(volume) || !(volume > 0.0)) throw std::invalid_argument("Stress reduction needs a finite positive volume.");
        if (!edge_receivers || !edge_sources || !edge_forces || !xyz || !atom_forces || !stress9)
            throw std::invalid_argument("Force reduction arguments must not be NULL.");
        const size_t E = static_cast<size_t>(num_edges);
        const int blocks = static_cast<int>((num_edges + kReduceThreads - 1) / kReduceThreads);
        DeviceBuffer<int> recv, src, flag;
        DeviceBuffer<double> f, r, out, stress, scratch;
        recv.reserve(E); src.reserve(E); f.reserve(3 * E); r.reserve(3 * E);
        out.reserve(3 * static_cast<size_t>(num_nodes)); stress.reserve(9); scratch.reserve(static_cast<size_t>(blocks) * 9 + 9);
        flag.reserve(1);
        cudaStream_t stream = nullptr;
        SXB_CUDA(cudaMemcpyAsync(recv.ptr, edge_receivers, E * sizeof(int), cudaMemcpyHostToDevice, stream));
        SXB_CUDA(cudaMemcpyAsync(src.ptr, edge_sources, E * sizeof(int), cudaMemcpyHostToDevice, stream));
        SXB_CUDA(cudaMemcpyAsync(f.ptr, edge_forces, 3 * E * sizeof(double), cudaMemcpyHostToDevice, stream));
        SXB_CUDA(cudaMemcpyAsync(r.ptr, xyz, 3 * E * sizeof(double), cudaMemcpyHostToDevice, stream));
        launch_reduce_edge_forces(num_edges, num_nodes, recv.ptr, src.ptr, f.ptr, r.ptr, volume, out.ptr, stress.ptr, scratch.ptr,
                                  flag.ptr, stream);
        int host_flag = 0;
        SXB_CUDA(cudaMemcpyAsync(atom_forces, out.ptr, 3 * sizeof(double) * num_nodes, cudaMemcpyDeviceToHost, stream));
        SXB_CUDA(cudaMemcpyAsync(stress9, stress.ptr, 9 * sizeof(double), cudaMemcpyDeviceToHost, stream));
        SXB_CUDA(cudaMemcpyAsync(&host_flag, flag.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream));
        SXB_CUDA(cudaStreamSynchronize(stream));
        if (host_flag) throw std::invalid_argument("Force reduction: an edge names a node outside [0, num_nodes).");
        return SXB_OK;
    } catch (const std::invalid_argument& e) {
        set_last_error(e.what());
        return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return SXB_ERR_RUNTIME;
    }
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that must not allocate device memory.  Two kinds of callers of this library
// are in that position: a molecular-dynamics engine that has handed the whole device to its own
// memory pool (LAMMPS/Kokkos, or a Python driver under a caching allocator), where a raw
// cudaMalloc can fail although the pool still has room; and a force callback in the middle of a
// time step, where cudaMalloc / cudaFree would stall every stream of the device because they
// synchronise it.  For them the per-block virial partials (and a status word) live in a file-scope
// device array that every GPU loading this library holds until the process exits.
namespace sxb {

constexpr long kStaticMaxEdges = 4194304;                                   // 2^22 directed edges per call
constexpr int kStaticMaxBlocks = static_cast<int>(kStaticMaxEdges / kReduceThreads);
// 16,384 blocks x 9 doubles = 1.18 MB per GPU
static __device__ __align__(256) double g_static_partials[static_cast<long>(kStaticMaxBlocks) * 9];
static __device__ __align__(256) int g_static_status[64];

// In host code the array names above are host-side stand-ins, not device addresses: the device
// address is looked up once per device (with that device current) and kept here.
struct StaticScratch {
    double* partials = nullptr;
    int* status = nullptr;
    bool ready = false;
};
constexpr int kMaxDevices = 64;
static StaticScratch g_static_scratch[kMaxDevices];
static std::mutex g_static_mutex;

static const StaticScratch& static_scratch_for_current_device()
{
    int device = -1;
    SXB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) throw std::invalid_argument("CUDA device ordinal is outside the supported range.");
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticScratch& entry = g_static_scratch[device];
    if (!entry.ready) {
        void* partials = nullptr;
        void* status = nullptr;
        SXB_CUDA(cudaGetSymbolAddress(&partials, g_static_partials));
        SXB_CUDA(cudaGetSymbolAddress(&status, g_static_status));
        entry.partials = static_cast<double*>(partials);
        entry.status = static_cast<int*>(status);
        entry.ready = true;
    }
    return entry;
}

}  // namespace sxb

extern "C" int sxb_reduce_edge_forces_static(int32_t num_nodes, int64_t num_edges, const int32_t* device_receivers,
                                             const int32_t* device_sources, const double* device_edge_forces,
                                             const double* device_xyz, double volume, double* device_atom_forces,
                                             double* device_stress9, int32_t* device_status, void* stream)
{
    using namespace sxb;
    try {
        if (num_nodes <= 0 || num_edges < 0) throw std::invalid_argument("Force reduction extents must be positive.");
        if (num_edges > kStaticMaxEdges)
            throw std::invalid_argument("sxb_reduce_edge_forces_static handles at most 4,194,304 edges per call (" +
                                        std::to_string(num_edges) + " given); split the edge list or use sxb_reduce_edge_forces.");
        if (!std::isfinite(volume) || !(volume > 0.0)) throw std::invalid_argument("Stress reduction needs a finite positive volume.");
        if (!device_receivers || !device_sources || !device_edge_forces || !device_xyz || !device_atom_forces || !device_stress9)
            throw std::invalid_argument("Force reduction arguments must not be NULL.");
        const StaticScratch& scratch = static_scratch_for_current_device();
        // every partial the second kernel reads is rewritten by the first one, so nothing in the
        // scratch has to be cleared; the status word and the output forces are zeroed on the stream
        launch_reduce_edge_forces(num_edges, num_nodes, device_receivers, device_sources, device_edge_forces, device_xyz, volume,
                                  device_atom_forces, device_stress9, scratch.partials,
                                  device_status != nullptr ? device_status : scratch.status, static_cast<cudaStream_t>(stream));
        return SXB_OK;
    } catch (const std::invalid_argument& e) {
        set_last_error(e.what());
        return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return SXB_ERR_RUNTIME;
    }
}
