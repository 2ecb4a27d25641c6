// Two small probes that give the edge kernels' rooflines a measured denominator on the GPU at hand:
//   * FP32 FMA issue rate of the CUDA cores (the layer-1 gradient kernel is bound by it), and
//   * L2-to-SM read bandwidth on a table that stays resident in L2, read with the access shape of
//     the edge kernels (one 128-bit load per lane, 512 contiguous bytes per warp, warp-random rows)
//     (the forward edge kernels are bound by the delivery of spline coefficients from L2).
// Each probe runs a few milliseconds, is timed with CUDA events on its own stream and changes no
// device setting.  The reference has no counterpart; its documentation quotes vendor peaks.
#include "../../include/symmetrix_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <stdexcept>
#include <string>
#include <vector>

#include "common.cuh"

namespace sxb {

void set_last_error(const std::string& message);   // c_api.cu

namespace {

constexpr int kFmaChains = 8;

// Every thread advances kFmaChains independent FMA chains `iterations` times.
__global__ void __launch_bounds__(256) fma_probe_kernel(int iterations, float seed, float* __restrict__ sink)
{
    float a[kFmaChains];
#pragma unroll
    for (int q = 0; q < kFmaChains; ++q) a[q] = seed + static_cast<float>(threadIdx.x + q);
    const float m = 0.999f + seed * 1e-6f, c = 1e-3f;
    for (int it = 0; it < iterations; ++it) {
#pragma unroll
        for (int rep = 0; rep < 16; ++rep)
#pragma unroll
            for (int q = 0; q < kFmaChains; ++q) a[q] = fmaf(a[q], m, c);
    }
    float total = 0.0f;
#pragma unroll
    for (int q = 0; q < kFmaChains; ++q) total += a[q];
    if (total == 12345.678f) sink[0] = total;   // never true in practice; keeps the chains alive
}

// Every warp reads `reads` rows of 512 bytes (a float4 per lane) at pseudo-random row positions of a
// table of `rows` rows.
__global__ void __launch_bounds__(256) l2_read_probe_kernel(const float4* __restrict__ table, unsigned rows, int reads,
                                                            float* __restrict__ sink)
{
    const unsigned warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31u;
    unsigned state = warp * 2654435761u + 12345u;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int it = 0; it < reads; it += 4) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            state = state * 1664525u + 1013904223u;
            const unsigned row = (state >> 8) % rows;
            v[u] = table[static_cast<size_t>(row) * 32u + lane];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
    }
    if (acc.x + acc.y + acc.z + acc.w == 12345.678f) sink[0] = acc.x;
}

}  // namespace
}  // namespace sxb

extern "C" int sxb_measure_device_peaks(int32_t device_ordinal, double* fp32_fma_tflops, double* l2_read_gbs)
{
    using namespace sxb;
    try {
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) throw std::runtime_error("No CUDA device is available.");
        if (device_ordinal < 0 || device_ordinal >= count) throw std::invalid_argument("CUDA device ordinal is out of range.");
        SXB_CUDA(cudaSetDevice(device_ordinal));
        int sms = 0;
        SXB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device_ordinal));
        cudaStream_t stream;
        SXB_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
        cudaEvent_t begin, end;
        SXB_CUDA(cudaEventCreate(&begin));
        SXB_CUDA(cudaEventCreate(&end));
        DeviceBuffer<float> sink;
        sink.reserve(4);
        float best_ms = 0.0f;
        if (fp32_fma_tflops != nullptr) {
            const int blocks = sms * 8, iterations = 2048;
            best_ms = 1e30f;
            for (int rep = 0; rep < 4; ++rep) {      // the first repetition warms the clocks up
                SXB_CUDA(cudaEventRecord(begin, stream));
                fma_probe_kernel<<<blocks, 256, 0, stream>>>(iterations, 0.5f, sink.ptr);
                SXB_CUDA(cudaEventRecord(end, stream));
                SXB_CUDA(cudaEventSynchronize(end));
                float ms = 0.0f;
                SXB_CUDA(cudaEventElapsedTime(&ms, begin, end));
                if (rep > 0) best_ms = std::min(best_ms, ms);
            }
            const double flop = 2.0 * static_cast<double>(blocks) * 256.0 * kFmaChains * 16.0 * iterations;
            *fp32_fma_tflops = flop / (best_ms * 1e-3) / 1e12;
        }
        if (l2_read_gbs != nullptr) {
            const unsigned rows = 65536;                       // 32 MB: inside the L2, as the spline tables are
            DeviceBuffer<float4> table;
            table.reserve(static_cast<size_t>(rows) * 32);
            SXB_CUDA(cudaMemsetAsync(table.ptr, 0, static_cast<size_t>(rows) * 512, stream));
            const int blocks = sms * 8, reads = 2048;
            best_ms = 1e30f;
            for (int rep = 0; rep < 4; ++rep) {      // the first repetition brings the table into L2
                SXB_CUDA(cudaEventRecord(begin, stream));
                l2_read_probe_kernel<<<blocks, 256, 0, stream>>>(table.ptr, rows, reads, sink.ptr);
                SXB_CUDA(cudaEventRecord(end, stream));
                SXB_CUDA(cudaEventSynchronize(end));
                float ms = 0.0f;
                SXB_CUDA(cudaEventElapsedTime(&ms, begin, end));
                if (rep > 0) best_ms = std::min(best_ms, ms);
            }
            const double bytes = static_cast<double>(blocks) * 8.0 * reads * 512.0;
            *l2_read_gbs = bytes / (best_ms * 1e-3) / 1e9;
        }
        SXB_CUDA(cudaGetLastError());
        cudaEventDestroy(begin);
        cudaEventDestroy(end);
        cudaStreamDestroy(stream);
        return SXB_OK;
    } catch (const std::invalid_argument& e) {
        set_last_error(e.what());
        return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return SXB_ERR_RUNTIME;
    }
}
