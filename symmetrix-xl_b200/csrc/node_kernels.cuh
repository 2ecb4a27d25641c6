// Node-local kernels of the force path: symmetric contraction (forward and gradient),
// channel-mixing linears, readout.  Reference statements: symmetric contraction
// libsymmetrix/source/mace.cpp:1639-1688 and 2461-2513 (polynomial
// multivariate_polynomial.cpp:322-353), linears mace.cpp:1691-1757, 2305-2378 and
// 2516-2588, readout mace.cpp:2622-2657 with the MLP of multilayer_perceptron.cpp:34-80.
#pragma once

#include "common.cuh"
#include "row_map.hpp"
#include "generated/structures.h"

namespace sxb {

// ---------------------------------------------------------------------------------------------
// Symmetric contraction.  One thread per (node, channel): the 16 inputs sit in registers and
// every monomial of the compiled structure is one straight-line statement; weights are laid
// out [element][term][channel] so a warp reads 128 contiguous bytes per term.
#define SXB_POLY_F1(out, term, a) o[out] = fmaf(w[(term) * C], x[a], o[out]);
#define SXB_POLY_F2(out, term, a, b) o[out] = fmaf(w[(term) * C], x[a] * x[b], o[out]);
#define SXB_POLY_F3(out, term, a, b, c) o[out] = fmaf(w[(term) * C], x[a] * x[b] * x[c], o[out]);
#define SXB_POLY_R1(out, term, a) g[a] = fmaf(w[(term) * C], adj[out], g[a]);
#define SXB_POLY_R2(out, term, a, b)                      \
    {                                                     \
        const float s_ = w[(term) * C] * adj[out];        \
        g[a] = fmaf(s_, x[b], g[a]);                      \
        g[b] = fmaf(s_, x[a], g[b]);                      \
    }
#define SXB_POLY_R3(out, term, a, b, c)                   \
    {                                                     \
        const float s_ = w[(term) * C] * adj[out];        \
        g[a] = fmaf(s_, x[b] * x[c], g[a]);               \
        g[b] = fmaf(s_, x[a] * x[c], g[b]);               \
        g[c] = fmaf(s_, x[a] * x[b], g[c]);               \
    }

constexpr int kPolyWarps = 8;

#define SXB_DEFINE_POLY_KERNELS(NAME)                                                                               \
    /* M0[node][LM][k] from A0[node][16][k] */                                                                      \
    __global__ void __launch_bounds__(32 * kPolyWarps)                                                              \
    m0_forward_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A0, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, float* __restrict__ M0)                             \
    {                                                                                                               \
        constexpr int NH = SXB_##NAME##_NUM_HIDDEN, NT = SXB_##NAME##_M0_NUM_TERMS;                                 \
        const int node = blockIdx.x * kPolyWarps + (threadIdx.x >> 5);                                              \
        const int k = blockIdx.y * 32 + (threadIdx.x & 31);                                                         \
        if (node >= num_nodes) return;                                                                              \
        const float* in = A0 + static_cast<size_t>(node) * 16 * C + k;                                              \
        float x[16];                                                                                                \
        _Pragma("unroll") for (int q = 0; q < 16; ++q) x[q] = in[q * C];                                            \
        const float* w = weights + static_cast<size_t>(element[node]) * NT * C + k;                                 \
        float o[NH];                                                                                                \
        _Pragma("unroll") for (int q = 0; q < NH; ++q) o[q] = 0.0f;                                                 \
        SXB_##NAME##_M0_TERMS(SXB_POLY_F1, SXB_POLY_F2, SXB_POLY_F3)                                                \
        float* out = M0 + static_cast<size_t>(node) * NH * C + k;                                                   \
        _Pragma("unroll") for (int q = 0; q < NH; ++q) out[q * C] = o[q];                                           \
    }                                                                                                               \
    /* A0_adj[node][16][k] = sum_LM M0_adj[node][LM][k] dM0[LM]/dA0 */                                              \
    __global__ void __launch_bounds__(32 * kPolyWarps)                                                              \
    m0_reverse_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A0, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, const float* __restrict__ M0_adj,                   \
                             float* __restrict__ A0_adj)                                                            \
    {                                                                                                               \
        constexpr int NH = SXB_##NAME##_NUM_HIDDEN, NT = SXB_##NAME##_M0_NUM_TERMS;                                 \
        const int node = blockIdx.x * kPolyWarps + (threadIdx.x >> 5);                                              \
        const int k = blockIdx.y * 32 + (threadIdx.x & 31);                                                         \
        if (node >= num_nodes) return;                                                                              \
        const float* in = A0 + static_cast<size_t>(node) * 16 * C + k;                                              \
        float x[16], g[16];                                                                                         \
        _Pragma("unroll") for (int q = 0; q < 16; ++q) { x[q] = in[q * C]; g[q] = 0.0f; }                           \
        const float* w = weights + static_cast<size_t>(element[node]) * NT * C + k;                                 \
        float adj[NH];                                                                                              \
        const float* ain = M0_adj + static_cast<size_t>(node) * NH * C + k;                                         \
        _Pragma("unroll") for (int q = 0; q < NH; ++q) adj[q] = ain[q * C];                                         \
        SXB_##NAME##_M0_TERMS(SXB_POLY_R1, SXB_POLY_R2, SXB_POLY_R3)                                                \
        float* out = A0_adj + static_cast<size_t>(node) * 16 * C + k;                                               \
        _Pragma("unroll") for (int q = 0; q < 16; ++q) out[q * C] = g[q];                                           \
    }                                                                                                               \
    /* M1[node][k] from A1[node][16][k] */                                                                          \
    __global__ void __launch_bounds__(32 * kPolyWarps)                                                              \
    m1_forward_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A1, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, float* __restrict__ M1)                             \
    {                                                                                                               \
        constexpr int NT = SXB_##NAME##_M1_NUM_TERMS;                                                               \
        const int node = blockIdx.x * kPolyWarps + (threadIdx.x >> 5);                                              \
        const int k = blockIdx.y * 32 + (threadIdx.x & 31);                                                         \
        if (node >= num_nodes) return;                                                                              \
        const float* in = A1 + static_cast<size_t>(node) * 16 * C + k;                                              \
        float x[16];                                                                                                \
        _Pragma("unroll") for (int q = 0; q < 16; ++q) x[q] = in[q * C];                                            \
        const float* w = weights + static_cast<size_t>(element[node]) * NT * C + k;                                 \
        float o[1] = {0.0f};                                                                                        \
        SXB_##NAME##_M1_TERMS(SXB_POLY_F1, SXB_POLY_F2, SXB_POLY_F3)                                                \
        M1[static_cast<size_t>(node) * C + k] = o[0];                                                               \
    }                                                                                                               \
    /* A1_adj[node][16][k] = M1_adj[node][k] dM1/dA1 */                                                             \
    __global__ void __launch_bounds__(32 * kPolyWarps)                                                              \
    m1_reverse_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A1, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, const float* __restrict__ M1_adj,                   \
                             float* __restrict__ A1_adj)                                                            \
    {                                                                                                               \
        constexpr int NT = SXB_##NAME##_M1_NUM_TERMS;                                                               \
        const int node = blockIdx.x * kPolyWarps + (threadIdx.x >> 5);                                              \
        const int k = blockIdx.y * 32 + (threadIdx.x & 31);                                                         \
        if (node >= num_nodes) return;                                                                              \
        const float* in = A1 + static_cast<size_t>(node) * 16 * C + k;                                              \
        float x[16], g[16];                                                                                         \
        _Pragma("unroll") for (int q = 0; q < 16; ++q) { x[q] = in[q * C]; g[q] = 0.0f; }                           \
        const float* w = weights + static_cast<size_t>(element[node]) * NT * C + k;                                 \
        float adj[1] = {M1_adj[static_cast<size_t>(node) * C + k]};                                                 \
        SXB_##NAME##_M1_TERMS(SXB_POLY_R1, SXB_POLY_R2, SXB_POLY_R3)                                                \
        float* out = A1_adj + static_cast<size_t>(node) * 16 * C + k;                                               \
        _Pragma("unroll") for (int q = 0; q < 16; ++q) out[q * C] = g[q];                                           \
    }

SXB_DEFINE_POLY_KERNELS(S0)
SXB_DEFINE_POLY_KERNELS(S1)

// ---------------------------------------------------------------------------------------------
// Channel-mixing linear as a tiled FP32 GEMM with structured rows.
//   C[row(g)][n] (+)= sum_k A[row(g)][k] * B[k][n]      (B stored [K][N], or [N][K] when transposed)
// Logical row g of a node tensor (node, component, channel): node = first_node + g / components,
// m = g % components, address = node*node_stride + offset + m*component_stride.
struct GemmArgs {
    const float* A;
    const float* B;
    float* C;
    const float* bias;      // optional [N], added when not accumulating
    RowMap a_rows, c_rows;
    int first_node;
    int M, N, K;            // M = logical rows
    int ldb;
    int b_transposed;       // 0: B[k*ldb + n], 1: B[n*ldb + k]
    int accumulate;         // 1: C += A B
};

__device__ __forceinline__ long row_address(const RowMap& map, int first_node, int g)
{
    const int node = first_node + g / map.components;
    const int m = g % map.components;
    return static_cast<long>(node) * map.node_stride + map.offset + static_cast<long>(m) * map.component_stride;
}

constexpr int kGemmBM = 64, kGemmBN = 64, kGemmBK = 16;

__global__ void __launch_bounds__(256) gemm_rows_kernel(const GemmArgs args)
{
    __shared__ float As[kGemmBK][kGemmBM + 4];
    __shared__ float Bs[kGemmBK][kGemmBN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    const int row0 = blockIdx.x * kGemmBM, col0 = blockIdx.y * kGemmBN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    // loader mapping: A tile 64 rows x 16 k: thread -> (row = tid/4, k4 = (tid%4)*4)
    const int a_row = tid >> 2, a_k = (tid & 3) * 4;
    const bool a_valid = row0 + a_row < args.M;
    const float* a_ptr = a_valid ? args.A + row_address(args.a_rows, args.first_node, row0 + a_row) : nullptr;
    for (int k0 = 0; k0 < args.K; k0 += kGemmBK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int kk = k0 + a_k + q;
            As[a_k + q][a_row] = (a_valid && kk < args.K) ? a_ptr[kk] : 0.0f;
        }
        if (!args.b_transposed) {
            // B tile 16 k x 64 n: thread -> (k = tid/16, n4 = (tid%16)*4)
            const int bk = tid >> 4, bn = (tid & 15) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int kk = k0 + bk, nn = col0 + bn + q;
                Bs[bk][bn + q] = (kk < args.K && nn < args.N) ? args.B[static_cast<long>(kk) * args.ldb + nn] : 0.0f;
            }
        } else {
            // stored [N][K]: thread -> (n = tid/4, k4 = (tid%4)*4)
            const int bn = tid >> 2, bk = (tid & 3) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int kk = k0 + bk + q, nn = col0 + bn;
                Bs[bk + q][bn] = (kk < args.K && nn < args.N) ? args.B[static_cast<long>(nn) * args.ldb + kk] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kGemmBK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int g = row0 + ty * 4 + i;
        if (g >= args.M) continue;
        float* c_ptr = args.C + row_address(args.c_rows, args.first_node, g);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = col0 + tx * 4 + j;
            if (n >= args.N) continue;
            float v = acc[i][j];
            if (args.accumulate) v += c_ptr[n];
            else if (args.bias != nullptr) v += args.bias[n];
            c_ptr[n] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Readout: E_i = E0[element] + q . xs_i + MLP(H2_i), MLP [C, hidden, 1] with hidden activation
// s*z*sigmoid(z); also the adjoint of H2.  One warp per node.
__global__ void __launch_bounds__(256)
readout_kernel(int num_nodes, int C, int hidden, float act_scale, const float* __restrict__ M0, int num_hidden_lm,
               const float* __restrict__ H2, const unsigned char* __restrict__ element,
               const double* __restrict__ atomic_energies, const float* __restrict__ q,
               const float* __restrict__ W1 /*[hidden][C]*/, const float* __restrict__ W2 /*[hidden]*/,
               double* __restrict__ node_energies, float* __restrict__ H2_adj, double* __restrict__ energy_slots)
{
    const int node = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (node >= num_nodes) return;
    const float* xs = M0 + static_cast<size_t>(node) * num_hidden_lm * C;   // scalar block of M0
    const float* h2 = H2 + static_cast<size_t>(node) * C;
    float e1 = 0.0f;
    for (int k = lane; k < C; k += 32) e1 = fmaf(q[k], xs[k], e1);
    float e2 = 0.0f;
    float coeff[64];   // V2[h] * dact[h], hidden <= 64
    for (int h = 0; h < hidden; ++h) {
        float z = 0.0f;
        for (int k = lane; k < C; k += 32) z = fmaf(W1[h * C + k], h2[k], z);
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) z += __shfl_xor_sync(0xffffffffu, z, offset);
        const float sig = 1.0f / (1.0f + expf(-z));
        e2 = fmaf(W2[h], act_scale * z * sig, e2);
        coeff[h] = W2[h] * (act_scale * sig + act_scale * z * sig * (1.0f - sig));
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) e1 += __shfl_xor_sync(0xffffffffu, e1, offset);
    for (int k = lane; k < C; k += 32) {
        float g = 0.0f;
        for (int h = 0; h < hidden; ++h) g = fmaf(coeff[h], W1[h * C + k], g);
        H2_adj[static_cast<size_t>(node) * C + k] = g;
    }
    if (lane == 0) {
        const double e = atomic_energies[element[node]] + static_cast<double>(e1) + static_cast<double>(e2);
        node_energies[node] = e;
        atomicAdd(energy_slots + (node % kVirialSlots), e);
    }
}

__global__ void finalize_kernel(const double* __restrict__ energy_slots, const double* __restrict__ virial_slots,
                                double* __restrict__ totals /* [0]=energy, [1..9]=virial sum f (x) xyz */)
{
    const int t = threadIdx.x;
    if (t < 10) {
        double s = 0.0;
        for (int slot = 0; slot < kVirialSlots; ++slot)
            s += (t == 0) ? energy_slots[slot] : virial_slots[slot * 9 + (t - 1)];
        totals[t] = s;
    }
}

}  // namespace sxb
