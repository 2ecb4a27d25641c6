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
// Symmetric contraction.  One thread per (group of G consecutive nodes, channel): the 16 inputs of
// every node of the group sit in registers and every monomial of the compiled structure is one
// straight-line statement.  Weights are laid out [element][term][channel].  A block covers
// kPolyNodesPerBlock consecutive nodes and 32 channels; it first copies the [term][32] weight slice
// of its first node's element to shared memory, and every group whose nodes all have that element
// (nodes are sorted by element, so nearly all do) reads its weights from there - a mixed group is
// evaluated node by node from global memory.  At one node per warp and weights from global memory
// these kernels are bound by re-reading the weight slice from L2 (216 KB per node for the 422-term
// structure); sharing a slice among the nodes of a block removes that traffic.
#define SXB_POLY_F1(out, term, a)                                                                     \
    {                                                                                                 \
        const float w_ = w[(term) * ws];                                                              \
        _Pragma("unroll") for (int n_ = 0; n_ < G; ++n_) o[n_][out] = fmaf(w_, x[n_][a], o[n_][out]); \
    }
#define SXB_POLY_F2(out, term, a, b)                                                                  \
    {                                                                                                 \
        const float w_ = w[(term) * ws];                                                              \
        _Pragma("unroll") for (int n_ = 0; n_ < G; ++n_)                                              \
            o[n_][out] = fmaf(w_, x[n_][a] * x[n_][b], o[n_][out]);                                   \
    }
#define SXB_POLY_F3(out, term, a, b, c)                                                               \
    {                                                                                                 \
        const float w_ = w[(term) * ws];                                                              \
        _Pragma("unroll") for (int n_ = 0; n_ < G; ++n_)                                              \
            o[n_][out] = fmaf(w_, x[n_][a] * x[n_][b] * x[n_][c], o[n_][out]);                        \
    }
#define SXB_POLY_R1(out, term, a)                                                                     \
    {                                                                                                 \
        const float w_ = w[(term) * ws];                                                              \
        _Pragma("unroll") for (int n_ = 0; n_ < G; ++n_) g[n_][a] = fmaf(w_, adj[n_][out], g[n_][a]); \
    }
#define SXB_POLY_R2(out, term, a, b)                                                                  \
    {                                                                                                 \
        const float w_ = w[(term) * ws];                                                              \
        _Pragma("unroll") for (int n_ = 0; n_ < G; ++n_) {                                            \
            const float s_ = w_ * adj[n_][out];                                                       \
            g[n_][a] = fmaf(s_, x[n_][b], g[n_][a]);                                                  \
            g[n_][b] = fmaf(s_, x[n_][a], g[n_][b]);                                                  \
        }                                                                                             \
    }
#define SXB_POLY_R3(out, term, a, b, c)                                                               \
    {                                                                                                 \
        const float w_ = w[(term) * ws];                                                              \
        _Pragma("unroll") for (int n_ = 0; n_ < G; ++n_) {                                            \
            const float s_ = w_ * adj[n_][out];                                                       \
            g[n_][a] = fmaf(s_, x[n_][b] * x[n_][c], g[n_][a]);                                       \
            g[n_][b] = fmaf(s_, x[n_][a] * x[n_][c], g[n_][b]);                                       \
            g[n_][c] = fmaf(s_, x[n_][a] * x[n_][b], g[n_][c]);                                       \
        }                                                                                             \
    }

constexpr int kPolyWarps = 8;
constexpr int kPolyNodesPerBlock = 32;

// Density-scaled models: dot[node] += sum over (lm, channels of this warp) of A_adj * A, the quantity
// the reference forms per node before the density force (libsymmetrix/source/mace.cpp:1611-1614,
// 2430-2433).  Called by a whole warp; one atomic per warp and node.
__device__ __forceinline__ void poly_accumulate_dot(const float* g, const float* x, float* __restrict__ dot, int node, int num_nodes)
{
    float partial = 0.0f;
#pragma unroll
    for (int q = 0; q < 16; ++q) partial = fmaf(g[q], x[q], partial);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, offset);
    if ((threadIdx.x & 31) == 0 && node < num_nodes) atomicAdd(dot + node, partial);
}

// Copies the [terms][32] weight slice of one element into shared memory (all threads of the block).
__device__ __forceinline__ void stage_poly_weights(float* __restrict__ dst, const float* __restrict__ weights, int type,
                                                   int terms, int C, int k_base)
{
    const float* src = weights + static_cast<size_t>(type) * terms * C + k_base;
    for (int idx = threadIdx.x; idx < terms * 32; idx += blockDim.x) dst[idx] = src[(idx >> 5) * C + (idx & 31)];
    __syncthreads();
}

// Walks the node groups of one block: BODY(node0, count_is_full_group_of_block_element, w, ws).
#define SXB_POLY_WALK(G, NT, CALL_GROUP, CALL_SINGLE)                                                               \
    extern __shared__ float w_s[];                                                                                  \
    const int block_node0 = blockIdx.x * kPolyNodesPerBlock;                                                        \
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;                                                     \
    const int k = blockIdx.y * 32 + lane;                                                                           \
    const int type0 = element[block_node0];                                                                         \
    stage_poly_weights(w_s, weights, type0, NT, C, blockIdx.y * 32);                                                \
    const int block_end = min(block_node0 + kPolyNodesPerBlock, num_nodes);                                         \
    for (int node0 = block_node0 + warp * G; node0 < block_end; node0 += kPolyWarps * G) {                          \
        bool same = true;                                                                                           \
        _Pragma("unroll") for (int n = 0; n < G; ++n) same = same && element[min(node0 + n, num_nodes - 1)] == type0; \
        if (same) {                                                                                                 \
            const float* w = w_s + lane;                                                                            \
            constexpr int ws = 32;                                                                                  \
            CALL_GROUP;                                                                                             \
        } else {                                                                                                    \
            for (int n = node0; n < min(node0 + G, block_end); ++n) {                                               \
                const float* w = weights + static_cast<size_t>(element[n]) * NT * C + k;                            \
                const int ws = C;                                                                                   \
                CALL_SINGLE;                                                                                        \
            }                                                                                                       \
        }                                                                                                           \
    }

#define SXB_DEFINE_POLY_KERNELS(NAME)                                                                               \
    /* M0[node][LM][k] from A0[node][16][k] for the nodes [node0, node0 + G) that exist */                          \
    template <int G>                                                                                                \
    __device__ __forceinline__ void m0_forward_group_##NAME(int node0, int num_nodes, int C, int k,                 \
                                                            const float* __restrict__ A0, const float* w, int ws,   \
                                                            float* __restrict__ M0)                                 \
    {                                                                                                               \
        constexpr int NH = SXB_##NAME##_NUM_HIDDEN;                                                                 \
        float x[G][16], o[G][NH];                                                                                   \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            const float* in = A0 + static_cast<size_t>(min(node0 + n, num_nodes - 1)) * 16 * C + k;                 \
            _Pragma("unroll") for (int q = 0; q < 16; ++q) x[n][q] = in[q * C];                                     \
            _Pragma("unroll") for (int q = 0; q < NH; ++q) o[n][q] = 0.0f;                                          \
        }                                                                                                           \
        SXB_##NAME##_M0_TERMS(SXB_POLY_F1, SXB_POLY_F2, SXB_POLY_F3)                                                \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            if (node0 + n < num_nodes) {                                                                            \
                float* out = M0 + static_cast<size_t>(node0 + n) * NH * C + k;                                      \
                _Pragma("unroll") for (int q = 0; q < NH; ++q) out[q * C] = o[n][q];                                \
            }                                                                                                       \
        }                                                                                                           \
    }                                                                                                               \
    template <int G>                                                                                                \
    __global__ void __launch_bounds__(32 * kPolyWarps, 2)                                                            \
    m0_forward_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A0, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, float* __restrict__ M0)                             \
    {                                                                                                               \
        SXB_POLY_WALK(G, SXB_##NAME##_M0_NUM_TERMS,                                                                 \
                      m0_forward_group_##NAME<G>(node0, num_nodes, C, k, A0, w, ws, M0),                            \
                      m0_forward_group_##NAME<1>(n, num_nodes, C, k, A0, w, ws, M0))                                \
    }                                                                                                               \
    /* A0_adj[node][16][k] = sum_LM M0_adj[node][LM][k] dM0[LM]/dA0 */                                              \
    template <int G>                                                                                                \
    __device__ __forceinline__ void m0_reverse_group_##NAME(int node0, int num_nodes, int C, int k,                 \
                                                            const float* __restrict__ A0, const float* w, int ws,   \
                                                            const float* __restrict__ M0_adj, float* __restrict__ A0_adj, \
                                                            float* __restrict__ dot)                                \
    {                                                                                                               \
        constexpr int NH = SXB_##NAME##_NUM_HIDDEN;                                                                 \
        float x[G][16], g[G][16], adj[G][NH];                                                                       \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            const size_t node = static_cast<size_t>(min(node0 + n, num_nodes - 1));                                 \
            const float* in = A0 + node * 16 * C + k;                                                               \
            _Pragma("unroll") for (int q = 0; q < 16; ++q) { x[n][q] = in[q * C]; g[n][q] = 0.0f; }                 \
            const float* ain = M0_adj + node * NH * C + k;                                                          \
            _Pragma("unroll") for (int q = 0; q < NH; ++q) adj[n][q] = ain[q * C];                                  \
        }                                                                                                           \
        SXB_##NAME##_M0_TERMS(SXB_POLY_R1, SXB_POLY_R2, SXB_POLY_R3)                                                \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            if (node0 + n < num_nodes) {                                                                            \
                float* out = A0_adj + static_cast<size_t>(node0 + n) * 16 * C + k;                                  \
                _Pragma("unroll") for (int q = 0; q < 16; ++q) out[q * C] = g[n][q];                                \
            }                                                                                                       \
            if (dot != nullptr) poly_accumulate_dot(g[n], x[n], dot, node0 + n, num_nodes);                         \
        }                                                                                                           \
    }                                                                                                               \
    template <int G>                                                                                                \
    __global__ void __launch_bounds__(32 * kPolyWarps, 1)                                                            \
    m0_reverse_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A0, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, const float* __restrict__ M0_adj,                   \
                             float* __restrict__ A0_adj, float* __restrict__ dot)                                   \
    {                                                                                                               \
        SXB_POLY_WALK(G, SXB_##NAME##_M0_NUM_TERMS,                                                                 \
                      m0_reverse_group_##NAME<G>(node0, num_nodes, C, k, A0, w, ws, M0_adj, A0_adj, dot),                \
                      m0_reverse_group_##NAME<1>(n, num_nodes, C, k, A0, w, ws, M0_adj, A0_adj, dot))                    \
    }                                                                                                               \
    /* M1[node][k] from A1[node][16][k] */                                                                          \
    template <int G>                                                                                                \
    __device__ __forceinline__ void m1_forward_group_##NAME(int node0, int num_nodes, int C, int k,                 \
                                                            const float* __restrict__ A1, const float* w, int ws,   \
                                                            float* __restrict__ M1)                                 \
    {                                                                                                               \
        float x[G][16], o[G][1];                                                                                    \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            const float* in = A1 + static_cast<size_t>(min(node0 + n, num_nodes - 1)) * 16 * C + k;                 \
            _Pragma("unroll") for (int q = 0; q < 16; ++q) x[n][q] = in[q * C];                                     \
            o[n][0] = 0.0f;                                                                                         \
        }                                                                                                           \
        SXB_##NAME##_M1_TERMS(SXB_POLY_F1, SXB_POLY_F2, SXB_POLY_F3)                                                \
        _Pragma("unroll") for (int n = 0; n < G; ++n)                                                               \
            if (node0 + n < num_nodes) M1[static_cast<size_t>(node0 + n) * C + k] = o[n][0];                        \
    }                                                                                                               \
    template <int G>                                                                                                \
    __global__ void __launch_bounds__(32 * kPolyWarps, 2)                                                            \
    m1_forward_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A1, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, float* __restrict__ M1)                             \
    {                                                                                                               \
        SXB_POLY_WALK(G, SXB_##NAME##_M1_NUM_TERMS,                                                                 \
                      m1_forward_group_##NAME<G>(node0, num_nodes, C, k, A1, w, ws, M1),                            \
                      m1_forward_group_##NAME<1>(n, num_nodes, C, k, A1, w, ws, M1))                                \
    }                                                                                                               \
    /* A1_adj[node][16][k] = M1_adj[node][k] dM1/dA1 */                                                             \
    template <int G>                                                                                                \
    __device__ __forceinline__ void m1_reverse_group_##NAME(int node0, int num_nodes, int C, int k,                 \
                                                            const float* __restrict__ A1, const float* w, int ws,   \
                                                            const float* __restrict__ M1_adj, float* __restrict__ A1_adj, \
                                                            float* __restrict__ dot)                                \
    {                                                                                                               \
        float x[G][16], g[G][16], adj[G][1];                                                                        \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            const size_t node = static_cast<size_t>(min(node0 + n, num_nodes - 1));                                 \
            const float* in = A1 + node * 16 * C + k;                                                               \
            _Pragma("unroll") for (int q = 0; q < 16; ++q) { x[n][q] = in[q * C]; g[n][q] = 0.0f; }                 \
            adj[n][0] = M1_adj[node * C + k];                                                                       \
        }                                                                                                           \
        SXB_##NAME##_M1_TERMS(SXB_POLY_R1, SXB_POLY_R2, SXB_POLY_R3)                                                \
        _Pragma("unroll") for (int n = 0; n < G; ++n) {                                                             \
            if (node0 + n < num_nodes) {                                                                            \
                float* out = A1_adj + static_cast<size_t>(node0 + n) * 16 * C + k;                                  \
                _Pragma("unroll") for (int q = 0; q < 16; ++q) out[q * C] = g[n][q];                                \
            }                                                                                                       \
            if (dot != nullptr) poly_accumulate_dot(g[n], x[n], dot, node0 + n, num_nodes);                         \
        }                                                                                                           \
    }                                                                                                               \
    template <int G>                                                                                                \
    __global__ void __launch_bounds__(32 * kPolyWarps, 2)                                                            \
    m1_reverse_kernel_##NAME(int num_nodes, int C, const float* __restrict__ A1, const unsigned char* __restrict__ element, \
                             const float* __restrict__ weights, const float* __restrict__ M1_adj,                   \
                             float* __restrict__ A1_adj, float* __restrict__ dot)                                   \
    {                                                                                                               \
        SXB_POLY_WALK(G, SXB_##NAME##_M1_NUM_TERMS,                                                                 \
                      m1_reverse_group_##NAME<G>(node0, num_nodes, C, k, A1, w, ws, M1_adj, A1_adj, dot),                \
                      m1_reverse_group_##NAME<1>(n, num_nodes, C, k, A1, w, ws, M1_adj, A1_adj, dot))                    \
    }

SXB_DEFINE_POLY_KERNELS(S0)
SXB_DEFINE_POLY_KERNELS(S1)
SXB_DEFINE_POLY_KERNELS(S2)

// ---------------------------------------------------------------------------------------------
// Readout polynomial of a single-layer model: M1[node][k] = sum_t w[element][t][k] prod_q H1[node][idx_t,q][k]
// over monomials of degree 1 to 3 in the hidden components, read as data (reference:
// libsymmetrix/source/mace.cpp:2460-2482 with the polynomial input switched to H1, and its gradient
// 2485-2512, which adds to H1_adj).  One thread per (node, channel); the monomial list is short (the
// invariants of at most nine components), so it is walked from global memory.
constexpr int kMaxHidden = 9;

template <bool kReverse>
__global__ void __launch_bounds__(128) hidden_poly_kernel(int num_nodes, int C, int num_hidden, int num_terms,
                                                          const int4* __restrict__ terms, const float* __restrict__ H1,
                                                          const unsigned char* __restrict__ element,
                                                          const float* __restrict__ weights, float* __restrict__ M1,
                                                          const float* __restrict__ M1_adj, float* __restrict__ H1_adj)
{
    const long index = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long>(num_nodes) * C) return;
    const int node = static_cast<int>(index / C), k = static_cast<int>(index - static_cast<long>(node) * C);
    float x[kMaxHidden], g[kMaxHidden];
#pragma unroll
    for (int q = 0; q < kMaxHidden; ++q) {
        x[q] = q < num_hidden ? H1[(static_cast<size_t>(node) * num_hidden + q) * C + k] : 0.0f;
        g[q] = 0.0f;
    }
    const float* w = weights + static_cast<size_t>(element[node]) * num_terms * C + k;
    float value = 0.0f;
    for (int t = 0; t < num_terms; ++t) {
        const int4 m = terms[t];
        const float wt = w[static_cast<size_t>(t) * C];
        const float a = x[m.x], b = m.y >= 0 ? x[m.y] : 1.0f, c = m.z >= 0 ? x[m.z] : 1.0f;
        if (!kReverse) {
            value = fmaf(wt, a * b * c, value);
        } else {
            g[m.x] = fmaf(wt, b * c, g[m.x]);
            if (m.y >= 0) g[m.y] = fmaf(wt, a * c, g[m.y]);
            if (m.z >= 0) g[m.z] = fmaf(wt, a * b, g[m.z]);
        }
    }
    if (!kReverse) {
        M1[static_cast<size_t>(node) * C + k] = value;
    } else {
        const float adj = M1_adj[static_cast<size_t>(node) * C + k];
        for (int q = 0; q < num_hidden; ++q) H1_adj[(static_cast<size_t>(node) * num_hidden + q) * C + k] += adj * g[q];
    }
}

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
        if (energy_slots != nullptr) atomicAdd(energy_slots + (node % kVirialSlots), e);
    }
}

// The same readout for the common head shape (16 hidden units, C a multiple of 32, at most 256): the 16
// pre-activations of a node are formed together, each lane holding its channels' partial sums, and
// summed over the warp by a butterfly that halves the number of live values at every step (16 shuffles
// instead of 80); lane L ends up with hidden unit L / 2.  No per-thread array is indexed at run time.
template <int kChunks>   // C / 32
__global__ void __launch_bounds__(256)
readout16_kernel(int num_nodes, float act_scale, const float* __restrict__ M0, int num_hidden_lm,
                 const float* __restrict__ H2, const unsigned char* __restrict__ element,
                 const double* __restrict__ atomic_energies, const float* __restrict__ q,
                 const float* __restrict__ W1 /*[16][C]*/, const float* __restrict__ W2 /*[16]*/,
                 double* __restrict__ node_energies, float* __restrict__ H2_adj, double* __restrict__ energy_slots)
{
    constexpr int C = 32 * kChunks, kHidden = 16;
    const int node = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (node >= num_nodes) return;
    const float* xs = M0 + static_cast<size_t>(node) * num_hidden_lm * C;   // scalar block of M0
    const float* h2 = H2 + static_cast<size_t>(node) * C;
    float hv[kChunks];
    float e1 = 0.0f;
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
        hv[j] = h2[lane + 32 * j];
        e1 = fmaf(q[lane + 32 * j], xs[lane + 32 * j], e1);
    }
    float v[kHidden];
#pragma unroll
    for (int h = 0; h < kHidden; ++h) {
        float z = 0.0f;
#pragma unroll
        for (int j = 0; j < kChunks; ++j) z = fmaf(W1[h * C + lane + 32 * j], hv[j], z);
        v[h] = z;
    }
#pragma unroll
    for (int offset = 16, live = kHidden; offset >= 2; offset >>= 1, live >>= 1) {
        const bool upper = (lane & offset) != 0;
        const int half = live / 2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < half) {
                const float send = upper ? v[i] : v[i + half];
                const float recv = __shfl_xor_sync(0xffffffffu, send, offset);
                v[i] = (upper ? v[i + half] : v[i]) + recv;
            }
        }
    }
    const float z = v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);      // lanes 2h and 2h+1: hidden unit h
    const int unit = lane >> 1;
    const float sig = 1.0f / (1.0f + expf(-z));
    const float w2 = W2[unit];
    float e2 = (lane & 1) ? 0.0f : w2 * (act_scale * z * sig);
    const float coeff = w2 * (act_scale * sig + act_scale * z * sig * (1.0f - sig));
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        e1 += __shfl_xor_sync(0xffffffffu, e1, offset);
        e2 += __shfl_xor_sync(0xffffffffu, e2, offset);
    }
    float g[kChunks];
#pragma unroll
    for (int j = 0; j < kChunks; ++j) g[j] = 0.0f;
#pragma unroll
    for (int h = 0; h < kHidden; ++h) {
        const float c = __shfl_sync(0xffffffffu, coeff, 2 * h);
#pragma unroll
        for (int j = 0; j < kChunks; ++j) g[j] = fmaf(c, W1[h * C + lane + 32 * j], g[j]);
    }
#pragma unroll
    for (int j = 0; j < kChunks; ++j) H2_adj[static_cast<size_t>(node) * C + lane + 32 * j] = g[j];
    if (lane == 0) {
        const double e = atomic_energies[element[node]] + static_cast<double>(e1) + static_cast<double>(e2);
        node_energies[node] = e;
        if (energy_slots != nullptr) atomicAdd(energy_slots + (node % kVirialSlots), e);
    }
}

// tensor[node][0][k] = values[k] for the first num_nodes nodes of a (node, component, channel) tensor.
__global__ void fill_scalar_block_kernel(int num_nodes, int C, long node_stride, const float* __restrict__ values,
                                         float* __restrict__ tensor)
{
    const long index = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long>(num_nodes) * C) return;
    const long node = index / C, k = index - node * C;
    tensor[node * node_stride + k] = values[k];
}

// tensor[node][:] += table[element[node]][:] over rows of row_floats values (element-dependent constants).
__global__ void add_element_rows_kernel(int num_nodes, int row_floats, const unsigned char* __restrict__ element,
                                        const float* __restrict__ table, float* __restrict__ tensor)
{
    const long index = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (index >= static_cast<long>(num_nodes) * row_floats) return;
    const long node = index / row_floats, k = index - node * row_floats;
    tensor[index] += table[static_cast<long>(element[node]) * row_floats + k];
}

// Closing kernel of an evaluation, one thread per output value: sums the energy / virial slots into
// totals[10] and writes node energies and node forces in the caller's node order.  When `host` is
// given the same values are also published straight into mapped pinned host memory, laid out
// [status word, totals[10], energies[num_receivers], forces[num_nodes][3]] (consecutive threads write
// consecutive words, so the writes cross the bus in full segments), and the caller needs no
// device-to-host copy.  Only the first `host_values` values go to the host (a caller that keeps the forces
// on the device asks for status and totals alone and saves the bus traffic).
__global__ void publish_results_kernel(int num_receivers, int num_nodes, const int* __restrict__ internal_of,
                                       const double* __restrict__ energy_slots, const double* __restrict__ virial_slots,
                                       const double* __restrict__ node_energies, const double* __restrict__ forces,
                                       const int* __restrict__ status, double* __restrict__ totals,
                                       double* __restrict__ energies_out, double* __restrict__ forces_out,
                                       double* __restrict__ host, long host_values)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long total = 11 + static_cast<long>(num_receivers) + 3 * static_cast<long>(num_nodes);
    if (idx >= total) return;
    double value;
    if (idx == 0) {
        value = static_cast<double>(status[0]);
    } else if (idx < 11) {
        const int t = static_cast<int>(idx) - 1;
        value = 0.0;
        for (int slot = 0; slot < kVirialSlots; ++slot) value += (t == 0) ? energy_slots[slot] : virial_slots[slot * 9 + (t - 1)];
        totals[t] = value;
    } else if (idx < 11 + num_receivers) {
        const long o = idx - 11;
        value = node_energies[internal_of[o]];
        energies_out[o] = value;
    } else {
        const long j = idx - 11 - num_receivers;
        const long o = j / 3, q = j % 3;
        value = forces[3 * static_cast<long>(internal_of[o]) + q];
        forces_out[j] = value;
    }
    if (host != nullptr && idx < host_values) host[idx] = value;
}

}  // namespace sxb
