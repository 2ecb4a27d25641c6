// Layer-1 edge kernels for coupling structures whose row count does not fit one thread's
// registers (hidden irreps up to l = 2: 17 paths, 243 rows, 71 outputs).  The paths are split at
// generation time into sets with equal row counts; one kernel instance handles one set for all
// receivers: it evaluates only that set's radial functions, keeps only that set's row sums (or
// row adjoints) in registers and writes only the outputs that set feeds - every output component
// belongs to exactly one path, so the sets write disjoint parts of Phi1 and read disjoint parts of
// dPhi1.  What the sets share is accumulated atomically: the source adjoint H1_adj (as in the
// unsplit kernel), the edge forces, the receiver force and the virial.
// Thread mapping, edge chunking and the math are those of edge_kernels.cuh (layer 1 forward and
// fused gradient, libsymmetrix/source/mace.cpp:2023-2083 and 2199-2302).
#pragma once

#include "edge_kernels.cuh"

namespace sxb {

#define SXB_DEFINE_L1_SPLIT_KERNELS(NAME, G)                                                                         \
    template <int kC>                                                                                                \
    __global__ void __launch_bounds__(kC)                                                                            \
    l1_forward_split_kernel_##NAME##_##G(int num_nodes, int node0, const int* __restrict__ first,                    \
                                         const int* __restrict__ sources, const EdgeGeom* __restrict__ geom,         \
                                         const unsigned char* __restrict__ atype, SplineGrid grid,                   \
                                         const float4* __restrict__ table4, const float* __restrict__ H1,            \
                                         const __grid_constant__ CouplingConstants cgc, float* __restrict__ Phi1,    \
                                         const float* __restrict__ inv_scale, int pair_types)                        \
    {                                                                                                                \
        constexpr int C = kC;                                                                                        \
        constexpr int NP = SXB_##NAME##_NUM_PATHS, NH = SXB_##NAME##_NUM_HIDDEN, NE = SXB_##NAME##_NUM_LME;          \
        constexpr int NPG = SXB_##NAME##_##G##_NUM_PATHS, NRG = SXB_##NAME##_##G##_NUM_ROWS;                         \
        constexpr int NEG = SXB_##NAME##_##G##_NUM_LME;                                                              \
        constexpr int path_of[NPG] = SXB_##NAME##_##G##_PATH_LIST;                                                   \
        constexpr int lme_of[NEG] = SXB_##NAME##_##G##_LME_LIST;                                                     \
        constexpr int F = NP * C;                                                                                    \
        __shared__ ChunkState<false> s;                                                                              \
        const int local = blockIdx.x, i = node0 + local;                                                             \
        const int k = threadIdx.x;                                                                                   \
        const int begin = first[i], end = first[i + 1];                                                              \
        float acc[NRG];                                                                                              \
        _Pragma("unroll") for (int r_ = 0; r_ < NRG; ++r_) acc[r_] = 0.0f;                                           \
        for (int chunk = begin; chunk < end; chunk += kEdgeChunk) {                                                  \
            const int count = min(kEdgeChunk, end - chunk);                                                          \
            __syncthreads();                                                                                         \
            fill_chunk<false, false>(s, chunk, count, sources, geom, atype, atype[i], pair_types, grid, F);          \
            __syncthreads();                                                                                         \
            for (int t = 0; t < count; ++t) {                                                                        \
                const int2 id = s.index[t];                                                                          \
                if (id.x < 0) continue;                                                                              \
                const float x = s.misc[t].x, xx = x * x, xxx = xx * x;                                               \
                const float4* c4 = table4 + (id.x >> 2) + k;                                                         \
                float R[NPG];                                                                                        \
                _Pragma("unroll") for (int q = 0; q < NPG; ++q) {                                                    \
                    const float4 c = c4[path_of[q] * C];                                                             \
                    R[q] = cubic(c.x, c.y, c.z, c.w, x, xx, xxx);                                                    \
                }                                                                                                    \
                const float* hsrc = H1 + static_cast<size_t>(id.y) * NH * C + k;                                     \
                float h[NH];                                                                                         \
                _Pragma("unroll") for (int q = 0; q < NH; ++q)                                                       \
                    h[q] = ((SXB_##NAME##_##G##_SOURCE_MASK >> q) & 1u) ? hsrc[q * C] : 0.0f;                         \
                float y[16];                                                                                         \
                load16(s.y[t], y);                                                                                   \
                SXB_##NAME##_##G##_FORWARD_BODY                                                                      \
            }                                                                                                        \
        }                                                                                                            \
        float out_lme[NEG];                                                                                          \
        _Pragma("unroll") for (int q = 0; q < NEG; ++q) out_lme[q] = 0.0f;                                           \
        SXB_##NAME##_##G##_TERMS(SXB_TERM_FORWARD)                                                                   \
        const float scale = inv_scale != nullptr ? inv_scale[i] : 1.0f;                                              \
        float* out = Phi1 + static_cast<size_t>(local) * NE * C + k;                                                 \
        _Pragma("unroll") for (int q = 0; q < NEG; ++q) out[lme_of[q] * C] = out_lme[q] * scale;                     \
    }                                                                                                                \
                                                                                                                     \
    template <int kC>                                                                                                \
    __global__ void __launch_bounds__(kC)                                                                            \
    l1_reverse_split_kernel_##NAME##_##G(int num_nodes, int node0, const int* __restrict__ first,                    \
                                         const int* __restrict__ sources, const EdgeGeom* __restrict__ geom,         \
                                         const unsigned char* __restrict__ atype, SplineGrid grid,                   \
                                         const float4* __restrict__ table4, const float* __restrict__ H1,            \
                                         const float* __restrict__ dPhi1,                                            \
                                         const __grid_constant__ CouplingConstants cgc, float* __restrict__ H1_adj,  \
                                         ForceOutputs out, DensityScale density, int pair_types)                     \
    {                                                                                                                \
        constexpr int C = kC;                                                                                        \
        constexpr int NP = SXB_##NAME##_NUM_PATHS, NH = SXB_##NAME##_NUM_HIDDEN, NE = SXB_##NAME##_NUM_LME;          \
        constexpr int NPG = SXB_##NAME##_##G##_NUM_PATHS, NRG = SXB_##NAME##_##G##_NUM_ROWS;                         \
        constexpr int NEG = SXB_##NAME##_##G##_NUM_LME;                                                              \
        constexpr int path_of[NPG] = SXB_##NAME##_##G##_PATH_LIST;                                                   \
        constexpr int lme_of[NEG] = SXB_##NAME##_##G##_LME_LIST;                                                     \
        constexpr int F = NP * C;                                                                                    \
        constexpr int kWarps = kC / 32;                                                                              \
        __shared__ ChunkState<true> s;                                                                               \
        __shared__ ForceScratch<kWarps> fs;                                                                          \
        const int local = blockIdx.x, i = node0 + local;                                                             \
        const int k = threadIdx.x;                                                                                   \
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;                                                  \
        const int begin = first[i], end = first[i + 1];                                                              \
        if (threadIdx.x < 3) fs.receiver[threadIdx.x] = 0.0;                                                         \
        if (threadIdx.x < 9) fs.virial[threadIdx.x] = 0.0;                                                           \
        const float scale = density.table != nullptr ? density.inv_scale[i] : 1.0f;                                  \
        /* the density force is one term per edge: the first path set carries it */                                 \
        const float density_coef =                                                                                   \
            (density.table != nullptr && SXB_##NAME##_##G##_HAS_PATH0) ? density.dot[i] * scale : 0.0f;              \
        float adj[NRG];                                                                                              \
        {                                                                                                            \
            float dphi[NEG];                                                                                         \
            const float* in = dPhi1 + static_cast<size_t>(local) * NE * C + k;                                       \
            _Pragma("unroll") for (int q = 0; q < NEG; ++q) dphi[q] = in[lme_of[q] * C] * scale;                     \
            _Pragma("unroll") for (int r_ = 0; r_ < NRG; ++r_) adj[r_] = 0.0f;                                       \
            SXB_##NAME##_##G##_TERMS(SXB_TERM_TRANSPOSE)                                                             \
        }                                                                                                            \
        for (int chunk = begin; chunk < end; chunk += kEdgeChunk) {                                                  \
            const int count = min(kEdgeChunk, end - chunk);                                                          \
            __syncthreads();                                                                                         \
            fill_chunk<true, false>(s, chunk, count, sources, geom, atype, atype[i], pair_types, grid, F,            \
                                    density.table, density.types);                                                   \
            __syncthreads();                                                                                         \
            for (int t = 0; t < count; ++t) {                                                                        \
                const int2 id = s.index[t];                                                                          \
                if (id.x < 0) continue;                                                                              \
                const float4 m = s.misc[t];                                                                          \
                const float x = m.x, xx = x * x, xxx = xx * x, x2 = 2.0f * x, xx3 = 3.0f * xx;                       \
                const float4* c4 = table4 + (id.x >> 2) + k;                                                         \
                float R[NPG], dR[NPG];                                                                               \
                _Pragma("unroll") for (int q = 0; q < NPG; ++q) {                                                    \
                    const float4 c = c4[path_of[q] * C];                                                             \
                    R[q] = cubic(c.x, c.y, c.z, c.w, x, xx, xxx);                                                    \
                    dR[q] = cubic_derivative(c.y, c.z, c.w, x2, xx3);                                                \
                }                                                                                                    \
                const size_t source_row = static_cast<size_t>(id.y) * NH * C + k;                                    \
                float h[NH], hadj[NH];                                                                               \
                _Pragma("unroll") for (int q = 0; q < NH; ++q) {                                                     \
                    h[q] = ((SXB_##NAME##_##G##_SOURCE_MASK >> q) & 1u) ? H1[source_row + q * C] : 0.0f;             \
                    hadj[q] = 0.0f;                                                                                  \
                }                                                                                                    \
                float y[16], ang[16];                                                                                \
                load16(s.y[t], y);                                                                                   \
                _Pragma("unroll") for (int q = 0; q < 16; ++q) ang[q] = 0.0f;                                        \
                float radial = 0.0f;                                                                                 \
                SXB_##NAME##_##G##_REVERSE_BODY                                                                      \
                _Pragma("unroll") for (int q = 0; q < NH; ++q)                                                       \
                    if ((SXB_##NAME##_##G##_SOURCE_MASK >> q) & 1u) atomicAdd(H1_adj + source_row + q * C, hadj[q]); \
                float fx = radial * m.y, fy = radial * m.z, fz = radial * m.w;                                       \
                {                                                                                                    \
                    float g[16];                                                                                     \
                    load16(s.gx[t], g);                                                                              \
                    _Pragma("unroll") for (int q = 0; q < 16; ++q)                                                   \
                        if ((SXB_##NAME##_##G##_EDGE_MASK >> q) & 1u) fx = fmaf(ang[q], g[q], fx);                   \
                    load16(s.gy[t], g);                                                                              \
                    _Pragma("unroll") for (int q = 0; q < 16; ++q)                                                   \
                        if ((SXB_##NAME##_##G##_EDGE_MASK >> q) & 1u) fy = fmaf(ang[q], g[q], fy);                   \
                    load16(s.gz[t], g);                                                                              \
                    _Pragma("unroll") for (int q = 0; q < 16; ++q)                                                   \
                        if ((SXB_##NAME##_##G##_EDGE_MASK >> q) & 1u) fz = fmaf(ang[q], g[q], fz);                   \
                }                                                                                                    \
                const float total = warp_reduce3_transposed(fx, fy, fz, lane);                                       \
                if ((lane & 7) == 0 && lane < 24) fs.partial[t][warp][lane >> 3] = total;                            \
            }                                                                                                        \
            __syncthreads();                                                                                         \
            flush_chunk_forces<kWarps>(fs, s, chunk, count, kWarps, out, density_coef);                              \
        }                                                                                                            \
        finish_receiver_forces<kWarps>(fs, i, out);                                                                  \
    }

SXB_DEFINE_L1_SPLIT_KERNELS(S2, G0)
SXB_DEFINE_L1_SPLIT_KERNELS(S2, G1)
SXB_DEFINE_L1_SPLIT_KERNELS(S2, G2)

}  // namespace sxb
