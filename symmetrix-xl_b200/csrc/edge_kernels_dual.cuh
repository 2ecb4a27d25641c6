// Fused layer-1 gradient with two threads per channel (hidden irreps 0e+1o, 10 paths / 88 rows).
//
// The one-thread-per-channel kernel keeps all 88 row adjoints of its channel in registers, which
// limits an SM to 12 warps.  Here the paths are split by the parity of the edge l into two sets
// (49 and 39 rows); a block of 2*C threads owns one receiver, thread (set, channel) keeps only its
// set's row adjoints, evaluates only its set's five radial functions and needs only its set's edge
// harmonics and harmonic gradients (an edge harmonic belongs to exactly one set).  Both sets share
// the per-chunk edge state in shared memory and the force bookkeeping; each adds its part of the
// source adjoint with red.global.add.  Same math as l1_reverse_kernel_S1 (edge_kernels.cuh; reference
// statement libsymmetrix/source/mace.cpp:2199-2302).
#pragma once

#include "edge_kernels.cuh"

namespace sxb {

#define SXB_DEFINE_PATH_SET(NAME, G)                                                                                  \
    struct PathSet_##NAME##_##G {                                                                                     \
        static constexpr int NP = SXB_##NAME##_NUM_PATHS, NH = SXB_##NAME##_NUM_HIDDEN, NE = SXB_##NAME##_NUM_LME;    \
        static constexpr int NPG = SXB_##NAME##_##G##_NUM_PATHS, NRG = SXB_##NAME##_##G##_NUM_ROWS;                   \
        static constexpr int NEG = SXB_##NAME##_##G##_NUM_LME;                                                        \
        static constexpr unsigned kEdgeMask = SXB_##NAME##_##G##_EDGE_MASK;                                           \
        static constexpr unsigned kSourceMask = SXB_##NAME##_##G##_SOURCE_MASK;                                       \
        static __device__ __forceinline__ int path(int q)                                                             \
        {                                                                                                             \
            constexpr int list[NPG] = SXB_##NAME##_##G##_PATH_LIST;                                                   \
            return list[q];                                                                                           \
        }                                                                                                             \
        static __device__ __forceinline__ int output(int q)                                                           \
        {                                                                                                             \
            constexpr int list[NEG] = SXB_##NAME##_##G##_LME_LIST;                                                    \
            return list[q];                                                                                           \
        }                                                                                                             \
        static __device__ __forceinline__ void transpose(const CouplingConstants& cgc, const float* __restrict__ dphi, \
                                                         float* __restrict__ adj)                                     \
        {                                                                                                             \
            SXB_##NAME##_##G##_TERMS(SXB_TERM_TRANSPOSE)                                                              \
        }                                                                                                             \
        static __device__ __forceinline__ void edge(const float* __restrict__ R, const float* __restrict__ dR,        \
                                                    const float* __restrict__ h, const float* __restrict__ y,         \
                                                    const float* __restrict__ adj, float* __restrict__ ang,           \
                                                    float* __restrict__ hadj, float& radial)                          \
        {                                                                                                             \
            SXB_##NAME##_##G##_REVERSE_BODY                                                                           \
        }                                                                                                             \
    };

SXB_DEFINE_PATH_SET(S1, G0)
SXB_DEFINE_PATH_SET(S1, G1)

// Reads the 16-float row of an edge as 128-bit shared loads, skipping the quarters no component of `kMask` lies in.
template <unsigned kMask>
__device__ __forceinline__ void load_rows(const float4* __restrict__ row, float* __restrict__ out)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        if ((kMask >> (4 * q)) & 0xFu) {
            const float4 v = row[q];
            out[4 * q] = v.x; out[4 * q + 1] = v.y; out[4 * q + 2] = v.z; out[4 * q + 3] = v.w;
        } else {
            out[4 * q] = out[4 * q + 1] = out[4 * q + 2] = out[4 * q + 3] = 0.0f;
        }
    }
}

struct L1ReverseArgs {
    const int* first;
    const int* sources;
    const EdgeGeom* geom;
    const unsigned char* atype;
    SplineGrid grid;
    const float4* table4;
    const float* H1;
    const float* dPhi1;
    float* H1_adj;
    ForceOutputs out;
    DensityScale density;
    int pair_types;
};

// Work of one (set, channel) thread for receiver i; every thread of the block runs this with its own Set,
// and all of them meet at the same barriers.
template <class Set, int kC, int kWarps>
__device__ __forceinline__ void l1_reverse_path_set(ChunkState<true>& s, ForceScratch<kWarps>& fs, const L1ReverseArgs& a,
                                                    const CouplingConstants& cgc, int local, int i, int k, int warp, int lane)
{
    constexpr int C = kC, NH = Set::NH, NE = Set::NE, NPG = Set::NPG, NRG = Set::NRG, NEG = Set::NEG;
    constexpr int F = Set::NP * C;
    const int begin = a.first[i], end = a.first[i + 1];
    const float scale = a.density.table != nullptr ? a.density.inv_scale[i] : 1.0f;
    const float density_coef = a.density.table != nullptr ? a.density.dot[i] * scale : 0.0f;   // applied once per edge in the flush
    float adj[NRG];
    {
        float dphi[NEG];
        const float* in = a.dPhi1 + static_cast<size_t>(local) * NE * C + k;
#pragma unroll
        for (int q = 0; q < NEG; ++q) dphi[q] = in[Set::output(q) * C] * scale;
#pragma unroll
        for (int r = 0; r < NRG; ++r) adj[r] = 0.0f;
        Set::transpose(cgc, dphi, adj);
    }
    for (int chunk = begin; chunk < end; chunk += kEdgeChunk) {
        const int count = min(kEdgeChunk, end - chunk);
        __syncthreads();
        fill_chunk<true, false>(s, chunk, count, a.sources, a.geom, a.atype, a.atype[i], a.pair_types, a.grid, F, a.density.table,
                                a.density.types);
        __syncthreads();
        for (int t = 0; t < count; ++t) {
            const int2 id = s.index[t];
            if (id.x < 0) continue;
            const float4 m = s.misc[t];
            const float x = m.x, xx = x * x, xxx = xx * x, x2 = 2.0f * x, xx3 = 3.0f * xx;
            const float4* c4 = a.table4 + (id.x >> 2) + k;
            float R[NPG], dR[NPG];
#pragma unroll
            for (int q = 0; q < NPG; ++q) {
                const float4 c = c4[Set::path(q) * C];
                R[q] = cubic(c.x, c.y, c.z, c.w, x, xx, xxx);
                dR[q] = cubic_derivative(c.y, c.z, c.w, x2, xx3);
            }
            const size_t source_row = static_cast<size_t>(id.y) * NH * C + k;
            float h[NH], hadj[NH];
#pragma unroll
            for (int q = 0; q < NH; ++q) {
                h[q] = ((Set::kSourceMask >> q) & 1u) ? a.H1[source_row + q * C] : 0.0f;
                hadj[q] = 0.0f;
            }
            // only the set's own edge harmonics are read from the chunk state
            float y[16], ang[16];
            load_rows<Set::kEdgeMask>(s.y[t], y);
#pragma unroll
            for (int q = 0; q < 16; ++q) ang[q] = 0.0f;
            float radial = 0.0f;
            Set::edge(R, dR, h, y, adj, ang, hadj, radial);
#pragma unroll
            for (int q = 0; q < NH; ++q)
                if ((Set::kSourceMask >> q) & 1u) atomicAdd(a.H1_adj + source_row + q * C, hadj[q]);
            float fx = radial * m.y, fy = radial * m.z, fz = radial * m.w;
            {
                float g[16];
                load_rows<Set::kEdgeMask>(s.gx[t], g);
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if ((Set::kEdgeMask >> q) & 1u) fx = fmaf(ang[q], g[q], fx);
                load_rows<Set::kEdgeMask>(s.gy[t], g);
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if ((Set::kEdgeMask >> q) & 1u) fy = fmaf(ang[q], g[q], fy);
                load_rows<Set::kEdgeMask>(s.gz[t], g);
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if ((Set::kEdgeMask >> q) & 1u) fz = fmaf(ang[q], g[q], fz);
            }
            const float total = warp_reduce3_transposed(fx, fy, fz, lane);
            if ((lane & 7) == 0 && lane < 24) fs.partial[t][warp][lane >> 3] = total;
        }
        __syncthreads();
        flush_chunk_forces<kWarps>(fs, s, chunk, count, kWarps, a.out, density_coef);
    }
    finish_receiver_forces<kWarps>(fs, i, a.out);
}

template <int kC>
__global__ void __launch_bounds__(2 * kC, 2)
l1_reverse_dual_kernel_S1(int num_nodes, int node0, L1ReverseArgs a, const __grid_constant__ CouplingConstants cgc)
{
    constexpr int kWarps = 2 * kC / 32;
    __shared__ ChunkState<true> s;
    __shared__ ForceScratch<kWarps> fs;
    const int local = blockIdx.x, i = node0 + local;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < 3) fs.receiver[threadIdx.x] = 0.0;
    if (threadIdx.x < 9) fs.virial[threadIdx.x] = 0.0;
    if (threadIdx.x < kC)
        l1_reverse_path_set<PathSet_S1_G0, kC, kWarps>(s, fs, a, cgc, local, i, threadIdx.x, warp, lane);
    else
        l1_reverse_path_set<PathSet_S1_G1, kC, kWarps>(s, fs, a, cgc, local, i, threadIdx.x - kC, warp, lane);
}

}  // namespace sxb
