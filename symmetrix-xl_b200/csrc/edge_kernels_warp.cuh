// Layer-0 edge kernels, warp-per-receiver form: one warp owns one receiver and every lane owns
// kVec consecutive channels (C = 32*kVec), so the channel-independent edge state read from shared
// memory, the gradient contraction and the 3-value force reduction are paid once per kVec channels,
// spline coefficients arrive as 128-bit loads, and a receiver needs no block-wide barrier at all.
// These kernels are bound by the load/store pipe (ncu: l1tex data-pipe wavefronts ~86 % of peak for
// the one-channel-per-thread form), which is what this layout relieves.
// Math and reference citations: see edge_kernels.cuh (layer 0 forward/reverse,
// libsymmetrix/source/mace.cpp:1356-1403 and 1486-1559).
#pragma once

#include "edge_kernels.cuh"

namespace sxb {

constexpr int kWarpChunk = 32;        // edges staged per pass: one per lane
constexpr int kWarpsPerBlock = 4;

template <bool kGradient>
struct alignas(16) WarpChunk {
    float4 y[kWarpChunk][4];
    float4 gx[kGradient ? kWarpChunk : 1][4];
    float4 gy[kGradient ? kWarpChunk : 1][4];
    float4 gz[kGradient ? kWarpChunk : 1][4];
    float4 misc[kWarpChunk];      // x = spline offset, yzw = unit direction
    int2 index[kWarpChunk];       // x = coefficient base or -1, y = source
    float len[kGradient ? kWarpChunk : 1];
    float dens[kGradient ? kWarpChunk : 1];   // d/dr of the density spline (0 without density scaling)
    float force[kGradient ? kWarpChunk : 1][3];
};

template <bool kGradient>
__device__ __forceinline__ void fill_warp_chunk(WarpChunk<kGradient>& s, int lane, int begin, int count,
                                                const int* __restrict__ sources, const EdgeGeom* __restrict__ geom,
                                                const unsigned char* __restrict__ atype, int type_i, int num_active,
                                                const SplineGrid& grid, int functions,
                                                const float* __restrict__ density_table = nullptr, int density_types = 1)
{
    if (lane < count) {
        const int e = begin + lane;
        const EdgeGeom g = geom[e];
        const int j = sources[e];
        if (!(g.r < grid.r_cut)) {
            s.index[lane] = make_int2(-1, j);
        } else {
            int interval;
            float x;
            spline_point(grid, g.r, interval, x);
            const int pair = type_i * num_active + atype[j];
            s.index[lane] = make_int2((pair * grid.intervals + interval) * 4 * functions, j);
            s.misc[lane] = make_float4(x, g.ux, g.uy, g.uz);
            const float inv_r = 1.0f / g.r;
            if constexpr (kGradient) {
                harmonics16<true>(g.ux, g.uy, g.uz, inv_r, reinterpret_cast<float*>(s.y[lane]), reinterpret_cast<float*>(s.gx[lane]),
                                  reinterpret_cast<float*>(s.gy[lane]), reinterpret_cast<float*>(s.gz[lane]));
                s.len[lane] = g.r;
                s.dens[lane] = density_table != nullptr
                                   ? scalar_spline_derivative(density_table, (type_i * density_types + (density_types > 1 ? atype[j] : 0)) * grid.intervals + interval, x)
                                   : 0.0f;
            } else {
                harmonics16<false>(g.ux, g.uy, g.uz, inv_r, reinterpret_cast<float*>(s.y[lane]), nullptr, nullptr, nullptr);
            }
        }
    }
}

template <int kVec>
struct VecLoad;
template <>
struct VecLoad<1> {
    static __device__ __forceinline__ void load(const float* p, float* out) { out[0] = *p; }
    static __device__ __forceinline__ void store(float* p, const float* in) { *p = in[0]; }
};
template <>
struct VecLoad<2> {
    static __device__ __forceinline__ void load(const float* p, float* out)
    {
        const float2 v = *reinterpret_cast<const float2*>(p);
        out[0] = v.x; out[1] = v.y;
    }
    static __device__ __forceinline__ void store(float* p, const float* in) { *reinterpret_cast<float2*>(p) = make_float2(in[0], in[1]); }
};
template <>
struct VecLoad<4> {
    static __device__ __forceinline__ void load(const float* p, float* out)
    {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* in)
    {
        *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    }
};

// ---------------------------------------------------------------------------------------------
template <int kVec>
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
l0_forward_warp_kernel(int num_nodes, int node0, const int* __restrict__ first, const int* __restrict__ sources,
                       const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype, int num_active,
                       SplineGrid grid, const float* __restrict__ table, float* __restrict__ A0,
                       const float* __restrict__ inv_scale)
{
    constexpr int C = 32 * kVec, F = 4 * C;
    __shared__ WarpChunk<false> chunks[kWarpsPerBlock];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int local = blockIdx.x * kWarpsPerBlock + warp;   // receiver inside the tile
    if (local >= num_nodes) return;
    const int i = node0 + local;                            // graph-wide receiver index
    WarpChunk<false>& s = chunks[warp];
    const int k = lane * kVec;
    const int type_i = atype[i];
    const int begin = first[i], end = first[i + 1];
    float acc[16][kVec];
#pragma unroll
    for (int lm = 0; lm < 16; ++lm)
#pragma unroll
        for (int v = 0; v < kVec; ++v) acc[lm][v] = 0.0f;
    for (int chunk = begin; chunk < end; chunk += kWarpChunk) {
        const int count = min(kWarpChunk, end - chunk);
        __syncwarp();
        fill_warp_chunk<false>(s, lane, chunk, count, sources, geom, atype, type_i, num_active, grid, F);
        __syncwarp();
        for (int t = 0; t < count; ++t) {
            const int base = s.index[t].x;
            if (base < 0) continue;
            const float x = s.misc[t].x, xx = x * x, xxx = xx * x;
            const float* c = table + base + k;
            float y[16];
            load16(s.y[t], y);
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                float c0[kVec], c1[kVec], c2[kVec], c3[kVec];
                VecLoad<kVec>::load(c + l * C, c0);
                VecLoad<kVec>::load(c + F + l * C, c1);
                VecLoad<kVec>::load(c + 2 * F + l * C, c2);
                VecLoad<kVec>::load(c + 3 * F + l * C, c3);
#pragma unroll
                for (int v = 0; v < kVec; ++v) {
                    const float R = cubic(c0[v], c1[v], c2[v], c3[v], x, xx, xxx);
#pragma unroll
                    for (int lm = l * l; lm < (l + 1) * (l + 1); ++lm) acc[lm][v] = fmaf(R, y[lm], acc[lm][v]);
                }
            }
        }
    }
    if (inv_scale != nullptr) {   // density scaling, mace.cpp:1562-1584
        const float scale = inv_scale[i];
#pragma unroll
        for (int lm = 0; lm < 16; ++lm)
#pragma unroll
            for (int v = 0; v < kVec; ++v) acc[lm][v] *= scale;
    }
    float* out = A0 + static_cast<size_t>(local) * 16 * C + k;
#pragma unroll
    for (int lm = 0; lm < 16; ++lm) VecLoad<kVec>::store(out + lm * C, acc[lm]);
}

// ---------------------------------------------------------------------------------------------
template <int kVec>
__global__ void __launch_bounds__(32 * kWarpsPerBlock)
l0_reverse_warp_kernel(int num_nodes, int node0, const int* __restrict__ first, const int* __restrict__ sources,
                       const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype, int num_active,
                       SplineGrid grid, const float* __restrict__ table, const float* __restrict__ A0_adj, ForceOutputs out,
                       DensityScale density)
{
    constexpr int C = 32 * kVec, F = 4 * C;
    __shared__ WarpChunk<true> chunks[kWarpsPerBlock];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int local = blockIdx.x * kWarpsPerBlock + warp;   // receiver inside the tile
    if (local >= num_nodes) return;
    const int i = node0 + local;                            // graph-wide receiver index
    WarpChunk<true>& s = chunks[warp];
    const int k = lane * kVec;
    const int type_i = atype[i];
    const int begin = first[i], end = first[i + 1];
    float adj[16][kVec];
    {
        const float* in = A0_adj + static_cast<size_t>(local) * 16 * C + k;
#pragma unroll
        for (int lm = 0; lm < 16; ++lm) VecLoad<kVec>::load(in + lm * C, adj[lm]);
    }
    // with density scaling the stored adjoint refers to the scaled A0: dE/dA0_unscaled = adj / (1 + rho_i)
    float density_coef = 0.0f;
    if (density.table != nullptr) {
        const float scale = density.inv_scale[i];
        density_coef = density.dot[i] * scale;
#pragma unroll
        for (int lm = 0; lm < 16; ++lm)
#pragma unroll
            for (int v = 0; v < kVec; ++v) adj[lm][v] *= scale;
    }
    // per-lane partial sums over the edges this lane finishes (lane t owns edge t of every chunk)
    double rfx = 0.0, rfy = 0.0, rfz = 0.0;
    double vir[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (int chunk = begin; chunk < end; chunk += kWarpChunk) {
        const int count = min(kWarpChunk, end - chunk);
        __syncwarp();
        fill_warp_chunk<true>(s, lane, chunk, count, sources, geom, atype, type_i, num_active, grid, F, density.table, density.types);
        __syncwarp();
        for (int t = 0; t < count; ++t) {
            const int base = s.index[t].x;
            if (base < 0) continue;
            const float4 m = s.misc[t];
            const float x = m.x, xx = x * x, xxx = xx * x, x2 = 2.0f * x, xx3 = 3.0f * xx;
            const float* c = table + base + k;
            float y[16], ang[16];
            load16(s.y[t], y);
            float radial = 0.0f;
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                float c0[kVec], c1[kVec], c2[kVec], c3[kVec];
                VecLoad<kVec>::load(c + l * C, c0);
                VecLoad<kVec>::load(c + F + l * C, c1);
                VecLoad<kVec>::load(c + 2 * F + l * C, c2);
                VecLoad<kVec>::load(c + 3 * F + l * C, c3);
#pragma unroll
                for (int lm = l * l; lm < (l + 1) * (l + 1); ++lm) ang[lm] = 0.0f;
#pragma unroll
                for (int v = 0; v < kVec; ++v) {
                    const float R = cubic(c0[v], c1[v], c2[v], c3[v], x, xx, xxx);
                    const float dR = cubic_derivative(c1[v], c2[v], c3[v], x2, xx3);
                    float ya = 0.0f;
#pragma unroll
                    for (int lm = l * l; lm < (l + 1) * (l + 1); ++lm) {
                        ya = fmaf(y[lm], adj[lm][v], ya);
                        ang[lm] = fmaf(R, adj[lm][v], ang[lm]);
                    }
                    radial = fmaf(dR, ya, radial);
                }
            }
            float fx = radial * m.y, fy = radial * m.z, fz = radial * m.w;
            {
                float g[16];
                load16(s.gx[t], g);
#pragma unroll
                for (int q = 0; q < 16; ++q) fx = fmaf(ang[q], g[q], fx);
                load16(s.gy[t], g);
#pragma unroll
                for (int q = 0; q < 16; ++q) fy = fmaf(ang[q], g[q], fy);
                load16(s.gz[t], g);
#pragma unroll
                for (int q = 0; q < 16; ++q) fz = fmaf(ang[q], g[q], fz);
            }
            const float total = warp_reduce3_transposed(fx, fy, fz, lane);
            if ((lane & 7) == 0 && lane < 24) s.force[t][lane >> 3] = total;
        }
        __syncwarp();
        // lane t finishes edge t: directed force dE/d(xyz_ij) = -(sum), scatter and virial
        if (lane < count && s.index[lane].x >= 0) {
            const float4 u = s.misc[lane];
            const float dens = density_coef * s.dens[lane];   // dE/d(xyz) += (A_adj . A) / (1 + rho) * s'(r) * rhat
            const double ex = -static_cast<double>(s.force[lane][0] - dens * u.y);
            const double ey = -static_cast<double>(s.force[lane][1] - dens * u.z);
            const double ez = -static_cast<double>(s.force[lane][2] - dens * u.w);
            const int j = s.index[lane].y;
            if (out.atom_forces != nullptr) {
                atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j), ex);
                atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j) + 1, ey);
                atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j) + 2, ez);
            }
            rfx -= ex; rfy -= ey; rfz -= ez;
            const double len = s.len[lane];
            const float4 m = s.misc[lane];
            const double rx = len * m.y, ry = len * m.z, rz = len * m.w;
            vir[0] += ex * rx; vir[1] += ex * ry; vir[2] += ex * rz;
            vir[3] += ey * rx; vir[4] += ey * ry; vir[5] += ey * rz;
            vir[6] += ez * rx; vir[7] += ez * ry; vir[8] += ez * rz;
            if (out.edge_forces != nullptr) {
                double* ef = out.edge_forces + 3 * static_cast<size_t>(chunk + lane);
                if (out.accumulate_edge) { ef[0] += ex; ef[1] += ey; ef[2] += ez; }
                else { ef[0] = ex; ef[1] = ey; ef[2] = ez; }
            }
        } else if (lane < count && out.edge_forces != nullptr && !out.accumulate_edge) {
            double* ef = out.edge_forces + 3 * static_cast<size_t>(chunk + lane);
            ef[0] = ef[1] = ef[2] = 0.0;
        }
    }
    // receiver total and virial: one reduction per receiver
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        rfx += __shfl_xor_sync(0xffffffffu, rfx, offset);
        rfy += __shfl_xor_sync(0xffffffffu, rfy, offset);
        rfz += __shfl_xor_sync(0xffffffffu, rfz, offset);
#pragma unroll
        for (int q = 0; q < 9; ++q) vir[q] += __shfl_xor_sync(0xffffffffu, vir[q], offset);
    }
    if (lane == 0 && out.atom_forces != nullptr) {
        atomicAdd(out.atom_forces + 3 * static_cast<size_t>(i), rfx);
        atomicAdd(out.atom_forces + 3 * static_cast<size_t>(i) + 1, rfy);
        atomicAdd(out.atom_forces + 3 * static_cast<size_t>(i) + 2, rfz);
        const int slot = i % kVirialSlots;
#pragma unroll
        for (int q = 0; q < 9; ++q) atomicAdd(out.virial_slots + slot * 9 + q, vir[q]);
    }
}

}  // namespace sxb
