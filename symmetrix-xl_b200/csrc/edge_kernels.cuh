// Receiver-sorted, warp-cooperative edge kernels of the force path (sm_100a).
//
// One thread block owns one receiver atom and has one thread per channel.  For a
// chunk of the receiver's edges the block first computes the channel-independent
// edge state once (spline interval and offset, spherical harmonics and, for the
// reverse kernels, their Cartesian gradients) into shared memory; then every thread
// walks the chunk for its own channel, evaluating the radial splines from the
// coefficient table (coalesced over channels) and accumulating in registers.  Edge
// state is regenerated here from the 16-byte geometry record and never stored
// graph-wide; the receiver's sums need no atomics.
//
// Reference statements of the same math: layer 0 forward/reverse
// libsymmetrix/source/mace.cpp:1356-1403 and 1486-1559 (with the H0 / W_A0 folding of
// mace_kokkos_factorized_lifecycle.cpp:3988-4047); layer 1 forward/reverse
// mace.cpp:2023-2083 and 2199-2302; harmonics mace.cpp:1269-1299; spline evaluation
// cubic_spline_set.cpp:33-80; force and virial reduction
// mace_kokkos_evaluate.cpp:92-106 and 157-186.
#pragma once

#include "common.cuh"
#include "generated/structures.h"

namespace sxb {

constexpr int kEdgeChunk = 64;

// ---------------------------------------------------------------------------------------------
// Real spherical harmonics up to l = 3 of a unit direction, model convention: the vector is
// permuted to (z, x, y), orthonormal harmonics are scaled by 2 sqrt(pi).  Each Y_lm is a
// homogeneous polynomial P of degree l, so dY/dX = (grad P - l P u) / r (Euler's theorem).
template <bool kGradient>
__device__ __forceinline__ void harmonics16(float dx, float dy, float dz, float inv_r, float* __restrict__ Y,
                                            float* __restrict__ gX, float* __restrict__ gY, float* __restrict__ gZ)
{
    // permuted frame and a second normalisation, as the reference's device path does
    const float n = rsqrtf(dx * dx + dy * dy + dz * dz);
    const float x = dz * n, y = dx * n, z = dy * n;
    const float x2 = x * x, y2 = y * y, z2 = z * z;
    // constants already multiplied by 2 sqrt(pi)
    constexpr float c1 = 1.7320508075688772f;     // sqrt(3)
    constexpr float a2 = 3.8729833462074170f;     // sqrt(15)
    constexpr float b2 = 1.1180339887498949f;     // sqrt(5)/2
    constexpr float h2 = 1.9364916731037085f;     // sqrt(15)/2
    constexpr float c3 = 2.0916500663351889f;     // sqrt(35/8)
    constexpr float d3 = 10.246950765959598f;     // sqrt(105)
    constexpr float e3 = 1.6201851746019651f;     // sqrt(21/8)
    constexpr float f3 = 1.3228756555322954f;     // sqrt(7)/2
    constexpr float k3 = 5.1234753829797990f;     // sqrt(105)/2
    const float q = 4.0f * z2 - x2 - y2;
    float P[16];
    P[0] = 1.0f;
    P[1] = c1 * y; P[2] = c1 * z; P[3] = c1 * x;
    P[4] = a2 * x * y; P[5] = a2 * y * z; P[6] = b2 * (2.0f * z2 - x2 - y2); P[7] = a2 * x * z; P[8] = h2 * (x2 - y2);
    P[9] = c3 * y * (3.0f * x2 - y2); P[10] = d3 * x * y * z; P[11] = e3 * y * q;
    P[12] = f3 * z * (2.0f * z2 - 3.0f * x2 - 3.0f * y2); P[13] = e3 * x * q; P[14] = k3 * z * (x2 - y2);
    P[15] = c3 * x * (x2 - 3.0f * y2);
#pragma unroll
    for (int i = 0; i < 16; ++i) Y[i] = P[i];
    if constexpr (kGradient) {
        float gx[16], gy[16], gz[16];   // polynomial gradients in the permuted frame
        gx[0] = gy[0] = gz[0] = 0.0f;
        gx[1] = 0.0f; gy[1] = c1; gz[1] = 0.0f;
        gx[2] = 0.0f; gy[2] = 0.0f; gz[2] = c1;
        gx[3] = c1; gy[3] = 0.0f; gz[3] = 0.0f;
        gx[4] = a2 * y; gy[4] = a2 * x; gz[4] = 0.0f;
        gx[5] = 0.0f; gy[5] = a2 * z; gz[5] = a2 * y;
        gx[6] = -2.0f * b2 * x; gy[6] = -2.0f * b2 * y; gz[6] = 4.0f * b2 * z;
        gx[7] = a2 * z; gy[7] = 0.0f; gz[7] = a2 * x;
        gx[8] = 2.0f * h2 * x; gy[8] = -2.0f * h2 * y; gz[8] = 0.0f;
        gx[9] = 6.0f * c3 * x * y; gy[9] = 3.0f * c3 * (x2 - y2); gz[9] = 0.0f;
        gx[10] = d3 * y * z; gy[10] = d3 * x * z; gz[10] = d3 * x * y;
        gx[11] = -2.0f * e3 * x * y; gy[11] = e3 * (q - 2.0f * y2); gz[11] = 8.0f * e3 * y * z;
        gx[12] = -6.0f * f3 * x * z; gy[12] = -6.0f * f3 * y * z; gz[12] = f3 * (6.0f * z2 - 3.0f * x2 - 3.0f * y2);
        gx[13] = e3 * (q - 2.0f * x2); gy[13] = -2.0f * e3 * x * y; gz[13] = 8.0f * e3 * x * z;
        gx[14] = 2.0f * k3 * x * z; gy[14] = -2.0f * k3 * y * z; gz[14] = k3 * (x2 - y2);
        gx[15] = 3.0f * c3 * (x2 - y2); gy[15] = -6.0f * c3 * x * y; gz[15] = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float l = i < 1 ? 0.0f : (i < 4 ? 1.0f : (i < 9 ? 2.0f : 3.0f));
            const float radial = l * P[i];
            // back to the original frame: X is the permuted y, Y the permuted z, Z the permuted x
            gX[i] = (gy[i] - y * radial) * inv_r;
            gY[i] = (gz[i] - z * radial) * inv_r;
            gZ[i] = (gx[i] - x * radial) * inv_r;
        }
    }
}

// Spline evaluation point in float, as the reference forms it (cubic_spline_set.cpp:33-47).
__device__ __forceinline__ void spline_point(const SplineGrid& g, float r, int& interval, float& x)
{
    interval = static_cast<int>(floorf((r - g.x0) / g.h));
    x = r - g.x0 - g.h * static_cast<float>(interval);
    if (interval < 0) {
        interval = 0;
        x = 0.0f;
    } else if (interval >= g.intervals) {
        interval = g.intervals - 1;
        x = g.h;
    }
}

// ---------------------------------------------------------------------------------------------
// Per-step geometry: xyz_ij = r_j - r_i + shift * cell in double, then the float record.
// One warp per receiver, lanes over its edges.
static __global__ void geometry_from_positions_kernel(int num_nodes, const int* __restrict__ first,
                                               const int* __restrict__ sources, const int* __restrict__ shifts,
                                               const double* __restrict__ positions, const int* __restrict__ original,
                                               const double* __restrict__ cell, EdgeGeom* __restrict__ geom,
                                               int* __restrict__ error_flag)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= num_nodes) return;
    const int oi = original[warp];
    const double xi = positions[3 * oi], yi = positions[3 * oi + 1], zi = positions[3 * oi + 2];
    const int begin = first[warp], end = first[warp + 1];
    for (int e = begin + lane; e < end; e += 32) {
        const int oj = original[sources[e]];
        double dx = positions[3 * oj] - xi, dy = positions[3 * oj + 1] - yi, dz = positions[3 * oj + 2] - zi;
        if (shifts != nullptr) {   // graphs without periodic shifts (explicit ghost atoms, open systems): plain differences
            const size_t se = 3 * static_cast<size_t>(e);
            const double sx = shifts[se], sy = shifts[se + 1], sz = shifts[se + 2];
            dx += sx * cell[0] + sy * cell[3] + sz * cell[6];
            dy += sx * cell[1] + sy * cell[4] + sz * cell[7];
            dz += sx * cell[2] + sy * cell[5] + sz * cell[8];
        }
        const double r = sqrt(dx * dx + dy * dy + dz * dz);
        if (!(r > 0.0) || !isfinite(r)) atomicOr(error_flag, 1);
        EdgeGeom g;
        g.ux = static_cast<float>(dx / r);
        g.uy = static_cast<float>(dy / r);
        g.uz = static_cast<float>(dz / r);
        g.r = static_cast<float>(r);
        geom[e] = g;
    }
}

// Per-step geometry from a reference state (graphs built by the caller without integer shifts):
//   Cartesian  (kFractional = false): xyz_ij = ref_xyz_ij + d_j - d_i,  d = position - reference position
//   fractional (kFractional = true):  xyz_ij = (ref_fxyz_ij + f_j - f_i) . cell,  f = position . cell^-1 - reference
// where d / f are reduced to the nearest image along the periodic axes, so an atom that crossed the cell
// boundary since the reference keeps its edges (reference: update_prepared_factorized_positions_geometry,
// libsymmetrix/source/mace_kokkos_factorized_lifecycle.cpp:2915-3076).  One warp per receiver.
template <bool kFractional>
__global__ void geometry_from_reference_kernel(int num_nodes, const int* __restrict__ first, const int* __restrict__ sources,
                                               const double* __restrict__ positions, const int* __restrict__ original,
                                               const double* __restrict__ reference, const double* __restrict__ reference_xyz,
                                               const int* __restrict__ edge_map, const double* __restrict__ cell,
                                               const double* __restrict__ inv_cell, int pbc_mask, EdgeGeom* __restrict__ geom,
                                               int* __restrict__ error_flag)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= num_nodes) return;
    // displacement of a node from its reference, in fractional coordinates reduced to the nearest image
    auto displacement = [&](int caller_node, double* f) {
        const double px = positions[3 * caller_node], py = positions[3 * caller_node + 1], pz = positions[3 * caller_node + 2];
        double q[3];
        if (kFractional) {
            for (int a = 0; a < 3; ++a) q[a] = px * inv_cell[a] + py * inv_cell[3 + a] + pz * inv_cell[6 + a] - reference[3 * caller_node + a];
        } else {
            const double dx = px - reference[3 * caller_node], dy = py - reference[3 * caller_node + 1], dz = pz - reference[3 * caller_node + 2];
            for (int a = 0; a < 3; ++a) q[a] = dx * inv_cell[a] + dy * inv_cell[3 + a] + dz * inv_cell[6 + a];
        }
        for (int a = 0; a < 3; ++a) f[a] = ((pbc_mask >> a) & 1) ? q[a] - rint(q[a]) : q[a];
    };
    double fi[3];
    displacement(original[warp], fi);
    const int begin = first[warp], end = first[warp + 1];
    for (int e = begin + lane; e < end; e += 32) {
        double fj[3];
        displacement(original[sources[e]], fj);
        const size_t o = 3 * static_cast<size_t>(edge_map[e]);
        double dx, dy, dz;
        if (kFractional) {
            const double gx = reference_xyz[o] + fj[0] - fi[0], gy = reference_xyz[o + 1] + fj[1] - fi[1],
                         gz = reference_xyz[o + 2] + fj[2] - fi[2];
            dx = gx * cell[0] + gy * cell[3] + gz * cell[6];
            dy = gx * cell[1] + gy * cell[4] + gz * cell[7];
            dz = gx * cell[2] + gy * cell[5] + gz * cell[8];
        } else {
            const double gx = fj[0] - fi[0], gy = fj[1] - fi[1], gz = fj[2] - fi[2];
            dx = reference_xyz[o] + gx * cell[0] + gy * cell[3] + gz * cell[6];
            dy = reference_xyz[o + 1] + gx * cell[1] + gy * cell[4] + gz * cell[7];
            dz = reference_xyz[o + 2] + gx * cell[2] + gy * cell[5] + gz * cell[8];
        }
        const double r = sqrt(dx * dx + dy * dy + dz * dz);
        if (!(r > 0.0) || !isfinite(r)) atomicOr(error_flag, 1);
        EdgeGeom g;
        g.ux = static_cast<float>(dx / r);
        g.uy = static_cast<float>(dy / r);
        g.uz = static_cast<float>(dz / r);
        g.r = static_cast<float>(r);
        geom[e] = g;
    }
}

// Geometry from caller-supplied edge vectors (original edge order == internal edge order of
// each receiver; ``edge_map`` gives the caller's edge index of every internal edge).
static __global__ void geometry_from_vectors_kernel(long num_edges, const double* __restrict__ xyz,
                                             const int* __restrict__ edge_map, EdgeGeom* __restrict__ geom,
                                             int* __restrict__ error_flag)
{
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= num_edges) return;
    const long o = edge_map[e];
    const double dx = xyz[3 * o], dy = xyz[3 * o + 1], dz = xyz[3 * o + 2];
    const double r = sqrt(dx * dx + dy * dy + dz * dz);
    if (!(r > 0.0) || !isfinite(r)) atomicOr(error_flag, 1);
    EdgeGeom g;
    g.ux = static_cast<float>(dx / r);
    g.uy = static_cast<float>(dy / r);
    g.uz = static_cast<float>(dz / r);
    g.r = static_cast<float>(r);
    geom[e] = g;
}

// ---------------------------------------------------------------------------------------------
// Shared-memory edge state of one chunk; every row is 16-byte aligned so that a thread reads
// it with 128-bit shared loads (all threads read the same address: a broadcast).
template <bool kGradient>
struct alignas(16) ChunkState {
    float4 y[kEdgeChunk][4];
    float4 gx[kGradient ? kEdgeChunk : 1][4];
    float4 gy[kGradient ? kEdgeChunk : 1][4];
    float4 gz[kGradient ? kEdgeChunk : 1][4];
    float4 misc[kEdgeChunk];      // x = offset inside the spline interval, yzw = unit direction
    int2 index[kEdgeChunk];       // x = first coefficient of (pair, interval) or -1 (inactive), y = source
    float len[kGradient ? kEdgeChunk : 1];
    float dens[kGradient ? kEdgeChunk : 1];   // d/dr of the density spline at the edge (0 without density scaling)
};

// Optional per-receiver density scaling of a layer's A tensor, A_i /= 1 + sum_j s(r_ij)
// (reference: libsymmetrix/source/mace.cpp:1562-1584 and 2381-2403; gradient 1587-1636, 2406-2458).
struct DensityScale {
    const float* table;       // cubic coefficients [interval][4] of s, nullptr when the model has none
    const float* inv_scale;   // [receiver] 1 / (1 + sum_j s(r_ij))
    const float* dot;         // [receiver] sum over (lm, k) of A_adj * A, both taken for the scaled A
    int types;                // active types the table distinguishes: table [type_i * types + type_j][interval][4]
};

// Derivative of a scalar spline stored [interval][4].
__device__ __forceinline__ float scalar_spline_derivative(const float* __restrict__ table, int interval, float x)
{
    const float4 c = reinterpret_cast<const float4*>(table)[interval];
    return fmaf(3.0f * c.w, x * x, fmaf(2.0f * c.z, x, c.y));
}
__device__ __forceinline__ float scalar_spline_value(const float* __restrict__ table, int interval, float x)
{
    const float4 c = reinterpret_cast<const float4*>(table)[interval];
    return fmaf(c.w, x * x * x, fmaf(c.z, x * x, fmaf(c.y, x, c.x)));
}

// inv_scale[i] = 1 / (1 + sum_j s(r_ij)) for the layer-0 and the layer-1 density spline (either table
// may be nullptr).  One warp per receiver; edge values in float as every radial function, summed in
// double.  Reference: libsymmetrix/source/mace.cpp:1562-1584 (layer 0), 2381-2403 (layer 1).
static __global__ void density_scale_kernel(int num_receivers, const int* __restrict__ first, const int* __restrict__ sources,
                                     const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype, int num_active,
                                     SplineGrid grid, const float* __restrict__ table0, const float* __restrict__ table1,
                                     float* __restrict__ inv_scale0, float* __restrict__ inv_scale1)
{
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (i >= num_receivers) return;
    const int type_i = atype[i];
    double rho0 = 0.0, rho1 = 0.0;
    for (int e = first[i] + lane; e < first[i + 1]; e += 32) {
        const float r = geom[e].r;
        if (!(r < grid.r_cut)) continue;
        int interval;
        float x;
        spline_point(grid, r, interval, x);
        const int row = (type_i * num_active + atype[sources[e]]) * grid.intervals + interval;   // table of the ordered pair
        if (table0 != nullptr) rho0 += scalar_spline_value(table0, row, x);
        if (table1 != nullptr) rho1 += scalar_spline_value(table1, row, x);
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        rho0 += __shfl_xor_sync(0xffffffffu, rho0, offset);
        rho1 += __shfl_xor_sync(0xffffffffu, rho1, offset);
    }
    if (lane == 0) {
        if (table0 != nullptr) inv_scale0[i] = static_cast<float>(1.0 / (1.0 + rho0));
        if (table1 != nullptr) inv_scale1[i] = static_cast<float>(1.0 / (1.0 + rho1));
    }
}

// Fills the chunk state for edges [begin, begin+count) of one receiver.
template <bool kGradient, bool kOrderedPairs, bool kGivenHarmonics = false>
__device__ __forceinline__ void fill_chunk(ChunkState<kGradient>& s, int begin, int count, const int* __restrict__ sources,
                                           const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype,
                                           int type_i, int num_active, const SplineGrid& grid, int functions,
                                           const float* __restrict__ density_table = nullptr, int density_types = 1,
                                           const float* __restrict__ given_harmonics = nullptr)
{
    for (int t = threadIdx.x; t < count; t += blockDim.x) {
        const int e = begin + t;
        const EdgeGeom g = geom[e];
        const int j = sources[e];
        if (!(g.r < grid.r_cut)) {
            s.index[t] = make_int2(-1, j);
            continue;
        }
        int interval;
        float x;
        spline_point(grid, g.r, interval, x);
        // layer 0: ordered pair (H0 of the source and W_A0 of the receiver are folded into the table);
        // layer 1: unordered pair, and a single table when the model has no distance transform (num_active == 1)
        int pair = 0, type_j = 0;
        if (kOrderedPairs || num_active > 1) type_j = atype[j];
        if constexpr (kOrderedPairs) {
            pair = type_i * num_active + type_j;
        } else if (num_active > 1) {
            const int a = min(type_i, type_j), b = max(type_i, type_j);
            pair = a * (2 * num_active - a - 1) / 2 + b;
        }
        s.index[t] = make_int2((pair * grid.intervals + interval) * 4 * functions, j);
        s.misc[t] = make_float4(x, g.ux, g.uy, g.uz);
        const float inv_r = 1.0f / g.r;
        if constexpr (kGradient) {
            harmonics16<true>(g.ux, g.uy, g.uz, inv_r, reinterpret_cast<float*>(s.y[t]), reinterpret_cast<float*>(s.gx[t]),
                              reinterpret_cast<float*>(s.gy[t]), reinterpret_cast<float*>(s.gz[t]));
            s.len[t] = g.r;
            // density tables are stored per ordered pair of the density_types active types
            s.dens[t] = density_table != nullptr
                            ? scalar_spline_derivative(density_table, (type_i * density_types + (density_types > 1 ? atype[j] : 0)) * grid.intervals + interval, x)
                            : 0.0f;
        } else if (kGivenHarmonics) {
            // the caller supplies Y_lm per edge [E][16] (the kernel-plugin interface passes them instead of directions)
            const float4* row = reinterpret_cast<const float4*>(given_harmonics + 16 * static_cast<size_t>(e));
            s.y[t][0] = row[0]; s.y[t][1] = row[1]; s.y[t][2] = row[2]; s.y[t][3] = row[3];
        } else {
            harmonics16<false>(g.ux, g.uy, g.uz, inv_r, reinterpret_cast<float*>(s.y[t]), nullptr, nullptr, nullptr);
        }
    }
}

__device__ __forceinline__ void load16(const float4* __restrict__ row, float* __restrict__ out)
{
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 v = row[q];
        out[4 * q] = v.x; out[4 * q + 1] = v.y; out[4 * q + 2] = v.z; out[4 * q + 3] = v.w;
    }
}

// value c0 + c1 x + c2 x^2 + c3 x^3 and derivative c1 + 2 c2 x + 3 c3 x^2 with shared powers
// (x2 = 2x and xx3 = 3x^2 are formed once per edge)
__device__ __forceinline__ float cubic(float c0, float c1, float c2, float c3, float x, float xx, float xxx)
{
    return fmaf(c3, xxx, fmaf(c2, xx, fmaf(c1, x, c0)));
}
__device__ __forceinline__ float cubic_derivative(float c1, float c2, float c3, float x2, float xx3)
{
    return fmaf(c3, xx3, fmaf(c2, x2, c1));
}

// ---------------------------------------------------------------------------------------------
// Layer 0 forward: A0_i[lm,k] = sum_j S0[pair(i,j), r_ij][l,k] * Y_ij[lm].
// kC > 0 fixes the channel count at compile time (all strides become immediates).
template <int kC>
__global__ void __launch_bounds__(kC > 0 ? kC : 256)
l0_forward_kernel(int num_nodes, int node0, int C_runtime, const int* __restrict__ first, const int* __restrict__ sources,
                  const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype, int num_active,
                  SplineGrid grid, const float* __restrict__ table, float* __restrict__ A0,
                  const float* __restrict__ inv_scale)
{
    __shared__ ChunkState<false> s;
    const int C = kC > 0 ? kC : C_runtime;
    const int local = blockIdx.x, i = node0 + local;   // tile-local and graph-wide receiver index
    const int k = threadIdx.x;
    const int F = 4 * C;
    const int type_i = atype[i];
    const int begin = first[i], end = first[i + 1];
    float acc[16];
#pragma unroll
    for (int lm = 0; lm < 16; ++lm) acc[lm] = 0.0f;
    for (int chunk = begin; chunk < end; chunk += kEdgeChunk) {
        const int count = min(kEdgeChunk, end - chunk);
        __syncthreads();
        fill_chunk<false, true>(s, chunk, count, sources, geom, atype, type_i, num_active, grid, F);
        __syncthreads();
        for (int t = 0; t < count; ++t) {
            const int base = s.index[t].x;
            if (base < 0) continue;
            const float x = s.misc[t].x, xx = x * x, xxx = xx * x;
            const float* c = table + base + k;
            float R[4];
#pragma unroll
            for (int l = 0; l < 4; ++l)
                R[l] = cubic(c[l * C], c[F + l * C], c[2 * F + l * C], c[3 * F + l * C], x, xx, xxx);
            float y[16];
            load16(s.y[t], y);
            acc[0] = fmaf(R[0], y[0], acc[0]);
#pragma unroll
            for (int lm = 1; lm < 4; ++lm) acc[lm] = fmaf(R[1], y[lm], acc[lm]);
#pragma unroll
            for (int lm = 4; lm < 9; ++lm) acc[lm] = fmaf(R[2], y[lm], acc[lm]);
#pragma unroll
            for (int lm = 9; lm < 16; ++lm) acc[lm] = fmaf(R[3], y[lm], acc[lm]);
        }
    }
    const float scale = inv_scale != nullptr ? inv_scale[i] : 1.0f;   // density scaling, mace.cpp:1562-1584
    float* out = A0 + static_cast<size_t>(local) * 16 * C + k;
#pragma unroll
    for (int lm = 0; lm < 16; ++lm) out[lm * C] = acc[lm] * scale;
}

// Block-level force bookkeeping shared by the two reverse kernels.  Each warp leaves its
// channel-partial edge force in ``partial``; after the chunk one thread per edge sums the warps,
// pushes +f to the source atom, adds -f to the receiver total and f (x) xyz to the virial.
struct ForceOutputs {
    double* atom_forces;     // [N][3], internal node order; nullptr in the reproducible mode (see below)
    double* virial_slots;    // [kVirialSlots][9]
    double* edge_forces;     // optional [E][3] directed forces dE/d(xyz_ij), may be nullptr
    int accumulate_edge;     // 0: overwrite edge_forces, 1: add, 2: add atomically (several kernels share an edge)
    // Reproducible mode: nothing is accumulated atomically.  The kernels leave the directed force of
    // every edge in edge_forces and the source adjoint of every edge in edge_source_adjoint
    // [E][num_hidden][C]; fixed-order passes over the source schedule (deterministic_kernels.cuh) sum them.
    float* edge_source_adjoint;
};

__device__ __forceinline__ void warp_reduce3(float& a, float& b, float& c)
{
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, offset);
        b += __shfl_xor_sync(0xffffffffu, b, offset);
        c += __shfl_xor_sync(0xffffffffu, c, offset);
    }
}

// Sums three values over the warp with 6 shuffles: the exchange at distance 16 halves the data
// (each half-warp keeps two of the four slots), the one at distance 8 halves it again, three more
// finish the sum.  On return lanes 0, 8 and 16 hold the totals of a, b and c respectively.
__device__ __forceinline__ float warp_reduce3_transposed(float a, float b, float c, int lane)
{
    const bool upper = lane & 16;
    // lower half keeps (a, b) and receives the partner's (a, b); upper half keeps (c, 0)
    const float send0 = upper ? a : c, send1 = upper ? b : 0.0f;
    const float recv0 = __shfl_xor_sync(0xffffffffu, send0, 16);
    const float recv1 = __shfl_xor_sync(0xffffffffu, send1, 16);
    float k0 = (upper ? c : a) + recv0;      // lower: a total of pair, upper: c total of pair
    float k1 = (upper ? 0.0f : b) + recv1;   // lower: b, upper: 0
    const bool second = lane & 8;
    const float send = second ? k0 : k1;
    const float recv = __shfl_xor_sync(0xffffffffu, send, 8);
    float v = (second ? k1 : k0) + recv;     // lanes 0-7: a, 8-15: b, 16-23: c, 24-31: 0
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v;
}

template <int kMaxWarps>
struct ForceScratch {
    float partial[kEdgeChunk][kMaxWarps][3];
    double receiver[3];
    double virial[9];
};

// kRecords = true: the caller knows at compile time that atom_forces is null (layer-1 gradient in the
// reproducible / plugin mode); false keeps the run-time test, which the other callers rely on.
template <int kMaxWarps, bool kRecords = false>
__device__ __forceinline__ void flush_chunk_forces(ForceScratch<kMaxWarps>& fs, const ChunkState<true>& s, int chunk_begin,
                                                   int count, int num_warps, const ForceOutputs& out,
                                                   float density_coef = 0.0f)
{
    // called by all threads after a __syncthreads(); threads t < count own one edge each
    double fx = 0.0, fy = 0.0, fz = 0.0;
    double v[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (int t = threadIdx.x; t < count; t += blockDim.x) {
        if (s.index[t].x < 0) {
            if (out.edge_forces != nullptr && !out.accumulate_edge) {
                double* ef = out.edge_forces + 3 * static_cast<size_t>(chunk_begin + t);
                ef[0] = ef[1] = ef[2] = 0.0;
            }
            continue;
        }
        float px = 0.0f, py = 0.0f, pz = 0.0f;
        for (int w = 0; w < num_warps; ++w) {
            px += fs.partial[t][w][0];
            py += fs.partial[t][w][1];
            pz += fs.partial[t][w][2];
        }
        {   // density scaling: dE/d(xyz_ij) += (A_adj . A) / (1 + rho_i) * s'(r) * rhat
            const float4 u = s.misc[t];
            const float d = density_coef * s.dens[t];
            px -= d * u.y; py -= d * u.z; pz -= d * u.w;
        }
        // directed force dE/d(xyz_ij) with the reference's sign: force -= adjoint * (...)
        const double ex = -static_cast<double>(px), ey = -static_cast<double>(py), ez = -static_cast<double>(pz);
        const int j = s.index[t].y;
        if (!kRecords && out.atom_forces != nullptr) {
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j), ex);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j) + 1, ey);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j) + 2, ez);
        }
        fx -= ex; fy -= ey; fz -= ez;
        const double len = s.len[t];
        const float4 m = s.misc[t];
        const double rx = len * m.y, ry = len * m.z, rz = len * m.w;
        v[0] += ex * rx; v[1] += ex * ry; v[2] += ex * rz;
        v[3] += ey * rx; v[4] += ey * ry; v[5] += ey * rz;
        v[6] += ez * rx; v[7] += ez * ry; v[8] += ez * rz;
        if (out.edge_forces != nullptr) {
            double* ef = out.edge_forces + 3 * static_cast<size_t>(chunk_begin + t);
            if (out.accumulate_edge == 2) { atomicAdd(ef, ex); atomicAdd(ef + 1, ey); atomicAdd(ef + 2, ez); }
            else if (out.accumulate_edge) { ef[0] += ex; ef[1] += ey; ef[2] += ez; }
            else { ef[0] = ex; ef[1] = ey; ef[2] = ez; }
        }
    }
    // only the first two warps can hold non-zero sums (count <= 64)
    if (threadIdx.x < kEdgeChunk) {
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            fx += __shfl_xor_sync(0xffffffffu, fx, offset);
            fy += __shfl_xor_sync(0xffffffffu, fy, offset);
            fz += __shfl_xor_sync(0xffffffffu, fz, offset);
#pragma unroll
            for (int q = 0; q < 9; ++q) v[q] += __shfl_xor_sync(0xffffffffu, v[q], offset);
        }
        if ((threadIdx.x & 31) == 0) {
            atomicAdd(&fs.receiver[0], fx);
            atomicAdd(&fs.receiver[1], fy);
            atomicAdd(&fs.receiver[2], fz);
#pragma unroll
            for (int q = 0; q < 9; ++q) atomicAdd(&fs.virial[q], v[q]);
        }
    }
}

template <int kMaxWarps, bool kRecords = false>
__device__ __forceinline__ void finish_receiver_forces(ForceScratch<kMaxWarps>& fs, int receiver, const ForceOutputs& out)
{
    __syncthreads();
    if (kRecords || out.atom_forces == nullptr) return;      // reproducible mode: forces and virial come from the per-edge records
    if (threadIdx.x < 3) atomicAdd(out.atom_forces + 3 * static_cast<size_t>(receiver) + threadIdx.x, fs.receiver[threadIdx.x]);
    if (threadIdx.x < 9) {
        const int slot = receiver % kVirialSlots;
        atomicAdd(out.virial_slots + slot * 9 + threadIdx.x, fs.virial[threadIdx.x]);
    }
}

// ---------------------------------------------------------------------------------------------
// Screened-Coulomb (ZBL) pair repulsion with a polynomial envelope, one half of the pair energy per
// directed edge: E_i += 0.5 env(r) V(r), force on the edge -dE/d(xyz_ij) = -rhat dE/dr
// (reference: libsymmetrix/source/zbl.cpp:24-139, evaluated in the model precision).  One warp per
// receiver, one lane per edge; the per-pair constants are tabulated on the host per active pair.
struct ZblPair {
    float inv_a;     // 1 / a,  a = a_prefactor * 0.529 / (Z_i^a_exp + Z_j^a_exp)
    float zz;        // 14.3996 * Z_i * Z_j
    float r_max;     // sum of the two covalent radii
    float pad;
};
struct ZblParams {
    const ZblPair* pairs;    // [active_i * num_active + active_j]
    float c[4];
    int p;
};

static __global__ void zbl_kernel(int num_receivers, const int* __restrict__ first, const int* __restrict__ sources,
                           const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype, int num_active,
                           ZblParams z, double* __restrict__ node_energies, double* __restrict__ energy_slots, ForceOutputs out)
{
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (i >= num_receivers) return;
    const int type_i = atype[i];
    double energy = 0.0, rfx = 0.0, rfy = 0.0, rfz = 0.0;
    double vir[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    for (int e = first[i] + lane; e < first[i + 1]; e += 32) {
        const EdgeGeom g = geom[e];
        const int j = sources[e];
        const ZblPair P = z.pairs[type_i * num_active + atype[j]];
        if (!(g.r < P.r_max)) continue;
        const float r = g.r, x = r * P.inv_a;
        const float e0 = z.c[0] * expf(-3.2f * x), e1 = z.c[1] * expf(-0.9423f * x);
        const float e2 = z.c[2] * expf(-0.4028f * x), e3 = z.c[3] * expf(-0.2016f * x);
        const float phi = e0 + e1 + e2 + e3;
        const float dphi = (-3.2f * e0 - 0.9423f * e1 - 0.4028f * e2 - 0.2016f * e3) * P.inv_a;
        const float v = P.zz / r * phi;
        const float dv = P.zz * (r * dphi - phi) / (r * r);
        const float u = r / P.r_max;
        float up = 1.0f;                                  // u^(p-1)
        for (int q = 1; q < z.p; ++q) up *= u;
        const float p = static_cast<float>(z.p);
        const float upp = up * u, uppp = upp * u, upppp = uppp * u;   // u^p, u^(p+1), u^(p+2)
        const float env = 1.0f - ((p + 1.0f) * (p + 2.0f) * 0.5f) * upp + p * (p + 2.0f) * uppp - (p * (p + 1.0f) * 0.5f) * upppp;
        const float denv = (-((p + 1.0f) * (p + 2.0f) * 0.5f) * p * up + p * (p + 2.0f) * (p + 1.0f) * upp -
                            (p * (p + 1.0f) * 0.5f) * (p + 2.0f) * uppp) / P.r_max;
        energy += static_cast<double>(0.5f * v * env);
        const float dEdr = 0.5f * (v * denv + dv * env);
        const double ex = -static_cast<double>(g.ux * dEdr), ey = -static_cast<double>(g.uy * dEdr), ez = -static_cast<double>(g.uz * dEdr);
        if (out.atom_forces != nullptr) {
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j), ex);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j) + 1, ey);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(j) + 2, ez);
        }
        rfx -= ex; rfy -= ey; rfz -= ez;
        const double rx = static_cast<double>(r) * g.ux, ry = static_cast<double>(r) * g.uy, rz = static_cast<double>(r) * g.uz;
        vir[0] += ex * rx; vir[1] += ex * ry; vir[2] += ex * rz;
        vir[3] += ey * rx; vir[4] += ey * ry; vir[5] += ey * rz;
        vir[6] += ez * rx; vir[7] += ez * ry; vir[8] += ez * rz;
        if (out.edge_forces != nullptr) {
            double* ef = out.edge_forces + 3 * static_cast<size_t>(e);
            ef[0] += ex; ef[1] += ey; ef[2] += ez;
        }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        energy += __shfl_xor_sync(0xffffffffu, energy, offset);
        rfx += __shfl_xor_sync(0xffffffffu, rfx, offset);
        rfy += __shfl_xor_sync(0xffffffffu, rfy, offset);
        rfz += __shfl_xor_sync(0xffffffffu, rfz, offset);
#pragma unroll
        for (int q = 0; q < 9; ++q) vir[q] += __shfl_xor_sync(0xffffffffu, vir[q], offset);
    }
    if (lane == 0) {
        node_energies[i] += energy;
        if (out.atom_forces != nullptr) {
            atomicAdd(energy_slots + (i % kVirialSlots), energy);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(i), rfx);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(i) + 1, rfy);
            atomicAdd(out.atom_forces + 3 * static_cast<size_t>(i) + 2, rfz);
            const int slot = i % kVirialSlots;
#pragma unroll
            for (int q = 0; q < 9; ++q) atomicAdd(out.virial_slots + slot * 9 + q, vir[q]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Layer 0 reverse: f_ij -= sum_{lm,k} A0_adj_i[lm,k] * (rhat S0' Y + S0 grad Y).
template <int kC>
__global__ void __launch_bounds__(kC > 0 ? kC : 256)
l0_reverse_kernel(int num_nodes, int node0, int C_runtime, const int* __restrict__ first, const int* __restrict__ sources,
                  const EdgeGeom* __restrict__ geom, const unsigned char* __restrict__ atype, int num_active,
                  SplineGrid grid, const float* __restrict__ table, const float* __restrict__ A0_adj, ForceOutputs out,
                  DensityScale density)
{
    __shared__ ChunkState<true> s;
    __shared__ ForceScratch<8> fs;
    const int C = kC > 0 ? kC : C_runtime;
    const int local = blockIdx.x, i = node0 + local;   // tile-local and graph-wide receiver index
    const int k = threadIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, num_warps = blockDim.x >> 5;
    const int F = 4 * C;
    const int type_i = atype[i];
    const int begin = first[i], end = first[i + 1];
    if (threadIdx.x < 3) fs.receiver[threadIdx.x] = 0.0;
    if (threadIdx.x < 9) fs.virial[threadIdx.x] = 0.0;
    // with density scaling the stored adjoint refers to the scaled A0: dE/dA0_unscaled = adj / (1 + rho_i)
    const float scale = density.table != nullptr ? density.inv_scale[i] : 1.0f;
    const float density_coef = density.table != nullptr ? density.dot[i] * scale : 0.0f;
    float adj[16];
    const float* in = A0_adj + static_cast<size_t>(local) * 16 * C + k;
#pragma unroll
    for (int lm = 0; lm < 16; ++lm) adj[lm] = in[lm * C] * scale;
    for (int chunk = begin; chunk < end; chunk += kEdgeChunk) {
        const int count = min(kEdgeChunk, end - chunk);
        __syncthreads();
        fill_chunk<true, true>(s, chunk, count, sources, geom, atype, type_i, num_active, grid, F, density.table, density.types);
        __syncthreads();
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
                const float c0 = c[l * C], c1 = c[F + l * C], c2 = c[2 * F + l * C], c3 = c[3 * F + l * C];
                const float R = cubic(c0, c1, c2, c3, x, xx, xxx);
                const float dR = cubic_derivative(c1, c2, c3, x2, xx3);
                float ya = 0.0f;
#pragma unroll
                for (int lm = l * l; lm < (l + 1) * (l + 1); ++lm) {
                    ya = fmaf(y[lm], adj[lm], ya);
                    ang[lm] = R * adj[lm];
                }
                radial = fmaf(dR, ya, radial);
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
            warp_reduce3(fx, fy, fz);
            if (lane == 0) {
                fs.partial[t][warp][0] = fx;
                fs.partial[t][warp][1] = fy;
                fs.partial[t][warp][2] = fz;
            }
        }
        __syncthreads();
        flush_chunk_forces<8>(fs, s, chunk, count, num_warps, out, density_coef);
    }
    finish_receiver_forces<8>(fs, i, out);
}

// ---------------------------------------------------------------------------------------------
// Layer 1 kernels, one instantiation per compiled coupling structure.  The coefficient table is
// laid out [interval][function][4] (function = path*C + channel): a thread fetches the cubic of one
// function with a single 128-bit load, a warp 512 contiguous bytes.
//   forward:  Phi1_i[lme,k] = sum_terms cg * sum_j R1_ij[path,k] Y_ij[lm1] H1_j[lm2,k]
//   reverse:  row adjoints from dPhi1_i, then per edge the force and the source adjoint
//             H1_adj_j[lm2,k] += sum R1 Y adj  (coalesced red.add into the source row)
#define SXB_TERM_FORWARD(term, row, lme) out_lme[lme] = fmaf(cgc.cg[term], acc[row], out_lme[lme]);
#define SXB_TERM_TRANSPOSE(term, row, lme) adj[row] = fmaf(cgc.cg[term], dphi[lme], adj[row]);

#define SXB_DEFINE_L1_KERNELS(NAME)                                                                                  \
    /* kGivenHarmonics: the caller passes Y_lm per edge [E][16] (the kernel-plugin interface) */                     \
    template <int kC, bool kGivenHarmonics = false>                                                                  \
    __global__ void __launch_bounds__(kC > 0 ? kC : 256)                                                             \
    l1_forward_kernel_##NAME(int num_nodes, int node0, int C_runtime, const int* __restrict__ first,                            \
                             const int* __restrict__ sources, const EdgeGeom* __restrict__ geom,                     \
                             const unsigned char* __restrict__ atype, SplineGrid grid,                               \
                             const float4* __restrict__ table4, const float* __restrict__ H1,                        \
                             const __grid_constant__ CouplingConstants cgc, float* __restrict__ Phi1,                \
                             const float* __restrict__ inv_scale, int pair_types,                                    \
                             const float* __restrict__ given_harmonics = nullptr)                                    \
    {                                                                                                                \
        constexpr int NP = SXB_##NAME##_NUM_PATHS, NR = SXB_##NAME##_NUM_ROWS, NH = SXB_##NAME##_NUM_HIDDEN;          \
        constexpr int NE = SXB_##NAME##_NUM_LME;                                                                     \
        __shared__ ChunkState<false> s;                                                                              \
        const int C = kC > 0 ? kC : C_runtime;                                                                       \
        const int local = blockIdx.x, i = node0 + local;                                                             \
        const int k = threadIdx.x;                                                                                   \
        const int F = NP * C;                                                                                        \
        const int begin = first[i], end = first[i + 1];                                                              \
        float acc[NR];                                                                                               \
        _Pragma("unroll") for (int r_ = 0; r_ < NR; ++r_) acc[r_] = 0.0f;                                            \
        for (int chunk = begin; chunk < end; chunk += kEdgeChunk) {                                                  \
            const int count = min(kEdgeChunk, end - chunk);                                                          \
            __syncthreads();                                                                                         \
            fill_chunk<false, false, kGivenHarmonics>(s, chunk, count, sources, geom, atype, atype[i], pair_types, grid, \
                                                      F, nullptr, 1, given_harmonics);                               \
            __syncthreads();                                                                                         \
            for (int t = 0; t < count; ++t) {                                                                        \
                const int2 id = s.index[t];                                                                          \
                if (id.x < 0) continue;                                                                              \
                const float x = s.misc[t].x, xx = x * x, xxx = xx * x;                                               \
                const float4* c4 = table4 + (id.x >> 2) + k;   /* the four coefficients of a function are adjacent */ \
                float R[NP];                                                                                         \
                _Pragma("unroll") for (int p = 0; p < NP; ++p) {                                                     \
                    const float4 c = c4[p * C];                                                                      \
                    R[p] = cubic(c.x, c.y, c.z, c.w, x, xx, xxx);                                                    \
                }                                                                                                    \
                const float* hsrc = H1 + static_cast<size_t>(id.y) * NH * C + k;                                     \
                float h[NH];                                                                                         \
                _Pragma("unroll") for (int q = 0; q < NH; ++q) h[q] = hsrc[q * C];                                   \
                float y[16];                                                                                         \
                load16(s.y[t], y);                                                                                   \
                SXB_##NAME##_L1_FORWARD_BODY                                                                         \
            }                                                                                                        \
        }                                                                                                            \
        float out_lme[NE];                                                                                           \
        _Pragma("unroll") for (int q = 0; q < NE; ++q) out_lme[q] = 0.0f;                                            \
        SXB_##NAME##_TERMS(SXB_TERM_FORWARD)                                                                         \
        /* density scaling of A1 = Phi1 W (mace.cpp:2381-2403) commutes with the linear: scale Phi1 */              \
        const float scale = inv_scale != nullptr ? inv_scale[i] : 1.0f;                                              \
        float* out = Phi1 + static_cast<size_t>(local) * NE * C + k;                                                 \
        _Pragma("unroll") for (int q = 0; q < NE; ++q) out[q * C] = out_lme[q] * scale;                              \
    }                                                                                                                \
                                                                                                                     \
    /* kMinBlocks caps the registers of the 128-channel build: 3 blocks per SM = at most 170 registers */           \
    /* kRecords: nothing is accumulated atomically; per-edge records are left for fixed-order passes */             \
    template <int kC, int kMinBlocks = 3, bool kRecords = false>                                                     \
    __global__ void __launch_bounds__(kC > 0 ? kC : 256, kC == 128 ? kMinBlocks : 1)                                 \
    l1_reverse_kernel_##NAME(int num_nodes, int node0, int C_runtime, const int* __restrict__ first,                            \
                             const int* __restrict__ sources, const EdgeGeom* __restrict__ geom,                     \
                             const unsigned char* __restrict__ atype, SplineGrid grid,                               \
                             const float4* __restrict__ table4, const float* __restrict__ H1,                        \
                             const float* __restrict__ dPhi1, const __grid_constant__ CouplingConstants cgc,         \
                             float* __restrict__ H1_adj, ForceOutputs out, DensityScale density, int pair_types)     \
    {                                                                                                                \
        constexpr int NP = SXB_##NAME##_NUM_PATHS, NR = SXB_##NAME##_NUM_ROWS, NH = SXB_##NAME##_NUM_HIDDEN;          \
        constexpr int NE = SXB_##NAME##_NUM_LME;                                                                     \
        __shared__ ChunkState<true> s;                                                                               \
        __shared__ ForceScratch<8> fs;                                                                               \
        const int C = kC > 0 ? kC : C_runtime;                                                                       \
        const int local = blockIdx.x, i = node0 + local;                                                             \
        const int k = threadIdx.x;                                                                                   \
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, num_warps = blockDim.x >> 5;                     \
        const int F = NP * C;                                                                                        \
        const int begin = first[i], end = first[i + 1];                                                              \
        if (threadIdx.x < 3) fs.receiver[threadIdx.x] = 0.0;                                                         \
        if (threadIdx.x < 9) fs.virial[threadIdx.x] = 0.0;                                                           \
        /* with density scaling dPhi1 holds the adjoint of the scaled Phi1: divide by 1 + rho_i once more */       \
        const float scale = density.table != nullptr ? density.inv_scale[i] : 1.0f;                                  \
        const float density_coef = density.table != nullptr ? density.dot[i] * scale : 0.0f;                         \
        float adj[NR];                                                                                               \
        {                                                                                                            \
            float dphi[NE];                                                                                          \
            const float* in = dPhi1 + static_cast<size_t>(local) * NE * C + k;                                       \
            _Pragma("unroll") for (int q = 0; q < NE; ++q) dphi[q] = in[q * C] * scale;                              \
            _Pragma("unroll") for (int r_ = 0; r_ < NR; ++r_) adj[r_] = 0.0f;                                        \
            SXB_##NAME##_TERMS(SXB_TERM_TRANSPOSE)                                                                   \
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
                float R[NP], dR[NP];                                                                                 \
                _Pragma("unroll") for (int p = 0; p < NP; ++p) {                                                     \
                    const float4 c = c4[p * C];                                                                      \
                    R[p] = cubic(c.x, c.y, c.z, c.w, x, xx, xxx);                                                    \
                    dR[p] = cubic_derivative(c.y, c.z, c.w, x2, xx3);                                                \
                }                                                                                                    \
                const size_t source_row = static_cast<size_t>(id.y) * NH * C + k;                                    \
                float h[NH], hadj[NH];                                                                               \
                _Pragma("unroll") for (int q = 0; q < NH; ++q) { h[q] = H1[source_row + q * C]; hadj[q] = 0.0f; }    \
                float y[16], ang[16];                                                                                \
                load16(s.y[t], y);                                                                                   \
                _Pragma("unroll") for (int q = 0; q < 16; ++q) ang[q] = 0.0f;                                        \
                float radial = 0.0f;                                                                                 \
                SXB_##NAME##_L1_REVERSE_BODY                                                                         \
                if (kRecords) {   /* reproducible mode: one record per edge, summed later */                         \
                    float* record = out.edge_source_adjoint + static_cast<size_t>(chunk + t) * NH * C + k;           \
                    _Pragma("unroll") for (int q = 0; q < NH; ++q) record[q * C] = hadj[q];                          \
                } else {                                                                                             \
                    _Pragma("unroll") for (int q = 0; q < NH; ++q) atomicAdd(H1_adj + source_row + q * C, hadj[q]);  \
                }                                                                                                    \
                float fx = radial * m.y, fy = radial * m.z, fz = radial * m.w;                                       \
                {                                                                                                    \
                    float g[16];                                                                                     \
                    load16(s.gx[t], g);                                                                              \
                    _Pragma("unroll") for (int q = 0; q < 16; ++q) fx = fmaf(ang[q], g[q], fx);                      \
                    load16(s.gy[t], g);                                                                              \
                    _Pragma("unroll") for (int q = 0; q < 16; ++q) fy = fmaf(ang[q], g[q], fy);                      \
                    load16(s.gz[t], g);                                                                              \
                    _Pragma("unroll") for (int q = 0; q < 16; ++q) fz = fmaf(ang[q], g[q], fz);                      \
                }                                                                                                    \
                const float total = warp_reduce3_transposed(fx, fy, fz, lane);   /* lanes 0, 8, 16: x, y, z */       \
                if ((lane & 7) == 0 && lane < 24) fs.partial[t][warp][lane >> 3] = total;                            \
            }                                                                                                        \
            __syncthreads();                                                                                         \
            flush_chunk_forces<8, kRecords>(fs, s, chunk, count, num_warps, out, density_coef);                      \
        }                                                                                                            \
        finish_receiver_forces<8, kRecords>(fs, i, out);                                                             \
    }

SXB_DEFINE_L1_KERNELS(S0)
SXB_DEFINE_L1_KERNELS(S1)

}  // namespace sxb
