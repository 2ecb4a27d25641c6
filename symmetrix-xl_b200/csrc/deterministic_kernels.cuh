// Fixed-order accumulation for the reproducible mode.
//
// By default the gradient kernels add the source adjoint H1_adj_j and the force on the source atom with
// atomics, whose order varies from run to run (results agree to rounding only).  The reference instead
// walks a source-sorted schedule (source_offsets / source_edges, libsymmetrix/source/
// mace_kokkos_factorized_lifecycle.cpp:2133-2195) so that every sum has one order.  In the reproducible
// mode the gradient kernels leave one record per edge (source adjoint, directed force) and the kernels
// below sum the records over that same schedule: edges of a source in ascending edge index.  Two
// evaluations of the same input then give identical bits.
#pragma once

#include "common.cuh"

namespace sxb {

// H1_adj[node] = sum over the edges whose source is `node`, in schedule order, of the edge's record.
// One block per node, one thread per four floats of the row.
__global__ void reduce_source_adjoint_kernel(int row_floats, const int* __restrict__ source_offsets, const int* __restrict__ source_edges,
                                             const EdgeGeom* __restrict__ geom, float r_cut, const float* __restrict__ records,
                                             float* __restrict__ H1_adj)
{
    const int node = blockIdx.x;
    const int begin = source_offsets[node], end = source_offsets[node + 1];
    for (int q = threadIdx.x; q < (row_floats >> 2); q += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = begin; k < end; ++k) {
            const int e = source_edges[k];
            if (!(geom[e].r < r_cut)) continue;        // list-skin edges leave no record
            const float4 v = reinterpret_cast<const float4*>(records + static_cast<size_t>(e) * row_floats)[q];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(H1_adj + static_cast<size_t>(node) * row_floats)[q] = acc;
    }
}

// forces[node] = - sum over the node's own edges (it is their receiver) + sum over the edges it is the
// source of, both in ascending edge order.  One thread per node.
__global__ void reduce_node_forces_kernel(int num_nodes, int num_receivers, const int* __restrict__ first,
                                          const int* __restrict__ source_offsets, const int* __restrict__ source_edges,
                                          const double* __restrict__ edge_forces, double* __restrict__ forces)
{
    const int node = blockIdx.x * blockDim.x + threadIdx.x;
    if (node >= num_nodes) return;
    double fx = 0.0, fy = 0.0, fz = 0.0;
    if (node < num_receivers)
        for (int e = first[node]; e < first[node + 1]; ++e) {
            fx -= edge_forces[3 * static_cast<size_t>(e)];
            fy -= edge_forces[3 * static_cast<size_t>(e) + 1];
            fz -= edge_forces[3 * static_cast<size_t>(e) + 2];
        }
    for (int k = source_offsets[node]; k < source_offsets[node + 1]; ++k) {
        const size_t e = static_cast<size_t>(source_edges[k]);
        fx += edge_forces[3 * e];
        fy += edge_forces[3 * e + 1];
        fz += edge_forces[3 * e + 2];
    }
    forces[3 * static_cast<size_t>(node)] = fx;
    forces[3 * static_cast<size_t>(node) + 1] = fy;
    forces[3 * static_cast<size_t>(node) + 2] = fz;
}

constexpr int kTotalsThreads = 256;

// Stage 1: block b sums f (x) xyz over its 256 edges and the node energies of its 256 receivers into
// partials[b][10] = [energy, virial 9]; the tree inside a block is the same on every run.
__global__ void __launch_bounds__(kTotalsThreads)
partial_totals_kernel(long num_edges, int num_receivers, const EdgeGeom* __restrict__ geom, const double* __restrict__ edge_forces,
                      const double* __restrict__ node_energies, double* __restrict__ partials)
{
    __shared__ double warp_sums[kTotalsThreads / 32][10];
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    double v[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (idx < num_receivers) v[0] = node_energies[idx];
    if (idx < num_edges) {
        const EdgeGeom g = geom[idx];
        const double len = g.r;
        const double rx = len * g.ux, ry = len * g.uy, rz = len * g.uz;
        const double ex = edge_forces[3 * idx], ey = edge_forces[3 * idx + 1], ez = edge_forces[3 * idx + 2];
        v[1] = ex * rx; v[2] = ex * ry; v[3] = ex * rz;
        v[4] = ey * rx; v[5] = ey * ry; v[6] = ey * rz;
        v[7] = ez * rx; v[8] = ez * ry; v[9] = ez * rz;
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
#pragma unroll
        for (int q = 0; q < 10; ++q) v[q] += __shfl_xor_sync(0xffffffffu, v[q], offset);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0)
#pragma unroll
        for (int q = 0; q < 10; ++q) warp_sums[warp][q] = v[q];
    __syncthreads();
    if (threadIdx.x < 10) {
        double s = 0.0;
        for (int w = 0; w < kTotalsThreads / 32; ++w) s += warp_sums[w][threadIdx.x];
        partials[static_cast<long>(blockIdx.x) * 10 + threadIdx.x] = s;
    }
}

// Stage 2: one thread per quantity adds the block partials in block order; the result goes to slot 0 of
// the energy / virial slots (the other slots stay zero in this mode), which the closing kernel sums.
__global__ void final_totals_kernel(int num_blocks, const double* __restrict__ partials, double* __restrict__ energy_slots,
                                    double* __restrict__ virial_slots)
{
    const int q = threadIdx.x;
    if (q >= 10) return;
    double s = 0.0;
    for (int b = 0; b < num_blocks; ++b) s += partials[static_cast<long>(b) * 10 + q];
    if (q == 0) energy_slots[0] = s;
    else virial_slots[q - 1] = s;
}

__global__ void count_sources_kernel(long num_edges, const int* __restrict__ sources, int* __restrict__ counts)
{
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e < num_edges) atomicAdd(counts + sources[e], 1);
}

__global__ void iota_kernel(long n, int* __restrict__ out)
{
    const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = static_cast<int>(i);
}

}  // namespace sxb
