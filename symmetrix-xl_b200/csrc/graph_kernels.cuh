// Periodic cell-list neighbor graph on the device, receiver-major CSR in the reference's
// stencil order.  Follows build_periodic_neighbor_graph_kokkos
// (libsymmetrix/source/neighbor_graph_kokkos.cpp:39-405): wrap -> bin -> sort inside bins by
// atom index -> count -> scan -> fill.  All double arithmetic on the acceptance path uses
// round-to-nearest add/mul intrinsics (never contracted into FMAs), so the accepted edge set is
// the one an IEEE evaluation of the reference's expressions gives.
#pragma once

#include "common.cuh"

namespace sxb {

struct CellList {
    int bins[3];
    int reach[3];
    int num_bins;
    double cutoff_squared;
};

__global__ void wrap_positions_kernel(int n, const double* __restrict__ positions, const double* __restrict__ inv_cell,
                                      const double* __restrict__ cell, double* __restrict__ wrapped_frac,
                                      double* __restrict__ wrapped_pos, int* __restrict__ wrap_shift)
{
    const int atom = blockIdx.x * blockDim.x + threadIdx.x;
    if (atom >= n) return;
    double frac[3];
    for (int axis = 0; axis < 3; ++axis) {
        double value = 0.0;
        for (int component = 0; component < 3; ++component)
            value = __dadd_rn(value, __dmul_rn(positions[3 * atom + component], inv_cell[3 * component + axis]));
        const int wrap = static_cast<int>(floor(value));
        value = __dadd_rn(value, -static_cast<double>(wrap));
        frac[axis] = value;
        wrapped_frac[3 * atom + axis] = value;
        wrap_shift[3 * atom + axis] = wrap;
    }
    for (int component = 0; component < 3; ++component) {
        double value = 0.0;
        for (int axis = 0; axis < 3; ++axis) value = __dadd_rn(value, __dmul_rn(frac[axis], cell[3 * axis + component]));
        wrapped_pos[3 * atom + component] = value;
    }
}

__global__ void count_bins_kernel(int n, CellList cl, const double* __restrict__ wrapped_frac, int* __restrict__ atom_bin,
                                  int* __restrict__ bin_sizes)
{
    const int atom = blockIdx.x * blockDim.x + threadIdx.x;
    if (atom >= n) return;
    const int x = min(cl.bins[0] - 1, static_cast<int>(__dmul_rn(wrapped_frac[3 * atom], static_cast<double>(cl.bins[0]))));
    const int y = min(cl.bins[1] - 1, static_cast<int>(__dmul_rn(wrapped_frac[3 * atom + 1], static_cast<double>(cl.bins[1]))));
    const int z = min(cl.bins[2] - 1, static_cast<int>(__dmul_rn(wrapped_frac[3 * atom + 2], static_cast<double>(cl.bins[2]))));
    const int bin = (z * cl.bins[1] + y) * cl.bins[0] + x;
    atom_bin[atom] = bin;
    atomicAdd(bin_sizes + bin, 1);
}

__global__ void fill_bins_kernel(int n, const int* __restrict__ atom_bin, int* __restrict__ cursors, int* __restrict__ bin_atoms)
{
    const int atom = blockIdx.x * blockDim.x + threadIdx.x;
    if (atom >= n) return;
    bin_atoms[atomicAdd(cursors + atom_bin[atom], 1)] = atom;
}

__global__ void sort_bins_kernel(int num_bins, const int* __restrict__ offsets, int* __restrict__ bin_atoms)
{
    const int bin = blockIdx.x * blockDim.x + threadIdx.x;
    if (bin >= num_bins) return;
    const int begin = offsets[bin], end = offsets[bin + 1];
    for (int index = begin + 1; index < end; ++index) {
        const int atom = bin_atoms[index];
        int insertion = index;
        while (insertion > begin && bin_atoms[insertion - 1] > atom) {
            bin_atoms[insertion] = bin_atoms[insertion - 1];
            --insertion;
        }
        bin_atoms[insertion] = atom;
    }
}

__device__ __forceinline__ int floor_div(int numerator, int denominator)
{
    const int quotient = numerator / denominator;
    const int remainder = numerator % denominator;
    return quotient - ((remainder != 0 && remainder < 0) ? 1 : 0);
}

// One thread per receiver; kFill = false counts, true writes sources and shifts at the
// receiver's offset.  The candidate order is the stencil order (z outermost) then the in-bin order.
template <bool kFill>
__global__ void neighbor_edges_kernel(int n, CellList cl, const int* __restrict__ atom_bin, const int* __restrict__ bin_offsets,
                                      const int* __restrict__ bin_atoms, const double* __restrict__ wrapped_pos,
                                      const int* __restrict__ wrap_shift, const double* __restrict__ cell,
                                      long long* __restrict__ counts, const int* __restrict__ receiver_offsets,
                                      int* __restrict__ sources, int* __restrict__ shifts)
{
    const int receiver = blockIdx.x * blockDim.x + threadIdx.x;
    if (receiver >= n) return;
    const int rb = atom_bin[receiver];
    const int rx = rb % cl.bins[0];
    const int ry = (rb / cl.bins[0]) % cl.bins[1];
    const int rz = rb / (cl.bins[0] * cl.bins[1]);
    const double px = wrapped_pos[3 * receiver], py = wrapped_pos[3 * receiver + 1], pz = wrapped_pos[3 * receiver + 2];
    double c[9];
    for (int q = 0; q < 9; ++q) c[q] = cell[q];
    long long local = 0;
    const long long base = kFill ? receiver_offsets[receiver] : 0;
    for (int dz = -cl.reach[2]; dz <= cl.reach[2]; ++dz) {
        const int raw_z = rz + dz;
        const int shift_z = floor_div(raw_z, cl.bins[2]);
        const int source_z = raw_z - shift_z * cl.bins[2];
        for (int dy = -cl.reach[1]; dy <= cl.reach[1]; ++dy) {
            const int raw_y = ry + dy;
            const int shift_y = floor_div(raw_y, cl.bins[1]);
            const int source_y = raw_y - shift_y * cl.bins[1];
            for (int dx = -cl.reach[0]; dx <= cl.reach[0]; ++dx) {
                const int raw_x = rx + dx;
                const int shift_x = floor_div(raw_x, cl.bins[0]);
                const int source_x = raw_x - shift_x * cl.bins[0];
                const int source_bin = (source_z * cl.bins[1] + source_y) * cl.bins[0] + source_x;
                const int image[3] = {shift_x, shift_y, shift_z};
                for (int index = bin_offsets[source_bin]; index < bin_offsets[source_bin + 1]; ++index) {
                    const int source = bin_atoms[index];
                    if (source == receiver && shift_x == 0 && shift_y == 0 && shift_z == 0) continue;
                    double distance_squared = 0.0;
                    const double rp[3] = {px, py, pz};
                    for (int component = 0; component < 3; ++component) {
                        double displacement = __dadd_rn(wrapped_pos[3 * source + component], -rp[component]);
                        for (int axis = 0; axis < 3; ++axis)
                            displacement = __dadd_rn(displacement, __dmul_rn(static_cast<double>(image[axis]), c[3 * axis + component]));
                        distance_squared = __dadd_rn(distance_squared, __dmul_rn(displacement, displacement));
                    }
                    if (distance_squared > cl.cutoff_squared) continue;
                    if constexpr (kFill) {
                        const long long edge = base + local;
                        sources[edge] = source;
                        for (int axis = 0; axis < 3; ++axis)
                            shifts[3 * edge + axis] = image[axis] - wrap_shift[3 * source + axis] + wrap_shift[3 * receiver + axis];
                    }
                    ++local;
                }
            }
        }
    }
    if constexpr (!kFill) counts[receiver] = local;
}

// Re-expresses a CSR graph given in caller node order in the internal order (nodes grouped by
// element): receiver ``new`` is caller node ``original[new]``; its edge list keeps its order and
// its sources are renumbered.  ``edge_map[new_edge]`` = caller edge index.
__global__ void permute_graph_kernel(int n, const int* __restrict__ original, const int* __restrict__ internal_of,
                                     const int* __restrict__ old_first, const int* __restrict__ old_sources,
                                     const int* __restrict__ old_shifts, const int* __restrict__ new_first,
                                     int* __restrict__ new_sources, int* __restrict__ new_shifts, int* __restrict__ edge_map)
{
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n) return;
    const int old_node = original[warp];
    const int ob = old_first[old_node], count = old_first[old_node + 1] - ob;
    const int nb = new_first[warp];
    for (int t = lane; t < count; t += 32) {
        new_sources[nb + t] = internal_of[old_sources[ob + t]];
        edge_map[nb + t] = ob + t;
        if (old_shifts != nullptr) {
            new_shifts[3 * (nb + t)] = old_shifts[3 * (ob + t)];
            new_shifts[3 * (nb + t) + 1] = old_shifts[3 * (ob + t) + 1];
            new_shifts[3 * (nb + t) + 2] = old_shifts[3 * (ob + t) + 2];
        }
    }
}

__global__ void gather_counts_kernel(int n, const int* __restrict__ original, const int* __restrict__ old_first,
                                     int* __restrict__ new_counts)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int o = original[i];
    new_counts[i] = old_first[o + 1] - old_first[o];
}

}  // namespace sxb
