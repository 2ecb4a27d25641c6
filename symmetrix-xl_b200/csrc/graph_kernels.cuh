// Periodic cell-list neighbor graph on the device: receiver-major CSR whose per-receiver edge order
// is bin-stencil order (z outermost, x innermost), atoms of a bin in ascending index.  That is the
// order and the accepted edge set of the reference's builder
// (libsymmetrix/source/neighbor_graph_kokkos.cpp:39-405); the work split is different:
//   * atoms are put in bin order by one stable radix sort of (bin, atom) pairs, so bins need no
//     per-bin sort and the candidates of x-adjacent bins are contiguous in memory;
//   * one warp owns a receiver; for each (z, y) row of the stencil it walks maximal runs of
//     x-adjacent bins that share a periodic image, 32 candidates at a time, and compacts the accepted
//     ones in order with a ballot and a prefix population count.
// The distance test is evaluated in double with round-to-nearest adds and multiplies that are never
// contracted into FMAs, in the operand order of the reference's expression, so that a pair at the
// cutoff is accepted or rejected exactly as an IEEE evaluation of that expression would.
#pragma once

#include "common.cuh"

namespace sxb {

struct CellGrid {
    int bins[3];
    int reach[3];
    int num_bins;
    double cutoff_squared;
};

// Fractional coordinates wrapped into [0, 1), the wrap count per axis, the wrapped Cartesian position
// and the atom's bin; a non-finite coordinate raises bit 2 of the status word.
__global__ void wrap_and_bin_kernel(int n, CellGrid grid, const double* __restrict__ positions,
                                    const double* __restrict__ inv_cell, const double* __restrict__ cell,
                                    double* __restrict__ wrapped_pos, int* __restrict__ wrap_count,
                                    int* __restrict__ atom_bin, int* __restrict__ atom_index, int* __restrict__ bin_sizes,
                                    int* __restrict__ status)
{
    const int atom = blockIdx.x * blockDim.x + threadIdx.x;
    if (atom >= n) return;
    atom_index[atom] = atom;
    const double p[3] = {positions[3 * atom], positions[3 * atom + 1], positions[3 * atom + 2]};
    if (!isfinite(p[0]) || !isfinite(p[1]) || !isfinite(p[2])) {
        atomicOr(status, 4);
        atom_bin[atom] = 0;
        atomicAdd(bin_sizes, 1);
        for (int c = 0; c < 3; ++c) {
            wrapped_pos[3 * atom + c] = 0.0;
            wrap_count[3 * atom + c] = 0;
        }
        return;
    }
    double f[3];
    int b[3];
#pragma unroll
    for (int axis = 0; axis < 3; ++axis) {
        double s = __dmul_rn(p[0], inv_cell[axis]);
        s = __dadd_rn(s, __dmul_rn(p[1], inv_cell[3 + axis]));
        s = __dadd_rn(s, __dmul_rn(p[2], inv_cell[6 + axis]));
        const int w = static_cast<int>(floor(s));
        f[axis] = __dadd_rn(s, -static_cast<double>(w));
        wrap_count[3 * atom + axis] = w;
        b[axis] = min(grid.bins[axis] - 1, static_cast<int>(__dmul_rn(f[axis], static_cast<double>(grid.bins[axis]))));
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) {
        double s = __dmul_rn(f[0], cell[c]);
        s = __dadd_rn(s, __dmul_rn(f[1], cell[3 + c]));
        s = __dadd_rn(s, __dmul_rn(f[2], cell[6 + c]));
        wrapped_pos[3 * atom + c] = s;
    }
    const int bin = (b[2] * grid.bins[1] + b[1]) * grid.bins[0] + b[0];
    atom_bin[atom] = bin;
    atomicAdd(bin_sizes + bin, 1);
}

// Wrapped positions gathered into bin order, so that a warp reads its candidates coalesced.
__global__ void gather_sorted_positions_kernel(int n, const int* __restrict__ sorted_atoms, const double* __restrict__ wrapped_pos,
                                               double* __restrict__ sorted_pos)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= n) return;
    const int atom = sorted_atoms[k];
    sorted_pos[3 * k] = wrapped_pos[3 * atom];
    sorted_pos[3 * k + 1] = wrapped_pos[3 * atom + 1];
    sorted_pos[3 * k + 2] = wrapped_pos[3 * atom + 2];
}

// Bin coordinate `raw` of an unbounded bin lattice folded into [0, extent): returns the folded
// coordinate and stores how many periods were removed (the periodic image of that bin).
__device__ __forceinline__ int fold_bin(int raw, int extent, int& image)
{
    image = raw >= 0 ? raw / extent : -((extent - 1 - raw) / extent);
    return raw - image * extent;
}

// kFill = false: counts[receiver] = number of accepted candidates.
// kFill = true:  writes sources / shifts from offsets[receiver] on, in candidate order.
template <bool kFill>
__global__ void __launch_bounds__(256)
receiver_edges_kernel(int num_receivers, CellGrid grid, const int* __restrict__ atom_bin, const int* __restrict__ bin_begin,
                      const int* __restrict__ sorted_atoms, const double* __restrict__ sorted_pos,
                      const double* __restrict__ wrapped_pos, const int* __restrict__ wrap_count,
                      const double* __restrict__ cell, long long* __restrict__ counts, const int* __restrict__ offsets,
                      int* __restrict__ sources, int* __restrict__ shifts)
{
    const int receiver = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const unsigned lane = threadIdx.x & 31u;
    if (receiver >= num_receivers) return;
    const int nx = grid.bins[0], ny = grid.bins[1], nz = grid.bins[2];
    const int home = atom_bin[receiver];
    const int hx = home % nx, hy = (home / nx) % ny, hz = home / (nx * ny);
    const double rx = wrapped_pos[3 * receiver], ry = wrapped_pos[3 * receiver + 1], rz = wrapped_pos[3 * receiver + 2];
    const int wrx = wrap_count[3 * receiver], wry = wrap_count[3 * receiver + 1], wrz = wrap_count[3 * receiver + 2];
    long long written = kFill ? offsets[receiver] : 0;

    for (int dz = -grid.reach[2]; dz <= grid.reach[2]; ++dz) {
        int iz;
        const int bz = fold_bin(hz + dz, nz, iz);
        // image translation, one product per (axis, component); the sums below add them one at a time
        const double zx = __dmul_rn(static_cast<double>(iz), cell[6]), zy = __dmul_rn(static_cast<double>(iz), cell[7]),
                     zz = __dmul_rn(static_cast<double>(iz), cell[8]);
        for (int dy = -grid.reach[1]; dy <= grid.reach[1]; ++dy) {
            int iy;
            const int by = fold_bin(hy + dy, ny, iy);
            const double yx = __dmul_rn(static_cast<double>(iy), cell[3]), yy = __dmul_rn(static_cast<double>(iy), cell[4]),
                         yz = __dmul_rn(static_cast<double>(iy), cell[5]);
            const int row = (bz * ny + by) * nx;
            int dx = -grid.reach[0];
            while (dx <= grid.reach[0]) {
                int ix;
                const int bx = fold_bin(hx + dx, nx, ix);
                // bins bx .. bx+run-1 of this row share the image ix and are contiguous in bin order
                const int run = min(grid.reach[0] - dx + 1, nx - bx);
                const double xx = __dmul_rn(static_cast<double>(ix), cell[0]), xy = __dmul_rn(static_cast<double>(ix), cell[1]),
                             xz = __dmul_rn(static_cast<double>(ix), cell[2]);
                const bool home_image = ix == 0 && iy == 0 && iz == 0;
                const int first = bin_begin[row + bx], last = bin_begin[row + bx + run];
                for (int k0 = first; k0 < last; k0 += 32) {
                    const int k = k0 + static_cast<int>(lane);
                    bool accept = false;
                    int source = -1;
                    if (k < last) {
                        source = sorted_atoms[k];
                        double d = __dadd_rn(sorted_pos[3 * k], -rx);
                        d = __dadd_rn(__dadd_rn(__dadd_rn(d, xx), yx), zx);
                        double d2 = __dmul_rn(d, d);
                        d = __dadd_rn(sorted_pos[3 * k + 1], -ry);
                        d = __dadd_rn(__dadd_rn(__dadd_rn(d, xy), yy), zy);
                        d2 = __dadd_rn(d2, __dmul_rn(d, d));
                        d = __dadd_rn(sorted_pos[3 * k + 2], -rz);
                        d = __dadd_rn(__dadd_rn(__dadd_rn(d, xz), yz), zz);
                        d2 = __dadd_rn(d2, __dmul_rn(d, d));
                        accept = !(d2 > grid.cutoff_squared) && !(home_image && source == receiver);
                    }
                    const unsigned taken = __ballot_sync(0xffffffffu, accept);
                    if constexpr (kFill) {
                        if (accept) {
                            const long long edge = written + __popc(taken & ((1u << lane) - 1u));
                            sources[edge] = source;
                            shifts[3 * edge] = ix - wrap_count[3 * source] + wrx;
                            shifts[3 * edge + 1] = iy - wrap_count[3 * source + 1] + wry;
                            shifts[3 * edge + 2] = iz - wrap_count[3 * source + 2] + wrz;
                        }
                    }
                    written += __popc(taken);
                }
                dx += run;
            }
        }
    }
    if constexpr (!kFill) {
        if (lane == 0) counts[receiver] = written;
    }
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
            const size_t to = 3 * static_cast<size_t>(nb + t), from = 3 * static_cast<size_t>(ob + t);
            new_shifts[to] = old_shifts[from];
            new_shifts[to + 1] = old_shifts[from + 1];
            new_shifts[to + 2] = old_shifts[from + 2];
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
