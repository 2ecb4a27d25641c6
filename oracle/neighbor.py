"""CPU restatement of the reference's periodic cell-list neighbor graph.

TEST INFRASTRUCTURE ONLY.  Follows build_periodic_neighbor_graph_kokkos
(libsymmetrix/source/neighbor_graph_kokkos.cpp:39-405) step by step in float64:
fractional = pos * inv_cell wrapped with floor (:122-151); bins per axis =
max(1, floor(face_height/cutoff)), reach = ceil(cutoff*|inv column|*bins)+1
(:153-176); bin = min(bins-1, int(frac*bins)) flattened (z*ny+y)*nx+x (:192-211);
atoms inside a bin in ascending index (:241-260); per receiver the stencil loops
dz, dy, dx in [-reach, reach] with z outermost, floor-division wrap giving the image
(:279-300); a candidate is skipped only when it is the receiver itself in the home
image (:303-306); the displacement is wrapped_source - wrapped_receiver + image*cell,
accepted when d^2 <= cutoff^2 (:307-321); shift = image - wrap(source) + wrap(receiver)
(:330-334).  Parity is unpinned by reference goldens (the Kokkos file cannot be built
here); it is pinned instead against a brute-force all-pairs search and the published
edge counts of the 5,000-atom SrTiO3 case (README.md:86-88).
"""
from __future__ import annotations

import numpy as np


def build_neighbor_graph(positions, cell, cutoff):
    """Returns (first_neigh[N+1] i32, sources[E] i32, shifts[E,3] i32) in reference order."""
    pos = np.asarray(positions, dtype=np.float64).reshape(-1, 3)
    cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
    inv = np.linalg.inv(cell)
    n = pos.shape[0]
    frac = np.zeros((n, 3))
    for axis in range(3):  # same summation order as the reference loop
        v = np.zeros(n)
        for comp in range(3):
            v = v + pos[:, comp] * inv[comp, axis]
        frac[:, axis] = v
    wrap = np.floor(frac).astype(np.int64)
    wfrac = frac - wrap
    wpos = np.zeros((n, 3))
    for comp in range(3):
        v = np.zeros(n)
        for axis in range(3):
            v = v + wfrac[:, axis] * cell[axis, comp]
        wpos[:, comp] = v
    bins = np.zeros(3, dtype=np.int64)
    reach = np.zeros(3, dtype=np.int64)
    for axis in range(3):
        inv_norm_sq = float((inv[:, axis] ** 2).sum())
        face_height = 1.0 / np.sqrt(inv_norm_sq)
        bins[axis] = max(1, int(np.floor(face_height / cutoff)))
        reach[axis] = max(1, int(np.ceil(cutoff * np.sqrt(inv_norm_sq) * bins[axis]) + 1.0))
    bx = np.minimum(bins[0] - 1, (wfrac[:, 0] * bins[0]).astype(np.int64))
    by = np.minimum(bins[1] - 1, (wfrac[:, 1] * bins[1]).astype(np.int64))
    bz = np.minimum(bins[2] - 1, (wfrac[:, 2] * bins[2]).astype(np.int64))
    atom_bin = (bz * bins[1] + by) * bins[0] + bx
    order = np.argsort(atom_bin, kind="stable")  # ascending atom index inside a bin
    nb = int(bins.prod())
    bin_offsets = np.concatenate([[0], np.cumsum(np.bincount(atom_bin, minlength=nb))])
    cut2 = cutoff * cutoff

    # vectorised over receivers per stencil offset, then re-ordered to (receiver, stencil, in-bin)
    recv_chunks, src_chunks, shift_chunks, key_chunks = [], [], [], []
    stencil_index = 0
    max_occ = int(np.diff(bin_offsets).max()) if n else 0
    for dz in range(-reach[2], reach[2] + 1):
        raw_z = bz + dz
        sz = np.floor_divide(raw_z, bins[2])
        cz = raw_z - sz * bins[2]
        for dy in range(-reach[1], reach[1] + 1):
            raw_y = by + dy
            sy = np.floor_divide(raw_y, bins[1])
            cy = raw_y - sy * bins[1]
            for dx in range(-reach[0], reach[0] + 1):
                raw_x = bx + dx
                sx = np.floor_divide(raw_x, bins[0])
                cx = raw_x - sx * bins[0]
                sbin = (cz * bins[1] + cy) * bins[0] + cx
                start, stop = bin_offsets[sbin], bin_offsets[sbin + 1]
                for slot in range(max_occ):
                    valid = start + slot < stop
                    if not valid.any():
                        break
                    recv = np.flatnonzero(valid)
                    src = order[start[recv] + slot]
                    img = np.stack([sx[recv], sy[recv], sz[recv]], axis=1)
                    keep = ~((src == recv) & (img == 0).all(axis=1))
                    recv, src, img = recv[keep], src[keep], img[keep]
                    d2 = np.zeros(len(recv))
                    for comp in range(3):
                        disp = wpos[src, comp] - wpos[recv, comp]
                        for axis in range(3):
                            disp = disp + img[:, axis] * cell[axis, comp]
                        d2 = d2 + disp * disp
                    ok = ~(d2 > cut2)
                    recv, src, img = recv[ok], src[ok], img[ok]
                    recv_chunks.append(recv)
                    src_chunks.append(src)
                    shift_chunks.append(img - wrap[src] + wrap[recv])
                    key_chunks.append(np.full(len(recv), stencil_index * max(max_occ, 1) + slot, dtype=np.int64))
                stencil_index += 1
    if recv_chunks:
        recv = np.concatenate(recv_chunks)
        src = np.concatenate(src_chunks)
        shifts = np.concatenate(shift_chunks)
        key = np.concatenate(key_chunks)
        perm = np.lexsort((key, recv))
        recv, src, shifts = recv[perm], src[perm], shifts[perm]
    else:
        recv = src = np.zeros(0, dtype=np.int64)
        shifts = np.zeros((0, 3), dtype=np.int64)
    first = np.concatenate([[0], np.cumsum(np.bincount(recv, minlength=n))]).astype(np.int32)
    return first, src.astype(np.int32), shifts.astype(np.int32)


def brute_force_edges(positions, cell, cutoff, max_image: int = 2):
    """All-pairs periodic search: set of (receiver, source, sx, sy, sz) with |r_j + S*cell - r_i| <= cutoff."""
    pos = np.asarray(positions, dtype=np.float64).reshape(-1, 3)
    cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
    n = len(pos)
    out = set()
    rng = range(-max_image, max_image + 1)
    for sx in rng:
        for sy in rng:
            for sz in rng:
                off = sx * cell[0] + sy * cell[1] + sz * cell[2]
                d = pos[None, :, :] + off[None, None, :] - pos[:, None, :]
                d2 = (d * d).sum(axis=2)
                ii, jj = np.nonzero(d2 <= cutoff * cutoff)
                for i, j in zip(ii, jj):
                    if i == j and sx == 0 and sy == 0 and sz == 0:
                        continue
                    out.add((int(i), int(j), sx, sy, sz))
    return out


def edge_vectors(positions, cell, first_neigh, sources, shifts):
    """xyz_ij = r_j - r_i + shift*cell per directed edge, receiver-major, float64."""
    pos = np.asarray(positions, dtype=np.float64).reshape(-1, 3)
    cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
    recv = np.repeat(np.arange(len(first_neigh) - 1), np.diff(first_neigh))
    return pos[sources] - pos[recv] + np.asarray(shifts, dtype=np.float64) @ cell
