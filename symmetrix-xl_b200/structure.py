"""Coupling structure of a compact two-layer MACE model, derived from first principles.

A compact model file carries three structural tables next to its weights
(reference loader: libsymmetrix/source/mace.cpp:2770-2786, 2850-2862, 2902-2914):

* the layer-1 edge tensor-product paths ``Phi1_l/l1/l2`` with their sparse
  Clebsch-Gordan table ``Phi1_lme / Phi1_lelm1lm2 / Phi1_clebsch_gordan``;
* the symmetric-contraction monomials ``M0_monomials`` (one list per output
  component LM) and ``M1_monomials`` (scalar output).

The reference obtains them from an e3nn/mace-torch checkpoint.  Here they are
computed directly: real spherical harmonics in the model's own convention (the
edge vector is permuted to (z, x, y) before the harmonics are taken and the
result is scaled by 2*sqrt(pi), mace.cpp:1269-1299), real Wigner matrices fitted
to those harmonics, coupling tensors as the invariant subspace of
D_l1 (x) D_l2 (x) D_l, and the monomial sets as the index triples on which a
symmetrised chain of two couplings does not vanish.  The sign of every coupling
tensor is a convention (a radial weight absorbs it); it is fixed here by making
the first non-zero entry positive.
"""
from __future__ import annotations

import hashlib
import itertools
import json
from functools import lru_cache

import numpy as np


# ----------------------------------------------------------------------------- harmonics
def real_harmonics(l_max: int, xyz: np.ndarray) -> np.ndarray:
    """Y_lm of the directions of ``xyz`` (n,3) in the model convention, lm = l*l+l+m.

    Orthonormal real harmonics of the permuted unit vector (z, x, y), times
    2*sqrt(pi) so that Y_00 = 1 (mace.cpp:1276-1290).
    """
    xyz = np.asarray(xyz, dtype=np.float64)
    r = np.linalg.norm(xyz, axis=1, keepdims=True)
    u = xyz / r
    x, y, z = u[:, 2], u[:, 0], u[:, 1]
    out = np.zeros((xyz.shape[0], (l_max + 1) ** 2))
    pi = np.pi
    out[:, 0] = 0.5 * np.sqrt(1.0 / pi)
    if l_max >= 1:
        c1 = np.sqrt(3.0 / (4.0 * pi))
        out[:, 1], out[:, 2], out[:, 3] = c1 * y, c1 * z, c1 * x
    if l_max >= 2:
        a = 0.5 * np.sqrt(15.0 / pi)
        b = 0.25 * np.sqrt(5.0 / pi)
        out[:, 4] = a * x * y
        out[:, 5] = a * y * z
        out[:, 6] = b * (2 * z * z - x * x - y * y)
        out[:, 7] = a * x * z
        out[:, 8] = 0.5 * a * (x * x - y * y)
    if l_max >= 3:
        c = 0.25 * np.sqrt(35.0 / (2.0 * pi))
        d = 0.5 * np.sqrt(105.0 / pi)
        e = 0.25 * np.sqrt(21.0 / (2.0 * pi))
        f = 0.25 * np.sqrt(7.0 / pi)
        q = 4 * z * z - x * x - y * y
        out[:, 9] = c * y * (3 * x * x - y * y)
        out[:, 10] = d * x * y * z
        out[:, 11] = e * y * q
        out[:, 12] = f * z * (2 * z * z - 3 * x * x - 3 * y * y)
        out[:, 13] = e * x * q
        out[:, 14] = 0.5 * d * z * (x * x - y * y)
        out[:, 15] = c * x * (x * x - 3 * y * y)
    if l_max >= 4:
        raise ValueError("harmonics are implemented for l_max <= 3")
    return out * (2.0 * np.sqrt(pi))


def _random_rotation(rng) -> np.ndarray:
    q, r = np.linalg.qr(rng.normal(size=(3, 3)))
    q = q * np.sign(np.diag(r))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return q


_SAMPLE_RNG_SEED = 20240611


@lru_cache(maxsize=None)
def _sample_points() -> np.ndarray:
    rng = np.random.default_rng(_SAMPLE_RNG_SEED)
    return rng.normal(size=(64, 3))


def _general_harmonics(l: int, xyz: np.ndarray) -> np.ndarray:
    """The 2l+1 real harmonics of degree ``l`` for any l, same convention as above.

    Built from the complex harmonics: m > 0 -> sqrt(2) (-1)^m Re Y_l^m, m < 0 ->
    sqrt(2) (-1)^m Im Y_l^|m|; equal to ``real_harmonics`` for l <= 3 (tested).  Needed
    only for intermediate irreps of the symmetric contraction (up to l = 6).
    """
    from scipy.special import sph_harm_y

    u = xyz / np.linalg.norm(xyz, axis=1, keepdims=True)
    x, y, z = u[:, 2], u[:, 0], u[:, 1]
    theta, phi = np.arccos(np.clip(z, -1.0, 1.0)), np.arctan2(y, x)
    out = np.zeros((xyz.shape[0], 2 * l + 1))
    for m in range(-l, l + 1):
        v = sph_harm_y(l, abs(m), theta, phi)
        if m == 0:
            out[:, l + m] = v.real
        elif m > 0:
            out[:, l + m] = np.sqrt(2.0) * (-1) ** m * v.real
        else:
            out[:, l + m] = np.sqrt(2.0) * (-1) ** m * v.imag
    return out * (2.0 * np.sqrt(np.pi))


def wigner_matrix(l: int, rotation: np.ndarray) -> np.ndarray:
    """Real matrix D with Y_l(R u) = D Y_l(u) for the harmonics above (least squares)."""
    pts = _sample_points()
    y0 = _general_harmonics(l, pts)
    y1 = _general_harmonics(l, pts @ rotation.T)
    d, *_ = np.linalg.lstsq(y0, y1, rcond=None)
    return d.T


@lru_cache(maxsize=None)
def coupling_tensor(l1: int, l2: int, l: int) -> np.ndarray | None:
    """Real Clebsch-Gordan tensor C[m1, m2, m] with sum_{m1 m2} C^2 = 1 for every m.

    The one-dimensional invariant subspace of D_l1 (x) D_l2 (x) D_l, found as the
    null space of (D (x) D (x) D - 1) stacked over a few random rotations.
    ``None`` when the triangle rule forbids the coupling.
    """
    if l < abs(l1 - l2) or l > l1 + l2:
        return None
    rng = np.random.default_rng(1000 * l1 + 100 * l2 + l + 7)
    n1, n2, n3 = 2 * l1 + 1, 2 * l2 + 1, 2 * l + 1
    rows = []
    for _ in range(4):
        rot = _random_rotation(rng)
        big = np.einsum("ai,bj,ck->abcijk", wigner_matrix(l1, rot), wigner_matrix(l2, rot),
                        wigner_matrix(l, rot)).reshape(n1 * n2 * n3, n1 * n2 * n3)
        rows.append(big - np.eye(n1 * n2 * n3))
    _, s, vt = np.linalg.svd(np.concatenate(rows, axis=0))
    if s[-1] > 1e-9 or (len(s) > 1 and s[-2] < 1e-6):
        raise RuntimeError(f"coupling ({l1},{l2},{l}) is not one-dimensional: {s[-3:]}")
    c = vt[-1].reshape(n1, n2, n3)
    c = c / np.sqrt(np.sum(c[:, :, 0] ** 2))
    c[np.abs(c) < 1e-12] = 0.0
    first = c.reshape(-1)[np.flatnonzero(c.reshape(-1))[0]]
    return c * np.sign(first)


# ----------------------------------------------------------------------------- layer-1 paths
def r1_structure(edge_l_max: int, source_l_max: int) -> dict:
    """Paths, row enumeration and sparse coupling table of the layer-1 edge tensor product.

    A path couples edge harmonic l1 with source irrep l2 (parity (-1)^l2) into an
    output irrep l <= edge_l_max of parity (-1)^l, i.e. l1 + l2 + l even.  Paths are
    ordered by (l, l2, l1); rows enumerate ``for path: for lm1: for lm2``
    (mace.cpp:2046-2064); the output index is group_begin(l) + m*eta_l + e so that
    Phi1[l] is a (2l+1) x (eta_l*C) row-major matrix (mace.cpp:2305-2340); terms are
    ordered by (lm1, lm2, path, output m).
    """
    paths = []
    for l in range(edge_l_max + 1):
        for l2 in range(source_l_max + 1):
            for l1 in range(edge_l_max + 1):
                if abs(l1 - l2) <= l <= l1 + l2 and (l1 + l2 + l) % 2 == 0:
                    paths.append((l, l1, l2))
    eta = [sum(1 for p in paths if p[0] == l) for l in range(edge_l_max + 1)]
    group_begin = np.concatenate([[0], np.cumsum([(2 * l + 1) * eta[l] for l in range(edge_l_max + 1)])])
    row_begin, rows = [], 0
    for (l, l1, l2) in paths:
        row_begin.append(rows)
        rows += (2 * l1 + 1) * (2 * l2 + 1)
    terms = []
    for p, (l, l1, l2) in enumerate(paths):
        c = coupling_tensor(l1, l2, l)
        e = [q for q in range(len(paths)) if paths[q][0] == l].index(p)
        for a in range(2 * l1 + 1):
            for b in range(2 * l2 + 1):
                for m in range(2 * l + 1):
                    if c[a, b, m] != 0.0:
                        lm1, lm2 = l1 * l1 + a, l2 * l2 + b
                        terms.append((lm1, lm2, p, m, int(group_begin[l]) + m * eta[l] + e,
                                      row_begin[p] + a * (2 * l2 + 1) + b, float(c[a, b, m])))
    terms.sort(key=lambda t: (t[0], t[1], t[2], t[3]))
    return {
        "edge_l_max": edge_l_max,
        "source_l_max": source_l_max,
        "Phi1_l": [p[0] for p in paths],
        "Phi1_l1": [p[1] for p in paths],
        "Phi1_l2": [p[2] for p in paths],
        "eta": eta,
        "num_rows": rows,
        "num_lme": int(group_begin[-1]),
        "Phi1_lme": [t[4] for t in terms],
        "Phi1_lelm1lm2": [t[5] for t in terms],
        "Phi1_clebsch_gordan": [t[6] for t in terms],
        "term_lm1": [t[0] for t in terms],
        "term_lm2": [t[1] for t in terms],
    }


# ----------------------------------------------------------------------------- symmetric contraction
def _l_of(lm: int) -> int:
    return int(np.floor(np.sqrt(lm + 0.5)))


@lru_cache(maxsize=None)
def contraction_basis(input_l_max: int, output_l: int, correlation: int = 3):
    """Monomials and an equivariant coefficient basis of the symmetric contraction.

    Inputs are the (input_l_max+1)^2 numbers A[lm] of one channel (irrep l has parity
    (-1)^l); the output irrep has parity (-1)^output_l.  Every chain of couplings
    (l_a (x) l_b -> l_mid) (x) l_c -> L defines one equivariant polynomial
    sum_{abc} T[a,b,c] x_a x_b x_c; collecting equal monomials symmetrises it.  A sorted
    index tuple belongs to component M when its collected coefficient is non-zero for
    some chain: the union of supports of a spanning set equals that of any basis of
    the equivariant polynomials, so the set does not depend on the basis a converter
    picks.

    Returns ``(monomials, chains)``: ``monomials[M]`` is the list of index tuples of
    component M = -L..L (linear, then quadratic, then cubic, each lexicographic);
    ``chains`` is a list of ``(degree, coeff)`` with ``coeff[M]`` a vector over
    ``monomials[M]``.  Using one weight per chain for all M gives an equivariant map.
    """
    L = output_l
    tol = 1e-9
    ls = range(input_l_max + 1)
    raw = []  # (degree, {key: vector over M})
    if correlation >= 1 and L <= input_l_max:
        raw.append((1, {(L * L + M,): np.eye(2 * L + 1)[M] for M in range(2 * L + 1)}))
    if correlation >= 2:
        for la, lb in itertools.product(ls, ls):
            if (la + lb + L) % 2 or la > lb:
                continue
            c = coupling_tensor(la, lb, L)
            if c is None:
                continue
            acc: dict = {}
            for a, b in itertools.product(range(2 * la + 1), range(2 * lb + 1)):
                key = tuple(sorted((la * la + a, lb * lb + b)))
                acc[key] = acc.get(key, 0.0) + c[a, b, :]
            raw.append((2, acc))
    if correlation >= 3:
        for la, lb, lc in itertools.product(ls, ls, ls):
            if (la + lb + lc + L) % 2:
                continue
            for l_mid in range(abs(la - lb), la + lb + 1):
                c1 = coupling_tensor(la, lb, l_mid)
                c2 = coupling_tensor(l_mid, lc, L)
                if c1 is None or c2 is None:
                    continue
                t = np.einsum("abu,ucm->abcm", c1, c2)
                acc = {}
                for a, b, c in itertools.product(range(2 * la + 1), range(2 * lb + 1), range(2 * lc + 1)):
                    key = tuple(sorted((la * la + a, lb * lb + b, lc * lc + c)))
                    acc[key] = acc.get(key, 0.0) + t[a, b, c, :]
                raw.append((3, acc))
    found: list[set] = [set() for _ in range(2 * L + 1)]
    kept = []
    for degree, acc in raw:
        nonzero = False
        for key, v in acc.items():
            for M in np.flatnonzero(np.abs(v) > tol):
                found[M].add(key)
                nonzero = True
        if nonzero:
            kept.append((degree, acc))
    monomials = [sorted(f, key=lambda k: (len(k), k)) for f in found]
    index = [{k: i for i, k in enumerate(m)} for m in monomials]
    chains = []
    for degree, acc in kept:
        coeff = [np.zeros(len(m)) for m in monomials]
        for key, v in acc.items():
            for M in np.flatnonzero(np.abs(v) > tol):
                coeff[M][index[M][key]] = v[M]
        norm = np.sqrt(sum(float(c @ c) for c in coeff) / (2 * L + 1))
        chains.append((degree, [c / norm for c in coeff]))
    return monomials, chains


def contraction_monomials(input_l_max: int, output_l: int, correlation: int = 3) -> list[list[list[int]]]:
    """Monomial index lists per component M of output irrep ``output_l`` (see contraction_basis)."""
    monomials, _ = contraction_basis(input_l_max, output_l, correlation)
    return [[list(k) for k in m] for m in monomials]


@lru_cache(maxsize=None)
def model_structure(edge_l_max: int, hidden_l_max: int, correlation: int = 3) -> dict:
    """All structural tables of a compact two-layer model with the given harmonics."""
    s = dict(r1_structure(edge_l_max, hidden_l_max))
    m0 = {}
    for L in range(hidden_l_max + 1):
        per_m = contraction_monomials(edge_l_max, L, correlation)
        for M, terms in enumerate(per_m):
            m0[str(L * L + M)] = terms
    s["M0_monomials"] = m0
    s["M1_monomials"] = m0["0"]
    s["l_max"] = edge_l_max
    s["L_max"] = hidden_l_max
    return s


def structure_fingerprint(s: dict) -> str:
    """SHA-256 over the integer tables and the coupling coefficients rounded to 1e-12."""
    blob = json.dumps(
        {
            "l": s["Phi1_l"], "l1": s["Phi1_l1"], "l2": s["Phi1_l2"],
            "lme": s["Phi1_lme"], "rows": s["Phi1_lelm1lm2"],
            "cg": [round(abs(v), 10) for v in s["Phi1_clebsch_gordan"]],
            "m0": {k: s["M0_monomials"][k] for k in sorted(s["M0_monomials"], key=int)},
            "m1": s["M1_monomials"],
        },
        separators=(",", ":"), sort_keys=True)
    return hashlib.sha256(blob.encode()).hexdigest()
