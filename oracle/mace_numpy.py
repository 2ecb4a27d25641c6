"""NumPy restatement of the reference's serial MACE evaluator (energy, forces, stress).

TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA path is compared with;
nothing in the product may import it.  Every stage follows MACECPU<double>
(libsymmetrix/source/mace.cpp) and cites the lines it restates.  It is pinned
against the reference's own evaluator compiled into oracle/_ref/ (all stage tensors
agree to ~1e-12, see tests/test_oracle.py) and against the golden fixtures under
tests/golden/.  Layout of every node tensor is (node, lm, channel), row-major.
"""
from __future__ import annotations

import json

import numpy as np

TWO_SQRT_PI = 2.0 * np.sqrt(np.pi)


def _silu_scaled(x, scale):
    return scale * x / (1.0 + np.exp(-x))


# ----------------------------------------------------------------------------- radial tables
class RadialTables:
    """Bessel x polynomial-cutoff features -> MLP -> nodal values -> cubic spline coefficients.

    compact_radial.cpp:227-267 (features), 269-289 (network), 326-366 (nodal derivatives:
    tridiagonal system with a left not-a-knot-like closure and a zero right derivative),
    cubic_spline_set.cpp:8-31 (coefficients c[(4*i+order)*F+f])."""

    def __init__(self, definition: dict, r_cut: float):
        self.x0 = float(definition["spline_grid_min"])
        self.points = int(definition["num_spline_points"])
        self.h = (r_cut - self.x0) / (self.points - 1)
        basis = definition["basis"]
        self.bessel_w = np.asarray(basis["weights"], dtype=np.float64)
        self.prefactor = float(basis["prefactor"])
        self.r_max = float(definition["cutoff"]["r_max"])
        self.p = int(definition["cutoff"]["p"])
        transform = definition["distance_transform"]                      # compact_radial.cpp:149-166
        self.agnesi = transform["type"] == "agnesi"
        if self.agnesi:
            self.agnesi_a, self.agnesi_q, self.agnesi_p = float(transform["a"]), float(transform["q"]), float(transform["p"])
            self.covalent_radii = np.asarray(transform["covalent_radii"], dtype=np.float64)
        elif transform["type"] != "none":
            raise NotImplementedError("unknown distance transform")
        self.networks = definition["networks"]
        self._cache = {}

    def features(self, type_i=0, type_j=0):
        """Bessel features on the spline grid; with the Agnesi transform the Bessel argument is the
        transformed distance of the species pair (compact_radial.cpp:227-267)."""
        r = self.x0 + np.arange(self.points) * self.h
        rt = r
        if self.agnesi:
            r0 = 0.5 * (self.covalent_radii[type_i] + self.covalent_radii[type_j])
            sr = r / r0
            rt = 1.0 / (1.0 + self.agnesi_a * sr ** self.agnesi_q / (1.0 + sr ** (self.agnesi_q - self.agnesi_p)))
        u = r / self.r_max
        p = float(self.p)
        cut = np.where(r < self.r_max,
                       1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * u ** self.p
                       + p * (p + 2.0) * u ** (self.p + 1)
                       - (p * (p + 1.0) / 2.0) * u ** (self.p + 2), 0.0)
        return self.prefactor * np.sin(self.bessel_w[None, :] * rt[:, None]) / rt[:, None] * cut[:, None]

    def mlp(self, name, x, penultimate=False):
        net = self.networks[name]
        shape, scale = net["shape"], float(net["activation_scale"])
        for layer in range(len(shape) - 2):
            w = np.asarray(net["weights"][layer], dtype=np.float64).reshape(shape[layer + 1], shape[layer])
            x = _silu_scaled(x @ w.T, scale)
        if penultimate:
            return x
        w = np.asarray(net["weights"][-1], dtype=np.float64).reshape(shape[-1], shape[-2])
        y = x @ w.T
        if net.get("postprocess") == "tanh-square":
            y = np.tanh(y * y)
        return y

    def nodal_derivatives(self, values):
        """values [points, F] -> derivatives [points, F] (compact_radial.cpp:326-366)."""
        P, h = self.points, self.h
        n = P - 2
        lower = np.zeros(n)
        diag = np.full(n, 4.0)
        upper = np.zeros(n)
        rhs = np.zeros((n, values.shape[1]))
        left = 2.0 * (-values[0] + 2.0 * values[1] - values[2]) / h
        upper[0] = 2.0
        rhs[0] = 3.0 * (values[2] - values[0]) / h - left
        for node in range(2, P - 1):
            row = node - 1
            lower[row] = 1.0
            if node + 1 <= P - 2:
                upper[row] = 1.0
            rhs[row] = 3.0 * (values[node + 1] - values[node - 1]) / h
        for row in range(1, n):
            f = lower[row] / diag[row - 1]
            diag[row] -= f * upper[row - 1]
            rhs[row] -= f * rhs[row - 1]
        sol = np.zeros_like(rhs)
        sol[-1] = rhs[-1] / diag[-1]
        for row in range(n - 2, -1, -1):
            sol[row] = (rhs[row] - upper[row] * sol[row + 1]) / diag[row]
        d = np.zeros_like(values)
        d[1:P - 1] = sol
        d[0] = d[2] + left
        d[-1] = 0.0
        return d

    def pair_coefficients(self, name, types):
        """[num_types, num_types, intervals, 4, F]: the table of every species pair (symmetric); without a
        distance transform all pairs share one table."""
        n = len(types)
        if not self.agnesi:
            c = self.coefficients(name)
            return np.broadcast_to(c, (n, n) + c.shape)
        out = None
        for a in range(n):
            for b in range(a, n):
                c = self.coefficients(name, types[a], types[b])
                if out is None:
                    out = np.zeros((n, n) + c.shape)
                out[a, b] = out[b, a] = c
        return out

    def coefficients(self, name, type_i=0, type_j=0):
        """[intervals, 4, F] cubic coefficients of network ``name`` (cubic_spline_set.cpp:8-31)."""
        key = (name, min(type_i, type_j), max(type_i, type_j)) if self.agnesi else (name, 0, 0)
        if key in self._cache:
            return self._cache[key]
        v = self.mlp(name, self.features(type_i, type_j))
        d = self.nodal_derivatives(v)
        h = self.h
        c = np.zeros((self.points - 1, 4, v.shape[1]))
        c[:, 0] = v[:-1]
        c[:, 1] = d[:-1]
        c[:, 2] = (-3 * v[:-1] - 2 * h * d[:-1] + 3 * v[1:] - h * d[1:]) / (h * h)
        c[:, 3] = (2 * v[:-1] + h * d[:-1] - 2 * v[1:] + h * d[1:]) / (h * h * h)
        self._cache[key] = c
        return c


class StoredPairTables:
    """Radial tables of the ``pair-splines`` representation: nodal values and derivatives per unordered element
    pair, read from the file (mace.cpp:2714-2737; density splines 2746-2761, 2884-2897), Hermite form
    cubic_spline_set.cpp:8-31.  Presents the interface of RadialTables with species-pair dependent tables."""

    agnesi = True      # tables depend on the species pair

    def __init__(self, model: dict, num_elements: int, single_layer: bool):
        self.h = float(model["radial_spline_h"])
        self.x0 = float(model.get("radial_spline_min", 0.0))
        self.num_elements = num_elements
        self._tables = {"R0": (model["radial_spline_values_0"], model["radial_spline_derivs_0"])}
        if not single_layer:
            self._tables["R1"] = (model["radial_spline_values_1"], model["radial_spline_derivs_1"])
        for name in ("A0", "A1"):
            if model.get(name + "_scaled", False):
                if float(model[name + "_spline_h"]) != self.h or float(model.get(name + "_spline_min", 0.0)) != self.x0:
                    raise NotImplementedError("density splines on a grid of their own are not restated")
                self._tables[name] = ([[v] for v in model[name + "_spline_values"]], [[d] for d in model[name + "_spline_derivs"]])
        self.points = len(model["radial_spline_values_0"][0][0])
        self._cache = {}

    def _pair(self, type_i, type_j):                                      # mace.cpp:216-229
        a, b = min(type_i, type_j), max(type_i, type_j)
        n = self.num_elements
        return a * (2 * n - a - 1) // 2 + b

    def coefficients(self, name, type_i=0, type_j=0):
        key = (name, self._pair(type_i, type_j))
        if key not in self._cache:
            values, derivs = self._tables[name]
            v = np.asarray(values[key[1]], dtype=np.float64).T                # [node, F]
            d = np.asarray(derivs[key[1]], dtype=np.float64).T
            h = self.h
            c = np.zeros((self.points - 1, 4, v.shape[1]))
            c[:, 0] = v[:-1]
            c[:, 1] = d[:-1]
            c[:, 2] = (-3 * v[:-1] - 2 * h * d[:-1] + 3 * v[1:] - h * d[1:]) / (h * h)
            c[:, 3] = (2 * v[:-1] + h * d[:-1] - 2 * v[1:] + h * d[1:]) / (h * h * h)
            self._cache[key] = c
        return self._cache[key]


def spline_eval(coeff, x0, h, r, dtype=np.float64):
    """Value and derivative of every function at every r (cubic_spline_set.cpp:33-80).

    The evaluation point is formed in ``dtype`` exactly as the templated reference does:
    interval = floor((r-x0)/h), x = r-x0-h*interval, clamped to the table."""
    r = np.asarray(r).astype(dtype)
    x0 = dtype(x0)
    h = dtype(h)
    n_int = coeff.shape[0]
    interval = np.floor((r - x0) / h).astype(np.int64)
    x = (r - x0 - h * interval.astype(dtype)).astype(dtype)
    low = interval < 0
    high = interval >= n_int
    interval = np.clip(interval, 0, n_int - 1)
    x = np.where(low, dtype(0), np.where(high, h, x)).astype(dtype)
    c = coeff.astype(dtype)[interval]  # [E,4,F]
    xx = x * x
    xxx = xx * x
    xe, xxe, xxxe = x[:, None], xx[:, None], xxx[:, None]
    value = c[:, 0] + c[:, 1] * xe + c[:, 2] * xxe + c[:, 3] * xxxe
    deriv = c[:, 1] + dtype(2.0) * c[:, 2] * xe + dtype(3.0) * c[:, 3] * xxe
    return value, deriv


# ----------------------------------------------------------------------------- harmonics
def harmonics(l_max, xyz, dtype=np.float64):
    """Y [E, num_lm] and dY/dxyz [E, 3, num_lm] (mace.cpp:1269-1299).

    The vector is permuted to (z, x, y), orthonormal real harmonics of its direction are
    taken (Y_00 = 0.28209...), everything is scaled by 2*sqrt(pi) and the gradient is
    permuted back.  Each harmonic is a homogeneous polynomial P of degree l of the unit
    vector u, and dY/dX = (grad P(u) - l P(u) u)/|X|."""
    v = np.asarray(xyz, dtype=np.float64).reshape(-1, 3).astype(dtype)
    s = np.stack([v[:, 2], v[:, 0], v[:, 1]], axis=1)
    rr = np.sqrt((s * s).sum(axis=1))
    inv = (dtype(1.0) / rr).astype(dtype)
    x, y, z = s[:, 0] * inv, s[:, 1] * inv, s[:, 2] * inv
    n = len(v)
    size = (l_max + 1) ** 2
    P = np.zeros((n, 16), dtype=dtype)
    G = np.zeros((n, 3, 16), dtype=dtype)  # polynomial gradients w.r.t. (x, y, z) of the permuted frame
    pi = np.pi
    P[:, 0] = 0.5 * np.sqrt(1.0 / pi)
    c1 = dtype(np.sqrt(3.0 / (4.0 * pi)))
    P[:, 1], P[:, 2], P[:, 3] = c1 * y, c1 * z, c1 * x
    G[:, 1, 1] = c1
    G[:, 2, 2] = c1
    G[:, 0, 3] = c1
    a = dtype(0.5 * np.sqrt(15.0 / pi))
    b = dtype(0.25 * np.sqrt(5.0 / pi))
    hh = dtype(0.25 * np.sqrt(15.0 / pi))
    x2, y2, z2 = x * x, y * y, z * z
    P[:, 4] = a * x * y; G[:, 0, 4] = a * y; G[:, 1, 4] = a * x
    P[:, 5] = a * y * z; G[:, 1, 5] = a * z; G[:, 2, 5] = a * y
    P[:, 6] = b * (2 * z2 - x2 - y2); G[:, 0, 6] = -2 * b * x; G[:, 1, 6] = -2 * b * y; G[:, 2, 6] = 4 * b * z
    P[:, 7] = a * x * z; G[:, 0, 7] = a * z; G[:, 2, 7] = a * x
    P[:, 8] = hh * (x2 - y2); G[:, 0, 8] = 2 * hh * x; G[:, 1, 8] = -2 * hh * y
    c = dtype(0.25 * np.sqrt(35.0 / (2.0 * pi)))
    d = dtype(0.5 * np.sqrt(105.0 / pi))
    e = dtype(0.25 * np.sqrt(21.0 / (2.0 * pi)))
    f = dtype(0.25 * np.sqrt(7.0 / pi))
    k = dtype(0.25 * np.sqrt(105.0 / pi))
    q = 4 * z2 - x2 - y2
    P[:, 9] = c * y * (3 * x2 - y2); G[:, 0, 9] = 6 * c * x * y; G[:, 1, 9] = 3 * c * (x2 - y2)
    P[:, 10] = d * x * y * z; G[:, 0, 10] = d * y * z; G[:, 1, 10] = d * x * z; G[:, 2, 10] = d * x * y
    P[:, 11] = e * y * q; G[:, 0, 11] = -2 * e * x * y; G[:, 1, 11] = e * (q - 2 * y2); G[:, 2, 11] = 8 * e * y * z
    P[:, 12] = f * z * (2 * z2 - 3 * x2 - 3 * y2)
    G[:, 0, 12] = -6 * f * x * z; G[:, 1, 12] = -6 * f * y * z; G[:, 2, 12] = f * (6 * z2 - 3 * x2 - 3 * y2)
    P[:, 13] = e * x * q; G[:, 0, 13] = e * (q - 2 * x2); G[:, 1, 13] = -2 * e * x * y; G[:, 2, 13] = 8 * e * x * z
    P[:, 14] = k * z * (x2 - y2); G[:, 0, 14] = 2 * k * x * z; G[:, 1, 14] = -2 * k * y * z; G[:, 2, 14] = k * (x2 - y2)
    P[:, 15] = c * x * (x2 - 3 * y2); G[:, 0, 15] = 3 * c * (x2 - y2); G[:, 1, 15] = -6 * c * x * y
    ldeg = np.array([0] + [1] * 3 + [2] * 5 + [3] * 7, dtype=dtype)
    u = np.stack([x, y, z], axis=1)
    grad = (G - u[:, :, None] * (ldeg[None, None, :] * P[:, None, :])) * inv[:, None, None]
    Y = (P[:, :size] * dtype(TWO_SQRT_PI)).astype(dtype)
    grad = (grad[:, :, :size] * dtype(TWO_SQRT_PI)).astype(dtype)
    # back to the original frame: d/dx <- g[1], d/dy <- g[2], d/dz <- g[0]
    Yg = np.stack([grad[:, 1], grad[:, 2], grad[:, 0]], axis=1)
    return Y, Yg


# ----------------------------------------------------------------------------- polynomial
class Polynomial:
    """Symmetric-contraction polynomial, sum_t w_t prod_{v in monomial t} x_v, with gradient
    (multivariate_polynomial.cpp:322-353, the closed-form pair evaluate_gradient_simple)."""

    def __init__(self, monomials):
        self.monomials = [list(m) for m in monomials]

    def evaluate(self, x, w):
        """x [N, V, C], w [N, T, C] -> value [N, C], gradient [N, V, C]."""
        value = np.zeros((x.shape[0], x.shape[2]), dtype=x.dtype)
        grad = np.zeros_like(x)
        for t, mono in enumerate(self.monomials):
            wt = w[:, t, :]
            prod = np.ones_like(value)
            for v in mono:
                prod = prod * x[:, v, :]
            value += wt * prod
            for j, v in enumerate(mono):
                partial = np.ones_like(value)
                for i, u in enumerate(mono):
                    if i != j:
                        partial = partial * x[:, u, :]
                grad[:, v, :] += wt * partial
        return value, grad


# ----------------------------------------------------------------------------- model
class NumpyMACE:
    """Compact MACE evaluated stage by stage: two interactions or one (single_layer_readout), radial networks or stored
    pair splines, and the three bases of the first readout and the H1 -> H2 skip (h1_affine_schema.hpp:5-30):
    ``m0_composite`` (format 4, scalar block of M0), ``pre_linear_up`` (format 4, M0 P0 + residual) and the old basis of
    formats 1 / 2 (scalar block of H1)."""

    def __init__(self, model, dtype=np.float64):
        if not isinstance(model, dict):
            with open(model) as fh:
                model = json.load(fh)
        m = model
        version = int(m.get("symmetrix_format_version", 1))
        self.basis = "legacy" if version in (1, 2) else m.get("h1_affine_mode")
        if self.basis not in ("legacy", "m0_composite", "pre_linear_up"):
            raise NotImplementedError("unknown h1 affine basis")
        radial = m.get("radial_representation", "pair-splines" if version == 1 else "")
        if radial not in ("compact", "pair-splines"):
            raise NotImplementedError("unknown radial representation")
        if m.get("has_field_coupling"):
            raise NotImplementedError("field coupling is not restated")
        self.single_layer = bool(m.get("single_layer_readout", False))
        self.residual = bool(m.get("first_interaction_residual", False))
        self.has_zbl = bool(m.get("has_zbl", False))
        if self.has_zbl:                                                 # mace.cpp:2690-2699
            self.zbl_a_exp, self.zbl_a_prefactor = float(m["zbl_a_exp"]), float(m["zbl_a_prefactor"])
            self.zbl_c = np.asarray(m["zbl_c"], dtype=np.float64)
            self.zbl_radii = np.asarray(m["zbl_covalent_radii"], dtype=np.float64)
            self.zbl_p = int(m["zbl_p"])
        self.atomic_numbers = np.asarray(m["atomic_numbers"], dtype=np.int64)
        self.dtype = dtype
        dt = dtype
        self.C = C = int(m["num_channels"])
        self.l_max, self.L_max = int(m["l_max"]), int(m["L_max"])
        self.num_lm, self.num_LM = (self.l_max + 1) ** 2, (self.L_max + 1) ** 2
        self.r_cut = float(m["r_cut"])
        self.A = A = int(m["num_elements"])
        self.atomic_energies = np.asarray(m["atomic_energies"], dtype=np.float64)
        self.tables = (RadialTables(m["compact_radial"], self.r_cut) if radial == "compact"
                       else StoredPairTables(m, A, self.single_layer))
        self.A0_scaled, self.A1_scaled = bool(m["A0_scaled"]), bool(m.get("A1_scaled", False))
        self.H0 = np.asarray(m["H0_weights"], dtype=dt).reshape(A, C)
        self.WA0 = np.asarray(m["A0_weights"], dtype=dt).reshape(A, self.l_max + 1, C, C)
        self.P0 = [Polynomial(m["M0_monomials"][str(lm)]) for lm in range(self.num_LM)]
        self.W0 = [np.asarray([[m["M0_weights"][str(a)][str(lm)][str(k)] for k in range(C)] for a in range(A)],
                              dtype=dt).transpose(0, 2, 1) for lm in range(self.num_LM)]  # [A, T, C]
        self.P1 = Polynomial(m["M1_monomials"])
        self.W1 = np.asarray([[m["M1_weights"][str(a)][str(k)] for k in range(C)] for a in range(A)],
                             dtype=dt).transpose(0, 2, 1)
        self.WH1 = np.asarray(m["H1_weights"], dtype=dt).reshape(self.L_max + 1, C, C)
        self.Phi1_l = list(m.get("Phi1_l", [])); self.Phi1_l1 = list(m.get("Phi1_l1", [])); self.Phi1_l2 = list(m.get("Phi1_l2", []))
        self.t_lme = np.asarray(m.get("Phi1_lme", [])); self.t_row = np.asarray(m.get("Phi1_lelm1lm2", []))
        self.t_cg = np.asarray(m.get("Phi1_clebsch_gordan", []), dtype=dt)
        self.num_lme = sum(2 * l + 1 for l in self.Phi1_l)
        self.eta = [sum(1 for l in self.Phi1_l if l == ll) for ll in range(self.l_max + 1)]
        if not self.single_layer:
            self.WA1 = [np.asarray(m["A1_weights"][l], dtype=dt).reshape(self.eta[l] * C, C) for l in range(self.l_max + 1)]
        # first readout q and skip T act on the basis' scalar input (keys: h1_affine_schema.hpp:62-74)
        skip_key = {"legacy": "H2_weights_for_H1", "m0_composite": "H2_weights_for_M0",
                    "pre_linear_up": "H2_weights_for_H1_pre_linear_up"}[self.basis]
        readout_key = {"legacy": "readout_1_weights", "m0_composite": "readout_1_weights_for_M0",
                       "pre_linear_up": "readout_1_weights_for_H1_pre_linear_up"}[self.basis]
        self.T = np.asarray(m[skip_key], dtype=dt).reshape(A, C, C)
        self.WM1 = np.asarray(m["H2_weights_for_M1"], dtype=dt).reshape(C, C)
        self.q = np.asarray(m[readout_key], dtype=dt)
        if self.basis == "pre_linear_up":                                # mace.cpp:1773-1778
            self.P0w = np.asarray(m["H1_product_weights"], dtype=dt).reshape(self.L_max + 1, C, C)[0]
        if self.residual:                                                # mace.cpp:2801-2829, 1845-1882
            R = np.asarray(m["H1_first_residual_weights"], dtype=dt).reshape(A, self.num_LM, C)
            U = np.asarray(m["H1_linear_up_weights"], dtype=dt).reshape(self.L_max + 1, C, C)
            L_of = np.array([int(np.floor(np.sqrt(lm + 0.5))) for lm in range(self.num_LM)])
            self.R_scalar = R[:, 0, :]
            self.R_fused = np.einsum("amk,mkj->amj", R, U[L_of])
        hid = int(m.get("readout_2_hidden_size", 16))
        self.V1 = np.asarray(m["readout_2_weights_1"], dtype=dt).reshape(hid, C)
        self.V2 = np.asarray(m["readout_2_weights_2"], dtype=dt).reshape(1, hid)
        self.act = dt(m["readout_2_scale_factor"])
        # rows: for path: for lm1: for lm2 (mace.cpp:2046-2064)
        rows = []
        for p, (l1, l2) in enumerate(zip(self.Phi1_l1, self.Phi1_l2)):
            for lm1 in range(l1 * l1, (l1 + 1) ** 2):
                for lm2 in range(l2 * l2, (l2 + 1) ** 2):
                    rows.append((p, lm1, lm2))
        self.rows = np.asarray(rows)
        self.stage = {}

    # -- forward + reverse ------------------------------------------------------------------
    def compute(self, node_types, first_neigh, sources, xyz, skip_beyond_cutoff=False):
        """Per-node energies and per-edge forces dE/d(xyz_ij) with the reference's sign
        (mace.cpp:232-319).  ``skip_beyond_cutoff`` drops edges with r >= r_cut the way the
        device kernels of the reference do (jit_codegen.py ``edge_is_active``)."""
        dt = self.dtype
        C, nlm, nLM = self.C, self.num_lm, self.num_LM
        typ = np.asarray(node_types)
        first = np.asarray(first_neigh)
        src = np.asarray(sources)
        N = len(typ)
        xyz = np.asarray(xyz, dtype=np.float64).reshape(-1, 3)
        recv = np.repeat(np.arange(N), np.diff(first))
        r = np.sqrt((xyz * xyz).sum(axis=1))
        active = (r < self.r_cut) if skip_beyond_cutoff else np.ones(len(r), dtype=bool)
        E = len(src)
        direction = (xyz / r[:, None]).astype(dt)                      # mace.cpp:2240-2242
        Y, Yg = harmonics(self.l_max, xyz, dt)                          # mace.cpp:1269-1299
        tj = typ[src]
        R0, dR0 = self._radial("R0", typ[recv], tj, r)                   # mace.cpp:1119-1144
        act = active[:, None].astype(dt)
        R0, dR0 = R0 * act, dR0 * act
        if not self.single_layer:
            R1, dR1 = self._radial("R1", typ[recv], tj, r)
            R1, dR1 = R1 * act, dR1 * act
        l_of_lm = np.array([int(np.floor(np.sqrt(lm + 0.5))) for lm in range(nlm)])
        tj = typ[src]

        # A0 (mace.cpp:1356-1403): Phi0 then the per-l channel mixing with W[type_i][l]
        R0e = R0.reshape(E, self.l_max + 1, C)[:, l_of_lm, :]            # [E, lm, C]
        msg0 = R0e * Y[:, :, None] * self.H0[tj][:, None, :]
        Phi0 = np.zeros((N, nlm, C), dtype=dt)
        np.add.at(Phi0, recv, msg0)
        Wl = self.WA0[typ][:, l_of_lm]                                   # [N, lm, C, C]
        A0 = np.einsum("nmk,nmkj->nmj", Phi0, Wl)
        scale0 = None
        if self.A0_scaled:                                               # mace.cpp:1562-1584
            s, ds = self._radial("A0", typ[recv], tj, r)
            scale0 = np.ones(N, dtype=dt)
            np.add.at(scale0, recv, s[:, 0])
            A0 = A0 / scale0[:, None, None]
        # M0 (mace.cpp:1639-1662)
        M0 = np.zeros((N, nLM, C), dtype=dt)
        M0g = np.zeros((N, nLM, nlm, C), dtype=dt)
        for lm in range(nLM):
            M0[:, lm], M0g[:, lm] = self.P0[lm].evaluate(A0, self.W0[lm][typ])
        L_of_LM = np.array([int(np.floor(np.sqrt(lm + 0.5))) for lm in range(nLM)])
        H1 = np.einsum("nmk,mkj->nmj", M0, self.WH1[L_of_LM])           # mace.cpp:1691-1724
        if self.residual:                                                # mace.cpp:1845-1861: H1 += R U of the node's element
            H1 = H1 + self.R_fused[typ]
        # scalar input of the first readout and the skip (mace.cpp:1759-1782, 1863-1873; old basis 2524-2525)
        if self.basis == "m0_composite":
            xs = M0[:, 0, :].copy()
        elif self.basis == "pre_linear_up":
            xs = M0[:, 0, :] @ self.P0w
            if self.residual:
                xs = xs + self.R_scalar[typ]
        else:
            xs = H1[:, 0, :].copy()
        if self.single_layer:
            return self._finish_single_layer(typ, recv, tj, r, direction, Y, Yg, R0, dR0, A0, scale0,
                                             ds if self.A0_scaled else None, M0, M0g, H1, xs, Wl, l_of_lm, L_of_LM)
        # Phi1 (mace.cpp:2023-2083)
        p_of_row, lm1_of_row, lm2_of_row = self.rows[:, 0], self.rows[:, 1], self.rows[:, 2]
        R1e = R1.reshape(E, len(self.Phi1_l), C)
        Hj = H1[src]                                                     # [E, LM, C]
        msg1 = R1e[:, p_of_row, :] * Y[:, lm1_of_row, None] * Hj[:, lm2_of_row, :]
        Phi1r = np.zeros((N, len(self.rows), C), dtype=dt)
        np.add.at(Phi1r, recv, msg1)
        Phi1 = np.zeros((N, self.num_lme, C), dtype=dt)
        for t in range(len(self.t_cg)):
            Phi1[:, self.t_lme[t]] += self.t_cg[t] * Phi1r[:, self.t_row[t]]
        # A1 (mace.cpp:2305-2340)
        A1 = np.zeros((N, nlm, C), dtype=dt)
        off = 0
        for l in range(self.l_max + 1):
            nm, ne = 2 * l + 1, self.eta[l]
            blk = Phi1[:, off:off + nm * ne].reshape(N, nm, ne * C)
            A1[:, l * l:l * l + nm] = blk @ self.WA1[l]
            off += nm * ne
        scale1 = None
        if self.A1_scaled:
            s1, ds1 = self._radial("A1", typ[recv], tj, r)
            scale1 = np.ones(N, dtype=dt)
            np.add.at(scale1, recv, s1[:, 0])
            A1 = A1 / scale1[:, None, None]
        M1, M1g = self.P1.evaluate(A1, self.W1[typ])                     # mace.cpp:2461-2484
        H2, H2_adj, energies, direct = self._readouts(typ, xs, M1)
        # reverse (mace.cpp:298-318)
        M1_adj = H2_adj @ self.WM1.T
        A1_adj = M1g * M1_adj[:, None, :]                                 # mace.cpp:2487-2513
        forces = np.zeros((E, 3), dtype=dt)
        if self.A1_scaled:                                               # mace.cpp:2406-2458
            dot = (A1_adj * A1).sum(axis=(1, 2))
            fs = (dot / scale1)[recv] * ds1[:, 0]
            forces += fs[:, None] * direction
            A1_adj = A1_adj / scale1[:, None, None]
        dPhi1 = np.zeros_like(Phi1)                                      # mace.cpp:2343-2378
        off = 0
        for l in range(self.l_max + 1):
            nm, ne = 2 * l + 1, self.eta[l]
            dPhi1[:, off:off + nm * ne] = (A1_adj[:, l * l:l * l + nm] @ self.WA1[l].T).reshape(N, nm * ne, C)
            off += nm * ne
        dPhi1r = np.zeros_like(Phi1r)                                    # mace.cpp:2211-2222
        for t in range(len(self.t_cg)):
            dPhi1r[:, self.t_row[t]] += self.t_cg[t] * dPhi1[:, self.t_lme[t]]
        adj = dPhi1r[recv]                                               # [E, rows, C]
        dR1e = dR1.reshape(E, len(self.Phi1_l), C)
        Hrow = Hj[:, lm2_of_row, :]
        radial = (adj * dR1e[:, p_of_row, :] * Y[:, lm1_of_row, None] * Hrow).sum(axis=(1, 2))
        ang = (adj * R1e[:, p_of_row, :] * Hrow).sum(axis=2)             # [E, rows]
        forces -= radial[:, None] * direction + np.einsum("er,edr->ed", ang, Yg[:, :, lm1_of_row])  # mace.cpp:2273-2296
        H1_adj = np.zeros_like(H1)
        contrib = adj * R1e[:, p_of_row, :] * Y[:, lm1_of_row, None]     # [E, rows, C]
        msg = np.zeros((E, nLM, C), dtype=dt)
        for row in range(len(self.rows)):
            msg[:, lm2_of_row[row]] += contrib[:, row]
        np.add.at(H1_adj, src, msg)
        if self.basis == "legacy":                                       # old basis: q and the skip's adjoint join H1_adj (mace.cpp:2588-2601, 2645-2646)
            H1_adj[:, 0, :] += direct
        M0_adj, A0_adj = self._reverse_layer0(typ, recv, tj, r, direction, Y, Yg, R0, dR0, A0, scale0,
                                              ds if self.A0_scaled else None, M0g, H1_adj, direct, Wl, l_of_lm, L_of_LM,
                                              energies, forces)
        self.stage = dict(Y=Y, Y_grad=Yg, A0=A0, M0=M0, H1=H1, Phi1=Phi1, A1=A1, M1=M1, H2=H2,
                          H2_adj=H2_adj, A1_adj=A1_adj, dPhi1=dPhi1, H1_adj=H1_adj, M0_adj=M0_adj,
                          A0_adj=A0_adj, node_energies=energies, node_forces=forces)
        return energies, forces

    def _readouts(self, typ, xs, M1):
        """H2, node energies and the adjoints leaving the readouts (mace.cpp:2516-2557, 2622-2657)."""
        H2 = np.einsum("nk,nkj->nj", xs, self.T[typ]) + M1 @ self.WM1
        z = H2 @ self.V1.T
        sig = 1.0 / (1.0 + np.exp(-z))
        hidden = self.act * z * sig
        e2 = (hidden @ self.V2.T)[:, 0]
        energies = self.atomic_energies[typ] + (xs @ self.q).astype(np.float64) + e2.astype(np.float64)
        dact = self.act * sig + self.act * z * sig * (1 - sig)
        H2_adj = (self.V2[0][None, :] * dact) @ self.V1
        direct = self.q[None, :] + np.einsum("nkj,nj->nk", self.T[typ], H2_adj)   # mace.cpp:2568-2580
        return H2, H2_adj, energies, direct

    def _reverse_layer0(self, typ, recv, tj, r, direction, Y, Yg, R0, dR0, A0, scale0, ds, M0g, H1_adj, direct, Wl, l_of_lm,
                        L_of_LM, energies, forces):
        """From H1_adj down to the edge forces of layer 0, plus the pair repulsion (mace.cpp:304-318); ``forces`` and
        ``energies`` are updated in place."""
        dt = self.dtype
        E, C = len(r), self.C
        M0_adj = np.einsum("nmj,mkj->nmk", H1_adj, self.WH1[L_of_LM])   # mace.cpp:1727-1757
        if self.basis == "m0_composite":
            M0_adj[:, 0, :] += direct                                    # mace.cpp:1785-1813
        elif self.basis == "pre_linear_up":
            M0_adj[:, 0, :] += direct @ self.P0w.T                       # mace.cpp:1799-1806
        A0_adj = np.einsum("nLmk,nLk->nmk", M0g, M0_adj)                 # mace.cpp:1665-1688
        if self.A0_scaled:                                               # mace.cpp:1587-1636
            dot = (A0_adj * A0).sum(axis=(1, 2))
            fs = (dot / scale0)[recv] * ds[:, 0]
            forces += fs[:, None] * direction
            A0_adj = A0_adj / scale0[:, None, None]
        Phi0_adj = np.einsum("nmj,nmkj->nmk", A0_adj, Wl)                # mace.cpp:1486-1503
        padj = Phi0_adj[recv]
        R0e = R0.reshape(E, self.l_max + 1, C)[:, l_of_lm, :]
        dR0e = dR0.reshape(E, self.l_max + 1, C)[:, l_of_lm, :]
        h0 = self.H0[tj][:, None, :]
        radial0 = (padj * dR0e * Y[:, :, None] * h0).sum(axis=(1, 2))
        ang0 = (padj * R0e * h0).sum(axis=2)
        forces -= radial0[:, None] * direction + np.einsum("em,edm->ed", ang0, Yg)   # mace.cpp:1505-1559
        if self.has_zbl:                                                 # zbl.cpp:24-139, called at mace.cpp:247-250
            ez, gz = self.zbl_pair(self.atomic_numbers[typ][recv], self.atomic_numbers[tj], r.astype(dt))
            np.add.at(energies, recv, ez.astype(np.float64))
            forces -= direction * gz[:, None].astype(dt)
        return M0_adj, A0_adj

    def _finish_single_layer(self, typ, recv, tj, r, direction, Y, Yg, R0, dR0, A0, scale0, ds, M0, M0g, H1, xs, Wl, l_of_lm,
                             L_of_LM):
        """One interaction: the readout polynomial acts on H1 and there is no second message step
        (mace.cpp:265-283; polynomial input 2465-2466, its adjoint adds to H1_adj 2499-2510)."""
        dt = self.dtype
        M1, M1g = self.P1.evaluate(H1, self.W1[typ])
        H2, H2_adj, energies, direct = self._readouts(typ, xs, M1)
        M1_adj = H2_adj @ self.WM1.T
        H1_adj = M1g * M1_adj[:, None, :]
        if self.basis == "legacy":
            # the serial evaluator clears H1_adj after the readouts on this path (mace.cpp:269), so the first readout's
            # own adjoint q does not reach the forces; exported single-layer files carry q = 0
            H1_adj[:, 0, :] += direct - self.q[None, :]
        forces = np.zeros((len(r), 3), dtype=dt)
        M0_adj, A0_adj = self._reverse_layer0(typ, recv, tj, r, direction, Y, Yg, R0, dR0, A0, scale0, ds, M0g, H1_adj, direct,
                                              Wl, l_of_lm, L_of_LM, energies, forces)
        self.stage = dict(Y=Y, Y_grad=Yg, A0=A0, M0=M0, H1=H1, M1=M1, H2=H2, H2_adj=H2_adj, H1_adj=H1_adj, M0_adj=M0_adj,
                          A0_adj=A0_adj, node_energies=energies, node_forces=forces)
        return energies, forces

    def _radial(self, name, type_i, type_j, r):
        """Spline values and derivatives [E, F] of network ``name`` at the edge lengths, with the table of
        each edge's species pair (mace.cpp:216-229 pair index, 1119-1144 evaluation)."""
        dt = self.dtype
        if not self.tables.agnesi:
            return spline_eval(self.tables.coefficients(name).astype(dt), self.tables.x0, self.tables.h, r, dt)
        value = deriv = None
        lo, hi = np.minimum(type_i, type_j), np.maximum(type_i, type_j)
        for a, b in sorted(set(zip(lo.tolist(), hi.tolist()))):
            mask = (lo == a) & (hi == b)
            v, d = spline_eval(self.tables.coefficients(name, a, b).astype(dt), self.tables.x0, self.tables.h, r[mask], dt)
            if value is None:
                value = np.zeros((len(r), v.shape[1]), dtype=v.dtype)
                deriv = np.zeros_like(value)
            value[mask], deriv[mask] = v, d
        return value, deriv

    def zbl_pair(self, Zu, Zv, r):
        """Screened-Coulomb pair energy (half per directed edge) and its radial derivative with the
        polynomial envelope (zbl.cpp:24-99)."""
        dt = r.dtype
        c_exps = np.array([-3.2, -0.9423, -0.4028, -0.2016], dtype=dt)      # zbl.hpp:47-50
        v_pref = dt.type(14.3996)                                            # zbl.hpp:51
        Zu_f, Zv_f = Zu.astype(dt), Zv.astype(dt)
        a = dt.type(self.zbl_a_prefactor) * dt.type(0.529) / (Zu_f ** dt.type(self.zbl_a_exp) + Zv_f ** dt.type(self.zbl_a_exp))
        x = r / a
        e = self.zbl_c.astype(dt)[None, :] * np.exp(c_exps[None, :] * x[:, None])
        phi = e.sum(axis=1)
        dphi = (e * c_exps[None, :]).sum(axis=1) / a
        v = v_pref * Zu_f * Zv_f / r * phi
        dv = v_pref * Zu_f * Zv_f * (r * dphi - phi) / (r * r)
        r_max = (self.zbl_radii[Zu] + self.zbl_radii[Zv]).astype(dt)
        p = self.zbl_p
        u = r / r_max
        inside = r < r_max
        env = np.where(inside, 1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * u ** p + p * (p + 2.0) * u ** (p + 1)
                       - (p * (p + 1.0) / 2.0) * u ** (p + 2), 0.0).astype(dt)
        denv = np.where(inside, (-((p + 1.0) * (p + 2.0) / 2.0) * p * u ** (p - 1) + p * (p + 2.0) * (p + 1.0) * u ** p
                                 - (p * (p + 1.0) / 2.0) * (p + 2.0) * u ** (p + 1)) / r_max, 0.0).astype(dt)
        return dt.type(0.5) * v * env, dt.type(0.5) * (v * denv + dv * env)

    def energy_forces_stress(self, node_types, positions, cell, first_neigh, sources, shifts,
                             skip_beyond_cutoff=True):
        """Total energy, atom forces [N,3] and stress [3,3] from positions and a shifted CSR graph.
        Force and stress reduction: mace_kokkos_evaluate.cpp:92-106, 157-186."""
        pos = np.asarray(positions, dtype=np.float64).reshape(-1, 3)
        cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        first = np.asarray(first_neigh)
        recv = np.repeat(np.arange(len(pos)), np.diff(first))
        xyz = pos[sources] - pos[recv] + np.asarray(shifts, dtype=np.float64) @ cell
        e, f = self.compute(node_types, first, sources, xyz, skip_beyond_cutoff)
        f = f.astype(np.float64)
        F = np.zeros((len(pos), 3))
        np.add.at(F, np.asarray(sources), f)
        np.add.at(F, recv, -f)
        stress = -(f[:, :, None] * xyz[:, None, :]).sum(axis=0) / abs(np.linalg.det(cell))
        return float(e.sum()), e, F, stress
