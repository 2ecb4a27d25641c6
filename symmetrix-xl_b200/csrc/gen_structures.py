"""Emits csrc/generated/structures.h: the coupling structure of each supported model
shape as X-macro lists, so that the CUDA kernels expand into straight-line code with
every row, coupling term and monomial index a compile-time constant.

Run from the repository root:  python symmetrix-xl_b200/csrc/gen_structures.py
The tables come from symmetrix-xl_b200/structure.py (first-principles derivation) plus
the extra zero-weight monomials modelgen.model_tables adds for the (3,1) shape.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
PKG = ROOT / "symmetrix-xl_b200"


def _load_pkg():
    spec = importlib.util.spec_from_file_location(
        "symmetrix_xl_b200", PKG / "__init__.py", submodule_search_locations=[str(PKG)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["symmetrix_xl_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


# (name, edge l_max, hidden L_max, number of path sets of the split layer-1 kernels, optional explicit sets)
# S2: set 0 = all paths with source l = 0 or 1 (88 rows, 4 source components), sets 1 and 2 share the
# source l = 2 paths (80 and 75 rows, 5 source components each)
SHAPES = [("S0", 3, 0, 1, None), ("S1", 3, 1, 1, None),
          ("S2", 3, 2, 3, [[0, 3, 8, 13, 1, 4, 5, 9, 10, 14], [7, 2, 6, 11], [16, 12, 15]])]


def reverse_path_lines(p, q, l, l1, l2, base):
    """Straight-line gradient code of one path for one (edge, channel): q = index of the path's radial
    function in R[] / dR[], base = first row adjoint of the path in adj[].  With w_a = sum_b h_b adj_ab and
    s_b = sum_a y_a adj_ab the path contributes
      ang_a += R w_a   (angular part of the force),   hadj_b += R s_b   (source adjoint),
      radial += dR * sum_a y_a w_a,   and   sum_a y_a w_a = sum_b h_b s_b.
    The radial sum runs over the shorter index set, and R is folded into that set's vector first, so
    that the other contraction accumulates straight into its target."""
    n1, n2 = 2 * l1 + 1, 2 * l2 + 1
    out = [f"    {{ /* path {p}: edge l={l1}, source l={l2} -> l={l} */"]
    out.append("      float yw = 0.0f;")
    if n2 < n1:
        for b in range(n2):
            out.append(f"      const float rh{b} = R[{q}] * h[{l2 * l2 + b}];")
        for a in range(n1):
            for b in range(n2):
                out.append(f"      ang[{l1 * l1 + a}] = fmaf(rh{b}, adj[{base + a * n2 + b}], ang[{l1 * l1 + a}]);")
        for b in range(n2):
            terms_ = [(f"y[{l1 * l1 + a}]", f"adj[{base + a * n2 + b}]") for a in range(n1)]
            expr = f"{terms_[0][0]} * {terms_[0][1]}"
            for yy, aa in terms_[1:]:
                expr = f"fmaf({yy}, {aa}, {expr})"
            out.append(f"      {{ const float s_ = {expr};")
            out.append(f"        hadj[{l2 * l2 + b}] = fmaf(R[{q}], s_, hadj[{l2 * l2 + b}]); yw = fmaf(h[{l2 * l2 + b}], s_, yw); }}")
    else:
        for a in range(n1):
            out.append(f"      const float ry{a} = R[{q}] * y[{l1 * l1 + a}];")
        for a in range(n1):
            terms_ = [(f"h[{l2 * l2 + b}]", f"adj[{base + a * n2 + b}]") for b in range(n2)]
            expr = f"{terms_[0][0]} * {terms_[0][1]}"
            for hh, aa in terms_[1:]:
                expr = f"fmaf({hh}, {aa}, {expr})"
            out.append(f"      {{ const float w = {expr};")
            out.append(f"        ang[{l1 * l1 + a}] = fmaf(R[{q}], w, ang[{l1 * l1 + a}]); yw = fmaf(y[{l1 * l1 + a}], w, yw); }}")
        for b in range(n2):
            for a in range(n1):
                out.append(f"      hadj[{l2 * l2 + b}] = fmaf(ry{a}, adj[{base + a * n2 + b}], hadj[{l2 * l2 + b}]);")
    out.append(f"      radial = fmaf(dR[{q}], yw, radial);")
    out.append("    }")
    return out


def emit_shape(name, l_max, L_max, tables, groups=1, by_edge_l=None):
    out = []
    paths = list(zip(tables["Phi1_l"], tables["Phi1_l1"], tables["Phi1_l2"]))
    num_lm, num_LM = (l_max + 1) ** 2, (L_max + 1) ** 2
    rows = []
    row_begin = []
    for p, (l, l1, l2) in enumerate(paths):
        row_begin.append(len(rows))
        for lm1 in range(l1 * l1, (l1 + 1) ** 2):
            for lm2 in range(l2 * l2, (l2 + 1) ** 2):
                rows.append((p, lm1, lm2))
    out.append(f"// ---- shape {name}: edge l_max={l_max}, hidden L_max={L_max}")
    out.append(f"#define SXB_{name}_LMAX {l_max}")
    out.append(f"#define SXB_{name}_HIDDEN_LMAX {L_max}")
    out.append(f"#define SXB_{name}_NUM_LM {num_lm}")
    out.append(f"#define SXB_{name}_NUM_HIDDEN {num_LM}")
    out.append(f"#define SXB_{name}_NUM_PATHS {len(paths)}")
    out.append(f"#define SXB_{name}_NUM_ROWS {len(rows)}")
    out.append(f"#define SXB_{name}_NUM_LME {tables['num_lme']}")
    out.append(f"#define SXB_{name}_NUM_TERMS {len(tables['Phi1_lme'])}")
    out.append(f"// X(path, l_out, l_edge, l_source, first_row)")
    out.append(f"#define SXB_{name}_PATHS(X) \\")
    out.append(" \\\n".join(f"    X({p}, {l}, {l1}, {l2}, {row_begin[p]})" for p, (l, l1, l2) in enumerate(paths)))
    out.append(f"// X(row, path, lm_edge, lm_source)")
    out.append(f"#define SXB_{name}_ROWS(X) \\")
    out.append(" \\\n".join(f"    X({r}, {p}, {lm1}, {lm2})" for r, (p, lm1, lm2) in enumerate(rows)))
    out.append(f"// X(term, row, lme): coefficient values live in constant memory, indexed by term")
    out.append(f"#define SXB_{name}_TERMS(X) \\")
    out.append(" \\\n".join(f"    X({t}, {row}, {lme})" for t, (row, lme) in
                            enumerate(zip(tables["Phi1_lelm1lm2"], tables["Phi1_lme"]))))
    out.append(f"// this library's own derivation of the coupling coefficients, by term (a model file carries its own)")
    out.append(f"#define SXB_{name}_DEFAULT_CG {{" + ", ".join(f"{float(v)!r}f" for v in tables["Phi1_clebsch_gordan"]) + "}")
    # symmetric contraction: weights laid out [type][term][channel], term = offset(LM) + index
    offset = 0
    lines1, lines2, lines3 = [], [], []
    offs = []
    for LM in range(num_LM):
        mons = tables["M0_monomials"][str(LM)]
        offs.append(offset)
        for t, mono in enumerate(mons):
            if len(mono) == 1:
                lines1.append(f"    X1({LM}, {offset + t}, {mono[0]})")
            elif len(mono) == 2:
                lines2.append(f"    X2({LM}, {offset + t}, {mono[0]}, {mono[1]})")
            else:
                lines3.append(f"    X3({LM}, {offset + t}, {mono[0]}, {mono[1]}, {mono[2]})")
        offset += len(mons)
    out.append(f"#define SXB_{name}_M0_NUM_TERMS {offset}")
    out.append(f"#define SXB_{name}_M0_OFFSETS {{{', '.join(map(str, offs + [offset]))}}}")
    out.append(f"// X1(out, term, a)  X2(out, term, a, b)  X3(out, term, a, b, c)")
    out.append(f"#define SXB_{name}_M0_TERMS(X1, X2, X3) \\")
    out.append(" \\\n".join(lines1 + lines2 + lines3))
    m1 = tables["M1_monomials"]
    out.append(f"#define SXB_{name}_M1_NUM_TERMS {len(m1)}")
    l1_, l2_, l3_ = [], [], []
    for t, mono in enumerate(m1):
        if len(mono) == 1:
            l1_.append(f"    X1(0, {t}, {mono[0]})")
        elif len(mono) == 2:
            l2_.append(f"    X2(0, {t}, {mono[0]}, {mono[1]})")
        else:
            l3_.append(f"    X3(0, {t}, {mono[0]}, {mono[1]}, {mono[2]})")
    out.append(f"#define SXB_{name}_M1_TERMS(X1, X2, X3) \\")
    out.append(" \\\n".join(l1_ + l2_ + l3_))
    # straight-line bodies of the layer-1 edge kernels (one channel per thread):
    #   R[p], dR[p]: radial value / derivative of path p;  y[lm]: edge harmonics;
    #   h[lm2]: source features;  acc[row] / adj[row]: receiver row sums / row adjoints
    fwd, rev = [], []
    for p, (l, l1, l2) in enumerate(paths):
        n1, n2 = 2 * l1 + 1, 2 * l2 + 1
        fwd.append(f"    {{ /* path {p}: edge l={l1}, source l={l2} -> l={l} */")
        for b in range(n2):
            fwd.append(f"      const float t{b} = R[{p}] * h[{l2 * l2 + b}];")
        for a in range(n1):
            for b in range(n2):
                row = row_begin[p] + a * n2 + b
                fwd.append(f"      acc[{row}] = fmaf(t{b}, y[{l1 * l1 + a}], acc[{row}]);")
        fwd.append("    }")
        rev.extend(reverse_path_lines(p, p, l, l1, l2, row_begin[p]))
    out.append(f"#define SXB_{name}_L1_FORWARD_BODY \\")
    out.append(" \\\n".join(fwd))
    out.append(f"#define SXB_{name}_L1_REVERSE_BODY \\")
    out.append(" \\\n".join(rev))
    if groups > 1:
        out.extend(emit_path_groups(name, paths, row_begin, tables, groups, by_edge_l))
    out.append("")
    return "\n".join(out)


def emit_path_groups(name, paths, row_begin, tables, groups, by_edge_l=None):
    """Splits the paths of a shape into `groups` sets with balanced row counts and emits, per set,
    the same straight-line bodies with rows, paths and outputs renumbered inside the set.  Every
    output component (lme) is fed by exactly one path, so the sets write disjoint outputs; a kernel
    instance that handles one set needs only that set's row accumulators in registers."""
    sizes = [(2 * l1 + 1) * (2 * l2 + 1) for (_, l1, l2) in paths]
    members = [[] for _ in range(groups)]
    load = [0] * groups
    if by_edge_l is not None:
        # explicit sets (lists of path indices), chosen so that a set touches few source components:
        # a set loads and atomically updates only the source components of its own paths
        assert sorted(p for group in by_edge_l for p in group) == list(range(len(paths)))
        members = [list(group) for group in by_edge_l]
    else:
        for p in sorted(range(len(paths)), key=lambda q: -sizes[q]):      # largest first, to the lightest set
            g = min(range(groups), key=lambda q: load[q])
            members[g].append(p)
            load[g] += sizes[p]
    row_path = []
    for p, n in enumerate(sizes):
        row_path += [p] * n
    lme_path = {}
    for row, lme in zip(tables["Phi1_lelm1lm2"], tables["Phi1_lme"]):
        assert lme_path.setdefault(lme, row_path[row]) == row_path[row]
    out = [f"#define SXB_{name}_NUM_GROUPS {groups}"]
    for g, plist in enumerate(members):
        plist = sorted(plist)
        local_row, rows_g = {}, 0
        for p in plist:
            for r in range(sizes[p]):
                local_row[row_begin[p] + r] = rows_g
                rows_g += 1
        lmes = sorted(lme for lme, p in lme_path.items() if p in plist)
        local_lme = {lme: i for i, lme in enumerate(lmes)}
        hmask, emask = 0, 0
        for p in plist:
            l1, l2 = paths[p][1], paths[p][2]
            for b in range(l2 * l2, (l2 + 1) ** 2):
                hmask |= 1 << b
            for a in range(l1 * l1, (l1 + 1) ** 2):
                emask |= 1 << a
        pre = f"SXB_{name}_G{g}"
        out.append(f"#define {pre}_NUM_PATHS {len(plist)}")
        out.append(f"#define {pre}_NUM_ROWS {rows_g}")
        out.append(f"#define {pre}_NUM_LME {len(lmes)}")
        out.append(f"#define {pre}_PATH_LIST {{{', '.join(map(str, plist))}}}")
        out.append(f"#define {pre}_LME_LIST {{{', '.join(map(str, lmes))}}}")
        out.append(f"#define {pre}_SOURCE_MASK {hmask}u   // source components lm2 the set touches")
        out.append(f"#define {pre}_EDGE_MASK {emask}u   // edge harmonics lm1 the set touches")
        out.append(f"#define {pre}_HAS_PATH0 {1 if 0 in plist else 0}")
        out.append(f"// X(term, row inside the set, output inside the set)")
        out.append(f"#define {pre}_TERMS(X) \\")
        out.append(" \\\n".join(f"    X({t}, {local_row[row]}, {local_lme[lme]})" for t, (row, lme) in
                                enumerate(zip(tables["Phi1_lelm1lm2"], tables["Phi1_lme"])) if row in local_row))
        fwd, rev = [], []
        for q, p in enumerate(plist):
            l, l1, l2 = paths[p]
            n1, n2 = 2 * l1 + 1, 2 * l2 + 1
            base = local_row[row_begin[p]]
            fwd.append(f"    {{ /* path {p}: edge l={l1}, source l={l2} -> l={l} */")
            for b in range(n2):
                fwd.append(f"      const float t{b} = R[{q}] * h[{l2 * l2 + b}];")
            for a in range(n1):
                for b in range(n2):
                    row = base + a * n2 + b
                    fwd.append(f"      acc[{row}] = fmaf(t{b}, y[{l1 * l1 + a}], acc[{row}]);")
            fwd.append("    }")
            rev.extend(reverse_path_lines(p, q, l, l1, l2, base))
        out.append(f"#define {pre}_FORWARD_BODY \\")
        out.append(" \\\n".join(fwd))
        out.append(f"#define {pre}_REVERSE_BODY \\")
        out.append(" \\\n".join(rev))
    return out


def main():
    pkg = _load_pkg()
    text = ["// Generated by symmetrix-xl_b200/csrc/gen_structures.py -- do not edit.",
            "// Coupling structure of the supported model shapes as X-macro lists.",
            "#pragma once", ""]
    for name, l_max, L_max, groups, by_edge_l in SHAPES:
        tables = pkg.modelgen.model_tables(l_max, L_max)
        text.append(emit_shape(name, l_max, L_max, tables, groups, by_edge_l))
    target = PKG / "csrc" / "generated" / "structures.h"
    target.write_text("\n".join(text))
    print("wrote", target)


if __name__ == "__main__":
    main()
