#include "model.hpp"

#include <algorithm>
#include <cmath>
#include <fstream>
#include <map>
#include <stdexcept>
#include <tuple>

#include "nlohmann/json.hpp"

#include "generated/structures.h"

namespace sxb {
namespace {

using json = nlohmann::json;

// ---------------------------------------------------------------- compiled shapes
#define SXB_PATH_PUSH(p, l, l1, l2, first_row) t.path_l.push_back(l); t.path_l1.push_back(l1); t.path_l2.push_back(l2);
#define SXB_TERM_PUSH(term, row, lme) t.term_row.push_back(row); t.term_lme.push_back(lme);
#define SXB_M_SET1(out, term, a) terms[term] = {a}; outs[term] = out;
#define SXB_M_SET2(out, term, a, b) terms[term] = {a, b}; outs[term] = out;
#define SXB_M_SET3(out, term, a, b, c) terms[term] = {a, b, c}; outs[term] = out;

#define SXB_DEFINE_SHAPE(NAME, ID)                                                      \
    ShapeTables make_##NAME()                                                            \
    {                                                                                    \
        ShapeTables t;                                                                   \
        t.name = #NAME; t.shape_id = ID;                                                 \
        t.l_max = SXB_##NAME##_LMAX; t.hidden_l_max = SXB_##NAME##_HIDDEN_LMAX;          \
        t.num_paths = SXB_##NAME##_NUM_PATHS; t.num_rows = SXB_##NAME##_NUM_ROWS;        \
        t.num_lme = SXB_##NAME##_NUM_LME; t.num_terms = SXB_##NAME##_NUM_TERMS;          \
        SXB_##NAME##_PATHS(SXB_PATH_PUSH)                                                \
        SXB_##NAME##_TERMS(SXB_TERM_PUSH)                                                \
        {                                                                                \
            std::vector<std::vector<int>> terms(SXB_##NAME##_M0_NUM_TERMS);              \
            std::vector<int> outs(SXB_##NAME##_M0_NUM_TERMS);                            \
            SXB_##NAME##_M0_TERMS(SXB_M_SET1, SXB_M_SET2, SXB_M_SET3)                    \
            t.m0_terms = terms; t.m0_out = outs;                                         \
        }                                                                                \
        {                                                                                \
            std::vector<std::vector<int>> terms(SXB_##NAME##_M1_NUM_TERMS);              \
            std::vector<int> outs(SXB_##NAME##_M1_NUM_TERMS);                            \
            SXB_##NAME##_M1_TERMS(SXB_M_SET1, SXB_M_SET2, SXB_M_SET3)                    \
            t.m1_terms = terms;                                                          \
        }                                                                                \
        return t;                                                                        \
    }

SXB_DEFINE_SHAPE(S0, 0)
SXB_DEFINE_SHAPE(S1, 1)
SXB_DEFINE_SHAPE(S2, 2)

const std::vector<ShapeTables>& all_shapes()
{
    static const std::vector<ShapeTables> shapes = {make_S0(), make_S1(), make_S2()};
    return shapes;
}

// ---------------------------------------------------------------- radial tables
struct Network {
    std::vector<int> shape;
    std::vector<std::vector<double>> weights;
    double activation_scale = 1.0;
    bool tanh_square = false;
};

Network parse_network(const json& def, const std::string& name)
{
    Network n;
    n.shape = def.at("shape").get<std::vector<int>>();
    n.weights = def.at("weights").get<std::vector<std::vector<double>>>();
    n.activation_scale = def.at("activation_scale").get<double>();
    const auto post = def.value("postprocess", std::string());
    if (!post.empty() && post != "tanh-square")
        throw std::invalid_argument("Compact radial network " + name + " has unsupported postprocessing.");
    n.tanh_square = post == "tanh-square";
    if (def.at("activation").get<std::string>() != "silu")
        throw std::invalid_argument("Compact radial network " + name + " must use SiLU.");
    if (n.shape.size() < 2 || n.weights.size() != n.shape.size() - 1)
        throw std::invalid_argument("Compact radial network " + name + " has an invalid shape.");
    for (std::size_t layer = 0; layer < n.weights.size(); ++layer)
        if (n.weights[layer].size() != static_cast<std::size_t>(n.shape[layer]) * n.shape[layer + 1])
            throw std::invalid_argument("Compact radial network " + name + " has invalid weights.");
    return n;
}

// values[node][out] for a batch of feature rows (weights are [out][in] row-major)
std::vector<double> run_network(const Network& n, const std::vector<double>& features, int batch)
{
    std::vector<double> x = features;
    for (std::size_t layer = 0; layer + 1 < n.shape.size(); ++layer) {
        const int in = n.shape[layer], out = n.shape[layer + 1];
        const bool last = layer + 2 == n.shape.size();
        std::vector<double> y(static_cast<std::size_t>(batch) * out);
        const auto& w = n.weights[layer];
        for (int b = 0; b < batch; ++b)
            for (int o = 0; o < out; ++o) {
                double s = 0.0;
                for (int i = 0; i < in; ++i)
                    s += x[static_cast<std::size_t>(b) * in + i] * w[static_cast<std::size_t>(o) * in + i];
                if (!last)
                    s = n.activation_scale * s / (1.0 + std::exp(-s));
                else if (n.tanh_square)
                    s = std::tanh(s * s);
                y[static_cast<std::size_t>(b) * out + o] = s;
            }
        x.swap(y);
    }
    return x;
}

// Cubic coefficients [interval][4][F] from nodal values [node][F]: nodal derivatives by
// the reference's tridiagonal system (left not-a-knot-like closure, zero right
// derivative), then the Hermite-to-monomial conversion.
std::vector<double> spline_coefficients(const std::vector<double>& values, int points, int F, double h)
{
    const int n = points - 2;
    std::vector<double> lower(n, 0.0), diag(n, 4.0), upper(n, 0.0);
    upper[0] = 2.0;
    for (int node = 2; node < points - 1; ++node) {
        const int row = node - 1;
        lower[row] = 1.0;
        if (node + 1 <= points - 2) upper[row] = 1.0;
    }
    std::vector<double> factor(n, 0.0);
    for (int row = 1; row < n; ++row) {
        factor[row] = lower[row] / diag[row - 1];
        diag[row] -= factor[row] * upper[row - 1];
    }
    std::vector<double> coeff(static_cast<std::size_t>(points - 1) * 4 * F);
    std::vector<double> rhs(n), d(points);
    for (int f = 0; f < F; ++f) {
        auto v = [&](int node) { return values[static_cast<std::size_t>(node) * F + f]; };
        const double left = 2.0 * (-v(0) + 2.0 * v(1) - v(2)) / h;
        rhs[0] = 3.0 * (v(2) - v(0)) / h - left;
        for (int node = 2; node < points - 1; ++node)
            rhs[node - 1] = 3.0 * (v(node + 1) - v(node - 1)) / h;
        for (int row = 1; row < n; ++row) rhs[row] -= factor[row] * rhs[row - 1];
        d[points - 2] = rhs[n - 1] / diag[n - 1];
        for (int row = n - 2; row >= 0; --row) d[row + 1] = (rhs[row] - upper[row] * d[row + 2]) / diag[row];
        d[0] = d[2] + left;
        d[points - 1] = 0.0;
        for (int i = 0; i < points - 1; ++i) {
            double* c = coeff.data() + static_cast<std::size_t>(i) * 4 * F + f;
            c[0] = v(i);
            c[F] = d[i];
            c[2 * F] = (-3 * v(i) - 2 * h * d[i] + 3 * v(i + 1) - h * d[i + 1]) / (h * h);
            c[3 * F] = (2 * v(i) + h * d[i] - 2 * v(i + 1) + h * d[i + 1]) / (h * h * h);
        }
    }
    return coeff;
}

// Parsed radial definition of a model: grid, basis, cutoff, optional Agnesi transform, networks,
// and the tables already built (per unordered species pair; key pair 0,0 without a transform).
struct RadialDefinition {
    int points = 0;
    double x0 = 0.0, h = 0.0;
    std::vector<double> bessel;
    double prefactor = 0.0, r_max = 0.0;
    int p = 0;
    bool agnesi = false;
    bool stored_pairs = false;   // tables were read from the file (pair-splines), nothing to build
    double agnesi_a = 0.0, agnesi_q = 0.0, agnesi_p = 0.0;
    std::vector<double> covalent_radii;   // per element type
    std::map<std::string, Network> networks;
    mutable std::map<std::tuple<std::string, int, int>, std::vector<double>> cache;
};

// Bessel x polynomial-cutoff features on the spline grid; with the Agnesi transform the Bessel argument
// is the transformed distance of the pair (libsymmetrix/source/compact_radial.cpp:227-267).
std::vector<double> radial_features(const RadialDefinition& d, int type_i, int type_j)
{
    const int nb = static_cast<int>(d.bessel.size());
    double r0 = 1.0;
    if (d.agnesi) r0 = 0.5 * (d.covalent_radii.at(type_i) + d.covalent_radii.at(type_j));
    std::vector<double> features(static_cast<std::size_t>(d.points) * nb);
    for (int node = 0; node < d.points; ++node) {
        const double r = d.x0 + node * d.h;
        double rt = r;
        if (d.agnesi) {
            const double sr = r / r0;
            rt = 1.0 / (1.0 + d.agnesi_a * std::pow(sr, d.agnesi_q) / (1.0 + std::pow(sr, d.agnesi_q - d.agnesi_p)));
        }
        double cut = 0.0;
        if (r < d.r_max) {
            const double u = r / d.r_max;
            cut = 1.0 - ((d.p + 1.0) * (d.p + 2.0) / 2.0) * std::pow(u, d.p) + d.p * (d.p + 2.0) * std::pow(u, d.p + 1)
                  - (d.p * (d.p + 1.0) / 2.0) * std::pow(u, d.p + 2);
        }
        for (int b = 0; b < nb; ++b)
            features[static_cast<std::size_t>(node) * nb + b] = d.prefactor * std::sin(d.bessel[b] * rt) / rt * cut;
    }
    return features;
}

template <typename T>
std::vector<T> to_vec(const std::vector<double>& v)
{
    std::vector<T> out(v.size());
    for (std::size_t i = 0; i < v.size(); ++i) {
        if (!std::isfinite(v[i])) throw std::invalid_argument("MACE model contains a non-finite value.");
        out[i] = static_cast<T>(v[i]);
    }
    return out;
}

}  // namespace

const ShapeTables& shape_tables(int shape_id) { return all_shapes().at(shape_id); }
int num_compiled_shapes() { return static_cast<int>(all_shapes().size()); }

namespace {
// Multi-head files keep the per-head parameters (atomic energies, both readouts, the ZBL
// coefficients) under prediction_heads.parameters[<name>]; the chosen head's values replace the
// top-level ones before anything else is parsed (reference: select_prediction_head,
// libsymmetrix/source/prediction_heads.hpp:10-90).  An empty request selects the file's default head.
void overlay_prediction_head(json& data, const std::string& requested, HostModel& m)
{
    const auto found = data.find("prediction_heads");
    if (found == data.end()) {
        const std::string only = data.value("head", std::string());
        if (!requested.empty() && requested != only)
            throw std::invalid_argument("Requested prediction head '" + requested + "' is unavailable; the file "
                                        + (only.empty() ? std::string("names no head.") : "holds '" + only + "'."));
        m.selected_head = only;
        if (!only.empty()) m.available_heads = {only};
        return;
    }
    const json section = *found;
    if (!section.is_object() || section.value("schema_version", 0) != 1)
        throw std::invalid_argument("prediction_heads has an unsupported schema version.");
    if (!section.contains("names") || !section.at("names").is_array())
        throw std::invalid_argument("prediction_heads.names must be an array.");
    const auto names = section.at("names").get<std::vector<std::string>>();
    std::vector<std::string> sorted_names(names);
    std::sort(sorted_names.begin(), sorted_names.end());
    const bool duplicated = std::adjacent_find(sorted_names.begin(), sorted_names.end()) != sorted_names.end();
    if (names.empty() || duplicated || sorted_names.front().empty())
        throw std::invalid_argument("prediction_heads.names must contain unique non-empty strings.");
    if (!section.contains("parameters") || !section.at("parameters").is_object()
        || section.at("parameters").size() != names.size())
        throw std::invalid_argument("prediction_heads.parameters must define every named head.");
    std::vector<std::string> expected = {"atomic_energies", "readout_1_weights_for_M0", "readout_2_weights_1",
                                         "readout_2_weights_2"};
    if (data.value("has_zbl", false)) expected.push_back("zbl_c");
    std::sort(expected.begin(), expected.end());
    for (const auto& name : names) {
        const auto& parameters = section.at("parameters");
        if (!parameters.contains(name) || !parameters.at(name).is_object())
            throw std::invalid_argument("prediction_heads.parameters must define every named head.");
        std::vector<std::string> fields;
        for (const auto& item : parameters.at(name).items()) fields.push_back(item.key());
        std::sort(fields.begin(), fields.end());
        if (fields != expected)
            throw std::invalid_argument("Every prediction-head payload must contain exactly the supported fields.");
    }
    const std::string fallback = section.value("default", std::string());
    if (!std::binary_search(sorted_names.begin(), sorted_names.end(), fallback))
        throw std::invalid_argument("prediction_heads.default must name a stored head.");
    const std::string chosen = requested.empty() ? fallback : requested;
    if (!std::binary_search(sorted_names.begin(), sorted_names.end(), chosen))
        throw std::invalid_argument("Requested prediction head '" + chosen + "' is unavailable.");
    for (const auto& item : section.at("parameters").at(chosen).items()) data[item.key()] = item.value();
    m.selected_head = chosen;
    m.available_heads = names;
}
// Stored pair splines (radial_representation "pair-splines": the exporter's nodal values and
// derivatives per unordered element pair, libsymmetrix/source/mace.cpp:2714-2737, 2746-2761; Hermite
// form cubic_spline_set.cpp:8-31).  Every pair's table goes straight into the definition's cache in
// the layout radial_coefficients() returns; the kernels then treat the model like one with a
// species-pair dependent distance transform.
void hermite_table(const std::vector<std::vector<double>>& values, const std::vector<std::vector<double>>& derivs, int points,
                   double h, const char* what, std::vector<double>& out)
{
    const std::size_t F = values.size();
    if (derivs.size() != F) throw std::invalid_argument(std::string(what) + ": values and derivatives differ in extent.");
    out.assign(static_cast<std::size_t>(points - 1) * 4 * F, 0.0);
    for (std::size_t f = 0; f < F; ++f) {
        const auto& v = values[f];
        const auto& d = derivs[f];
        if (static_cast<int>(v.size()) != points || static_cast<int>(d.size()) != points)
            throw std::invalid_argument(std::string(what) + ": every spline must hold one value and one derivative per node.");
        for (int i = 0; i < points; ++i)
            if (!std::isfinite(v[i]) || !std::isfinite(d[i])) throw std::invalid_argument(std::string(what) + " contains a non-finite value.");
        // the edge kernels skip edges at or beyond the cutoff, which is exact only for functions that end at zero
        const double scale = 1.0 + std::abs(v[points / 2]);
        if (std::abs(v[points - 1]) > 1e-6 * scale || std::abs(d[points - 1]) * h > 1e-6 * scale)
            throw std::invalid_argument(std::string(what) + " must vanish with zero slope at the cutoff.");
        for (int i = 0; i < points - 1; ++i) {
            double* c = out.data() + static_cast<std::size_t>(i) * 4 * F + f;
            c[0] = v[i];
            c[F] = d[i];
            c[2 * F] = (-3 * v[i] - 2 * h * d[i] + 3 * v[i + 1] - h * d[i + 1]) / (h * h);
            c[3 * F] = (2 * v[i] + h * d[i] - 2 * v[i + 1] + h * d[i + 1]) / (h * h * h);
        }
    }
}

void load_pair_splines(const json& file, HostModel& m)
{
    const int A = m.num_elements, C = m.channels, pairs = A * (A + 1) / 2;
    auto def = std::make_shared<RadialDefinition>();
    def->stored_pairs = true;
    def->h = file.at("radial_spline_h").get<double>();
    def->x0 = file.value("radial_spline_min", 0.0);
    using Table = std::vector<std::vector<std::vector<double>>>;   // [pair][function][node]
    const Table values0 = file.at("radial_spline_values_0").get<Table>(), derivs0 = file.at("radial_spline_derivs_0").get<Table>();
    Table values1, derivs1;
    if (!m.single_layer) {
        values1 = file.at("radial_spline_values_1").get<Table>();
        derivs1 = file.at("radial_spline_derivs_1").get<Table>();
    }
    if (static_cast<int>(values0.size()) != pairs || static_cast<int>(derivs0.size()) != pairs
        || (!m.single_layer && (static_cast<int>(values1.size()) != pairs || static_cast<int>(derivs1.size()) != pairs)))
        throw std::invalid_argument("Pair-spline tables must hold one entry per unordered element pair.");
    if (values0[0].empty() || values0[0][0].size() < 2) throw std::invalid_argument("Pair-spline tables are empty.");
    def->points = static_cast<int>(values0[0][0].size());
    if (!(def->h > 0.0) || !std::isfinite(def->h) || !(def->x0 >= 0.0) || !std::isfinite(def->x0))
        throw std::invalid_argument("Pair-spline grid is invalid.");
    if (std::abs(def->x0 + def->h * (def->points - 1) - m.r_cut) > 1e-9 * m.r_cut)
        throw std::invalid_argument("Pair-spline grid must end at the model cutoff.");
    m.spline_x0 = def->x0;
    m.spline_h = def->h;
    m.spline_points = def->points;
    m.a0_scaled = file.at("A0_scaled").get<bool>();
    m.a1_scaled = file.value("A1_scaled", false);
    // density splines: one per pair on a grid of their own, which must be the radial grid (mace.cpp:2746-2761)
    auto density = [&](const char* name, const char* prefix) {
        const std::string p(prefix);
        const double h = file.at(p + "_spline_h").get<double>(), x0 = file.value(p + "_spline_min", 0.0);
        if (std::abs(h - def->h) > 1e-12 * def->h || std::abs(x0 - def->x0) > 1e-12)
            throw std::invalid_argument(p + " density splines must use the grid of the radial splines.");
        const auto values = file.at(p + "_spline_values").get<std::vector<std::vector<double>>>();
        const auto derivs = file.at(p + "_spline_derivs").get<std::vector<std::vector<double>>>();
        if (static_cast<int>(values.size()) != pairs || static_cast<int>(derivs.size()) != pairs)
            throw std::invalid_argument(p + " density splines must hold one entry per unordered element pair.");
        int pair = 0;
        for (int a = 0; a < A; ++a)
            for (int b = a; b < A; ++b, ++pair)
                hermite_table({values[pair]}, {derivs[pair]}, def->points, def->h, (p + "_spline_values").c_str(),
                              def->cache[std::make_tuple(std::string(name), a, b)]);
    };
    int pair = 0;
    for (int a = 0; a < A; ++a)
        for (int b = a; b < A; ++b, ++pair) {   // the exporter's pair order: a <= b, row by row
            if (static_cast<int>(values0[pair].size()) != (m.l_max + 1) * C)
                throw std::invalid_argument("radial_spline_values_0 must hold (l_max+1)*num_channels splines per pair.");
            hermite_table(values0[pair], derivs0[pair], def->points, def->h, "radial_spline_values_0",
                          def->cache[std::make_tuple(std::string("R0"), a, b)]);
            if (m.single_layer) continue;
            if (static_cast<int>(values1[pair].size()) != m.num_paths * C)
                throw std::invalid_argument("radial_spline_values_1 must hold paths*num_channels splines per pair.");
            hermite_table(values1[pair], derivs1[pair], def->points, def->h, "radial_spline_values_1",
                          def->cache[std::make_tuple(std::string("R1"), a, b)]);
        }
    if (m.a0_scaled) density("A0", "A0");
    if (m.a1_scaled) density("A1", "A1");
    m.agnesi = true;   // tables depend on the species pair
    m.radial = def;
}
}  // namespace

HostModel load_model(const std::string& json_path, const std::string& head)
{
    std::ifstream stream(json_path);
    if (!stream) throw std::runtime_error("Could not open Symmetrix model file: " + json_path);
    json parsed = json::parse(stream);
    HostModel m;
    if (parsed.value("model_type", std::string("MACE")) == "MACE" && parsed.value("symmetrix_format_version", 1) == 4
        && parsed.value("h1_affine_mode", std::string()) == "m0_composite")
        overlay_prediction_head(parsed, head, m);
    const json& file = parsed;
    if (parsed.contains("prediction_heads") && parsed.value("h1_affine_mode", std::string()) == "pre_linear_up")
        throw std::invalid_argument("Multi-head files are supported in the m0_composite basis only.");

    if (file.value("model_type", std::string("MACE")) != "MACE")
        throw std::invalid_argument("Only the standard two-layer MACE model family is supported.");
    // H1 affine basis (libsymmetrix/source/h1_affine_schema.hpp:179-240): format 4 with the first readout and the
    // H1->H2 skip on the scalar block of M0, or format 1 / 2 with both on the scalar block of H1 (after linear_up)
    const int format_version = file.value("symmetrix_format_version", 1);
    if (format_version == 1 || format_version == 2) {
        for (const char* key : {"h1_affine_mode", "h1_affine_version", "readout_1_weights_for_M0", "H2_weights_for_M0",
                                "readout_1_weights_for_H1_pre_linear_up", "H2_weights_for_H1_pre_linear_up"})
            if (file.contains(key))
                throw std::invalid_argument("Symmetrix MACE format version " + std::to_string(format_version)
                                            + " must not declare h1_affine fields; they require format version 4.");
        if (file.contains("prediction_heads"))
            throw std::invalid_argument("Multi-head files are supported in format version 4 only.");
        m.legacy_h1_basis = true;
    } else if (format_version != 4) {
        throw std::invalid_argument("Unsupported Symmetrix model format version.");
    } else {
        const std::string mode = file.value("h1_affine_mode", std::string());
        if (mode != "m0_composite" && mode != "pre_linear_up")
            throw std::invalid_argument("Symmetrix MACE format version 4 requires h1_affine_mode 'm0_composite' or 'pre_linear_up'.");
        m.pre_linear_up = mode == "pre_linear_up";
        if (file.value("h1_affine_version", 0) != 1) throw std::invalid_argument("Unsupported h1_affine_version (supported: 1).");
        if (file.contains("readout_1_weights") || file.contains("H2_weights_for_H1"))
            throw std::invalid_argument("A format-version-4 MACE JSON must not contain the old-basis readout_1_weights or H2_weights_for_H1 fields.");
        const char* other_readout = m.pre_linear_up ? "readout_1_weights_for_M0" : "readout_1_weights_for_H1_pre_linear_up";
        const char* other_skip = m.pre_linear_up ? "H2_weights_for_M0" : "H2_weights_for_H1_pre_linear_up";
        if (file.contains(other_readout) || file.contains(other_skip))
            throw std::invalid_argument("A '" + mode + "' MACE JSON must not contain " + other_readout + " or " + other_skip + ".");
        const bool residual = file.value("first_interaction_residual", false);
        if (!m.pre_linear_up && !file.value("single_layer_readout", false) && residual)
            throw std::invalid_argument("The m0_composite basis cannot represent first-interaction residual features; such models use "
                                        "h1_affine_mode 'pre_linear_up'.");
        if (m.pre_linear_up && (file.value("single_layer_readout", false) || file.value("num_interactions", 2) != 2))
            throw std::invalid_argument("The pre_linear_up basis applies to two-interaction models only.");
        if (m.pre_linear_up && !file.contains("H1_product_weights"))
            throw std::invalid_argument("The pre_linear_up basis requires H1_product_weights.");
    }
    const std::string radial_representation =
        file.value("radial_representation", std::string(format_version == 1 ? "pair-splines" : ""));
    if (radial_representation != "compact" && radial_representation != "pair-splines")
        throw std::invalid_argument("Model must use the compact or the pair-splines radial representation.");
    m.single_layer = file.value("single_layer_readout", false);
    if (file.value("num_interactions", 2) != (m.single_layer ? 1 : 2))
        throw std::invalid_argument("MACE interaction count and single-layer readout metadata disagree.");
    if (file.value("has_field_coupling", false)) throw std::invalid_argument("MACEField models are not supported.");
    m.first_residual = file.value("first_interaction_residual", false);
    if (m.first_residual && !m.pre_linear_up)
        throw std::invalid_argument("Residual-first models are supported in the pre_linear_up basis of format version 4 only.");

    m.has_zbl = file.value("has_zbl", false);
    if (m.has_zbl) {   // libsymmetrix/source/mace.cpp:2690-2699
        m.zbl_a_exp = file.at("zbl_a_exp").get<double>();
        m.zbl_a_prefactor = file.at("zbl_a_prefactor").get<double>();
        m.zbl_c = file.at("zbl_c").get<std::vector<double>>();
        m.zbl_covalent_radii = file.at("zbl_covalent_radii").get<std::vector<double>>();
        m.zbl_p = file.at("zbl_p").get<int>();
        if (m.zbl_c.size() != 4 || m.zbl_p < 1) throw std::invalid_argument("ZBL parameters are malformed.");
    }
    m.num_elements = file.at("num_elements").get<int>();
    m.channels = file.at("num_channels").get<int>();
    m.r_cut = file.at("r_cut").get<double>();
    m.l_max = file.at("l_max").get<int>();
    m.hidden_l_max = file.at("L_max").get<int>();
    m.num_lm = (m.l_max + 1) * (m.l_max + 1);
    m.num_hidden = (m.hidden_l_max + 1) * (m.hidden_l_max + 1);
    m.atomic_numbers = file.at("atomic_numbers").get<std::vector<int>>();
    m.atomic_energies = file.at("atomic_energies").get<std::vector<double>>();
    const int A = m.num_elements, C = m.channels;
    if (static_cast<int>(m.atomic_numbers.size()) != A || static_cast<int>(m.atomic_energies.size()) != A)
        throw std::invalid_argument("atomic_numbers / atomic_energies do not match num_elements.");
    if (C % 32 != 0 || C > 256) throw std::invalid_argument("num_channels must be a multiple of 32, at most 256.");

    // ---- structure: match against a compiled shape
    // a single-layer model has no second message step: its file carries no Phi1 tables (mace.cpp:2860-2873)
    const std::vector<int> none;
    const auto phi_l = file.value("Phi1_l", none);
    const auto phi_l1 = file.value("Phi1_l1", none);
    const auto phi_l2 = file.value("Phi1_l2", none);
    const auto phi_lme = file.value("Phi1_lme", none);
    const auto phi_row = file.value("Phi1_lelm1lm2", none);
    const auto phi_cg = file.value("Phi1_clebsch_gordan", std::vector<double>());
    if (m.single_layer && !phi_l.empty()) throw std::invalid_argument("A single-layer model must not carry Phi1 tables.");
    const auto m0_monomials = file.at("M0_monomials").get<std::map<std::string, std::vector<std::vector<int>>>>();
    const auto m1_monomials = file.at("M1_monomials").get<std::vector<std::vector<int>>>();
    const ShapeTables* shape = nullptr;
    for (const auto& s : all_shapes())
        if (s.l_max == m.l_max && s.hidden_l_max == m.hidden_l_max
            && (m.single_layer || (s.path_l == phi_l && s.path_l1 == phi_l1 && s.path_l2 == phi_l2)))
            shape = &s;
    if (shape == nullptr)
        throw std::invalid_argument("Model coupling structure (l_max, L_max, paths) matches no compiled shape.");
    m.shape_id = shape->shape_id;
    m.num_paths = shape->num_paths;
    m.num_rows = shape->num_rows;
    m.num_lme = shape->num_lme;
    m.num_terms = shape->num_terms;
    if (phi_lme.size() != phi_row.size() || phi_lme.size() != phi_cg.size())
        throw std::invalid_argument("Phi1 sparse coupling arrays must have equal lengths.");
    m.cg.assign(shape->num_terms, 0.0f);
    {
        std::map<std::pair<int, int>, int> compiled;
        for (int t = 0; t < shape->num_terms; ++t) compiled[{shape->term_row[t], shape->term_lme[t]}] = t;
        for (std::size_t t = 0; t < phi_cg.size(); ++t) {
            auto it = compiled.find({phi_row[t], phi_lme[t]});
            if (it == compiled.end()) {
                if (phi_cg[t] == 0.0) continue;
                throw std::invalid_argument("Model has a Phi1 coupling term outside the compiled structure.");
            }
            m.cg[it->second] += static_cast<float>(phi_cg[t]);
        }
    }
    m.eta.assign(m.l_max + 1, 0);
    for (int l : (m.single_layer ? shape->path_l : phi_l)) m.eta[l] += 1;
    m.group_begin.assign(m.l_max + 2, 0);
    for (int l = 0; l <= m.l_max; ++l) m.group_begin[l + 1] = m.group_begin[l] + (2 * l + 1) * m.eta[l];

    // ---- symmetric contraction weights in compiled term order
    auto map_terms = [](const std::vector<std::vector<int>>& compiled, const std::vector<int>* outs, int out,
                        const std::vector<std::vector<int>>& given, const char* what) {
        std::map<std::vector<int>, int> where;
        for (std::size_t t = 0; t < compiled.size(); ++t)
            if (outs == nullptr || (*outs)[t] == out) where[compiled[t]] = static_cast<int>(t);
        std::vector<int> position(given.size());
        for (std::size_t t = 0; t < given.size(); ++t) {
            auto sorted = given[t];
            std::sort(sorted.begin(), sorted.end());
            auto it = where.find(sorted);
            if (it == where.end())
                throw std::invalid_argument(std::string(what) + " contains a monomial outside the compiled structure.");
            position[t] = it->second;
        }
        return position;
    };
    m.m0_num_terms = static_cast<int>(shape->m0_terms.size());
    m.m1_num_terms = static_cast<int>(shape->m1_terms.size());
    m.m0_weights.assign(static_cast<std::size_t>(A) * m.m0_num_terms * C, 0.0f);
    m.m1_weights.assign(static_cast<std::size_t>(A) * m.m1_num_terms * C, 0.0f);
    {
        const auto& weights = file.at("M0_weights");
        for (int lm = 0; lm < m.num_hidden; ++lm) {
            const auto position = map_terms(shape->m0_terms, &shape->m0_out, lm, m0_monomials.at(std::to_string(lm)),
                                            "M0_monomials");
            for (int a = 0; a < A; ++a)
                for (int k = 0; k < C; ++k) {
                    const auto w = weights.at(std::to_string(a)).at(std::to_string(lm)).at(std::to_string(k))
                                       .get<std::vector<double>>();
                    if (w.size() != position.size()) throw std::invalid_argument("M0_weights extent mismatch.");
                    for (std::size_t t = 0; t < w.size(); ++t)
                        m.m0_weights[(static_cast<std::size_t>(a) * m.m0_num_terms + position[t]) * C + k] +=
                            static_cast<float>(w[t]);
                }
        }
        const auto& w1 = file.at("M1_weights");
        if (m.single_layer) {
            // the readout polynomial acts on H1 (mace.cpp:2465-2466): its monomials index the hidden components and
            // are kept as data for the generic polynomial kernel, in the file's order
            const int terms = static_cast<int>(m1_monomials.size());
            m.hidden_poly_terms.assign(static_cast<std::size_t>(terms) * 4, -1);
            for (int t = 0; t < terms; ++t) {
                const auto& mono = m1_monomials[t];
                if (mono.empty() || mono.size() > 3) throw std::invalid_argument("M1_monomials must have degree 1 to 3.");
                for (std::size_t q = 0; q < mono.size(); ++q) {
                    if (mono[q] < 0 || mono[q] >= m.num_hidden) throw std::invalid_argument("M1_monomials index a component outside H1.");
                    m.hidden_poly_terms[static_cast<std::size_t>(t) * 4 + q] = mono[q];
                }
            }
            m.hidden_poly_weights.assign(static_cast<std::size_t>(A) * terms * C, 0.0f);
            for (int a = 0; a < A; ++a)
                for (int k = 0; k < C; ++k) {
                    const auto w = w1.at(std::to_string(a)).at(std::to_string(k)).get<std::vector<double>>();
                    if (static_cast<int>(w.size()) != terms) throw std::invalid_argument("M1_weights extent mismatch.");
                    for (int t = 0; t < terms; ++t)
                        m.hidden_poly_weights[(static_cast<std::size_t>(a) * terms + t) * C + k] = static_cast<float>(w[t]);
                }
        } else {
        const auto position = map_terms(shape->m1_terms, nullptr, 0, m1_monomials, "M1_monomials");
        for (int a = 0; a < A; ++a)
            for (int k = 0; k < C; ++k) {
                const auto w = w1.at(std::to_string(a)).at(std::to_string(k)).get<std::vector<double>>();
                if (w.size() != position.size()) throw std::invalid_argument("M1_weights extent mismatch.");
                for (std::size_t t = 0; t < w.size(); ++t)
                    m.m1_weights[(static_cast<std::size_t>(a) * m.m1_num_terms + position[t]) * C + k] +=
                        static_cast<float>(w[t]);
            }
        }
    }

    // ---- radial tables
    if (radial_representation == "pair-splines") {
        load_pair_splines(file, m);
    } else {
    const auto& radial = file.at("compact_radial");
    m.spline_x0 = radial.at("spline_grid_min").get<double>();
    m.spline_points = radial.at("num_spline_points").get<int>();
    if (!(m.spline_x0 > 0.0) || m.spline_points < 4)
        throw std::invalid_argument("Compact radial model has an invalid spline grid.");
    m.spline_h = (m.r_cut - m.spline_x0) / (m.spline_points - 1);
    const auto& basis = radial.at("basis");
    if (basis.at("type").get<std::string>() != "bessel")
        throw std::invalid_argument("Compact radial model only supports a Bessel basis.");
    const auto bessel = basis.at("weights").get<std::vector<double>>();
    const double prefactor = basis.at("prefactor").get<double>();
    const auto& cutoff = radial.at("cutoff");
    if (cutoff.at("type").get<std::string>() != "polynomial")
        throw std::invalid_argument("Compact radial model only supports a polynomial cutoff.");
    const double r_max = cutoff.at("r_max").get<double>();
    const int p = cutoff.at("p").get<int>();
    if (std::abs(r_max - m.r_cut) > 1e-12) throw std::invalid_argument("Compact radial cutoff does not match model r_cut.");
    auto def = std::make_shared<RadialDefinition>();
    def->points = m.spline_points;
    def->x0 = m.spline_x0;
    def->h = m.spline_h;
    def->bessel = bessel;
    def->prefactor = prefactor;
    def->r_max = r_max;
    def->p = p;
    const auto& transform = radial.at("distance_transform");
    const std::string transform_type = transform.at("type").get<std::string>();
    if (transform_type == "agnesi") {   // libsymmetrix/source/compact_radial.cpp:149-166
        def->agnesi = true;
        def->agnesi_a = transform.at("a").get<double>();
        def->agnesi_q = transform.at("q").get<double>();
        def->agnesi_p = transform.at("p").get<double>();
        def->covalent_radii = transform.at("covalent_radii").get<std::vector<double>>();
        if (static_cast<int>(def->covalent_radii.size()) != A)
            throw std::invalid_argument("Compact radial covalent radii do not match atomic numbers.");
        for (double rc : def->covalent_radii)
            if (!(rc > 0.0) || !std::isfinite(rc)) throw std::invalid_argument("Compact radial model has invalid Agnesi data.");
        if (!std::isfinite(def->agnesi_a) || !std::isfinite(def->agnesi_q) || !std::isfinite(def->agnesi_p))
            throw std::invalid_argument("Compact radial model has invalid Agnesi data.");
    } else if (transform_type != "none") {
        throw std::invalid_argument("Unknown radial distance transform: " + transform_type);
    }
    m.agnesi = def->agnesi;
    const int nb = static_cast<int>(bessel.size());
    const auto& networks = radial.at("networks");
    auto add_network = [&](const char* name, int expected) {
        const Network net = parse_network(networks.at(name), name);
        if (net.shape.front() != nb || net.shape.back() != expected)
            throw std::invalid_argument(std::string("Compact radial network ") + name + " has an invalid extent.");
        def->networks.emplace(name, net);
    };
    add_network("R0", (m.l_max + 1) * C);
    if (networks.contains("R1") == m.single_layer)   // compact_radial: has_R1() == single_layer is an error (mace.cpp:2768-2771)
        throw std::invalid_argument("Compact radial R1 network does not match single_layer_readout.");
    if (!m.single_layer) add_network("R1", m.num_paths * C);
    m.a0_scaled = file.at("A0_scaled").get<bool>();
    m.a1_scaled = file.value("A1_scaled", false);
    if (m.a0_scaled != networks.contains("A0") || m.a1_scaled != networks.contains("A1"))
        throw std::invalid_argument("Compact radial density networks do not match A0_scaled / A1_scaled.");
    if (m.a0_scaled) add_network("A0", 1);
    if (m.a1_scaled) add_network("A1", 1);
    m.radial = def;
    }

    // ---- dense weights
    m.h0 = file.at("H0_weights").get<std::vector<double>>();
    if (m.h0.size() != static_cast<std::size_t>(A) * C) throw std::invalid_argument("H0_weights extent mismatch.");
    {
        const auto w = file.at("A0_weights").get<std::vector<std::vector<std::vector<double>>>>();
        if (static_cast<int>(w.size()) != A) throw std::invalid_argument("A0_weights extent mismatch.");
        m.w_a0.reserve(static_cast<std::size_t>(A) * (m.l_max + 1) * C * C);
        for (const auto& per_element : w) {
            if (static_cast<int>(per_element.size()) != m.l_max + 1) throw std::invalid_argument("A0_weights extent mismatch.");
            for (const auto& block : per_element) {
                if (block.size() != static_cast<std::size_t>(C) * C) throw std::invalid_argument("A0_weights extent mismatch.");
                m.w_a0.insert(m.w_a0.end(), block.begin(), block.end());
            }
        }
    }
    m.w_h1 = to_vec<float>(file.at("H1_weights").get<std::vector<double>>());
    if (m.w_h1.size() != static_cast<std::size_t>(m.hidden_l_max + 1) * C * C)
        throw std::invalid_argument("H1_weights extent mismatch.");
    if (m.pre_linear_up) {
        // the first readout and the skip act on x = M0[l=0] P0 (+ the residual's scalar block): keep P0 = H1_product_weights[l=0]
        const auto product = file.at("H1_product_weights").get<std::vector<double>>();
        if (product.size() != m.w_h1.size())
            throw std::invalid_argument("The pre_linear_up basis requires H1_product_weights of the H1_weights extent.");
        m.w_product0.assign(product.begin(), product.begin() + static_cast<std::ptrdiff_t>(C) * C);
    } else if (file.contains("H1_first_residual_weights") && !file.at("H1_first_residual_weights").empty()) {
        throw std::invalid_argument("Non-residual MACE JSON must not contain H1 residual weights.");
    }
    if (m.first_residual) {
        // H1 += R U per element (the residual passes through linear_up, mace.cpp:2801-2829); x += R[l=0]
        const auto residual = file.at("H1_first_residual_weights").get<std::vector<double>>();
        const auto linear_up = file.at("H1_linear_up_weights").get<std::vector<double>>();
        const std::size_t NHs = static_cast<std::size_t>(m.num_hidden);
        if (residual.size() != static_cast<std::size_t>(A) * NHs * C) throw std::invalid_argument("Residual-first MACE JSON has an invalid H1 residual extent.");
        if (linear_up.size() != m.w_h1.size()) throw std::invalid_argument("Residual-first MACE JSON requires split H1 weights.");
        m.residual_fused.assign(residual.size(), 0.0f);
        m.residual_scalar.assign(static_cast<std::size_t>(A) * C, 0.0f);
        for (int a = 0; a < A; ++a) {
            for (int l = 0; l <= m.hidden_l_max; ++l)
                for (int mm = 0; mm < 2 * l + 1; ++mm) {
                    const std::size_t lm = static_cast<std::size_t>(l) * l + mm;
                    for (int out = 0; out < C; ++out) {
                        double sum = 0.0;
                        for (int in = 0; in < C; ++in)
                            sum += residual[(a * NHs + lm) * C + in] * linear_up[(static_cast<std::size_t>(l) * C + in) * C + out];
                        m.residual_fused[(a * NHs + lm) * C + out] = static_cast<float>(sum);
                    }
                }
            for (int k = 0; k < C; ++k) m.residual_scalar[static_cast<std::size_t>(a) * C + k] = static_cast<float>(residual[a * NHs * C + k]);
        }
    }
    if (!m.single_layer) {
        const auto w = file.at("A1_weights").get<std::vector<std::vector<double>>>();
        if (static_cast<int>(w.size()) != m.l_max + 1) throw std::invalid_argument("A1_weights extent mismatch.");
        for (int l = 0; l <= m.l_max; ++l) {
            if (w[l].size() != static_cast<std::size_t>(m.eta[l]) * C * C) throw std::invalid_argument("A1_weights extent mismatch.");
            m.w_a1.push_back(to_vec<float>(w[l]));
        }
    }
    {
        const char* skip_key = m.legacy_h1_basis ? "H2_weights_for_H1" : m.pre_linear_up ? "H2_weights_for_H1_pre_linear_up" : "H2_weights_for_M0";
        const auto w = file.at(skip_key).get<std::vector<std::vector<double>>>();
        if (static_cast<int>(w.size()) != A) throw std::invalid_argument("H2_weights_for_M0 extent mismatch.");
        for (const auto& block : w) {
            if (block.size() != static_cast<std::size_t>(C) * C) throw std::invalid_argument("H2_weights_for_M0 extent mismatch.");
            const auto f = to_vec<float>(block);
            m.h2_skip.insert(m.h2_skip.end(), f.begin(), f.end());
        }
    }
    m.h2_m1 = to_vec<float>(file.at("H2_weights_for_M1").get<std::vector<double>>());
    m.readout1 = to_vec<float>(file.at(m.legacy_h1_basis ? "readout_1_weights"
                                       : m.pre_linear_up ? "readout_1_weights_for_H1_pre_linear_up"
                                                         : "readout_1_weights_for_M0").get<std::vector<double>>());
    m.readout2_w1 = to_vec<float>(file.at("readout_2_weights_1").get<std::vector<double>>());
    m.readout2_w2 = to_vec<float>(file.at("readout_2_weights_2").get<std::vector<double>>());
    m.readout2_hidden = file.value("readout_2_hidden_size", 16);
    m.readout2_scale = static_cast<float>(file.at("readout_2_scale_factor").get<double>());
    if (m.single_layer && m.a1_scaled) throw std::invalid_argument("A single-layer model cannot scale a second message step (A1_scaled).");
    if (m.h2_m1.size() != static_cast<std::size_t>(C) * C || m.readout1.size() != static_cast<std::size_t>(C)
        || m.readout2_hidden <= 0 || m.readout2_hidden > 64
        || m.readout2_w1.size() != static_cast<std::size_t>(C) * m.readout2_hidden
        || m.readout2_w2.size() != static_cast<std::size_t>(m.readout2_hidden))
        throw std::invalid_argument("MACE readout weights do not match the declared sizes.");
    return m;
}

const std::vector<double>& radial_coefficients(const HostModel& m, const std::string& name, int type_i, int type_j)
{
    const auto& d = *static_cast<const RadialDefinition*>(m.radial.get());
    int a = 0, b = 0;
    if (d.agnesi || d.stored_pairs) { a = std::min(type_i, type_j); b = std::max(type_i, type_j); }
    const auto key = std::make_tuple(name, a, b);
    auto found = d.cache.find(key);
    if (found != d.cache.end()) return found->second;
    if (d.stored_pairs) throw std::invalid_argument("Pair-spline model holds no table " + name + " for the requested element pair.");
    const Network& net = d.networks.at(name);
    const auto values = run_network(net, radial_features(d, a, b), d.points);
    return d.cache.emplace(key, spline_coefficients(values, d.points, net.shape.back(), d.h)).first->second;
}

std::vector<float> build_r1_table(const HostModel& m, const std::vector<int>& active_types, int* num_pairs)
{
    const int n = m.agnesi ? static_cast<int>(active_types.size()) : 1;
    const int pairs = n * (n + 1) / 2;
    *num_pairs = pairs;
    const std::size_t F = static_cast<std::size_t>(m.num_paths) * m.channels;
    const std::size_t intervals = static_cast<std::size_t>(m.spline_points - 1);
    std::vector<float> out(static_cast<std::size_t>(pairs) * intervals * F * 4);
    int pair = 0;
    for (int a = 0; a < n; ++a)
        for (int b = a; b < n; ++b, ++pair) {   // pair index a*(2n-a-1)/2 + b
            const auto& c = radial_coefficients(m, "R1", m.agnesi ? active_types[a] : 0, m.agnesi ? active_types[b] : 0);
            float* table = out.data() + static_cast<std::size_t>(pair) * intervals * F * 4;
            for (std::size_t i = 0; i < intervals; ++i)
                for (std::size_t f = 0; f < F; ++f)
                    for (std::size_t q = 0; q < 4; ++q) table[(i * F + f) * 4 + q] = static_cast<float>(c[(i * 4 + q) * F + f]);
        }
    return out;
}

std::vector<float> build_density_table(const HostModel& m, const std::string& name, const std::vector<int>& active_types)
{
    const int n = static_cast<int>(active_types.size());
    const std::size_t rows = static_cast<std::size_t>(m.spline_points - 1) * 4;
    std::vector<float> out(static_cast<std::size_t>(n) * n * rows);
    for (int a = 0; a < n; ++a)
        for (int b = 0; b < n; ++b) {
            const auto& c = radial_coefficients(m, name, active_types[a], active_types[b]);   // [interval][4][1]
            for (std::size_t q = 0; q < rows; ++q) out[(static_cast<std::size_t>(a) * n + b) * rows + q] = static_cast<float>(c[q]);
        }
    return out;
}

std::vector<float> fold_r0_table(const HostModel& m, const std::vector<int>& active_types)
{
    const int n = static_cast<int>(active_types.size());
    const int C = m.channels, L = m.l_max + 1, F = L * C;
    const int rows = (m.spline_points - 1) * 4;
    std::vector<float> out(static_cast<std::size_t>(n) * n * rows * F);
    std::vector<double> scaled(C), acc(C);
    for (int ai = 0; ai < n; ++ai)
        for (int aj = 0; aj < n; ++aj) {
            const double* h0 = m.h0.data() + static_cast<std::size_t>(active_types[aj]) * C;
            float* table = out.data() + static_cast<std::size_t>(ai * n + aj) * rows * F;
            const std::vector<double>& r0_coeff = radial_coefficients(m, "R0", active_types[ai], active_types[aj]);
            for (int row = 0; row < rows; ++row)
                for (int l = 0; l < L; ++l) {
                    const double* c = r0_coeff.data() + static_cast<std::size_t>(row) * F + l * C;
                    const double* w = m.w_a0.data() + (static_cast<std::size_t>(active_types[ai]) * L + l) * C * C;
                    for (int k = 0; k < C; ++k) scaled[k] = c[k] * h0[k];
                    std::fill(acc.begin(), acc.end(), 0.0);
                    for (int k = 0; k < C; ++k) {
                        const double s = scaled[k];
                        const double* wk = w + static_cast<std::size_t>(k) * C;
                        for (int j = 0; j < C; ++j) acc[j] += s * wk[j];
                    }
                    float* o = table + static_cast<std::size_t>(row) * F + l * C;
                    for (int j = 0; j < C; ++j) o[j] = static_cast<float>(acc[j]);
                }
        }
    return out;
}

}  // namespace sxb
