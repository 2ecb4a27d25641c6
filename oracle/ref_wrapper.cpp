// C-ABI wrapper around the reference's own serial evaluator MACECPU<float|double>
// (libsymmetrix/source/mace.hpp:17-302), compiled in place from the reference
// checkout by oracle/Makefile into oracle/_ref/.  TEST INFRASTRUCTURE ONLY: it is
// the checker the CUDA path is compared against (and the timed CPU baseline); no
// product code path may call it.
//
// The wrapper adds no arithmetic of its own: it forwards the CSR graph and edge
// vectors to compute_node_energies_forces (mace.cpp:232-319) and copies public
// member vectors out as doubles.
#include <cstring>
#include <memory>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "mace.hpp"

namespace {
struct Handle {
    std::unique_ptr<MACECPU<float>> f;
    std::unique_ptr<MACECPU<double>> d;
    std::string error;
};

template <typename M>
void prepare_types(M& mace, const int* node_types, int num_nodes, const int* neigh_types, long num_edges)
{
    // The Python binding of the reference unions node and neighbor types before
    // preparing the radial cache (symmetrix/source/cpp/mace.cpp:36-57).
    std::vector<int> types(node_types, node_types + num_nodes);
    types.insert(types.end(), neigh_types, neigh_types + num_edges);
    mace.prepare_active_types(types);
}

template <typename V>
long copy_out(const V& v, double* out, long capacity)
{
    const long n = static_cast<long>(v.size());
    if (out == nullptr) return n;
    if (capacity < n) return -n;
    for (long i = 0; i < n; ++i) out[i] = static_cast<double>(v[i]);
    return n;
}

template <typename M>
long get_field(M& m, const std::string& name, double* out, long cap)
{
#define FIELD(x) if (name == #x) return copy_out(m.x, out, cap)
    FIELD(node_energies); FIELD(node_forces); FIELD(Y); FIELD(Y_grad);
    FIELD(A0); FIELD(A0_adj); FIELD(M0); FIELD(M0_adj); FIELD(H1); FIELD(H1_adj);
    FIELD(Phi1); FIELD(dPhi1); FIELD(A1); FIELD(A1_adj); FIELD(M1); FIELD(M1_adj);
    FIELD(H2); FIELD(H2_adj); FIELD(M0_direct_adj); FIELD(h1_affine_scalar);
    FIELD(R0); FIELD(R0_deriv); FIELD(R1); FIELD(R1_deriv);
#undef FIELD
    return -1;
}
}  // namespace

extern "C" {

void* symref_create(const char* json_path, int use_double, char* error, int error_size)
{
    auto h = std::make_unique<Handle>();
    try {
        if (use_double) h->d = std::make_unique<MACECPU<double>>(json_path);
        else h->f = std::make_unique<MACECPU<float>>(json_path);
    } catch (const std::exception& e) {
        if (error && error_size > 0) { std::strncpy(error, e.what(), error_size - 1); error[error_size - 1] = 0; }
        return nullptr;
    }
    return h.release();
}

void symref_destroy(void* handle) { delete static_cast<Handle*>(handle); }

const char* symref_last_error(void* handle) { return static_cast<Handle*>(handle)->error.c_str(); }

// mode: "materialized", "generic" (streamed A0 and Phi1) or "" to keep the
// constructor's default (direct on a compact model, mace.cpp:80-86).
int symref_compute(void* handle, int num_nodes, long num_edges, const int* node_types,
                   const int* num_neigh, const int* neigh_indices, const int* neigh_types,
                   const double* xyz, const double* r, const char* mode)
{
    auto* h = static_cast<Handle*>(handle);
    try {
        auto run = [&](auto& m) {
            if (mode && mode[0]) m.set_streamed_edges(mode);
            prepare_types(m, node_types, num_nodes, neigh_types, num_edges);
            m.compute_node_energies_forces(
                num_nodes,
                std::span<const int>(node_types, num_nodes),
                std::span<const int>(num_neigh, num_nodes),
                std::span<const int>(neigh_indices, num_edges),
                std::span<const int>(neigh_types, num_edges),
                std::span<const double>(xyz, 3 * num_edges),
                std::span<const double>(r, num_edges));
        };
        if (h->d) run(*h->d); else run(*h->f);
    } catch (const std::exception& e) {
        h->error = e.what();
        return 1;
    }
    return 0;
}

// Copies a public member vector out as doubles.  out == nullptr returns the
// element count; a too-small capacity returns minus the count; an unknown name -1.
long symref_get(void* handle, const char* name, double* out, long capacity)
{
    auto* h = static_cast<Handle*>(handle);
    return h->d ? get_field(*h->d, name, out, capacity) : get_field(*h->f, name, out, capacity);
}

int symref_info(void* handle, int* out8, double* r_cut)
{
    auto* h = static_cast<Handle*>(handle);
    auto fill = [&](auto& m) {
        out8[0] = m.num_elements; out8[1] = m.num_channels; out8[2] = m.l_max; out8[3] = m.L_max;
        out8[4] = m.num_lme; out8[5] = m.num_lelm1lm2; out8[6] = static_cast<int>(m.Phi1_l.size());
        out8[7] = m.has_zbl ? 1 : 0;
        *r_cut = m.r_cut;
    };
    if (h->d) fill(*h->d); else fill(*h->f);
    return 0;
}

}  // extern "C"
