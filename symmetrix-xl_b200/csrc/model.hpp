// Host-side model container: reads a format-v4 compact MACE JSON file and turns it
// into the flat tables the device kernels consume.  Mirrors what the reference's
// loader and radial-table builder produce (libsymmetrix/source/mace.cpp:2660-2959,
// compact_radial.cpp:227-366, cubic_spline_set.cpp:8-31), with the weights laid
// out for the kernels of this library.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace sxb {

// Coupling structure of one compiled model shape, expanded from the generated
// X-macro lists so that a model file can be matched against it at load time.
struct ShapeTables {
    const char* name;
    int shape_id;                 // 0: hidden 0e, 1: 0e+1o, 2: 0e+1o+2e
    int l_max, hidden_l_max;
    int num_paths, num_rows, num_lme, num_terms;
    std::vector<int> path_l, path_l1, path_l2;
    std::vector<int> term_row, term_lme;
    std::vector<std::vector<int>> m0_terms;   // compiled order, term index = position
    std::vector<int> m0_out;                  // output component of each compiled term
    std::vector<std::vector<int>> m1_terms;
};

const ShapeTables& shape_tables(int shape_id);
int num_compiled_shapes();

struct HostModel {
    int shape_id = -1;
    int num_elements = 0, channels = 0, l_max = 0, hidden_l_max = 0;
    int num_lm = 0, num_hidden = 0, num_paths = 0, num_rows = 0, num_lme = 0, num_terms = 0;
    double r_cut = 0.0;
    std::vector<int> atomic_numbers;
    std::vector<double> atomic_energies;
    std::string selected_head;               // prediction head in use ("" when the file names none)
    std::vector<std::string> available_heads;
    std::vector<int> eta;                    // paths per output l
    std::vector<int> group_begin;            // first lme of each output l

    // radial spline grid
    double spline_x0 = 0.0, spline_h = 0.0;
    int spline_points = 0;
    // Radial networks R0, R1 and the density networks A0, A1: kept in parsed form, because with the
    // Agnesi distance transform the spline tables depend on the species pair and are built per active
    // pair (radial_coefficients below).  Without a transform every pair shares one table.
    bool agnesi = false;
    std::shared_ptr<const void> radial;   // parsed definition, owned by model.cpp
    bool a0_scaled = false, a1_scaled = false;
    // optional screened-Coulomb pair repulsion (libsymmetrix/source/zbl.cpp)
    bool has_zbl = false;
    double zbl_a_exp = 0.0, zbl_a_prefactor = 0.0;
    std::vector<double> zbl_c, zbl_covalent_radii;   // radii indexed by atomic number
    int zbl_p = 0;

    std::vector<double> h0;                  // [A][C]
    std::vector<double> w_a0;                // [A][l][C_in][C_out]
    std::vector<float> m0_weights;           // [A][compiled term][C]
    std::vector<float> m1_weights;           // [A][compiled term][C]
    int m0_num_terms = 0, m1_num_terms = 0;
    std::vector<float> w_h1;                 // [L+1][C_in][C_out]
    std::vector<std::vector<float>> w_a1;    // per l: [eta_l*C][C]
    std::vector<float> h2_skip;              // T[A][C_in][C_out]
    std::vector<float> h2_m1;                // [C_in][C_out]
    std::vector<float> readout1;             // q[C]
    std::vector<float> readout2_w1;          // [hidden][C]
    std::vector<float> readout2_w2;          // [hidden]
    int readout2_hidden = 16;
    float readout2_scale = 1.0f;
    std::vector<float> cg;                   // [compiled term]
    // format versions 1 / 2: the first readout and the H1->H2 skip act on the scalar block of H1 (after the linear),
    // not of M0; h2_skip and readout1 then hold H2_weights_for_H1 and readout_1_weights
    bool legacy_h1_basis = false;
    // format version 4, h1_affine_mode pre_linear_up: both act on x = M0[l=0] P0 + residual[l=0] (P0 = H1_product_weights of
    // l = 0); with first_interaction_residual an element-dependent constant R U joins H1 (libsymmetrix/source/mace.cpp:1759-1888)
    bool pre_linear_up = false, first_residual = false;
    std::vector<float> w_product0;           // [C_in][C_out]
    std::vector<float> residual_fused;       // [A][num_hidden][C]: R U, added to H1
    std::vector<float> residual_scalar;      // [A][C]: R of the scalar block, added to x
    // single-layer models (single_layer_readout): no second message step, the readout polynomial acts on H1
    bool single_layer = false;
    std::vector<int> hidden_poly_terms;      // [term][4]: up to three hidden-component indices, -1 padded
    std::vector<float> hidden_poly_weights;  // [A][term][C]
};

// Throws std::runtime_error / std::invalid_argument with a message naming the key.
// ``head`` selects a prediction head of a multi-head file; empty = the file's default head.
HostModel load_model(const std::string& json_path, const std::string& head = std::string());

// Cubic coefficients [interval][4][functions] (double) of radial network ``name`` ("R0", "R1", "A0",
// "A1") for the species pair (type_i, type_j) - symmetric in the pair; reference:
// libsymmetrix/source/compact_radial.cpp:227-289, 326-366 and cubic_spline_set.cpp:8-31.  Tables are
// cached per unordered pair inside the model.
const std::vector<double>& radial_coefficients(const HostModel& model, const std::string& name, int type_i, int type_j);

// Layer-1 table for the given active types, repacked to [unordered pair][interval][function][4] in
// float; one pair when the model has no distance transform.  ``num_pairs`` receives the pair count.
std::vector<float> build_r1_table(const HostModel& model, const std::vector<int>& active_types, int* num_pairs);

// Density table [ordered pair ai*n+aj][interval][4] in float of network "A0" or "A1".
std::vector<float> build_density_table(const HostModel& model, const std::string& name, const std::vector<int>& active_types);

// Folds H0[type_j] and W_A0[type_i][l] into the layer-0 spline coefficients for the
// given active types (the reference does the same per ordered species pair,
// mace_kokkos_factorized_lifecycle.cpp:3988-4047), in double, rounded once to float.
// Output layout [pair = ai*n+aj][interval][4][(l_max+1)*C].
std::vector<float> fold_r0_table(const HostModel& model, const std::vector<int>& active_types);

}  // namespace sxb
