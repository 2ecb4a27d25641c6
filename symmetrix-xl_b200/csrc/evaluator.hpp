// Evaluator class behind the C ABI (include/symmetrix_b200.h).
#pragma once

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"
#include <cuda.h>

#include "model.hpp"
#include "row_map.hpp"

namespace sxb {


struct StaleGraph : std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};

class Evaluator {
public:
    Evaluator(const std::string& json_path, int device_ordinal, const std::string& head = std::string());
    ~Evaluator();
    Evaluator(const Evaluator&) = delete;
    Evaluator& operator=(const Evaluator&) = delete;

    const HostModel& model() const { return model_; }
    int num_nodes() const { return num_nodes_; }
    int num_receivers() const { return num_receivers_; }
    long num_edges() const { return num_edges_; }
    std::uint64_t generation() const { return generation_; }

    // num_receivers < num_nodes: only the first num_receivers nodes own edges (the others are ghosts)
    std::pair<std::uint64_t, long> prepare_periodic_graph(int num_nodes, const int* node_types, const double* positions,
                                                          const double* cell, const double* inverse_cell, double cutoff,
                                                          int num_receivers = -1);
    std::uint64_t prepare_graph(int num_nodes, const int* node_types, const int* num_neigh, const int* neigh_indices,
                                const int* shifts, const double* cell);
    std::uint64_t prepare_graph_csr(int num_receivers, int num_nodes, const int* node_types, const int* num_neigh,
                                    const int* neigh_indices, bool on_device);
    void prepare_reference_geometry(std::uint64_t generation, bool fractional, const double* reference_positions,
                                    const double* reference_xyz, const double* cell, const double* inverse_cell, const int* pbc);
    void update_cell(std::uint64_t generation, const double* cell, const double* inverse_cell);
    void get_graph(std::uint64_t generation, int* first, int* sources, int* shifts);
    void check_generation(std::uint64_t generation) const;

    void compute_positions(std::uint64_t generation, const double* positions, bool on_device);
    void compute_edge_vectors(std::uint64_t generation, const double* xyz);
    void synchronize();
    void distributed_begin(std::uint64_t generation, const double* device_positions);
    void distributed_begin_edge_vectors(std::uint64_t generation, const double* device_xyz);
    void distributed_continue();
    void distributed_finish();
    void pack_rows(int which, const int* device_indices, long count, float* device_out);
    void unpack_rows(int which, const int* device_indices, long count, const float* device_in, bool accumulate);
    void add_force_rows(const int* device_indices, long count, const double* device_in);
    void internal_rows(const int* device_indices, long count, int* device_out);
    void mark_phases_replayed(std::uint64_t generation, long launches);
    void abort_phases();
    void set_halo_plan(const int* send_indices, long num_send, float* send_rows, const float* received_rows, int world,
                       const int* ghost_begin, double* force_send);
    void get_halo_rows(int which, long first_row, long count, float* host_out);
    void put_halo_rows(int which, long first_row, long count, const float* host_in, bool accumulate);
    void distributed_begin_host(std::uint64_t generation, const double* host_positions);
    void gather_position_rows(const double* device_rows, const int* device_indices, long count, const double* device_offsets,
                              double* device_out);
    void pack_ghost_forces(int world, const int* device_ghost_begin, long num_ghosts, double* device_out);
    void unpack_ghost_forces(int world, const int* device_send_begin, const int* device_indices, long num_rows,
                             const double* device_in, double* device_totals_out);
    float* halo_tensor(int which);
    int halo_row_floats() const { return model_.num_hidden * model_.channels; }
    void set_stream(cudaStream_t stream);
    // Tiled streaming: receivers are processed in tiles of this many with one reusable workspace
    // (0 = one tile holding every receiver).  Takes effect at the next graph preparation.
    void set_tile_size(int receivers_per_tile);
    // Reproducible mode: every accumulation in a fixed order (no atomics); takes effect at the next graph preparation.
    void set_deterministic(bool enabled);
    int tile_capacity() const;

    void get_node_energies(double* out);
    void get_atom_forces(double* out);
    void get_edge_forces(double* out);
    void set_keep_edge_forces(bool enabled);
    void get_stress(double volume, double* out9);
    double energy() const;
    long get_stage(const std::string& name, double* out, long capacity);
    const double* device_energy() const { return totals_.ptr; }
    const double* device_forces() const { return forces_out_.ptr; }
    const double* device_virial() const { return totals_.ptr + 1; }
    long launches() const { return launches_; }
    std::size_t workspace_bytes() const
    {
        return geom_.bytes() + A0_.bytes() + A0_adj_.bytes() + M0_.bytes() + M0_adj_.bytes() + H1_.bytes() + H1_adj_.bytes() + Phi1_.bytes()
               + dPhi1_.bytes() + A1_.bytes() + A1_adj_.bytes() + M1_.bytes() + M1_adj_.bytes() + H2_.bytes() + H2_adj_.bytes()
               + first_.bytes() + sources_.bytes() + shifts_.bytes() + edge_map_.bytes() + first_caller_.bytes() + sources_caller_.bytes()
               + shifts_caller_.bytes() + forces_.bytes() + forces_out_.bytes() + positions_.bytes() + edge_forces_.bytes()
               + r0_table_.bytes() + r1_table_.bytes();
    }
    // Per-kernel device times of the last compute (CUDA events on the evaluator's stream), only
    // collected while profiling is switched on.
    void set_profiling(bool enabled) { profiling_ = enabled; }
    struct ProfileEntry { std::string name; float ms; int launches; };
    const std::vector<ProfileEntry>& profile() const { return profile_; }
    float last_ms() const { return last_ms_; }
    void require_results() const;

private:
    void prepare_active_types(const std::vector<int>& node_types);
    void install_graph(int num_receivers, int num_nodes, const std::vector<int>& node_types, long num_edges, bool has_shifts);
    void run_pipeline(int phases);
    void enqueue_phases(int phases, const double* positions, bool upload_staged);
    void drop_step_graphs();
    // one captured step per phase mask (7: whole evaluation; 1, 2, 4: the distributed phases)
    struct StepGraph {
        cudaGraphExec_t exec = nullptr;
        std::uint64_t generation = 0;
        const double* positions = nullptr;
        bool upload_staged = false;
        bool keep_edge_forces = false;
        long launches = 0;
    };
    std::map<int, StepGraph> step_graphs_;
    struct HaloPlan {
        bool active = false;
        const int* send_indices = nullptr;
        long num_send = 0;
        float* send_rows = nullptr;
        const float* received_rows = nullptr;
        int world = 0;
        const int* ghost_begin = nullptr;
        double* force_send = nullptr;
    };
    HaloPlan halo_plan_;
    bool use_graphs_ = true;
    void finish_compute();
    void launch_gemm(const float* A, const RowMap& a_rows, const float* B, int ldb, bool b_transposed, float* C,
                     const RowMap& c_rows, int first_node, int num_nodes, int N, int K, bool accumulate, const float* bias);

    int device_ = 0;
    cudaStream_t stream_ = nullptr;
    cudaEvent_t event_begin_ = nullptr, event_end_ = nullptr;
    HostModel model_;
    std::vector<int> active_types_;
    std::vector<int> type_begin_;

    // model tables on the device
    DeviceBuffer<float> density0_table_, density1_table_, inv_scale0_, inv_scale1_, dot0_, dot1_;
    DeviceBuffer<float> r0_table_, r1_table_, m0_weights_, m1_weights_, w_h1_, w_a1_[4], h2_skip_, h2_m1_;
    // pre_linear_up basis: x = M0[l=0] P0 (+ residual) and its adjoint per receiver; residual-first constants per element
    DeviceBuffer<float> scalar_input_, scalar_adjoint_, residual_fused_, residual_scalar_;
    DeviceBuffer<int> hidden_poly_terms_;          // single-layer models: monomials of the readout polynomial over H1
    DeviceBuffer<float> hidden_poly_weights_;
    DeviceBuffer<float> readout1_, readout2_w1_, readout2_w2_;
    // the same weights split into TF32-exact high part and residual, stored [N][K] (K contiguous)
    // for the product with W ("fwd", C = A W) and with W^T ("rev", C = A W^T)
    struct SplitWeight {
        DeviceBuffer<float> fwd_hi, fwd_lo, rev_hi, rev_lo, full;
        int rows = 0, cols = 0;   // W is [rows = K of fwd][cols = N of fwd]
        CUtensorMap map_fwd_hi, map_fwd_lo, map_rev_hi, map_rev_lo;   // [N][K] tensors, box [n_tile][32]
        CUtensorMap wide_fwd_hi, wide_fwd_lo, wide_rev_hi, wide_rev_lo;   // the same with box [min(N, 128)][32]
    };
    SplitWeight s_h1_[4], s_a1_[4], s_h2_m1_;
    std::vector<SplitWeight> s_h2_skip_;
    SplitWeight s_product0_;          // P0 of the pre_linear_up basis
    bool use_tensor_cores_ = true;
    int num_sms_ = 148;
    int r1_pair_types_ = 1;   // active types the layer-1 table distinguishes (1 without a distance transform)
    // scratch of the cell-list build and of the graph installation (kept between rebuilds)
    DeviceBuffer<double> nb_wrapped_pos_, nb_sorted_pos_;
    DeviceBuffer<int> nb_wrap_count_, nb_atom_bin_, nb_atom_index_, nb_sorted_bin_, nb_sorted_atoms_, nb_bin_sizes_, nb_bin_begin_, ig_counts_;
    DeviceBuffer<long long> nb_counts_, nb_offsets_;
    DeviceBuffer<unsigned char> nb_temp_, ig_temp_;
    DeviceBuffer<float> zbl_pairs_;    // [active pair][4]: 1/a, 14.3996 Z_i Z_j, r_max, pad (models with ZBL)
    bool use_tma_activations_ = true;   // operand-streaming form of the tensor-core linears (N in {32, 64, 128})
    int poly_g_forward_ = 1, poly_g_reverse_ = 1;   // nodes per thread in the symmetric-contraction kernels
    void upload_split(SplitWeight& out, const float* w, int rows, int cols);
    struct TcCall {
        const float* A; RowMap a_rows; const SplitWeight* w; bool reverse; float* C; RowMap c_rows;
        int first_node, num_nodes; bool accumulate; const float* bias;
    };
    void launch_tc(const std::vector<TcCall>& calls);
    DeviceBuffer<double> atomic_energies_;
    CouplingConstants coupling_;
    SplineGrid grid_;

    // prepared graph
    std::uint64_t generation_ = 0;
    int num_nodes_ = 0, num_receivers_ = 0;
    int phase_ = 0;
    int tile_size_ = 0;
    bool owns_stream_ = true;
    bool pending_finish_ = false;
    long num_edges_ = 0;
    bool has_shifts_ = false;
    DeviceBuffer<int> first_caller_, sources_caller_, shifts_caller_;
    DeviceBuffer<int> first_, sources_, shifts_, edge_map_, original_, internal_of_;
    DeviceBuffer<unsigned char> atype_, element_;
    DeviceBuffer<double> cell_, inv_cell_, positions_;
    // reference state of a caller-built graph: 0 none, 1 Cartesian, 2 fractional
    DeviceBuffer<double> reference_positions_, reference_xyz_;
    int geometry_mode_ = 0, pbc_mask_ = 0;

    // work buffers
    DeviceBuffer<EdgeGeom> geom_;
    DeviceBuffer<float> A0_, A0_adj_, M0_, M0_adj_, H1_, H1_adj_, Phi1_, dPhi1_, A1_, A1_adj_, M1_, M1_adj_, H2_, H2_adj_;
    DeviceBuffer<double> node_energies_, node_energies_out_, forces_, forces_out_, edge_forces_;
    DeviceBuffer<double> totals_, energy_slots_, virial_slots_;
    bool deterministic_ = false;
    DeviceBuffer<float> edge_source_adjoint_;                 // [E][num_hidden][C] records of the reproducible mode
    DeviceBuffer<int> source_offsets_, source_edges_;         // source schedule: edges sorted by source
    DeviceBuffer<int> det_sorted_sources_, det_edge_ids_, det_counts_;
    DeviceBuffer<double> det_partials_;
    DeviceBuffer<float> halo_stage_;         // rows of H1 / H1_adj on their way to or from host buffers
    DeviceBuffer<double> edge_scratch_;      // [E][3]: caller edge vectors on the way in, un-permuted edge forces on the way out
    DeviceBuffer<int> error_flag_;
    double host_totals_[10] = {0};
    // pinned host mirror of the per-node results, filled by calls that take host inputs so that the
    // result getters cost a host copy instead of a device copy and a synchronisation each
    double* host_results_ = nullptr;         // mapped: [status, totals[10], energies[receivers], forces[nodes][3]]
    double* host_stage_ = nullptr;           // pinned staging copy of the caller's positions
    std::size_t host_results_capacity_ = 0;  // doubles
    bool mirror_valid_ = false;
    bool keep_edge_forces_ = false;
    bool have_results_ = false;
    long launches_ = 0;
    float last_ms_ = 0.0f;
    bool profiling_ = false;
    struct Span { std::string name; cudaEvent_t begin, end; int launches; };
    std::vector<Span> spans_;
    std::vector<cudaEvent_t> event_pool_;
    std::size_t events_used_ = 0;
    std::vector<ProfileEntry> profile_;
    cudaEvent_t pooled_event();
    void span_begin(const char* name);
    void span_end();
    long span_launch_mark_ = 0;
};

}  // namespace sxb
