/* C ABI of the B200 (sm_100a) force-path library: energy, forces and stress of a compact
 * two-layer MACE model.  Plain pointers and sizes only; every array is caller-owned and is
 * copied in or out during the call.  Each entry point names the interface of the reference
 * (bonan-group/symmetrix-xl) that it replaces, by the file's path inside that project.
 *
 * Status: every function returns 0 on success, a negative SXB_ERR_* code otherwise;
 * sxb_last_error() returns the message of the calling thread's last failure.  An evaluator is
 * used by one host thread at a time and owns one CUDA stream.  There is no CPU fallback: a
 * missing or unusable CUDA device makes sxb_create fail.
 */
#ifndef SYMMETRIX_B200_H
#define SYMMETRIX_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SXB_OK 0
#define SXB_ERR_INVALID_ARGUMENT (-1) /* std::invalid_argument in the reference (ValueError in Python) */
#define SXB_ERR_RUNTIME (-2)          /* std::runtime_error / CUDA failure (RuntimeError) */
#define SXB_ERR_STALE_GRAPH (-3)      /* graph generation token does not name the prepared graph */
#define SXB_ERR_CAPACITY (-4)         /* graph exceeds 32-bit edge indexing (std::length_error) */

typedef struct sxb_evaluator sxb_evaluator;

typedef struct sxb_model_info {
    int32_t num_elements;
    int32_t num_channels;
    int32_t l_max;          /* edge harmonics */
    int32_t hidden_l_max;   /* hidden irreps (L_max) */
    int32_t num_paths;      /* layer-1 tensor-product paths */
    int32_t num_lme;        /* layer-1 output components */
    int32_t shape_id;       /* compiled coupling structure in use */
    int32_t single_layer;   /* 1: single_layer_readout model (no second message step) */
    int32_t h1_basis;       /* input of the first readout and the skip: 0 M0 (m0_composite), 1 H1 (format 1 / 2), 2 M0 P0 + residual (pre_linear_up) */
    int32_t reserved;
    double r_cut;
} sxb_model_info;

/* Replaces the evaluator constructor MACEKokkos<float>(filename)
 * (libsymmetrix/source/mace_kokkos_model.cpp:146; loader twin mace.cpp:2660-2959; Python binding
 * symmetrix/source/cpp/mace_kokkos.cpp:262).  Reads a model JSON (format version 4 in the m0_composite or
 * pre_linear_up basis, or format versions 1 / 2; radial networks or stored pair splines; one or two
 * interactions), builds the spline tables and uploads the weights to CUDA device `device_ordinal`. */
int sxb_create(const char* model_json_path, int device_ordinal, sxb_evaluator** out);
/* The same with a named prediction head of a multi-head model file (the `head` argument of the
 * reference constructor; select_prediction_head, libsymmetrix/source/prediction_heads.hpp:10-90):
 * the head's atomic energies, readout weights and ZBL coefficients replace the top-level ones.
 * head NULL or "" selects the file's default head.  sxb_selected_head copies the name in use
 * (empty for a file without heads) into out[capacity]. */
int sxb_create_with_head(const char* model_json_path, int device_ordinal, const char* head, sxb_evaluator** out);
int sxb_selected_head(const sxb_evaluator* evaluator, char* out, int32_t capacity);
/* The names of all heads the file carries (attribute available_heads, symmetrix/source/cpp/mace_kokkos.cpp:2088-2100),
 * joined by newlines into out[capacity]; empty for a file without heads. */
int sxb_available_heads(const sxb_evaluator* evaluator, char* out, int32_t capacity);
/* Parses and validates a model file on the host only (no CUDA device is touched): the structure it
 * would run with, the head that would be selected and that head's atomic energies.  Counterpart of
 * the reference's metadata inspection (libsymmetrix/source/model_metadata.cpp).  Any output pointer
 * may be NULL. */
int sxb_model_file_info(const char* model_json_path, const char* head, sxb_model_info* info, char* selected_head,
                        int32_t head_capacity, double* atomic_energies, int32_t energies_capacity);
void sxb_destroy(sxb_evaluator* evaluator);
const char* sxb_last_error(void);
/* Number of CUDA devices this process can use (0 when there is none or the driver is missing); a
 * multi-rank host maps its ranks onto them (the reference leaves this to Kokkos' device selection). */
int sxb_device_count(void);
/* What the evaluator's `device_cuda_environment` attribute reports about its device
 * (symmetrix/source/cpp/mace_kokkos.cpp:807-828): name, and values[6] = compute capability code (100 for
 * sm_100), multiprocessor count, warp width, CUDA runtime version, driver version, device memory in MiB. */
int sxb_device_properties(int32_t device_ordinal, char* name, int32_t name_capacity, int64_t* values6);

/* Attributes atomic_numbers, atomic_energies, r_cut, num_channels ... of the Python class
 * (symmetrix/source/cpp/mace_kokkos.cpp:2040-2087). */
int sxb_model_info_get(const sxb_evaluator* evaluator, sxb_model_info* out);
int sxb_atomic_numbers(const sxb_evaluator* evaluator, int32_t* out, int32_t capacity);
int sxb_atomic_energies(const sxb_evaluator* evaluator, double* out, int32_t capacity);
/* Bytes of device memory the evaluator's graph and work buffers hold, and the device's free / total
 * memory: the numbers behind the reference's execution-plan report (libsymmetrix/source/execution_plan.hpp:
 * 32-50: estimated_bytes, available_bytes).  Any output may be NULL. */
int sxb_memory_report(const sxb_evaluator* evaluator, int64_t* workspace_bytes, int64_t* device_free_bytes,
                      int64_t* device_total_bytes);

/* Replaces _prepare_periodic_factorized_graph(node_types, positions, cell, inverse_cell,
 * neighbor_cutoff) -> {generation, num_edges} (symmetrix/source/cpp/mace_kokkos.cpp:1580-1603;
 * MACEKokkos::prepare_periodic_factorized_graph, mace_kokkos_factorized_lifecycle.cpp:1934-2316;
 * cell list libsymmetrix/source/neighbor_graph_kokkos.cpp:39-405).  Host arrays:
 * node_types int32[num_nodes] (indices into the model's element list), positions f64[3*num_nodes],
 * cell and inverse_cell f64[9] row-major. */
int sxb_prepare_periodic_graph(sxb_evaluator* evaluator, int32_t num_nodes, const int32_t* node_types,
                               const double* positions, const double* cell, const double* inverse_cell,
                               double neighbor_cutoff, uint64_t* generation, int64_t* num_edges);

/* Replaces _prepare_factorized_graph(num_nodes, node_types, num_neigh, neigh_indices, neigh_types)
 * (symmetrix/source/cpp/mace_kokkos.cpp:1561-1579): a receiver-major CSR graph built by the caller.
 * `shifts` (int32[3*num_edges], periodic image of each source) and `cell` may be NULL when the
 * graph will only be evaluated from explicit edge vectors (sxb_compute_edge_vectors). */
int sxb_prepare_graph(sxb_evaluator* evaluator, int32_t num_nodes, const int32_t* node_types,
                      const int32_t* num_neigh, const int32_t* neigh_indices, const int32_t* shifts,
                      const double* cell, uint64_t* generation);

/* Replace _prepare_factorized_geometry / _prepare_factorized_fractional_geometry (fractional != 0) and
 * _update_factorized_cell (symmetrix/source/cpp/mace_kokkos.cpp:1608-1685; device side
 * update_prepared_factorized_positions_geometry, mace_kokkos_factorized_lifecycle.cpp:2915-3076) for a
 * graph prepared with sxb_prepare_graph without shifts (the calculator's host-graph branch, used for
 * non-periodic and mixed-periodic systems, calculator.py:3274-3359): the reference positions
 * f64[3*num_nodes] (Cartesian, or fractional), the edge vectors of that state f64[3*num_edges] in the
 * caller's edge order (Cartesian, or fractional), the cell pair and the periodic axes int32[3].
 * sxb_compute_positions then moves the edges with the atoms: xyz_ij = ref_xyz_ij + d_j - d_i with the
 * displacements reduced to the nearest image along periodic axes.  sxb_update_cell swaps the cell of a
 * fractional reference (an affine deformation keeps the graph) or of a graph with integer shifts. */
int sxb_prepare_reference_geometry(sxb_evaluator* evaluator, uint64_t generation, int32_t fractional,
                                   const double* reference_positions, const double* reference_xyz, const double* cell,
                                   const double* inverse_cell, const int32_t* pbc);
int sxb_update_cell(sxb_evaluator* evaluator, uint64_t generation, const double* cell, const double* inverse_cell);

/* Copies the prepared graph out in the caller's node order and the reference's edge order
 * (the arrays KokkosNeighborGraph holds: receiver_offsets, sources, shifts;
 * libsymmetrix/source/neighbor_graph_kokkos.hpp:13-23).  first_neigh int32[num_nodes+1],
 * sources int32[num_edges], shifts int32[3*num_edges] (may be NULL). */
int sxb_get_graph(sxb_evaluator* evaluator, uint64_t generation, int32_t* first_neigh, int32_t* sources,
                  int32_t* shifts);

/* Replaces _compute_prepared_factorized_positions(generation, positions)
 * (symmetrix/source/cpp/mace_kokkos.cpp:1828-1836; MACEKokkos::compute_prepared_factorized_positions,
 * mace_kokkos_factorized_lifecycle.cpp:3089-3123 -> compute_node_energies_forces,
 * mace_kokkos_evaluate.cpp:314-611).  positions: host f64[3*num_nodes].  Copies positions to the
 * device, runs the whole forward + reverse pipeline and the force/stress reduction. */
int sxb_compute_positions(sxb_evaluator* evaluator, uint64_t generation, const double* positions);

/* Same evaluation with positions already resident in device memory (f64[3*num_nodes] on the
 * evaluator's device); nothing is copied to the host.  Device-view counterpart of the call above
 * (MACEKokkos::compute_prepared_factorized_positions takes device views inside LAMMPS,
 * pair_symmetrix/pair_symmetrix_mace_kokkos.cpp:1532-1568). */
int sxb_compute_positions_device(sxb_evaluator* evaluator, uint64_t generation, const double* device_positions);

/* Replaces _compute_prepared_factorized(generation, xyz, r) and the one-shot
 * compute_node_energies_forces(num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r)
 * (symmetrix/source/cpp/mace_kokkos.cpp:1817-1827, 2169-2204): edge vectors xyz f64[3*num_edges] in
 * the caller's edge order. */
int sxb_compute_edge_vectors(sxb_evaluator* evaluator, uint64_t generation, const double* xyz);

int sxb_synchronize(sxb_evaluator* evaluator);

/* Results of the last compute, caller node / edge order, all f64.
 * node_energies: property node_energies (mace_kokkos.cpp:2088-2095), [num_nodes].
 * edge_forces:   property node_forces, the directed forces dE/d(xyz_ij) (2096-2102), [3*num_edges];
 *                only filled when enabled with sxb_set_keep_edge_forces.
 * atom forces:   _reduce_atom_forces (2103-2133), [num_nodes][3].
 * stress:        _reduce_stress(volume) (2134-2154), [3][3] = -(1/volume) sum f_ij (x) xyz_ij.
 * energy:        sum of node energies (calculator.py:3821-3858 sums them in f64). */
int sxb_get_node_energies(sxb_evaluator* evaluator, double* out, int64_t capacity);
int sxb_set_keep_edge_forces(sxb_evaluator* evaluator, int32_t enabled);
int sxb_get_edge_forces(sxb_evaluator* evaluator, double* out, int64_t capacity);
int sxb_reduce_atom_forces(sxb_evaluator* evaluator, uint64_t generation, double* out, int64_t capacity);
int sxb_reduce_stress(sxb_evaluator* evaluator, uint64_t generation, double volume, double* out9);
int sxb_get_energy(sxb_evaluator* evaluator, double* out);

/* Graph-less reduction of caller-held directed edge forces: F_j += f_ij, F_i -= f_ij and
 * stress = -(1/volume) sum f_ij (x) xyz_ij.  Replaces _reduce_atom_forces(num_nodes, edge_receivers,
 * edge_sources) and _reduce_stress(volume, xyz) with execution_graph_generation = 0
 * (symmetrix/source/cpp/mace_kokkos.cpp:2103-2154; MACEKokkos::reduce_node_forces / reduce_stress,
 * libsymmetrix/source/mace_kokkos_evaluate.cpp:92-106, 157-186).  Host arrays: edge_receivers,
 * edge_sources int32[num_edges]; edge_forces, xyz f64[3*num_edges]; atom_forces f64[3*num_nodes];
 * stress9 f64[9].  Runs on the current CUDA device and allocates its device buffers per call. */
int sxb_reduce_edge_forces(int32_t num_nodes, int64_t num_edges, const int32_t* edge_receivers,
                           const int32_t* edge_sources, const double* edge_forces, const double* xyz, double volume,
                           double* atom_forces, double* stress9);

/* The same reduction for callers that cannot allocate device memory.  It has no counterpart in
 * the reference.  It exists for hosts that have given all device memory to a pool of their own
 * (a raw cudaMalloc may then fail although the pool has room) and for force callbacks inside a
 * time step, where cudaMalloc / cudaFree would stall the whole device because they synchronise it.
 * Every pointer is a DEVICE pointer on the current CUDA device and the work is only enqueued on
 * `stream` (results are ready once the stream reaches them).  Scratch (per-block virial partials)
 * lives in a static device array inside the library: 1.18 MB per GPU, held until the process
 * exits, enough for at most 4,194,304 edges per call -- larger edge counts are rejected with
 * SXB_ERR_INVALID_ARGUMENT.  The call itself performs no cudaMalloc / cudaFree.  The first call on
 * each device looks up the array's device address; make that first call before any stream capture
 * is open on the device.  All calls share the one array, which keeps the previous call's contents
 * (nothing in it needs clearing: each call rewrites every entry it later reads), so two calls whose
 * kernels can overlap on the GPU -- different streams, or the same stream from two host threads
 * without ordering -- race on it; serialise them.  device_status (may be NULL) receives 1 when an
 * edge names a node outside [0, num_nodes), 0 otherwise; such edges are skipped. */
int sxb_reduce_edge_forces_static(int32_t num_nodes, int64_t num_edges, const int32_t* device_receivers,
                                  const int32_t* device_sources, const double* device_edge_forces,
                                  const double* device_xyz, double volume, double* device_atom_forces,
                                  double* device_stress9, int32_t* device_status, void* stream);

/* Device addresses of the last results (valid until the next prepare/compute): energy f64[1],
 * forces f64[3*num_nodes] in caller order, virial f64[9] = sum f_ij (x) xyz_ij. */
int sxb_device_results(sxb_evaluator* evaluator, const double** energy, const double** forces,
                       const double** virial);

/* Stage tensors of the last compute for parity tests, caller node order, converted to f64:
 * "A0","M0","H1","Phi1","A1","M1","H2","H2_adj","A1_adj","dPhi1","H1_adj","M0_adj","A0_adj"
 * (the public member vectors of the reference's serial evaluator, libsymmetrix/source/mace.hpp).
 * Returns the element count through `count`; out may be NULL to query it. */
int sxb_get_stage(sxb_evaluator* evaluator, const char* name, double* out, int64_t capacity, int64_t* count);

/* Number of kernels this library launched since creation, and device time of the last compute in
 * milliseconds (CUDA events on the evaluator's stream). */
int sxb_launch_count(const sxb_evaluator* evaluator, int64_t* out);
int sxb_last_compute_ms(const sxb_evaluator* evaluator, float* out);

/* ---- Domain-decomposed evaluation (one process per GPU) ------------------------------------------
 * A rank holds `num_receivers` owned atoms followed by its ghost atoms (copies of atoms owned by
 * other ranks, or periodic images of its own, within the halo), num_nodes in total.  Only owned atoms
 * are receivers; ghosts carry H1, H1_adj, a type, a position and a force row.
 *
 * sxb_prepare_local_graph replaces MACEKokkos::prepare_factorized_graph_device(num_receivers,
 * num_feature_nodes, ...) as the LAMMPS pair style calls it
 * (pair_symmetrix/pair_symmetrix_mace_kokkos.cpp:1464-1476; libsymmetrix/source/mace_kokkos.hpp:672-697),
 * building the receiver-major graph of the open (non-periodic) local node set on the device.
 * positions: host f64[3*num_nodes] with ghosts already displaced to their image positions.
 *
 * sxb_distributed_begin / _continue / _finish replace begin_ / continue_ /
 * finish_factorized_distributed_evaluation (libsymmetrix/source/mace_kokkos_evaluate.cpp:1658-1833,
 * 1836-1983, 1986-2101; call sites pair_symmetrix_mace_kokkos.cpp:1568, 1690, 1705):
 *   begin:    geometry, layer 0, M0, H1 of the owned atoms          -> exchange H1 rows of ghosts
 *   continue: layer 1 forward ... fused layer-1 gradient            -> return H1_adj rows of ghosts
 *   finish:   rest of the reverse pass, forces on owned and ghost nodes, energy, virial.
 * Calling them out of order fails with SXB_ERR_INVALID_ARGUMENT and resets the phase (the reference
 * throws std::logic_error).  device_positions: f64[3*num_nodes] on the evaluator's device.
 *
 * sxb_halo_pack / sxb_halo_unpack replace the pair style's pack/unpack_forward_comm_kokkos and
 * pack/unpack_reverse_comm_kokkos kernels (pair_symmetrix_mace_kokkos.cpp:737-1005): rows of H1
 * (which = 0) or H1_adj (which = 1), FP32, [count][num_hidden*num_channels], for the caller-order
 * node indices in device_indices; unpack with accumulate != 0 adds (owners summing ghost adjoints).
 * sxb_add_force_rows adds returned ghost forces f64[count][3] into the owners' force rows after
 * finish (the pair style's force reverse communication, pair_symmetrix_mace_kokkos.cpp:1853-1876).
 * sxb_set_stream makes the evaluator enqueue on the caller's stream (e.g. the one NCCL uses). */
int sxb_prepare_local_graph(sxb_evaluator* evaluator, int32_t num_receivers, int32_t num_nodes, const int32_t* node_types,
                            const double* positions, double neighbor_cutoff, uint64_t* generation, int64_t* num_edges);
int sxb_distributed_begin(sxb_evaluator* evaluator, uint64_t generation, const double* device_positions);
/* The pair style's own form of the two calls above: it hands over ITS neighbor list and, each step,
 * ITS edge vectors.  sxb_prepare_local_graph_csr replaces prepare_factorized_graph_device(num_receivers,
 * num_feature_nodes, node_types, num_neigh, neigh_indices, neigh_types)
 * (libsymmetrix/source/mace_kokkos.hpp:399-413; pair_symmetrix_mace_kokkos.cpp:1380-1476): owned atoms
 * first, ghosts after; num_neigh int32[num_receivers], neigh_indices int32[sum num_neigh] index all
 * num_nodes local nodes; node_types int32[num_nodes].  The three arrays are host pointers, or device
 * pointers on the evaluator's device when pointers_on_device != 0 (Kokkos views in the reference).
 * sxb_distributed_begin_edge_vectors replaces begin_factorized_distributed_evaluation(..., xyz, r,
 * generation) (mace_kokkos.hpp:672-677; pair_symmetrix_mace_kokkos.cpp:1532-1568): device_xyz
 * f64[3*num_edges] in the caller's edge order.  Edges at or beyond the model cutoff (list skin)
 * contribute nothing, whether or not the caller has clamped them to the cutoff as the pair style does. */
int sxb_prepare_local_graph_csr(sxb_evaluator* evaluator, int32_t num_receivers, int32_t num_nodes, const int32_t* node_types,
                                const int32_t* num_neigh, const int32_t* neigh_indices, int32_t pointers_on_device,
                                uint64_t* generation);
int sxb_distributed_begin_edge_vectors(sxb_evaluator* evaluator, uint64_t generation, const double* device_xyz);
/* Host-buffer forms for a plain (non-Kokkos) LAMMPS pair style, whose halo exchange runs through the
 * host callbacks pack/unpack_forward_comm and pack/unpack_reverse_comm
 * (pair_symmetrix/pair_symmetrix_mace.cpp:261-307, 443-646): sxb_distributed_begin_host takes host
 * positions f64[3*num_nodes] (a graph without periodic shifts uses plain differences x_j - x_i, the
 * ghosts being explicit atoms); sxb_halo_rows_get / _put copy the caller-order rows
 * [first_row, first_row + count) of H1 (which = 0) or H1_adj (which = 1) to / from host floats
 * [count][num_hidden*num_channels]; put with accumulate != 0 adds. */
int sxb_distributed_begin_host(sxb_evaluator* evaluator, uint64_t generation, const double* host_positions);
int sxb_halo_rows_get(sxb_evaluator* evaluator, int32_t which, int64_t first_row, int64_t count, float* host_out);
int sxb_halo_rows_put(sxb_evaluator* evaluator, int32_t which, int64_t first_row, int64_t count, const float* host_in,
                      int32_t accumulate);
int sxb_distributed_continue(sxb_evaluator* evaluator);
int sxb_distributed_finish(sxb_evaluator* evaluator);
int sxb_halo_pack(sxb_evaluator* evaluator, int32_t which, const int32_t* device_indices, int64_t count, float* device_out);
int sxb_halo_unpack(sxb_evaluator* evaluator, int32_t which, const int32_t* device_indices, int64_t count,
                    const float* device_in, int32_t accumulate);
int sxb_add_force_rows(sxb_evaluator* evaluator, const int32_t* device_indices, int64_t count, const double* device_in);
/* Exchange without staging copies.  Ghost nodes follow the receivers in every node tensor, in the
 * caller's ghost order, so a rank that orders its ghosts by owner can receive H1 rows straight into,
 * and send H1_adj rows straight from, the tail of the tensor: sxb_halo_tensor returns the device
 * address of H1 (which = 0) or H1_adj (which = 1), the floats per row and the row at which the ghosts
 * start (counterpart of the public views H1 / H1_adj of MACEKokkos, libsymmetrix/source/mace_kokkos.hpp:
 * 672-708, that the pair style packs from and unpacks into).
 * sxb_gather_position_rows: out[k] = rows[indices[k]] (+ offsets[k]), three doubles per row -- the
 * positions of the owned atoms that other ranks hold as ghosts, displaced to their images (the pair
 * style leaves this to LAMMPS' own forward communication of x).
 * sxb_pack_ghost_forces / sxb_unpack_ghost_forces: the closing exchange after finish.  The send buffer
 * holds, per peer p, the force rows of the ghosts p owns (ghost_begin[p] .. ghost_begin[p+1]) followed
 * by four rows carrying this rank's energy and virial; unpack adds the returned rows into the owners'
 * force rows (send_begin / indices = the rank's send list) and sums the totals of all ranks in rank
 * order into totals_out f64[10], so the energy / virial reduction needs no collective of its own
 * (pair style: reverse communication of f, pair_symmetrix_mace_kokkos.cpp:1853-1876, and LAMMPS' own
 * reductions of eng_vdwl / virial).  Buffers: f64[(rows + 4*world)*3]; the *_begin arrays are device
 * int32[world+1]. */
int sxb_halo_tensor(sxb_evaluator* evaluator, int32_t which, float** device_tensor, int64_t* row_floats, int64_t* first_ghost_row);
int sxb_gather_position_rows(sxb_evaluator* evaluator, const double* device_rows, const int32_t* device_indices, int64_t count,
                             const double* device_offsets, double* device_out);
int sxb_pack_ghost_forces(sxb_evaluator* evaluator, int32_t world, const int32_t* device_ghost_begin, int64_t num_ghosts,
                          double* device_out);
int sxb_unpack_ghost_forces(sxb_evaluator* evaluator, int32_t world, const int32_t* device_send_begin,
                            const int32_t* device_indices, int64_t num_rows, const double* device_in, double* device_totals_out);
/* Folds the packing into the phases (and into their captured CUDA graphs): with a plan set, begin ends
 * by gathering the H1 rows `device_send_indices` into `device_send_rows`, finish starts by adding
 * `device_received_rows` into the H1_adj rows of those same atoms and ends by filling
 * `device_force_send` as sxb_pack_ghost_forces does.  The caller then only moves buffers between the
 * phases.  Device pointers, valid until the next graph preparation (which clears the plan); calling
 * with num_send = 0 and NULL indices also clears it.  The reference's pair style keeps the equivalent
 * send lists inside LAMMPS' Comm (pair_symmetrix_mace_kokkos.cpp:737-1005). */
int sxb_set_halo_plan(sxb_evaluator* evaluator, const int32_t* device_send_indices, int64_t num_send, float* device_send_rows,
                      const float* device_received_rows, int32_t world, const int32_t* device_ghost_begin,
                      double* device_force_send);
/* For a caller that captured one whole decomposed step (the three phases and its own exchanges) into a
 * CUDA graph on the evaluator's stream and now replays it: declares that the phases have run, so that
 * sxb_synchronize and the result getters behave as after sxb_distributed_finish; `launches` = kernels of
 * this library inside the replayed graph (added to sxb_launch_count).  No counterpart in the reference,
 * which launches its kernels one by one. */
int sxb_distributed_replayed(sxb_evaluator* evaluator, uint64_t generation, int64_t launches);
/* Abandons an evaluation that is open between the phases (the reference resets its phase when a phase
 * call throws, libsymmetrix/source/mace_kokkos_evaluate.cpp:1737-1746): the next call must be a begin. */
int sxb_distributed_abort(sxb_evaluator* evaluator);
int sxb_set_stream(sxb_evaluator* evaluator, void* stream);

/* ---- Halo exchange over NVLink peer memory ---------------------------------------------------------
 * Replaces the MPI brick swaps of the reference's pair style (pair_symmetrix_mace_kokkos.cpp:737-1005,
 * 1568-1705) inside one node: every rank maps its peers' receive buffers (CUDA IPC) and an exchange is a
 * push kernel (16-byte stores into the peers' buffers, then a release store of an arrival flag) followed
 * by a wait kernel with a time limit; no collective, no staging copy, capturable into a CUDA graph.
 *   sxb_device_alloc / _free   plain cudaMalloc'd, zeroed buffers (IPC handles exist only for those)
 *   sxb_ipc_export             64-byte handle of such a buffer (or of sxb_halo_tensor's allocation)
 *   sxb_peer_create            this rank's exchange object; sxb_peer_flags = its flag table (export it)
 *   sxb_peer_open              maps a peer's buffer from its handle (closed by sxb_peer_destroy)
 *   sxb_peer_plan              exchange `phase` (0..3): my outgoing rows `send` ordered by destination
 *                              (send_begin int64[world+1], rows of row_bytes), the address of my segment in
 *                              every peer's receive buffer, and every peer's flag table; optionally a gather
 *                              list over a local tensor, a scatter list into the peers' tensors, and add mode
 *   sxb_peer_advance           enqueue: next step (once per evaluation, before its first exchange)
 *   sxb_peer_exchange          enqueue: push my rows of `phase`, then wait for every peer's
 *   sxb_peer_status            after a synchronisation: 0, or 32 when a wait ran out (ten seconds unless
 *                              sxb_peer_set_wait_limit changed it); the results of that step are then invalid,
 *                              the CUDA context stays usable
 * Every rank must run the same sequence of exchanges. */
typedef struct PeerExchange sxb_peer_exchange_t;
int sxb_device_alloc(int32_t device_ordinal, int64_t bytes, void** out);
int sxb_device_free(void* pointer);
int sxb_ipc_export(const void* device_pointer, unsigned char* handle64);
int sxb_peer_create(int32_t device_ordinal, int32_t rank, int32_t world, sxb_peer_exchange_t** out);
int sxb_peer_flags(sxb_peer_exchange_t* exchange, void** flags);
int sxb_peer_status(sxb_peer_exchange_t* exchange, int32_t* out);
int sxb_peer_open(sxb_peer_exchange_t* exchange, const unsigned char* handle64, void** out);
int sxb_peer_plan(sxb_peer_exchange_t* exchange, int32_t phase, const void* send, const int64_t* send_begin, int32_t row_bytes,
                  void* const* remote_pointers, void* const* remote_flags, const int32_t* device_row_source,
                  const int32_t* device_row_dest, int32_t accumulate);
/* out[k] = row of the evaluator's node tensors (H1, H1_adj) that holds caller-order node indices[k]; device
 * arrays.  Lets an exchange gather from, or add into, those tensors directly (row_source / row_dest above). */
int sxb_internal_rows(sxb_evaluator* evaluator, const int32_t* device_indices, int64_t count, int32_t* device_out);
int sxb_peer_advance(sxb_peer_exchange_t* exchange, void* stream);
int sxb_peer_exchange(sxb_peer_exchange_t* exchange, int32_t phase, void* stream);
int sxb_peer_set_wait_limit(sxb_peer_exchange_t* exchange, double seconds);
int sxb_peer_destroy(sxb_peer_exchange_t* exchange);

/* Tiled streaming (the reference's fixed-workspace dual-layer plan, allow_fixed_workspace:
 * libsymmetrix/source/mace_kokkos_evaluate.cpp:755-1148, workspace
 * mace_kokkos_factorized_lifecycle.cpp:1353-1569): receivers are processed in tiles of
 * `receivers_per_tile` with one reusable workspace in three sweeps (layer 0 -> H1; layer 1 forward
 * and its fused gradient; layer-0 forward recomputed, then the layer-0 gradient).  Graph-wide state
 * is H1, H1_adj, M0, the readout adjoint and the outputs only.  0 switches tiling off.  The setting
 * invalidates the prepared graph; prepare again afterwards. */
int sxb_set_tile_size(sxb_evaluator* evaluator, int32_t receivers_per_tile);

/* Reproducible mode (off by default).  The default kernels add the source adjoint H1_adj and the forces
 * on source atoms with atomics, whose order -- and so the last bits of the results -- varies between
 * runs.  With this mode on, the kernels leave one record per edge and fixed-order passes sum them over a
 * source-sorted schedule, the device counterpart of the reference's source schedule and source-owner
 * accumulation (source_offsets / source_edges, libsymmetrix/source/mace_kokkos_factorized_lifecycle.cpp:
 * 2133-2195; symmetrix/source/symmetrix/jit_codegen.py:1018-1109): two evaluations of one input give
 * identical bits.  Costs 4*num_hidden*num_channels bytes per edge (refused above 16 GB), so it is meant
 * for small and medium systems; not available for hidden irreps 0e+1o+2e or density-scaled models.
 * The setting invalidates the prepared graph; prepare again afterwards. */
int sxb_set_deterministic(sxb_evaluator* evaluator, int32_t enabled);

/* Per-stage device times of the last compute (CUDA events on the evaluator's stream around each
 * kernel group), collected only while profiling is enabled; counterpart of the reference's per-stage
 * counters (factorized_last_evaluation_ms ..., libsymmetrix/source/mace_kokkos.hpp:1431-1454).
 * sxb_profile_entry returns the number of entries through `count`; index outside [0,count) only
 * reports the count. */
int sxb_set_profiling(sxb_evaluator* evaluator, int32_t enabled);
int sxb_profile_entry(const sxb_evaluator* evaluator, int32_t index, char* name, int32_t name_capacity, float* ms,
                      int32_t* launches, int32_t* count);

/* Measured denominators for the rooflines of the edge kernels on CUDA device `device_ordinal`: the
 * FP32 FMA rate of the CUDA cores (TFLOP/s, 2 flop per FMA) and the L2-to-SM read bandwidth on an
 * L2-resident 32 MB table read 512 contiguous bytes per warp at warp-random rows (GB/s), each from a
 * probe kernel of a few milliseconds timed with CUDA events.  No counterpart in the reference (its
 * documentation quotes vendor peaks).  Either output pointer may be NULL to skip that probe. */
int sxb_measure_device_peaks(int32_t device_ordinal, double* fp32_fma_tflops, double* l2_read_gbs);

#ifdef __cplusplus
}
#endif
#endif
