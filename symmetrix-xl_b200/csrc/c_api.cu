// extern "C" boundary (include/symmetrix_b200.h): translates exceptions into status codes and a
// thread-local message, the way the reference's Python binding turns C++ exceptions into
// ValueError / RuntimeError (symmetrix/source/cpp/mace_kokkos.cpp).
#include "../../include/symmetrix_b200.h"

#include <algorithm>
#include <cstring>
#include <vector>
#include <new>
#include <string>

#include "evaluator.hpp"

struct sxb_evaluator {
    sxb::Evaluator impl;
    sxb_evaluator(const char* path, int device, const char* head) : impl(path, device, head ? head : "") {}
};

namespace {
thread_local std::string g_last_error;
}  // namespace

namespace sxb {
void set_last_error(const std::string& message) { g_last_error = message; }
}  // namespace sxb

namespace {

template <typename F>
int guarded(F&& body)
{
    try {
        body();
        return SXB_OK;
    } catch (const sxb::StaleGraph& e) {
        g_last_error = e.what();
        return SXB_ERR_STALE_GRAPH;
    } catch (const std::length_error& e) {
        g_last_error = e.what();
        return SXB_ERR_CAPACITY;
    } catch (const std::invalid_argument& e) {
        g_last_error = e.what();
        return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::logic_error& e) {
        g_last_error = e.what();
        return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return SXB_ERR_RUNTIME;
    } catch (...) {
        g_last_error = "unknown failure";
        return SXB_ERR_RUNTIME;
    }
}

void require(const void* p, const char* what)
{
    if (p == nullptr) throw std::invalid_argument(std::string(what) + " must not be NULL.");
}
}  // namespace

extern "C" {

const char* sxb_last_error(void) { return g_last_error.c_str(); }

int sxb_device_count(void)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return count;
}

int sxb_device_properties(int32_t device_ordinal, char* name, int32_t name_capacity, int64_t* values6)
{
    return guarded([&] {
        if (name == nullptr || name_capacity <= 0 || values6 == nullptr) throw std::invalid_argument("NULL output argument.");
        int count = 0;
        if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
            cudaGetLastError();
            throw std::runtime_error("No CUDA device is available.");
        }
        if (device_ordinal < 0 || device_ordinal >= count) throw std::invalid_argument("CUDA device ordinal is out of range.");
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) throw std::runtime_error("cudaGetDeviceProperties failed.");
        std::snprintf(name, static_cast<std::size_t>(name_capacity), "%s", prop.name);
        int runtime = 0, driver = 0;
        cudaRuntimeGetVersion(&runtime);
        cudaDriverGetVersion(&driver);
        values6[0] = prop.major * 10 + prop.minor;
        values6[1] = prop.multiProcessorCount;
        values6[2] = prop.warpSize;
        values6[3] = runtime;
        values6[4] = driver;
        values6[5] = static_cast<int64_t>(prop.totalGlobalMem >> 20);
    });
}

int sxb_create(const char* model_json_path, int device_ordinal, sxb_evaluator** out)
{
    return guarded([&] {
        require(model_json_path, "model_json_path");
        require(out, "out");
        *out = new sxb_evaluator(model_json_path, device_ordinal, nullptr);
    });
}

int sxb_create_with_head(const char* model_json_path, int device_ordinal, const char* head, sxb_evaluator** out)
{
    return guarded([&] {
        require(model_json_path, "model_json_path");
        require(out, "out");
        *out = new sxb_evaluator(model_json_path, device_ordinal, head);
    });
}

int sxb_model_file_info(const char* model_json_path, const char* head, sxb_model_info* info, char* selected_head,
                        int32_t head_capacity, double* atomic_energies, int32_t energies_capacity)
{
    return guarded([&] {
        require(model_json_path, "model_json_path");
        const sxb::HostModel m = sxb::load_model(model_json_path, head ? head : "");
        if (info != nullptr) {
            info->num_elements = m.num_elements; info->num_channels = m.channels; info->l_max = m.l_max;
            info->hidden_l_max = m.hidden_l_max; info->num_paths = m.num_paths; info->num_lme = m.num_lme;
            info->shape_id = m.shape_id; info->single_layer = m.single_layer ? 1 : 0; info->h1_basis = m.legacy_h1_basis ? 1 : m.pre_linear_up ? 2 : 0; info->reserved = 0; info->r_cut = m.r_cut;
        }
        if (selected_head != nullptr) {
            if (head_capacity <= static_cast<int32_t>(m.selected_head.size()))
                throw std::invalid_argument("head name buffer is too small.");
            std::memcpy(selected_head, m.selected_head.c_str(), m.selected_head.size() + 1);
        }
        if (atomic_energies != nullptr) {
            if (energies_capacity < m.num_elements) throw std::invalid_argument("atomic_energies buffer is too small.");
            for (int a = 0; a < m.num_elements; ++a) atomic_energies[a] = m.atomic_energies[a];
        }
    });
}

int sxb_selected_head(const sxb_evaluator* ev, char* out, int32_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator");
        require(out, "out");
        const std::string& name = ev->impl.model().selected_head;
        if (capacity <= static_cast<int32_t>(name.size())) throw std::invalid_argument("head name buffer is too small.");
        std::memcpy(out, name.c_str(), name.size() + 1);
    });
}

int sxb_available_heads(const sxb_evaluator* ev, char* out, int32_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator");
        require(out, "out");
        std::string joined;
        for (const std::string& name : ev->impl.model().available_heads) {
            if (!joined.empty()) joined += '\n';
            joined += name;
        }
        if (capacity <= static_cast<int32_t>(joined.size())) throw std::invalid_argument("head name buffer is too small.");
        std::memcpy(out, joined.c_str(), joined.size() + 1);
    });
}

void sxb_destroy(sxb_evaluator* evaluator) { delete evaluator; }

int sxb_model_info_get(const sxb_evaluator* ev, sxb_model_info* out)
{
    return guarded([&] {
        require(ev, "evaluator");
        require(out, "out");
        const auto& m = ev->impl.model();
        out->num_elements = m.num_elements;
        out->num_channels = m.channels;
        out->l_max = m.l_max;
        out->hidden_l_max = m.hidden_l_max;
        out->num_paths = m.num_paths;
        out->num_lme = m.num_lme;
        out->shape_id = m.shape_id;
        out->single_layer = m.single_layer ? 1 : 0;
        out->h1_basis = m.legacy_h1_basis ? 1 : m.pre_linear_up ? 2 : 0;
        out->reserved = 0;
        out->r_cut = m.r_cut;
    });
}

int sxb_atomic_numbers(const sxb_evaluator* ev, int32_t* out, int32_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator");
        require(out, "out");
        const auto& z = ev->impl.model().atomic_numbers;
        if (capacity < static_cast<int32_t>(z.size())) throw std::invalid_argument("atomic_numbers buffer is too small.");
        for (std::size_t i = 0; i < z.size(); ++i) out[i] = z[i];
    });
}

int sxb_atomic_energies(const sxb_evaluator* ev, double* out, int32_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator");
        require(out, "out");
        const auto& e = ev->impl.model().atomic_energies;
        if (capacity < static_cast<int32_t>(e.size())) throw std::invalid_argument("atomic_energies buffer is too small.");
        for (std::size_t i = 0; i < e.size(); ++i) out[i] = e[i];
    });
}

int sxb_memory_report(const sxb_evaluator* ev, int64_t* workspace_bytes, int64_t* device_free_bytes, int64_t* device_total_bytes)
{
    return guarded([&] {
        require(ev, "evaluator");
        std::size_t free_bytes = 0, total_bytes = 0;
        SXB_CUDA(cudaMemGetInfo(&free_bytes, &total_bytes));
        if (workspace_bytes) *workspace_bytes = static_cast<int64_t>(ev->impl.workspace_bytes());
        if (device_free_bytes) *device_free_bytes = static_cast<int64_t>(free_bytes);
        if (device_total_bytes) *device_total_bytes = static_cast<int64_t>(total_bytes);
    });
}

int sxb_prepare_periodic_graph(sxb_evaluator* ev, int32_t num_nodes, const int32_t* node_types, const double* positions,
                               const double* cell, const double* inverse_cell, double neighbor_cutoff, uint64_t* generation,
                               int64_t* num_edges)
{
    return guarded([&] {
        require(ev, "evaluator"); require(node_types, "node_types"); require(positions, "positions");
        require(cell, "cell"); require(inverse_cell, "inverse_cell"); require(generation, "generation");
        const auto result = ev->impl.prepare_periodic_graph(num_nodes, node_types, positions, cell, inverse_cell, neighbor_cutoff);
        *generation = result.first;
        if (num_edges != nullptr) *num_edges = result.second;
    });
}

int sxb_prepare_graph(sxb_evaluator* ev, int32_t num_nodes, const int32_t* node_types, const int32_t* num_neigh,
                      const int32_t* neigh_indices, const int32_t* shifts, const double* cell, uint64_t* generation)
{
    return guarded([&] {
        require(ev, "evaluator"); require(node_types, "node_types"); require(num_neigh, "num_neigh");
        require(neigh_indices, "neigh_indices"); require(generation, "generation");
        *generation = ev->impl.prepare_graph(num_nodes, node_types, num_neigh, neigh_indices, shifts, cell);
    });
}

int sxb_prepare_reference_geometry(sxb_evaluator* ev, uint64_t generation, int32_t fractional, const double* reference_positions,
                                   const double* reference_xyz, const double* cell, const double* inverse_cell, const int32_t* pbc)
{
    return guarded([&] {
        require(ev, "evaluator"); require(reference_positions, "reference_positions"); require(cell, "cell");
        require(inverse_cell, "inverse_cell"); require(pbc, "pbc");
        if (ev->impl.num_edges() > 0) require(reference_xyz, "reference_xyz");
        ev->impl.prepare_reference_geometry(generation, fractional != 0, reference_positions, reference_xyz, cell, inverse_cell, pbc);
    });
}

int sxb_update_cell(sxb_evaluator* ev, uint64_t generation, const double* cell, const double* inverse_cell)
{
    return guarded([&] {
        require(ev, "evaluator"); require(cell, "cell"); require(inverse_cell, "inverse_cell");
        ev->impl.update_cell(generation, cell, inverse_cell);
    });
}

int sxb_get_graph(sxb_evaluator* ev, uint64_t generation, int32_t* first_neigh, int32_t* sources, int32_t* shifts)
{
    return guarded([&] {
        require(ev, "evaluator"); require(first_neigh, "first_neigh"); require(sources, "sources");
        ev->impl.get_graph(generation, first_neigh, sources, shifts);
    });
}

int sxb_compute_positions(sxb_evaluator* ev, uint64_t generation, const double* positions)
{
    return guarded([&] {
        require(ev, "evaluator"); require(positions, "positions");
        ev->impl.compute_positions(generation, positions, false);
    });
}

int sxb_compute_positions_device(sxb_evaluator* ev, uint64_t generation, const double* device_positions)
{
    return guarded([&] {
        require(ev, "evaluator"); require(device_positions, "device_positions");
        ev->impl.compute_positions(generation, device_positions, true);
    });
}

int sxb_compute_edge_vectors(sxb_evaluator* ev, uint64_t generation, const double* xyz)
{
    return guarded([&] {
        require(ev, "evaluator"); require(xyz, "xyz");
        ev->impl.compute_edge_vectors(generation, xyz);
    });
}

int sxb_synchronize(sxb_evaluator* ev)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.synchronize(); });
}

int sxb_get_node_energies(sxb_evaluator* ev, double* out, int64_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator"); require(out, "out");
        if (capacity < ev->impl.num_receivers()) throw std::invalid_argument("node_energies buffer is too small.");
        ev->impl.get_node_energies(out);
    });
}

int sxb_set_keep_edge_forces(sxb_evaluator* ev, int32_t enabled)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.set_keep_edge_forces(enabled != 0); });
}

int sxb_get_edge_forces(sxb_evaluator* ev, double* out, int64_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator"); require(out, "out");
        if (capacity < 3 * ev->impl.num_edges()) throw std::invalid_argument("edge_forces buffer is too small.");
        ev->impl.get_edge_forces(out);
    });
}

int sxb_reduce_atom_forces(sxb_evaluator* ev, uint64_t generation, double* out, int64_t capacity)
{
    return guarded([&] {
        require(ev, "evaluator"); require(out, "out");
        ev->impl.check_generation(generation);
        if (capacity < 3L * ev->impl.num_nodes()) throw std::invalid_argument("atom_forces buffer is too small.");
        ev->impl.get_atom_forces(out);
    });
}

int sxb_reduce_stress(sxb_evaluator* ev, uint64_t generation, double volume, double* out9)
{
    return guarded([&] {
        require(ev, "evaluator"); require(out9, "out9");
        ev->impl.check_generation(generation);
        ev->impl.get_stress(volume, out9);
    });
}

int sxb_get_energy(sxb_evaluator* ev, double* out)
{
    return guarded([&] { require(ev, "evaluator"); require(out, "out"); *out = ev->impl.energy(); });
}

int sxb_device_results(sxb_evaluator* ev, const double** energy, const double** forces, const double** virial)
{
    return guarded([&] {
        require(ev, "evaluator");
        ev->impl.require_results();
        if (energy) *energy = ev->impl.device_energy();
        if (forces) *forces = ev->impl.device_forces();
        if (virial) *virial = ev->impl.device_virial();
    });
}

int sxb_get_stage(sxb_evaluator* ev, const char* name, double* out, int64_t capacity, int64_t* count)
{
    return guarded([&] {
        require(ev, "evaluator"); require(name, "name");
        const long n = ev->impl.get_stage(name, out, capacity);
        if (count) *count = n;
    });
}

int sxb_launch_count(const sxb_evaluator* ev, int64_t* out)
{
    return guarded([&] { require(ev, "evaluator"); require(out, "out"); *out = ev->impl.launches(); });
}

int sxb_last_compute_ms(const sxb_evaluator* ev, float* out)
{
    return guarded([&] { require(ev, "evaluator"); require(out, "out"); *out = ev->impl.last_ms(); });
}

int sxb_prepare_local_graph(sxb_evaluator* ev, int32_t num_receivers, int32_t num_nodes, const int32_t* node_types,
                            const double* positions, double neighbor_cutoff, uint64_t* generation, int64_t* num_edges)
{
    return guarded([&] {
        require(ev, "evaluator"); require(node_types, "node_types"); require(positions, "positions"); require(generation, "generation");
        if (num_nodes <= 0) throw std::invalid_argument("Neighbor graph needs at least one node.");
        // open (non-periodic) set of nodes: a box around them with a margin wider than the cutoff, so
        // that no periodic image of the box can come within reach and every shift is zero
        double lo[3] = {positions[0], positions[1], positions[2]}, hi[3] = {positions[0], positions[1], positions[2]};
        for (int i = 0; i < num_nodes; ++i)
            for (int d = 0; d < 3; ++d) {
                lo[d] = std::min(lo[d], positions[3 * i + d]);
                hi[d] = std::max(hi[d], positions[3 * i + d]);
            }
        double cell[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0}, inverse[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
        const double margin = neighbor_cutoff + 1.0;
        for (int d = 0; d < 3; ++d) {
            cell[4 * d] = (hi[d] - lo[d]) + 2.0 * margin;
            inverse[4 * d] = 1.0 / cell[4 * d];
        }
        std::vector<double> shifted(3 * static_cast<std::size_t>(num_nodes));
        for (int i = 0; i < num_nodes; ++i)
            for (int d = 0; d < 3; ++d) shifted[3 * i + d] = positions[3 * i + d] - lo[d] + margin;
        const auto result = ev->impl.prepare_periodic_graph(num_nodes, node_types, shifted.data(), cell, inverse, neighbor_cutoff,
                                                            num_receivers);
        *generation = result.first;
        if (num_edges != nullptr) *num_edges = result.second;
    });
}

int sxb_distributed_begin(sxb_evaluator* ev, uint64_t generation, const double* device_positions)
{
    return guarded([&] {
        require(ev, "evaluator"); require(device_positions, "device_positions");
        ev->impl.distributed_begin(generation, device_positions);
    });
}

int sxb_prepare_local_graph_csr(sxb_evaluator* ev, int32_t num_receivers, int32_t num_nodes, const int32_t* node_types,
                                const int32_t* num_neigh, const int32_t* neigh_indices, int32_t pointers_on_device, uint64_t* generation)
{
    return guarded([&] {
        require(ev, "evaluator"); require(node_types, "node_types"); require(num_neigh, "num_neigh"); require(generation, "generation");
        *generation = ev->impl.prepare_graph_csr(num_receivers, num_nodes, node_types, num_neigh, neigh_indices, pointers_on_device != 0);
    });
}

int sxb_distributed_begin_edge_vectors(sxb_evaluator* ev, uint64_t generation, const double* device_xyz)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (ev->impl.num_edges() > 0) require(device_xyz, "device_xyz");
        ev->impl.distributed_begin_edge_vectors(generation, device_xyz);
    });
}

int sxb_distributed_begin_host(sxb_evaluator* ev, uint64_t generation, const double* host_positions)
{
    return guarded([&] {
        require(ev, "evaluator"); require(host_positions, "host_positions");
        ev->impl.distributed_begin_host(generation, host_positions);
    });
}

int sxb_halo_rows_get(sxb_evaluator* ev, int32_t which, int64_t first_row, int64_t count, float* host_out)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) require(host_out, "host_out");
        ev->impl.get_halo_rows(which, first_row, count, host_out);
    });
}

int sxb_halo_rows_put(sxb_evaluator* ev, int32_t which, int64_t first_row, int64_t count, const float* host_in, int32_t accumulate)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) require(host_in, "host_in");
        ev->impl.put_halo_rows(which, first_row, count, host_in, accumulate != 0);
    });
}

int sxb_distributed_continue(sxb_evaluator* ev)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.distributed_continue(); });
}

int sxb_distributed_finish(sxb_evaluator* ev)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.distributed_finish(); });
}

int sxb_halo_pack(sxb_evaluator* ev, int32_t which, const int32_t* device_indices, int64_t count, float* device_out)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) { require(device_indices, "device_indices"); require(device_out, "device_out"); }
        ev->impl.pack_rows(which, device_indices, count, device_out);
    });
}

int sxb_halo_unpack(sxb_evaluator* ev, int32_t which, const int32_t* device_indices, int64_t count, const float* device_in,
                    int32_t accumulate)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) { require(device_indices, "device_indices"); require(device_in, "device_in"); }
        ev->impl.unpack_rows(which, device_indices, count, device_in, accumulate != 0);
    });
}

int sxb_add_force_rows(sxb_evaluator* ev, const int32_t* device_indices, int64_t count, const double* device_in)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) { require(device_indices, "device_indices"); require(device_in, "device_in"); }
        ev->impl.add_force_rows(device_indices, count, device_in);
    });
}

int sxb_halo_tensor(sxb_evaluator* ev, int32_t which, float** device_tensor, int64_t* row_floats, int64_t* first_ghost_row)
{
    return guarded([&] {
        require(ev, "evaluator"); require(device_tensor, "device_tensor");
        *device_tensor = ev->impl.halo_tensor(which);
        if (row_floats) *row_floats = ev->impl.halo_row_floats();
        if (first_ghost_row) *first_ghost_row = ev->impl.num_receivers();
    });
}

int sxb_gather_position_rows(sxb_evaluator* ev, const double* device_rows, const int32_t* device_indices, int64_t count,
                             const double* device_offsets, double* device_out)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) { require(device_rows, "device_rows"); require(device_indices, "device_indices"); require(device_out, "device_out"); }
        ev->impl.gather_position_rows(device_rows, device_indices, count, device_offsets, device_out);
    });
}

int sxb_pack_ghost_forces(sxb_evaluator* ev, int32_t world, const int32_t* device_ghost_begin, int64_t num_ghosts, double* device_out)
{
    return guarded([&] {
        require(ev, "evaluator"); require(device_ghost_begin, "device_ghost_begin"); require(device_out, "device_out");
        ev->impl.pack_ghost_forces(world, device_ghost_begin, num_ghosts, device_out);
    });
}

int sxb_unpack_ghost_forces(sxb_evaluator* ev, int32_t world, const int32_t* device_send_begin, const int32_t* device_indices,
                            int64_t num_rows, const double* device_in, double* device_totals_out)
{
    return guarded([&] {
        require(ev, "evaluator"); require(device_send_begin, "device_send_begin"); require(device_in, "device_in");
        require(device_totals_out, "device_totals_out");
        if (num_rows > 0) require(device_indices, "device_indices");
        ev->impl.unpack_ghost_forces(world, device_send_begin, device_indices, num_rows, device_in, device_totals_out);
    });
}

int sxb_set_halo_plan(sxb_evaluator* ev, const int32_t* device_send_indices, int64_t num_send, float* device_send_rows,
                      const float* device_received_rows, int32_t world, const int32_t* device_ghost_begin, double* device_force_send)
{
    return guarded([&] {
        require(ev, "evaluator");
        ev->impl.set_halo_plan(device_send_indices, num_send, device_send_rows, device_received_rows, world, device_ghost_begin,
                               device_force_send);
    });
}

int sxb_internal_rows(sxb_evaluator* ev, const int32_t* device_indices, int64_t count, int32_t* device_out)
{
    return guarded([&] {
        require(ev, "evaluator");
        if (count > 0) { require(device_indices, "device_indices"); require(device_out, "device_out"); }
        ev->impl.internal_rows(device_indices, count, device_out);
    });
}

int sxb_distributed_abort(sxb_evaluator* ev)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.abort_phases(); });
}

int sxb_distributed_replayed(sxb_evaluator* ev, uint64_t generation, int64_t launches)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.mark_phases_replayed(generation, launches); });
}

int sxb_set_deterministic(sxb_evaluator* ev, int32_t enabled)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.set_deterministic(enabled != 0); });
}

int sxb_set_tile_size(sxb_evaluator* ev, int32_t receivers_per_tile)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.set_tile_size(receivers_per_tile); });
}

int sxb_set_stream(sxb_evaluator* ev, void* stream)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.set_stream(static_cast<cudaStream_t>(stream)); });
}

int sxb_set_profiling(sxb_evaluator* ev, int32_t enabled)
{
    return guarded([&] { require(ev, "evaluator"); ev->impl.set_profiling(enabled != 0); });
}

int sxb_profile_entry(const sxb_evaluator* ev, int32_t index, char* name, int32_t name_capacity, float* ms, int32_t* launches,
                      int32_t* count)
{
    return guarded([&] {
        require(ev, "evaluator");
        const auto& profile = ev->impl.profile();
        if (count) *count = static_cast<int32_t>(profile.size());
        if (index < 0 || index >= static_cast<int32_t>(profile.size())) return;
        const auto& entry = profile[index];
        if (name != nullptr && name_capacity > 0) {
            std::strncpy(name, entry.name.c_str(), name_capacity - 1);
            name[name_capacity - 1] = 0;
        }
        if (ms) *ms = entry.ms;
        if (launches) *launches = entry.launches;
    });
}

}  // extern "C"
