// Evaluator: owns the model tables, the prepared graph and the work buffers on one B200, and
// sequences the forward + reverse pipeline of the force path on one stream.  Stage order follows
// the reference driver (libsymmetrix/source/mace_kokkos_evaluate.cpp:314-611 and the serial
// statement libsymmetrix/source/mace.cpp:232-319).
#include "evaluator.hpp"

#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <numeric>

#include "deterministic_kernels.cuh"
#include "edge_kernels.cuh"
#include "edge_kernels_split.cuh"
#include "edge_kernels_warp.cuh"
#include "graph_kernels.cuh"
#include "node_kernels.cuh"
#include "tc_gemm.cuh"
#include "tc_gemm_tma.cuh"

namespace sxb {

namespace {

template <typename T>
void upload(DeviceBuffer<T>& buffer, const std::vector<T>& host, cudaStream_t stream)
{
    buffer.reserve(host.size());
    if (!host.empty())
        SXB_CUDA(cudaMemcpyAsync(buffer.ptr, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice, stream));
}

__global__ void unpermute_stage_kernel(long n, long row, const int* __restrict__ original, const float* __restrict__ in,
                                       double* __restrict__ out)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= n * row) return;
    const long node = idx / row, q = idx % row;
    out[static_cast<long>(original[node]) * row + q] = static_cast<double>(in[idx]);
}

__global__ void unpermute_edges_kernel(long num_edges, const int* __restrict__ edge_map, const double* __restrict__ in,
                                       double* __restrict__ out)
{
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= num_edges) return;
    const long o = edge_map[e];
    out[3 * o] = in[3 * e];
    out[3 * o + 1] = in[3 * e + 1];
    out[3 * o + 2] = in[3 * e + 2];
}

__global__ void narrow_offsets_kernel(int n, const long long* __restrict__ wide, int* __restrict__ narrow)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= n) narrow[i] = static_cast<int>(wide[i]);
}

inline int blocks_for(long n, int threads) { return static_cast<int>((n + threads - 1) / threads); }

// Launches KERNEL<kC> with the channel count fixed at compile time for the common widths.
#define SXB_LAUNCH_BY_CHANNELS(KERNEL, C, GRID, STREAM, ...)                         \
    do {                                                                              \
        if ((C) == 128) KERNEL<128><<<(GRID), 128, 0, (STREAM)>>>(__VA_ARGS__);       \
        else if ((C) == 32) KERNEL<32><<<(GRID), 32, 0, (STREAM)>>>(__VA_ARGS__);     \
        else KERNEL<0><<<(GRID), (C), 0, (STREAM)>>>(__VA_ARGS__);                    \
    } while (0)

// Launches a symmetric-contraction kernel with G nodes per thread (G in {1, 2}); the dynamic
// shared memory holds the [terms][32] weight slice of the block's element.
#define SXB_LAUNCH_POLY(KERNEL, G, TERMS, T, C, STREAM, ...)                                                 \
    do {                                                                                                     \
        const dim3 grid_(blocks_for((T), kPolyNodesPerBlock), (C) / 32);                                     \
        const std::size_t smem_ = static_cast<std::size_t>(TERMS) * 32 * sizeof(float);                      \
        if ((G) == 2) KERNEL<2><<<grid_, 32 * kPolyWarps, smem_, (STREAM)>>>(__VA_ARGS__);                   \
        else KERNEL<1><<<grid_, 32 * kPolyWarps, smem_, (STREAM)>>>(__VA_ARGS__);                            \
    } while (0)

// Opts a contraction kernel into the dynamic shared memory its weight slice needs (once, at start-up).
#define SXB_ALLOW_POLY_SMEM(KERNEL, TERMS)                                                                   \
    do {                                                                                                     \
        const int smem_ = static_cast<int>(static_cast<std::size_t>(TERMS) * 32 * sizeof(float));            \
        SXB_CUDA(cudaFuncSetAttribute(KERNEL<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_));       \
        SXB_CUDA(cudaFuncSetAttribute(KERNEL<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_));       \
    } while (0)

}  // namespace

Evaluator::Evaluator(const std::string& json_path, int device_ordinal, const std::string& head) : device_(device_ordinal)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0)
        throw std::runtime_error("No CUDA device is available; this library has no CPU fallback.");
    if (device_ordinal < 0 || device_ordinal >= count) throw std::invalid_argument("CUDA device ordinal is out of range.");
    SXB_CUDA(cudaSetDevice(device_));
    model_ = load_model(json_path, head);
    if (model_.shape_id > 2) throw std::invalid_argument("This build carries kernels for hidden irreps up to 0e+1o+2e only.");
    if (model_.shape_id == 2 && model_.channels != 128)
        throw std::invalid_argument("Hidden irreps 0e+1o+2e are compiled for 128 channels only.");
    SXB_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    SXB_CUDA(cudaEventCreate(&event_begin_));
    SXB_CUDA(cudaEventCreate(&event_end_));

    const int C = model_.channels;
    // the layer-1 table [pair][interval][paths*C][4] and the density tables depend on the active species
    // pairs when the model uses a distance transform: they are built in prepare_active_types
    upload(m0_weights_, model_.m0_weights, stream_);
    upload(m1_weights_, model_.m1_weights, stream_);
    upload(w_h1_, model_.w_h1, stream_);
    if (!model_.single_layer)
        for (int l = 0; l <= model_.l_max; ++l) upload(w_a1_[l], model_.w_a1[l], stream_);
    else {
        if (model_.num_hidden > kMaxHidden) throw std::invalid_argument("Single-layer models are supported for hidden irreps up to l = 2.");
        upload(hidden_poly_terms_, model_.hidden_poly_terms, stream_);
        upload(hidden_poly_weights_, model_.hidden_poly_weights, stream_);
    }
    upload(h2_skip_, model_.h2_skip, stream_);
    upload(h2_m1_, model_.h2_m1, stream_);
    upload(readout1_, model_.readout1, stream_);
    upload(readout2_w1_, model_.readout2_w1, stream_);
    upload(readout2_w2_, model_.readout2_w2, stream_);
    upload(atomic_energies_, model_.atomic_energies, stream_);
    if (const char* env = std::getenv("SXB_SIMT_LINEARS")) use_tensor_cores_ = !(env[0] == '1');
    if (const char* env = std::getenv("SXB_CUDA_GRAPHS")) use_graphs_ = env[0] != '0';
    if (const char* env = std::getenv("SXB_POLY_GROUP")) {   // nodes per thread in the contraction kernels: "<forward><reverse>"
        if (env[0] == '1' || env[0] == '2') poly_g_forward_ = env[0] - '0';
        if (env[0] != 0 && (env[1] == '1' || env[1] == '2')) poly_g_reverse_ = env[1] - '0';
    }
    for (int l = 0; l <= model_.hidden_l_max; ++l)
        upload_split(s_h1_[l], model_.w_h1.data() + static_cast<std::size_t>(l) * C * C, C, C);
    if (!model_.single_layer)
        for (int l = 0; l <= model_.l_max; ++l) upload_split(s_a1_[l], model_.w_a1[l].data(), model_.eta[l] * C, C);
    s_h2_skip_.resize(model_.num_elements);
    for (int a = 0; a < model_.num_elements; ++a)
        upload_split(s_h2_skip_[a], model_.h2_skip.data() + static_cast<std::size_t>(a) * C * C, C, C);
    upload_split(s_h2_m1_, model_.h2_m1.data(), C, C);
    if (model_.pre_linear_up) upload_split(s_product0_, model_.w_product0.data(), C, C);
    if (model_.first_residual) {
        upload(residual_fused_, model_.residual_fused, stream_);
        upload(residual_scalar_, model_.residual_scalar, stream_);
    }
    SXB_ALLOW_POLY_SMEM(m0_forward_kernel_S0, SXB_S0_M0_NUM_TERMS); SXB_ALLOW_POLY_SMEM(m0_reverse_kernel_S0, SXB_S0_M0_NUM_TERMS);
    SXB_ALLOW_POLY_SMEM(m0_forward_kernel_S1, SXB_S1_M0_NUM_TERMS); SXB_ALLOW_POLY_SMEM(m0_reverse_kernel_S1, SXB_S1_M0_NUM_TERMS);
    SXB_ALLOW_POLY_SMEM(m0_forward_kernel_S2, SXB_S2_M0_NUM_TERMS); SXB_ALLOW_POLY_SMEM(m0_reverse_kernel_S2, SXB_S2_M0_NUM_TERMS);
    SXB_ALLOW_POLY_SMEM(m1_forward_kernel_S0, SXB_S0_M1_NUM_TERMS); SXB_ALLOW_POLY_SMEM(m1_reverse_kernel_S0, SXB_S0_M1_NUM_TERMS);
    SXB_ALLOW_POLY_SMEM(m1_forward_kernel_S1, SXB_S1_M1_NUM_TERMS); SXB_ALLOW_POLY_SMEM(m1_reverse_kernel_S1, SXB_S1_M1_NUM_TERMS);
    SXB_ALLOW_POLY_SMEM(m1_forward_kernel_S2, SXB_S2_M1_NUM_TERMS); SXB_ALLOW_POLY_SMEM(m1_reverse_kernel_S2, SXB_S2_M1_NUM_TERMS);
    SXB_CUDA(cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
    SXB_CUDA(cudaFuncSetAttribute(tc_gemm_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kT3SmemBytes));
    SXB_CUDA(cudaDeviceGetAttribute(&num_sms_, cudaDevAttrMultiProcessorCount, device_));
    if (const char* env = std::getenv("SXB_TMA_ACTIVATIONS")) use_tma_activations_ = env[0] != '0';
    std::memset(&coupling_, 0, sizeof(coupling_));
    if (model_.num_terms > 256) throw std::invalid_argument("Too many coupling terms.");
    for (int t = 0; t < model_.num_terms; ++t) coupling_.cg[t] = model_.cg[t];
    grid_.x0 = static_cast<float>(model_.spline_x0);
    grid_.h = static_cast<float>(model_.spline_h);
    grid_.r_cut = static_cast<float>(model_.r_cut);
    grid_.intervals = model_.spline_points - 1;
    totals_.reserve(10);
    energy_slots_.reserve(kVirialSlots);
    virial_slots_.reserve(kVirialSlots * 9);
    error_flag_.reserve(1);
    cell_.reserve(9);
    inv_cell_.reserve(9);
    SXB_CUDA(cudaStreamSynchronize(stream_));
    (void)C;
}

Evaluator::~Evaluator()
{
    cudaSetDevice(device_);
    drop_step_graphs();
    if (event_begin_) cudaEventDestroy(event_begin_);
    if (event_end_) cudaEventDestroy(event_end_);
    for (auto e : event_pool_) cudaEventDestroy(e);
    if (stream_ && owns_stream_) cudaStreamDestroy(stream_);
    if (host_results_) cudaFreeHost(host_results_);
    if (host_stage_) cudaFreeHost(host_stage_);
}

void Evaluator::prepare_active_types(const std::vector<int>& node_types)
{
    std::vector<int> requested(node_types);
    std::sort(requested.begin(), requested.end());
    requested.erase(std::unique(requested.begin(), requested.end()), requested.end());
    if (requested.empty()) throw std::invalid_argument("MACE compact radial cache requires at least one active type.");
    for (int t : requested)
        if (t < 0 || t >= model_.num_elements) throw std::invalid_argument("MACE active type index is out of range.");
    if (requested.size() > 255) throw std::invalid_argument("More than 255 active element types.");
    if (requested == active_types_) return;
    active_types_ = requested;
    const auto table = fold_r0_table(model_, active_types_);
    if (table.size() > static_cast<std::size_t>(std::numeric_limits<int>::max()))
        throw std::length_error("Layer-0 spline table exceeds 32-bit indexing; too many active element types.");
    upload(r0_table_, table, stream_);
    {
        if (!model_.single_layer) {
            int pairs = 1;
            const auto r1 = build_r1_table(model_, active_types_, &pairs);
            if (r1.size() > static_cast<std::size_t>(std::numeric_limits<int>::max()))
                throw std::length_error("Layer-1 spline table exceeds 32-bit indexing; too many active element types.");
            upload(r1_table_, r1, stream_);
        }
        r1_pair_types_ = model_.agnesi ? static_cast<int>(active_types_.size()) : 1;
        if (model_.a0_scaled) upload(density0_table_, build_density_table(model_, "A0", active_types_), stream_);
        if (model_.a1_scaled) upload(density1_table_, build_density_table(model_, "A1", active_types_), stream_);
    }
    if (model_.has_zbl) {
        // per-pair constants in the model precision, as the reference forms them (zbl.cpp:24-45)
        const std::size_t n = active_types_.size();
        std::vector<float> pairs(n * n * 4, 0.0f);
        for (std::size_t a = 0; a < n; ++a)
            for (std::size_t b = 0; b < n; ++b) {
                const int Zu = model_.atomic_numbers[active_types_[a]], Zv = model_.atomic_numbers[active_types_[b]];
                if (Zu < 0 || Zv < 0 || static_cast<std::size_t>(std::max(Zu, Zv)) >= model_.zbl_covalent_radii.size())
                    throw std::invalid_argument("ZBL covalent radii do not cover the model's atomic numbers.");
                const float zu = static_cast<float>(Zu), zv = static_cast<float>(Zv);
                const float a_exp = static_cast<float>(model_.zbl_a_exp);
                const float aa = static_cast<float>(model_.zbl_a_prefactor) * 0.529f / (std::pow(zu, a_exp) + std::pow(zv, a_exp));
                float* p = pairs.data() + (a * n + b) * 4;
                p[0] = 1.0f / aa;
                p[1] = 14.3996f * zu * zv;
                p[2] = static_cast<float>(model_.zbl_covalent_radii[Zu]) + static_cast<float>(model_.zbl_covalent_radii[Zv]);
            }
        upload(zbl_pairs_, pairs, stream_);
    }
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

// Installs a caller-order CSR graph that already sits on the device, re-expressed in the internal
// node order (stable sort by element type).
void Evaluator::install_graph(int num_receivers, int num_nodes, const std::vector<int>& node_types, long num_edges, bool has_shifts)
{
    // Receivers (nodes that own edges and readouts) come first in the caller's order; the nodes
    // after them are feature-only nodes (ghost atoms of a domain decomposition): they carry H1,
    // H1_adj, a type, a position and a force row, nothing else.
    num_receivers_ = num_receivers;
    num_nodes_ = num_nodes;
    num_edges_ = num_edges;
    has_shifts_ = has_shifts;
    prepare_active_types(node_types);
    std::vector<int> type_to_active(model_.num_elements, -1);
    for (std::size_t a = 0; a < active_types_.size(); ++a) type_to_active[active_types_[a]] = static_cast<int>(a);
    // internal order: receivers stably grouped by element (a counting sort), feature-only nodes after them
    std::vector<int> original(num_nodes);
    std::iota(original.begin(), original.end(), 0);
    {
        std::vector<int> cursor(static_cast<std::size_t>(model_.num_elements) + 1, 0);
        for (int i = 0; i < num_receivers; ++i) cursor[node_types[i] + 1] += 1;
        for (int t = 0; t < model_.num_elements; ++t) cursor[t + 1] += cursor[t];
        for (int i = 0; i < num_receivers; ++i) original[cursor[node_types[i]]++] = i;
    }
    std::vector<int> internal_of(num_nodes);
    std::vector<unsigned char> atype(num_nodes), element(num_nodes);
    type_begin_.assign(active_types_.size() + 1, 0);
    for (int i = 0; i < num_nodes; ++i) {
        internal_of[original[i]] = i;
        atype[i] = static_cast<unsigned char>(type_to_active[node_types[original[i]]]);
        element[i] = static_cast<unsigned char>(node_types[original[i]]);
        if (i < num_receivers) type_begin_[atype[i] + 1] += 1;
    }
    for (std::size_t a = 0; a < active_types_.size(); ++a) type_begin_[a + 1] += type_begin_[a];
    if (model_.num_elements > 255) throw std::invalid_argument("More than 255 element types.");
    upload(original_, original, stream_);
    upload(internal_of_, internal_of, stream_);
    upload(atype_, atype, stream_);
    upload(element_, element, stream_);

    // internal CSR
    const int R = num_receivers;
    first_.reserve(R + 1);
    sources_.reserve_with_slack(num_edges);
    if (has_shifts) shifts_.reserve_with_slack(3 * num_edges);
    edge_map_.reserve_with_slack(num_edges);
    DeviceBuffer<int>& counts = ig_counts_;
    counts.reserve(R + 1);
    SXB_CUDA(cudaMemsetAsync(counts.ptr, 0, (R + 1) * sizeof(int), stream_));
    gather_counts_kernel<<<blocks_for(R, 256), 256, 0, stream_>>>(R, original_.ptr, first_caller_.ptr, counts.ptr);
    launches_ += 1;
    std::size_t temp_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, counts.ptr, first_.ptr, R + 1, stream_);
    DeviceBuffer<unsigned char>& temp = ig_temp_;
    temp.reserve(temp_bytes);
    cub::DeviceScan::ExclusiveSum(temp.ptr, temp_bytes, counts.ptr, first_.ptr, R + 1, stream_);
    permute_graph_kernel<<<blocks_for(static_cast<long>(R) * 32, 256), 256, 0, stream_>>>(
        R, original_.ptr, internal_of_.ptr, first_caller_.ptr, sources_caller_.ptr,
        has_shifts ? shifts_caller_.ptr : nullptr, first_.ptr, sources_.ptr, has_shifts ? shifts_.ptr : nullptr, edge_map_.ptr);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());

    // work buffers
    // graph-wide state: H1, H1_adj (all nodes), M0, H2_adj, energies (receivers), forces (all nodes);
    // everything else lives in a workspace sized for one tile of receivers and is reused tile by tile
    const std::size_t N = num_receivers, ALL = num_nodes, C = model_.channels, NH = model_.num_hidden, NE = model_.num_lme;
    const std::size_t T = static_cast<std::size_t>(tile_capacity());
    geom_.reserve_with_slack(num_edges);
    A0_.reserve(T * 16 * C);
    A0_adj_.reserve(T * 16 * C);
    M0_.reserve(N * NH * C);
    M0_adj_.reserve(T * NH * C);
    H1_.reserve(ALL * NH * C);
    H1_adj_.reserve(ALL * NH * C);
    Phi1_.reserve(T * NE * C);
    dPhi1_.reserve(T * NE * C);
    A1_.reserve(T * 16 * C);
    A1_adj_.reserve(T * 16 * C);
    M1_.reserve(T * C);
    M1_adj_.reserve(T * C);
    H2_.reserve(T * C);
    H2_adj_.reserve(N * C);
    if (model_.pre_linear_up) {   // scalar input of the first readout and the skip, and its adjoint, for every receiver
        scalar_input_.reserve(N * C);
        scalar_adjoint_.reserve(N * C);
    }
    node_energies_.reserve(N);
    if (model_.a0_scaled) { inv_scale0_.reserve(N); dot0_.reserve(N); }
    if (model_.a1_scaled) { inv_scale1_.reserve(N); dot1_.reserve(N); }
    node_energies_out_.reserve(N);
    forces_.reserve(ALL * 3);
    forces_out_.reserve(ALL * 3);
    positions_.reserve(ALL * 3);
    if (deterministic_) {
        // source schedule: edge ids sorted by source (stable, so ascending edge index inside a source) and the
        // offsets of each source's run; plus one record per edge for the source adjoint and the directed force
        if (model_.shape_id == 2) throw std::invalid_argument("The reproducible mode is not available for hidden irreps 0e+1o+2e.");
        if (model_.single_layer) throw std::invalid_argument("The reproducible mode is not available for single-layer models.");
        if (model_.legacy_h1_basis) throw std::invalid_argument("The reproducible mode is not available for format-version 1 / 2 models.");
        if (model_.pre_linear_up) throw std::invalid_argument("The reproducible mode is not available for pre_linear_up models.");
        if (model_.a0_scaled || model_.a1_scaled)
            throw std::invalid_argument("The reproducible mode is not available for density-scaled models.");
        const std::size_t record_floats = static_cast<std::size_t>(num_edges) * NH * C;
        if (record_floats * sizeof(float) > (16ull << 30))
            throw std::length_error("The reproducible mode keeps one source-adjoint record per edge; this graph would need more than 16 GB.");
        keep_edge_forces_ = true;
        edge_source_adjoint_.reserve_with_slack(std::max<std::size_t>(record_floats, 1));
        source_offsets_.reserve(ALL + 1);
        source_edges_.reserve_with_slack(std::max<long>(num_edges, 1));
        det_sorted_sources_.reserve_with_slack(std::max<long>(num_edges, 1));
        det_edge_ids_.reserve_with_slack(std::max<long>(num_edges, 1));
        det_counts_.reserve(ALL + 1);
        const long blocks_e = blocks_for(std::max<long>(num_edges, 1), 256);
        det_partials_.reserve(static_cast<std::size_t>(std::max<long>(blocks_e, blocks_for(R, 256))) * 10);
        SXB_CUDA(cudaMemsetAsync(det_counts_.ptr, 0, (ALL + 1) * sizeof(int), stream_));
        if (num_edges > 0) {
            count_sources_kernel<<<blocks_e, 256, 0, stream_>>>(num_edges, sources_.ptr, det_counts_.ptr);
            iota_kernel<<<blocks_e, 256, 0, stream_>>>(num_edges, det_edge_ids_.ptr);
        }
        std::size_t scan_bytes = 0, sort_bytes = 0;
        int key_bits = 1;
        while ((1ll << key_bits) < static_cast<long long>(ALL)) ++key_bits;
        cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, det_counts_.ptr, source_offsets_.ptr, static_cast<int>(ALL + 1), stream_);
        cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, sources_.ptr, det_sorted_sources_.ptr, det_edge_ids_.ptr, source_edges_.ptr,
                                        static_cast<int>(num_edges), 0, key_bits, stream_);
        ig_temp_.reserve(std::max(scan_bytes, sort_bytes));
        cub::DeviceScan::ExclusiveSum(ig_temp_.ptr, scan_bytes, det_counts_.ptr, source_offsets_.ptr, static_cast<int>(ALL + 1), stream_);
        if (num_edges > 0)
            cub::DeviceRadixSort::SortPairs(ig_temp_.ptr, sort_bytes, sources_.ptr, det_sorted_sources_.ptr, det_edge_ids_.ptr,
                                            source_edges_.ptr, static_cast<int>(num_edges), 0, key_bits, stream_);
        launches_ += 2;
        SXB_CUDA(cudaGetLastError());
    }
    if (keep_edge_forces_) edge_forces_.reserve_with_slack(3 * static_cast<std::size_t>(num_edges));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    // pinned host side of an evaluation: a staging copy of the positions (uploaded by a copy node of the
    // captured step) and the result block the closing kernel writes through the mapping
    constexpr std::size_t kHostBlockLimit = 4u << 20;   // doubles (32 MB): beyond this the getters copy on demand
    const std::size_t result_doubles = 11 + N + 3 * ALL;
    if (result_doubles <= kHostBlockLimit) {
        if (host_results_capacity_ < result_doubles) {
            if (host_results_) SXB_CUDA(cudaFreeHost(host_results_));
            if (host_stage_) SXB_CUDA(cudaFreeHost(host_stage_));
            host_results_ = host_stage_ = nullptr;
            host_results_capacity_ = 0;
            const std::size_t grown = result_doubles + result_doubles / 16;
            SXB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&host_results_), sizeof(double) * grown, cudaHostAllocMapped));
            SXB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&host_stage_), sizeof(double) * grown, cudaHostAllocDefault));
            host_results_capacity_ = grown;
        }
    } else if (host_results_) {
        SXB_CUDA(cudaFreeHost(host_results_));
        SXB_CUDA(cudaFreeHost(host_stage_));
        host_results_ = host_stage_ = nullptr;
        host_results_capacity_ = 0;
    }
    generation_ += 1;
    have_results_ = false;
    mirror_valid_ = false;
    phase_ = 0;
    halo_plan_ = HaloPlan{};      // buffers of a decomposed run belong to the previous graph
    geometry_mode_ = 0;           // a reference geometry belongs to the graph it was given for
}

namespace {
// Bins and stencil reach of the cell list.  Per axis: the spacing of the lattice planes is
// 1 / |column of the inverse cell|; bins = floor(spacing / cutoff), at least one, so a bin is never
// thinner than the cutoff; reach = ceil(cutoff * bins / spacing) + 1 bins on either side.  These are
// the extents of the reference's builder (libsymmetrix/source/neighbor_graph_kokkos.cpp:84-120), which
// fixes the candidate order.
void validate_cell_pair(const double* cell, const double* inverse_cell);
CellGrid finish_cell_grid(const double* inverse_cell, double cutoff);

CellGrid plan_cell_grid(const double* cell, const double* inverse_cell, double cutoff)
{
    if (!std::isfinite(cutoff) || !(cutoff > 0.0)) throw std::invalid_argument("Neighbor cutoff must be finite and positive.");
    validate_cell_pair(cell, inverse_cell);
    return finish_cell_grid(inverse_cell, cutoff);
}

void validate_cell_pair(const double* cell, const double* inverse_cell)
{
    double worst = 0.0;
    bool finite = true;
    for (int q = 0; q < 9; ++q) finite = finite && std::isfinite(cell[q]) && std::isfinite(inverse_cell[q]);
    if (!finite) throw std::invalid_argument("Cell and inverse cell must be finite.");
    for (int r = 0; r < 3; ++r)
        for (int c = 0; c < 3; ++c) {
            const double dot = cell[3 * r] * inverse_cell[c] + cell[3 * r + 1] * inverse_cell[3 + c] + cell[3 * r + 2] * inverse_cell[6 + c];
            worst = std::max(worst, std::abs(dot - (r == c ? 1.0 : 0.0)));
        }
    if (worst > 1e-9) throw std::invalid_argument("inverse_cell is not the inverse of cell.");
}

CellGrid finish_cell_grid(const double* inverse_cell, double cutoff)
{
    CellGrid grid;
    std::size_t total = 1;
    for (int axis = 0; axis < 3; ++axis) {
        const double inverse_spacing = std::sqrt(inverse_cell[axis] * inverse_cell[axis] + inverse_cell[3 + axis] * inverse_cell[3 + axis]
                                                 + inverse_cell[6 + axis] * inverse_cell[6 + axis]);
        if (!(inverse_spacing > 0.0)) throw std::invalid_argument("Cell is singular.");
        const double whole_bins = std::floor((1.0 / inverse_spacing) / cutoff);
        if (whole_bins >= static_cast<double>(std::numeric_limits<int>::max()))
            throw std::length_error("Cell list needs more bins along one axis than 32-bit indexing allows.");
        grid.bins[axis] = std::max(1, static_cast<int>(whole_bins));
        grid.reach[axis] = std::max(1, static_cast<int>(std::ceil(cutoff * inverse_spacing * grid.bins[axis]) + 1.0));
        total *= static_cast<std::size_t>(grid.bins[axis]);
        if (total >= static_cast<std::size_t>(std::numeric_limits<int>::max()))
            throw std::length_error("Cell list needs more bins than 32-bit indexing allows.");
    }
    grid.num_bins = static_cast<int>(total);
    grid.cutoff_squared = cutoff * cutoff;
    return grid;
}
}  // namespace

std::pair<std::uint64_t, long> Evaluator::prepare_periodic_graph(int num_nodes, const int* node_types, const double* positions,
                                                                 const double* cell, const double* inverse_cell, double cutoff,
                                                                 int num_receivers)
{
    SXB_CUDA(cudaSetDevice(device_));
    if (num_nodes <= 0) throw std::invalid_argument("Neighbor graph needs at least one node.");
    if (num_receivers < 0) num_receivers = num_nodes;
    if (num_receivers == 0 || num_receivers > num_nodes) throw std::invalid_argument("Receiver count must lie in [1, num_nodes].");
    const CellGrid grid = plan_cell_grid(cell, inverse_cell, cutoff);
    const int n = num_nodes, nr = num_receivers, threads = 256;
    const std::size_t num_bins = static_cast<std::size_t>(grid.num_bins);

    positions_.reserve(3 * static_cast<std::size_t>(n));
    SXB_CUDA(cudaMemcpyAsync(positions_.ptr, positions, 3 * sizeof(double) * n, cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaMemcpyAsync(cell_.ptr, cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaMemcpyAsync(inv_cell_.ptr, inverse_cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    // cell-list scratch lives in members: a rebuild allocates nothing once the sizes have settled
    nb_wrapped_pos_.reserve(3 * static_cast<std::size_t>(n));
    nb_sorted_pos_.reserve(3 * static_cast<std::size_t>(n));
    nb_wrap_count_.reserve(3 * static_cast<std::size_t>(n));
    nb_atom_bin_.reserve(n);
    nb_atom_index_.reserve(n);
    nb_sorted_bin_.reserve(n);
    nb_sorted_atoms_.reserve(n);
    nb_bin_sizes_.reserve(num_bins + 1);
    nb_bin_begin_.reserve(num_bins + 1);
    nb_counts_.reserve(nr + 1);
    nb_offsets_.reserve(nr + 1);
    int key_bits = 1;
    while ((1ll << key_bits) < static_cast<long long>(num_bins)) ++key_bits;
    std::size_t scan_bins_bytes = 0, scan_edges_bytes = 0, sort_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bins_bytes, nb_bin_sizes_.ptr, nb_bin_begin_.ptr, grid.num_bins + 1, stream_);
    cub::DeviceScan::ExclusiveSum(nullptr, scan_edges_bytes, nb_counts_.ptr, nb_offsets_.ptr, nr + 1, stream_);
    cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, nb_atom_bin_.ptr, nb_sorted_bin_.ptr, nb_atom_index_.ptr, nb_sorted_atoms_.ptr, n,
                                    0, key_bits, stream_);
    nb_temp_.reserve(std::max(sort_bytes, std::max(scan_bins_bytes, scan_edges_bytes)));

    SXB_CUDA(cudaMemsetAsync(nb_bin_sizes_.ptr, 0, (num_bins + 1) * sizeof(int), stream_));
    SXB_CUDA(cudaMemsetAsync(nb_counts_.ptr, 0, (nr + 1) * sizeof(long long), stream_));
    SXB_CUDA(cudaMemsetAsync(error_flag_.ptr, 0, sizeof(int), stream_));
    wrap_and_bin_kernel<<<blocks_for(n, threads), threads, 0, stream_>>>(n, grid, positions_.ptr, inv_cell_.ptr, cell_.ptr,
                                                                          nb_wrapped_pos_.ptr, nb_wrap_count_.ptr, nb_atom_bin_.ptr,
                                                                          nb_atom_index_.ptr, nb_bin_sizes_.ptr, error_flag_.ptr);
    cub::DeviceScan::ExclusiveSum(nb_temp_.ptr, scan_bins_bytes, nb_bin_sizes_.ptr, nb_bin_begin_.ptr, grid.num_bins + 1, stream_);
    // stable sort by bin: inside a bin the atoms stay in ascending index
    cub::DeviceRadixSort::SortPairs(nb_temp_.ptr, sort_bytes, nb_atom_bin_.ptr, nb_sorted_bin_.ptr, nb_atom_index_.ptr,
                                    nb_sorted_atoms_.ptr, n, 0, key_bits, stream_);
    gather_sorted_positions_kernel<<<blocks_for(n, threads), threads, 0, stream_>>>(n, nb_sorted_atoms_.ptr, nb_wrapped_pos_.ptr,
                                                                                     nb_sorted_pos_.ptr);
    const int warp_blocks = blocks_for(static_cast<long>(nr) * 32, threads);
    receiver_edges_kernel<false><<<warp_blocks, threads, 0, stream_>>>(nr, grid, nb_atom_bin_.ptr, nb_bin_begin_.ptr, nb_sorted_atoms_.ptr,
                                                                        nb_sorted_pos_.ptr, nb_wrapped_pos_.ptr, nb_wrap_count_.ptr,
                                                                        cell_.ptr, nb_counts_.ptr, nullptr, nullptr, nullptr);
    cub::DeviceScan::ExclusiveSum(nb_temp_.ptr, scan_edges_bytes, nb_counts_.ptr, nb_offsets_.ptr, nr + 1, stream_);
    long long total = 0;
    int status = 0;
    SXB_CUDA(cudaMemcpyAsync(&total, nb_offsets_.ptr + nr, sizeof(long long), cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaMemcpyAsync(&status, error_flag_.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    if (status & 4) throw std::invalid_argument("Neighbor graph positions must be finite.");
    if (total > static_cast<long long>(std::numeric_limits<int>::max()))
        throw std::length_error("Neighbor graph exceeds 32-bit edge indexing.");
    first_caller_.reserve(nr + 1);
    sources_caller_.reserve_with_slack(static_cast<std::size_t>(total));
    shifts_caller_.reserve_with_slack(3 * static_cast<std::size_t>(total));
    narrow_offsets_kernel<<<blocks_for(nr + 1, threads), threads, 0, stream_>>>(nr, nb_offsets_.ptr, first_caller_.ptr);
    receiver_edges_kernel<true><<<warp_blocks, threads, 0, stream_>>>(nr, grid, nb_atom_bin_.ptr, nb_bin_begin_.ptr, nb_sorted_atoms_.ptr,
                                                                       nb_sorted_pos_.ptr, nb_wrapped_pos_.ptr, nb_wrap_count_.ptr,
                                                                       cell_.ptr, nullptr, first_caller_.ptr, sources_caller_.ptr,
                                                                       shifts_caller_.ptr);
    launches_ += 5;
    SXB_CUDA(cudaGetLastError());
    std::vector<int> types(node_types, node_types + n);
    install_graph(nr, n, types, static_cast<long>(total), true);
    return {generation_, static_cast<long>(total)};
}

std::uint64_t Evaluator::prepare_graph(int num_nodes, const int* node_types, const int* num_neigh, const int* neigh_indices,
                                       const int* shifts, const double* cell)
{
    SXB_CUDA(cudaSetDevice(device_));
    if (num_nodes <= 0) throw std::invalid_argument("Graph needs at least one node.");
    std::vector<int> first(num_nodes + 1, 0);
    for (int i = 0; i < num_nodes; ++i) {
        if (num_neigh[i] < 0) throw std::invalid_argument("num_neigh must be non-negative.");
        const long long next = static_cast<long long>(first[i]) + num_neigh[i];
        if (next > std::numeric_limits<int>::max()) throw std::length_error("Graph exceeds 32-bit edge indexing.");
        first[i + 1] = static_cast<int>(next);
    }
    const long E = first[num_nodes];
    for (long e = 0; e < E; ++e)
        if (neigh_indices[e] < 0 || neigh_indices[e] >= num_nodes) throw std::invalid_argument("neigh_indices entry is out of range.");
    if ((shifts == nullptr) != (cell == nullptr)) throw std::invalid_argument("shifts and cell must be given together.");
    upload(first_caller_, first, stream_);
    sources_caller_.reserve(E);
    SXB_CUDA(cudaMemcpyAsync(sources_caller_.ptr, neigh_indices, E * sizeof(int), cudaMemcpyHostToDevice, stream_));
    if (shifts != nullptr) {
        shifts_caller_.reserve(3 * E);
        SXB_CUDA(cudaMemcpyAsync(shifts_caller_.ptr, shifts, 3 * E * sizeof(int), cudaMemcpyHostToDevice, stream_));
        SXB_CUDA(cudaMemcpyAsync(cell_.ptr, cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    }
    std::vector<int> types(node_types, node_types + num_nodes);
    install_graph(num_nodes, num_nodes, types, E, shifts != nullptr);
    return generation_;
}

namespace {
__global__ void widen_counts_kernel(int n, const int* __restrict__ counts, long long* __restrict__ wide, int* __restrict__ status)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i > n) return;
    const int c = i < n ? counts[i] : 0;
    if (c < 0) atomicOr(status, 8);
    wide[i] = c < 0 ? 0 : c;
}

__global__ void check_indices_kernel(long num_edges, int num_nodes, const int* __restrict__ indices, int* __restrict__ status)
{
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= num_edges) return;
    const int j = indices[e];
    if (j < 0 || j >= num_nodes) atomicOr(status, 16);
}
}  // namespace

// A caller-built receiver-major CSR over num_nodes nodes of which the first num_receivers own edge
// lists (the others are ghosts: feature-only nodes).  Host or device arrays; evaluated from per-step
// edge vectors.  This is the graph a LAMMPS pair style holds: owned atoms first, ghosts after, the
// full neighbor list of the owned atoms (reference: MACEKokkos::prepare_factorized_graph_device,
// libsymmetrix/source/mace_kokkos.hpp:399-413; call site pair_symmetrix_mace_kokkos.cpp:1464-1476).
std::uint64_t Evaluator::prepare_graph_csr(int num_receivers, int num_nodes, const int* node_types, const int* num_neigh,
                                           const int* neigh_indices, bool on_device)
{
    SXB_CUDA(cudaSetDevice(device_));
    if (num_nodes <= 0) throw std::invalid_argument("Graph needs at least one node.");
    if (num_receivers <= 0 || num_receivers > num_nodes) throw std::invalid_argument("Receiver count must lie in [1, num_nodes].");
    const int R = num_receivers, threads = 256;
    std::vector<int> types(num_nodes);
    if (on_device) SXB_CUDA(cudaMemcpyAsync(types.data(), node_types, sizeof(int) * num_nodes, cudaMemcpyDeviceToHost, stream_));
    else std::copy(node_types, node_types + num_nodes, types.begin());
    ig_counts_.reserve(R + 1);
    SXB_CUDA(cudaMemcpyAsync(ig_counts_.ptr, num_neigh, sizeof(int) * R, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream_));
    nb_counts_.reserve(R + 1);
    nb_offsets_.reserve(R + 1);
    SXB_CUDA(cudaMemsetAsync(error_flag_.ptr, 0, sizeof(int), stream_));
    widen_counts_kernel<<<blocks_for(R + 1, threads), threads, 0, stream_>>>(R, ig_counts_.ptr, nb_counts_.ptr, error_flag_.ptr);
    std::size_t scan_bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, nb_counts_.ptr, nb_offsets_.ptr, R + 1, stream_);
    nb_temp_.reserve(scan_bytes);
    cub::DeviceScan::ExclusiveSum(nb_temp_.ptr, scan_bytes, nb_counts_.ptr, nb_offsets_.ptr, R + 1, stream_);
    long long total = 0;
    SXB_CUDA(cudaMemcpyAsync(&total, nb_offsets_.ptr + R, sizeof(long long), cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    if (total > static_cast<long long>(std::numeric_limits<int>::max())) throw std::length_error("Graph exceeds 32-bit edge indexing.");
    const long E = static_cast<long>(total);
    first_caller_.reserve(R + 1);
    narrow_offsets_kernel<<<blocks_for(R + 1, threads), threads, 0, stream_>>>(R, nb_offsets_.ptr, first_caller_.ptr);
    sources_caller_.reserve_with_slack(static_cast<std::size_t>(E));
    if (E > 0) {
        SXB_CUDA(cudaMemcpyAsync(sources_caller_.ptr, neigh_indices, sizeof(int) * E, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream_));
        check_indices_kernel<<<blocks_for(E, threads), threads, 0, stream_>>>(E, num_nodes, sources_caller_.ptr, error_flag_.ptr);
    }
    int status = 0;
    SXB_CUDA(cudaMemcpyAsync(&status, error_flag_.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    launches_ += 3;
    if (status & 8) throw std::invalid_argument("num_neigh must be non-negative.");
    if (status & 16) throw std::invalid_argument("neigh_indices entry is out of range.");
    install_graph(R, num_nodes, types, E, false);
    return generation_;
}

// Reference state for graphs the caller built without integer shifts: reference positions (Cartesian
// or fractional), the edge vectors of that state in the caller's edge order, the cell and the periodic
// axes.  Evaluations from positions then follow the atoms from that reference
// (reference: prepare_factorized_geometry / prepare_factorized_fractional_geometry / update_factorized_cell,
// symmetrix/source/cpp/mace_kokkos.cpp:1608-1685).
void Evaluator::prepare_reference_geometry(std::uint64_t generation, bool fractional, const double* reference_positions,
                                           const double* reference_xyz, const double* cell, const double* inverse_cell, const int* pbc)
{
    check_generation(generation);
    if (has_shifts_) throw std::invalid_argument("The prepared graph carries periodic shifts; it needs no reference geometry.");
    SXB_CUDA(cudaSetDevice(device_));
    validate_cell_pair(cell, inverse_cell);
    reference_positions_.reserve(3 * static_cast<std::size_t>(num_nodes_));
    reference_xyz_.reserve_with_slack(3 * static_cast<std::size_t>(std::max<long>(num_edges_, 1)));
    SXB_CUDA(cudaMemcpyAsync(reference_positions_.ptr, reference_positions, sizeof(double) * 3 * num_nodes_, cudaMemcpyHostToDevice, stream_));
    if (num_edges_ > 0)
        SXB_CUDA(cudaMemcpyAsync(reference_xyz_.ptr, reference_xyz, sizeof(double) * 3 * num_edges_, cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaMemcpyAsync(cell_.ptr, cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaMemcpyAsync(inv_cell_.ptr, inverse_cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    pbc_mask_ = (pbc[0] ? 1 : 0) | (pbc[1] ? 2 : 0) | (pbc[2] ? 4 : 0);
    geometry_mode_ = fractional ? 2 : 1;
    drop_step_graphs();
    have_results_ = false;
}

void Evaluator::update_cell(std::uint64_t generation, const double* cell, const double* inverse_cell)
{
    check_generation(generation);
    if (geometry_mode_ != 2 && !has_shifts_)
        throw std::invalid_argument("A cell update needs fractional reference geometry or a graph with periodic shifts.");
    SXB_CUDA(cudaSetDevice(device_));
    validate_cell_pair(cell, inverse_cell);
    SXB_CUDA(cudaMemcpyAsync(cell_.ptr, cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaMemcpyAsync(inv_cell_.ptr, inverse_cell, 9 * sizeof(double), cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    have_results_ = false;
}

void Evaluator::check_generation(std::uint64_t generation) const
{
    if (generation == 0 || generation != generation_)
        throw StaleGraph("Prepared graph generation is stale or invalid.");
}

void Evaluator::get_graph(std::uint64_t generation, int* first, int* sources, int* shifts)
{
    check_generation(generation);
    SXB_CUDA(cudaSetDevice(device_));
    SXB_CUDA(cudaMemcpyAsync(first, first_caller_.ptr, (num_receivers_ + 1) * sizeof(int), cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaMemcpyAsync(sources, sources_caller_.ptr, num_edges_ * sizeof(int), cudaMemcpyDeviceToHost, stream_));
    if (shifts != nullptr) {
        if (!has_shifts_) throw std::invalid_argument("The prepared graph carries no periodic shifts.");
        SXB_CUDA(cudaMemcpyAsync(shifts, shifts_caller_.ptr, 3 * num_edges_ * sizeof(int), cudaMemcpyDeviceToHost, stream_));
    }
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::launch_gemm(const float* A, const RowMap& a_rows, const float* B, int ldb, bool b_transposed, float* Cout,
                            const RowMap& c_rows, int first_node, int num_nodes, int N, int K, bool accumulate, const float* bias)
{
    if (num_nodes <= 0) return;
    GemmArgs args;
    args.A = A; args.B = B; args.C = Cout; args.bias = bias;
    args.a_rows = a_rows; args.c_rows = c_rows;
    args.first_node = first_node;
    args.M = num_nodes * a_rows.components;
    args.N = N; args.K = K; args.ldb = ldb;
    args.b_transposed = b_transposed ? 1 : 0;
    args.accumulate = accumulate ? 1 : 0;
    dim3 grid(blocks_for(args.M, kGemmBM), blocks_for(N, kGemmBN));
    gemm_rows_kernel<<<grid, 256, 0, stream_>>>(args);
    launches_ += 1;
}

cudaEvent_t Evaluator::pooled_event()
{
    if (events_used_ == event_pool_.size()) {
        cudaEvent_t e;
        SXB_CUDA(cudaEventCreate(&e));
        event_pool_.push_back(e);
    }
    return event_pool_[events_used_++];
}

void Evaluator::span_begin(const char* name)
{
    if (!profiling_) return;
    Span s;
    s.name = name;
    s.begin = pooled_event();
    s.end = pooled_event();
    s.launches = 0;
    span_launch_mark_ = launches_;
    SXB_CUDA(cudaEventRecord(s.begin, stream_));
    spans_.push_back(s);
}

void Evaluator::span_end()
{
    if (!profiling_) return;
    spans_.back().launches = static_cast<int>(launches_ - span_launch_mark_);
    SXB_CUDA(cudaEventRecord(spans_.back().end, stream_));
}

namespace {
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled_entry()
{
    static EncodeTiled fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        SXB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result));
        if (ptr == nullptr || result != cudaDriverEntryPointSuccess)
            throw std::runtime_error("cuTensorMapEncodeTiled is not available from the CUDA driver.");
        return reinterpret_cast<EncodeTiled>(ptr);
    }();
    return fn;
}

// Tensor map of a row-major FP32 matrix [n][k] (k contiguous): box [n_tile rows][32 floats], 128-byte swizzle.
CUtensorMap make_weight_map(const float* device_ptr, int n, int k, int n_tile)
{
    CUtensorMap map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * sizeof(float)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTcChunk), static_cast<cuuint32_t>(n_tile)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode_tiled_entry()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(device_ptr), dims, strides,
                                             box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed for a weight matrix.");
    return map;
}
}  // namespace

// Splits W [rows][cols] into a TF32-exact high part (low 13 mantissa bits cleared) and the
// residual, in both orientations the tensor-core kernel needs ([N][K], K contiguous).
void Evaluator::upload_split(SplitWeight& out, const float* w, int rows, int cols)
{
    out.rows = rows;
    out.cols = cols;
    const std::size_t n = static_cast<std::size_t>(rows) * cols;
    std::vector<float> hi(n), lo(n), thi(n), tlo(n);
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            const float v = w[static_cast<std::size_t>(r) * cols + c];
            // high part rounded to nearest TF32 (not truncated): the residual then has either sign, so the one product
            // the three-pass scheme drops, a_lo * w_lo, carries no systematic sign (the activations' high part is the
            // hardware's truncation, whose residual always has the sign of the value)
            std::uint32_t bits;
            std::memcpy(&bits, &v, 4);
            if ((bits & 0x7f800000u) != 0x7f800000u) bits += 0x00001000u;
            bits &= 0xffffe000u;
            float h;
            std::memcpy(&h, &bits, 4);
            const float l = v - h;
            hi[static_cast<std::size_t>(r) * cols + c] = h;      // rev: Bt[n = r][k = c] = W[r][c]
            lo[static_cast<std::size_t>(r) * cols + c] = l;
            thi[static_cast<std::size_t>(c) * rows + r] = h;     // fwd: Bt[n = c][k = r] = W[r][c]
            tlo[static_cast<std::size_t>(c) * rows + r] = l;
        }
    upload(out.full, std::vector<float>(w, w + n), stream_);
    upload(out.rev_hi, hi, stream_);
    upload(out.rev_lo, lo, stream_);
    upload(out.fwd_hi, thi, stream_);
    upload(out.fwd_lo, tlo, stream_);
    SXB_CUDA(cudaStreamSynchronize(stream_));
    // forward product: N = cols, K = rows; reverse product: N = rows, K = cols
    if (rows % kTcChunk != 0 || cols % kTcChunk != 0)
        throw std::invalid_argument("Linear extents must be multiples of 32 for the tensor-core kernel.");
    out.map_fwd_hi = make_weight_map(out.fwd_hi.ptr, cols, rows, std::min(cols, kTcNTile));
    out.map_fwd_lo = make_weight_map(out.fwd_lo.ptr, cols, rows, std::min(cols, kTcNTile));
    out.map_rev_hi = make_weight_map(out.rev_hi.ptr, rows, cols, std::min(rows, kTcNTile));
    out.map_rev_lo = make_weight_map(out.rev_lo.ptr, rows, cols, std::min(rows, kTcNTile));
    out.wide_fwd_hi = make_weight_map(out.fwd_hi.ptr, cols, rows, std::min(cols, 128));
    out.wide_fwd_lo = make_weight_map(out.fwd_lo.ptr, cols, rows, std::min(cols, 128));
    out.wide_rev_hi = make_weight_map(out.rev_hi.ptr, rows, cols, std::min(rows, 128));
    out.wide_rev_lo = make_weight_map(out.rev_lo.ptr, rows, cols, std::min(rows, 128));
}

// Runs a group of independent linears as one tensor-core launch (or as FP32 SIMT launches when the
// tensor-core path is switched off for comparison).
namespace {
// Rank-3 view [node][component][K] of the A rows of a linear (K contiguous floats per row), boxes of
// whole nodes: box = [nodes_per_tile][components][32 floats], 128-byte swizzle.
CUtensorMap make_activation_map(const float* A, const RowMap& rows, int first_node, int num_nodes, int K, int nodes_per_tile)
{
    CUtensorMap map;
    const float* base = A + rows.offset + static_cast<long>(first_node) * rows.node_stride;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows.components), static_cast<cuuint64_t>(num_nodes)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(rows.component_stride) * sizeof(float),
                                   static_cast<cuuint64_t>(rows.node_stride) * sizeof(float)};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(kTcChunk), static_cast<cuuint32_t>(rows.components),
                               static_cast<cuuint32_t>(nodes_per_tile)};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult rc = encode_tiled_entry()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, elem,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed for an activation tensor.");
    return map;
}
}  // namespace

void Evaluator::launch_tc(const std::vector<TcCall>& calls)
{
    if (!use_tensor_cores_) {
        for (const auto& c : calls) {
            const int N = c.reverse ? c.w->rows : c.w->cols, K = c.reverse ? c.w->cols : c.w->rows;
            launch_gemm(c.A, c.a_rows, c.w->full.ptr, c.w->cols, c.reverse, c.C, c.c_rows, c.first_node, c.num_nodes, N, K,
                        c.accumulate, c.bias);
        }
        return;
    }
    bool streaming = use_tma_activations_;
    for (const auto& c : calls) {
        const int N = c.reverse ? c.w->rows : c.w->cols;
        const int n_tile = std::min(N, 128);
        if ((n_tile != 32 && n_tile != 64 && n_tile != 128) || N % n_tile != 0) streaming = false;
    }
    if (streaming) {
        std::size_t next = 0;
        while (next < calls.size()) {
            Tc3Batch batch;
            std::memset(static_cast<void*>(&batch), 0, sizeof(batch));
            int tiles = 0, count = 0;
            for (; next < calls.size() && count < kT3MaxProblems; ++next) {
                const auto& c = calls[next];
                if (c.num_nodes <= 0) continue;
                Tc3Problem& p = batch.problem[count];
                p.N = c.reverse ? c.w->rows : c.w->cols;
                p.K = c.reverse ? c.w->cols : c.w->rows;
                if (p.K % kTcChunk != 0) throw std::invalid_argument("Linear extents are not supported by the tensor-core kernel.");
                p.n_tile = std::min(p.N, 128);
                p.n_tiles = p.N / p.n_tile;
                p.nodes_per_tile = kTcRows / c.a_rows.components;
                p.rows_per_tile = p.nodes_per_tile * c.a_rows.components;
                p.map_a = make_activation_map(c.A, c.a_rows, c.first_node, c.num_nodes, p.K, p.nodes_per_tile);
                p.map_hi = c.reverse ? c.w->wide_rev_hi : c.w->wide_fwd_hi;
                p.map_lo = c.reverse ? c.w->wide_rev_lo : c.w->wide_fwd_lo;
                p.C = c.C;
                p.bias = c.bias;
                p.c_rows = c.c_rows;
                p.first_node = c.first_node;
                p.M = c.num_nodes * c.a_rows.components;
                p.accumulate = c.accumulate ? 1 : 0;
                p.m_tiles = (c.num_nodes + p.nodes_per_tile - 1) / p.nodes_per_tile;
                p.tile_begin = tiles;
                tiles += p.m_tiles * p.n_tiles;
                ++count;
            }
            if (count == 0) continue;
            batch.count = count;
            batch.total_tiles = tiles;
            tc_gemm_tma_kernel<<<std::min(tiles, num_sms_), kT3Threads, kT3SmemBytes, stream_>>>(batch, error_flag_.ptr);
            launches_ += 1;
        }
        return;
    }
    std::size_t begin = 0;
    while (begin < calls.size()) {
        TcBatch batch;
        std::memset(static_cast<void*>(&batch), 0, sizeof(batch));
        int tiles = 0, count = 0;
        for (; begin < calls.size() && count < kTcMaxProblems; ++begin) {
            const auto& c = calls[begin];
            if (c.num_nodes <= 0) continue;
            TcProblem& p = batch.problem[count];
            p.A = c.A;
            p.map_hi = c.reverse ? c.w->map_rev_hi : c.w->map_fwd_hi;
            p.map_lo = c.reverse ? c.w->map_rev_lo : c.w->map_fwd_lo;
            p.C = c.C;
            p.bias = c.bias;
            p.a_rows = c.a_rows;
            p.c_rows = c.c_rows;
            p.first_node = c.first_node;
            p.M = c.num_nodes * c.a_rows.components;
            p.N = c.reverse ? c.w->rows : c.w->cols;
            p.K = c.reverse ? c.w->cols : c.w->rows;
            p.accumulate = c.accumulate ? 1 : 0;
            p.n_tile = std::min(p.N, kTcNTile);
            if (p.K % kTcChunk != 0 || p.N % p.n_tile != 0 || p.n_tile % 32 != 0)
                throw std::invalid_argument("Linear extents are not supported by the tensor-core kernel.");
            p.m_tiles = (p.M + kTcRows - 1) / kTcRows;
            p.n_tiles = p.N / p.n_tile;
            p.tile_begin = tiles;
            tiles += p.m_tiles * p.n_tiles;
            ++count;
        }
        if (count == 0) continue;
        batch.count = count;
        batch.total_tiles = tiles;
        tc_gemm_kernel<<<tiles, kTcThreads, kTcSmemBytes, stream_>>>(batch, error_flag_.ptr);
        launches_ += 1;
    }
}

// phases: bit 0 = up to H1 of the receivers, bit 1 = layer 1 forward .. fused layer-1 gradient,
// bit 2 = the rest of the reverse pass.  Between the phases a domain-decomposed run exchanges the
// H1 rows and then the H1_adj rows of its ghost nodes (reference: begin / continue /
// finish_factorized_distributed_evaluation, libsymmetrix/source/mace_kokkos_evaluate.cpp:1658-2101).
void Evaluator::run_pipeline(int phases)
{
    const int R = num_receivers_, ALL = num_nodes_, C = model_.channels, NH = model_.num_hidden, NE = model_.num_lme;
    const int n_active = static_cast<int>(active_types_.size());
    const int tile_cap = tile_capacity();
    const bool tiled = tile_cap < R;
    const std::size_t rowH = static_cast<std::size_t>(NH) * C;
    const RowMap scalar_rows{static_cast<long>(NH) * C, C, 0, 1};
    const RowMap flat_rows{static_cast<long>(C), C, 0, 1};
    ForceOutputs fo;
    fo.atom_forces = forces_.ptr;
    fo.virial_slots = virial_slots_.ptr;
    fo.edge_forces = keep_edge_forces_ ? edge_forces_.ptr : nullptr;
    fo.accumulate_edge = 0;
    fo.edge_source_adjoint = nullptr;
    if (deterministic_) {       // no atomics: per-edge records, summed over the source schedule
        fo.atom_forces = nullptr;
        fo.edge_source_adjoint = edge_source_adjoint_.ptr;
    }
    double* const energy_slots = deterministic_ ? nullptr : energy_slots_.ptr;
    const int warp_threads = 32 * kWarpsPerBlock;

    // launch helpers for one tile of T receivers starting at t0 (tile tensors are indexed from 0)
    const float* inv0 = model_.a0_scaled ? inv_scale0_.ptr : nullptr;
    const float* inv1 = model_.a1_scaled ? inv_scale1_.ptr : nullptr;
    const DensityScale density0{model_.a0_scaled ? density0_table_.ptr : nullptr, inv_scale0_.ptr, dot0_.ptr, n_active};
    const DensityScale density1{model_.a1_scaled ? density1_table_.ptr : nullptr, inv_scale1_.ptr, dot1_.ptr, n_active};
    auto l0_forward = [&](int t0, int T) {
        const int warp_grid = blocks_for(T, kWarpsPerBlock);
        if (C == 128)
            l0_forward_warp_kernel<4><<<warp_grid, warp_threads, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_.ptr, inv0);
        else if (C == 64)
            l0_forward_warp_kernel<2><<<warp_grid, warp_threads, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_.ptr, inv0);
        else if (C == 32)
            l0_forward_warp_kernel<1><<<warp_grid, warp_threads, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_.ptr, inv0);
        else
            l0_forward_kernel<0><<<T, C, 0, stream_>>>(T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_.ptr, inv0);
        launches_ += 1;
    };
    // per-element node ranges intersected with the tile
    auto for_type_ranges = [&](int t0, int T, auto&& body) {
        for (int a = 0; a < n_active; ++a) {
            const int begin = std::max(type_begin_[a], t0), end = std::min(type_begin_[a + 1], t0 + T);
            if (end > begin) body(a, begin, end - begin);
        }
    };

    if (phases & 1) {
        spans_.clear();
        events_used_ = 0;
        SXB_CUDA(cudaMemsetAsync(forces_.ptr, 0, sizeof(double) * 3 * ALL, stream_));
        SXB_CUDA(cudaMemsetAsync(H1_adj_.ptr, 0, sizeof(float) * static_cast<std::size_t>(ALL) * rowH, stream_));
        if (model_.legacy_h1_basis) {   // old basis: dE/dH1 starts from the first readout's weights on the scalar block
            fill_scalar_block_kernel<<<blocks_for(static_cast<long>(R) * C, 256), 256, 0, stream_>>>(R, C, static_cast<long>(rowH),
                                                                                                    readout1_.ptr, H1_adj_.ptr);
            launches_ += 1;
        }
        SXB_CUDA(cudaMemsetAsync(energy_slots_.ptr, 0, sizeof(double) * kVirialSlots, stream_));
        SXB_CUDA(cudaMemsetAsync(virial_slots_.ptr, 0, sizeof(double) * kVirialSlots * 9, stream_));
        if (model_.a0_scaled || model_.a1_scaled) {
            if (model_.a0_scaled) SXB_CUDA(cudaMemsetAsync(dot0_.ptr, 0, sizeof(float) * R, stream_));
            if (model_.a1_scaled) SXB_CUDA(cudaMemsetAsync(dot1_.ptr, 0, sizeof(float) * R, stream_));
            span_begin("density_scales");
            density_scale_kernel<<<blocks_for(static_cast<long>(R) * 32, 256), 256, 0, stream_>>>(
                R, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, density0.table, density1.table, inv_scale0_.ptr,
                inv_scale1_.ptr);
            launches_ += 1;
            span_end();
        }
        for (int t0 = 0; t0 < R; t0 += tile_cap) {
            const int T = std::min(tile_cap, R - t0);
            span_begin("l0_forward");
            l0_forward(t0, T);
            span_end();
            span_begin("m0_forward");
            float* m0 = M0_.ptr + t0 * rowH;
            if (model_.shape_id == 0)
                SXB_LAUNCH_POLY(m0_forward_kernel_S0, poly_g_forward_, SXB_S0_M0_NUM_TERMS, T, C, stream_, T, C, A0_.ptr, element_.ptr + t0, m0_weights_.ptr, m0);
            else if (model_.shape_id == 1)
                SXB_LAUNCH_POLY(m0_forward_kernel_S1, poly_g_forward_, SXB_S1_M0_NUM_TERMS, T, C, stream_, T, C, A0_.ptr, element_.ptr + t0, m0_weights_.ptr, m0);
            else
                SXB_LAUNCH_POLY(m0_forward_kernel_S2, poly_g_forward_, SXB_S2_M0_NUM_TERMS, T, C, stream_, T, C, A0_.ptr, element_.ptr + t0, m0_weights_.ptr, m0);
            launches_ += 1;
            span_end();
            // H1_il = M0_il W_l
            span_begin("gemm_h1");
            std::vector<TcCall> calls;
            for (int l = 0; l <= model_.hidden_l_max; ++l) {
                const RowMap rows{static_cast<long>(NH) * C, C, static_cast<long>(l) * l * C, 2 * l + 1};
                calls.push_back({m0, rows, &s_h1_[l], false, H1_.ptr + t0 * rowH, rows, 0, T, false, nullptr});
            }
            // one tile: the element-dependent skip term of H2 (x_i T_element) only needs M0, so it rides in this launch
            if (!tiled && !model_.legacy_h1_basis && !model_.pre_linear_up)
                for_type_ranges(t0, T, [&](int a, int begin, int count) {
                    calls.push_back({M0_.ptr + begin * rowH, scalar_rows, &s_h2_skip_[active_types_[a]], false,
                                     H2_.ptr + static_cast<std::size_t>(begin - t0) * C, flat_rows, 0, count, false, nullptr});
                });
            if (model_.pre_linear_up)   // x = M0[l=0] P0, the scalar input of the first readout and the skip
                calls.push_back({m0, scalar_rows, &s_product0_, false, scalar_input_.ptr + static_cast<std::size_t>(t0) * C, flat_rows, 0, T,
                                 false, nullptr});
            launch_tc(calls);
            if (model_.first_residual) {   // element-dependent constants: R U joins H1, R of the scalar block joins x
                add_element_rows_kernel<<<blocks_for(static_cast<long>(T) * rowH, 256), 256, 0, stream_>>>(
                    T, static_cast<int>(rowH), element_.ptr + t0, residual_fused_.ptr, H1_.ptr + t0 * rowH);
                add_element_rows_kernel<<<blocks_for(static_cast<long>(T) * C, 256), 256, 0, stream_>>>(
                    T, C, element_.ptr + t0, residual_scalar_.ptr, scalar_input_.ptr + static_cast<std::size_t>(t0) * C);
                launches_ += 2;
            }
            span_end();
        }
        if (phases != 7 && halo_plan_.active && halo_plan_.send_rows != nullptr) {   // forward halo: my owned rows that peers hold as ghosts
            span_begin("halo_pack");
            pack_rows(0, halo_plan_.send_indices, halo_plan_.num_send, halo_plan_.send_rows);
            span_end();
        }
    }
    if (phases & 2) {
        if (model_.shape_id == 2 && fo.edge_forces != nullptr)   // the split gradient kernels accumulate into it
            SXB_CUDA(cudaMemsetAsync(fo.edge_forces, 0, sizeof(double) * 3 * static_cast<std::size_t>(num_edges_), stream_));
        for (int t0 = 0; t0 < R; t0 += tile_cap) {
            const int T = std::min(tile_cap, R - t0);
            if (model_.single_layer) {
                // no second message step: the readout polynomial acts on H1 of the receivers
                span_begin("m1_forward");
                hidden_poly_kernel<false><<<blocks_for(static_cast<long>(T) * C, 128), 128, 0, stream_>>>(
                    T, C, NH, static_cast<int>(model_.hidden_poly_terms.size() / 4), reinterpret_cast<const int4*>(hidden_poly_terms_.ptr),
                    H1_.ptr + t0 * rowH, element_.ptr + t0, hidden_poly_weights_.ptr, M1_.ptr, nullptr, nullptr);
                launches_ += 1;
                span_end();
            } else {
            span_begin("l1_forward");
            if (model_.shape_id == 0)
                SXB_LAUNCH_BY_CHANNELS(l1_forward_kernel_S0, C, T, stream_, T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_,
                                       reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, coupling_, Phi1_.ptr, inv1, r1_pair_types_);
            else if (model_.shape_id == 1)
                SXB_LAUNCH_BY_CHANNELS(l1_forward_kernel_S1, C, T, stream_, T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_,
                                       reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, coupling_, Phi1_.ptr, inv1, r1_pair_types_);
            else {
                // one launch per path set; the sets write disjoint components of Phi1
#define SXB_SPLIT_FORWARD(SET)                                                                                            \
                l1_forward_split_kernel_S2_##SET<128><<<T, 128, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_, \
                    reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, coupling_, Phi1_.ptr, inv1, r1_pair_types_)
                SXB_SPLIT_FORWARD(G0);
                SXB_SPLIT_FORWARD(G1);
                SXB_SPLIT_FORWARD(G2);
#undef SXB_SPLIT_FORWARD
                launches_ += 2;
            }
            launches_ += 1;
            span_end();
            // A1_il = Phi1_il W_l
            span_begin("gemm_a1");
            {
                std::vector<TcCall> calls;
                for (int l = 0; l <= model_.l_max; ++l) {
                    const int eta = model_.eta[l];
                    const RowMap a_rows{static_cast<long>(NE) * C, static_cast<long>(eta) * C, static_cast<long>(model_.group_begin[l]) * C, 2 * l + 1};
                    const RowMap c_rows{16L * C, C, static_cast<long>(l) * l * C, 2 * l + 1};
                    calls.push_back({Phi1_.ptr, a_rows, &s_a1_[l], false, A1_.ptr, c_rows, 0, T, false, nullptr});
                }
                launch_tc(calls);
            }
            span_end();
            span_begin("m1_forward");
            if (model_.shape_id == 0)
                SXB_LAUNCH_POLY(m1_forward_kernel_S0, poly_g_forward_, SXB_S0_M1_NUM_TERMS, T, C, stream_, T, C, A1_.ptr, element_.ptr + t0, m1_weights_.ptr, M1_.ptr);
            else if (model_.shape_id == 1)
                SXB_LAUNCH_POLY(m1_forward_kernel_S1, poly_g_forward_, SXB_S1_M1_NUM_TERMS, T, C, stream_, T, C, A1_.ptr, element_.ptr + t0, m1_weights_.ptr, M1_.ptr);
            else
                SXB_LAUNCH_POLY(m1_forward_kernel_S2, poly_g_forward_, SXB_S2_M1_NUM_TERMS, T, C, stream_, T, C, A1_.ptr, element_.ptr + t0, m1_weights_.ptr, M1_.ptr);
            launches_ += 1;
            span_end();
            }
            // H2 = xs T_element + M1 W
            span_begin("gemm_h2");
            {
                if (tiled || model_.legacy_h1_basis || model_.pre_linear_up) {
                    const float* skip_input = model_.legacy_h1_basis ? H1_.ptr : M0_.ptr;   // old basis: the skip reads H1
                    std::vector<TcCall> calls;
                    for_type_ranges(t0, T, [&](int a, int begin, int count) {
                        if (model_.pre_linear_up)
                            calls.push_back({scalar_input_.ptr + static_cast<std::size_t>(begin) * C, flat_rows, &s_h2_skip_[active_types_[a]],
                                             false, H2_.ptr + static_cast<std::size_t>(begin - t0) * C, flat_rows, 0, count, false, nullptr});
                        else
                            calls.push_back({skip_input + begin * rowH, scalar_rows, &s_h2_skip_[active_types_[a]], false,
                                             H2_.ptr + static_cast<std::size_t>(begin - t0) * C, flat_rows, 0, count, false, nullptr});
                    });
                    launch_tc(calls);
                }
                launch_tc({{M1_.ptr, flat_rows, &s_h2_m1_, false, H2_.ptr, flat_rows, 0, T, true, nullptr}});
            }
            span_end();
            span_begin("readout");
            // scalar block the first readout acts on, and the stride between nodes in components
            const float* readout_input = model_.pre_linear_up ? scalar_input_.ptr : model_.legacy_h1_basis ? H1_.ptr : M0_.ptr;
            const int readout_stride = model_.pre_linear_up ? 1 : NH;
            const std::size_t readout_row = static_cast<std::size_t>(readout_stride) * C;
            if (model_.readout2_hidden == 16 && (C == 128 || C == 32)) {
#define SXB_READOUT16(CHUNKS)                                                                                             \
                readout16_kernel<CHUNKS><<<blocks_for(static_cast<long>(T) * 32, 256), 256, 0, stream_>>>(                 \
                    T, model_.readout2_scale, readout_input + t0 * readout_row, readout_stride, H2_.ptr, element_.ptr + t0,         \
                    atomic_energies_.ptr,                                                                                 \
                    readout1_.ptr, readout2_w1_.ptr, readout2_w2_.ptr, node_energies_.ptr + t0,                            \
                    H2_adj_.ptr + static_cast<std::size_t>(t0) * C, energy_slots)
                if (C == 128) SXB_READOUT16(4);
                else SXB_READOUT16(1);
#undef SXB_READOUT16
            } else
                readout_kernel<<<blocks_for(static_cast<long>(T) * 32, 256), 256, 0, stream_>>>(
                    T, C, model_.readout2_hidden, model_.readout2_scale, readout_input + t0 * readout_row, readout_stride, H2_.ptr, element_.ptr + t0,
                    atomic_energies_.ptr, readout1_.ptr, readout2_w1_.ptr, readout2_w2_.ptr, node_energies_.ptr + t0,
                    H2_adj_.ptr + static_cast<std::size_t>(t0) * C, energy_slots);
            launches_ += 1;
            span_end();
            // reverse
            span_begin("gemm_h2_reverse");
            {
                std::vector<TcCall> calls{{H2_adj_.ptr + static_cast<std::size_t>(t0) * C, flat_rows, &s_h2_m1_, true, M1_adj_.ptr,
                                           flat_rows, 0, T, false, nullptr}};
                // one tile: the direct adjoint of the scalar block of M0, q + T_element H2_adj, is known here already;
                // the reverse of the H1 linear adds to it later
                if (model_.pre_linear_up)   // adjoint of x: q + S_element H2_adj, multiplied by P0^T in the last phase
                    for_type_ranges(t0, T, [&](int a, int begin, int count) {
                        calls.push_back({H2_adj_.ptr + static_cast<std::size_t>(begin) * C, flat_rows, &s_h2_skip_[active_types_[a]], true,
                                         scalar_adjoint_.ptr + static_cast<std::size_t>(begin) * C, flat_rows, 0, count, false, readout1_.ptr});
                    });
                else if (!tiled && !model_.legacy_h1_basis)
                    for_type_ranges(t0, T, [&](int a, int begin, int count) {
                        calls.push_back({H2_adj_.ptr + static_cast<std::size_t>(begin) * C, flat_rows, &s_h2_skip_[active_types_[a]], true,
                                         M0_adj_.ptr + (begin - t0) * rowH, scalar_rows, 0, count, false, readout1_.ptr});
                    });
                launch_tc(calls);
            }
            span_end();
            if (model_.single_layer) {
                span_begin("m1_reverse");
                hidden_poly_kernel<true><<<blocks_for(static_cast<long>(T) * C, 128), 128, 0, stream_>>>(
                    T, C, NH, static_cast<int>(model_.hidden_poly_terms.size() / 4), reinterpret_cast<const int4*>(hidden_poly_terms_.ptr),
                    H1_.ptr + t0 * rowH, element_.ptr + t0, hidden_poly_weights_.ptr, nullptr, M1_adj_.ptr, H1_adj_.ptr + t0 * rowH);
                launches_ += 1;
                span_end();
                continue;
            }
            span_begin("m1_reverse");
            if (model_.shape_id == 0)
                SXB_LAUNCH_POLY(m1_reverse_kernel_S0, poly_g_reverse_, SXB_S0_M1_NUM_TERMS, T, C, stream_, T, C, A1_.ptr, element_.ptr + t0, m1_weights_.ptr, M1_adj_.ptr, A1_adj_.ptr, model_.a1_scaled ? dot1_.ptr + t0 : nullptr);
            else if (model_.shape_id == 1)
                SXB_LAUNCH_POLY(m1_reverse_kernel_S1, poly_g_reverse_, SXB_S1_M1_NUM_TERMS, T, C, stream_, T, C, A1_.ptr, element_.ptr + t0, m1_weights_.ptr, M1_adj_.ptr, A1_adj_.ptr, model_.a1_scaled ? dot1_.ptr + t0 : nullptr);
            else
                SXB_LAUNCH_POLY(m1_reverse_kernel_S2, poly_g_reverse_, SXB_S2_M1_NUM_TERMS, T, C, stream_, T, C, A1_.ptr, element_.ptr + t0, m1_weights_.ptr, M1_adj_.ptr, A1_adj_.ptr, model_.a1_scaled ? dot1_.ptr + t0 : nullptr);
            launches_ += 1;
            span_end();
            span_begin("gemm_a1_reverse");
            {
                std::vector<TcCall> calls;
                for (int l = 0; l <= model_.l_max; ++l) {
                    const int eta = model_.eta[l];
                    const RowMap a_rows{16L * C, C, static_cast<long>(l) * l * C, 2 * l + 1};
                    const RowMap c_rows{static_cast<long>(NE) * C, static_cast<long>(eta) * C, static_cast<long>(model_.group_begin[l]) * C, 2 * l + 1};
                    calls.push_back({A1_adj_.ptr, a_rows, &s_a1_[l], true, dPhi1_.ptr, c_rows, 0, T, false, nullptr});
                }
                launch_tc(calls);
            }
            span_end();
            span_begin("l1_reverse");
            if (deterministic_ && model_.shape_id == 0)      // records instead of atomics: the build with the channel count at run time
                l1_reverse_kernel_S0<0, 3, true><<<T, C, 0, stream_>>>(T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_,
                    reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, dPhi1_.ptr, coupling_, H1_adj_.ptr, fo, density1, r1_pair_types_);
            else if (deterministic_ && model_.shape_id == 1)
                l1_reverse_kernel_S1<0, 3, true><<<T, C, 0, stream_>>>(T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_,
                    reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, dPhi1_.ptr, coupling_, H1_adj_.ptr, fo, density1, r1_pair_types_);
            else if (model_.shape_id == 0)
                SXB_LAUNCH_BY_CHANNELS(l1_reverse_kernel_S0, C, T, stream_, T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_,
                                       reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, dPhi1_.ptr, coupling_, H1_adj_.ptr, fo, density1, r1_pair_types_);
            else if (model_.shape_id == 1)
                SXB_LAUNCH_BY_CHANNELS(l1_reverse_kernel_S1, C, T, stream_, T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_,
                                       reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, dPhi1_.ptr, coupling_, H1_adj_.ptr, fo, density1, r1_pair_types_);
            else {
                // one launch per path set; the sets add into the same edge forces, so those are cleared
                // first and accumulated atomically
                ForceOutputs split = fo;
                split.accumulate_edge = 2;
#define SXB_SPLIT_REVERSE(SET)                                                                                            \
                l1_reverse_split_kernel_S2_##SET<128><<<T, 128, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, grid_, \
                    reinterpret_cast<const float4*>(r1_table_.ptr), H1_.ptr, dPhi1_.ptr, coupling_, H1_adj_.ptr, split, density1, r1_pair_types_)
                SXB_SPLIT_REVERSE(G0);
                SXB_SPLIT_REVERSE(G1);
                SXB_SPLIT_REVERSE(G2);
#undef SXB_SPLIT_REVERSE
                launches_ += 2;
            }
            launches_ += 1;
            span_end();
        }
        if (deterministic_ && !model_.single_layer) {
            span_begin("source_adjoint_schedule");
            reduce_source_adjoint_kernel<<<ALL, 128, 0, stream_>>>(NH * C, source_offsets_.ptr, source_edges_.ptr, geom_.ptr, grid_.r_cut,
                                                                  edge_source_adjoint_.ptr, H1_adj_.ptr);
            launches_ += 1;
            span_end();
        }
    }
    if (phases & 4) {
        fo.accumulate_edge = model_.single_layer ? 0 : 1;   // the layer-1 gradient wrote the edge forces first
        if (phases != 7 && halo_plan_.active && halo_plan_.received_rows != nullptr) {   // reverse halo: adjoints my atoms collected as ghosts of the peers
            span_begin("halo_unpack");
            unpack_rows(1, halo_plan_.send_indices, halo_plan_.num_send, halo_plan_.received_rows, true);
            span_end();
        }
        for (int t0 = 0; t0 < R; t0 += tile_cap) {
            const int T = std::min(tile_cap, R - t0);
            if (tiled) {
                // the tile workspace no longer holds this tile's A0: regenerate it
                span_begin("l0_forward_recompute");
                l0_forward(t0, T);
                span_end();
            }
            span_begin("gemm_h1_reverse");
            // M0_adj_il = H1_adj_il W_l^T, then the direct adjoint q + T_element H2_adj on the scalar block
            if (model_.pre_linear_up) {
                // M0_adj = H1_adj W^T, then the scalar block gains (q + S_element H2_adj) P0^T
                std::vector<TcCall> calls;
                for (int l = 0; l <= model_.hidden_l_max; ++l) {
                    const RowMap rows{static_cast<long>(NH) * C, C, static_cast<long>(l) * l * C, 2 * l + 1};
                    calls.push_back({H1_adj_.ptr + t0 * rowH, rows, &s_h1_[l], true, M0_adj_.ptr, rows, 0, T, false, nullptr});
                }
                launch_tc(calls);
                launch_tc({{scalar_adjoint_.ptr + static_cast<std::size_t>(t0) * C, flat_rows, &s_product0_, true, M0_adj_.ptr, scalar_rows, 0, T,
                            true, nullptr}});
            } else if (model_.legacy_h1_basis) {
                // old basis: the skip's adjoint S_element H2_adj joins H1_adj (which started from q) before the linear
                std::vector<TcCall> calls;
                for_type_ranges(t0, T, [&](int a, int begin, int count) {
                    calls.push_back({H2_adj_.ptr + static_cast<std::size_t>(begin) * C, flat_rows, &s_h2_skip_[active_types_[a]], true,
                                     H1_adj_.ptr + begin * rowH, scalar_rows, 0, count, true, nullptr});
                });
                launch_tc(calls);
                calls.clear();
                for (int l = 0; l <= model_.hidden_l_max; ++l) {
                    const RowMap rows{static_cast<long>(NH) * C, C, static_cast<long>(l) * l * C, 2 * l + 1};
                    calls.push_back({H1_adj_.ptr + t0 * rowH, rows, &s_h1_[l], true, M0_adj_.ptr, rows, 0, T, false, nullptr});
                }
                launch_tc(calls);
            } else {
                std::vector<TcCall> calls;
                for (int l = 0; l <= model_.hidden_l_max; ++l) {
                    const RowMap rows{static_cast<long>(NH) * C, C, static_cast<long>(l) * l * C, 2 * l + 1};
                    if (tiled)
                        calls.push_back({H1_adj_.ptr + t0 * rowH, rows, &s_h1_[l], true, M0_adj_.ptr, rows, 0, T, false,
                                         l == 0 ? readout1_.ptr : nullptr});
                    else   // the scalar block already holds the direct adjoint (written with the H2 reverse linear)
                        calls.push_back({H1_adj_.ptr + t0 * rowH, rows, &s_h1_[l], true, M0_adj_.ptr, rows, 0, T, l == 0, nullptr});
                }
                launch_tc(calls);
                if (tiled) {
                    calls.clear();
                    for_type_ranges(t0, T, [&](int a, int begin, int count) {
                        calls.push_back({H2_adj_.ptr + static_cast<std::size_t>(begin) * C, flat_rows, &s_h2_skip_[active_types_[a]], true,
                                         M0_adj_.ptr + (begin - t0) * rowH, scalar_rows, 0, count, true, nullptr});
                    });
                    launch_tc(calls);
                }
            }
            span_end();
            span_begin("m0_reverse");
            if (model_.shape_id == 0)
                SXB_LAUNCH_POLY(m0_reverse_kernel_S0, poly_g_reverse_, SXB_S0_M0_NUM_TERMS, T, C, stream_, T, C, A0_.ptr, element_.ptr + t0, m0_weights_.ptr, M0_adj_.ptr, A0_adj_.ptr, model_.a0_scaled ? dot0_.ptr + t0 : nullptr);
            else if (model_.shape_id == 1)
                SXB_LAUNCH_POLY(m0_reverse_kernel_S1, poly_g_reverse_, SXB_S1_M0_NUM_TERMS, T, C, stream_, T, C, A0_.ptr, element_.ptr + t0, m0_weights_.ptr, M0_adj_.ptr, A0_adj_.ptr, model_.a0_scaled ? dot0_.ptr + t0 : nullptr);
            else
                SXB_LAUNCH_POLY(m0_reverse_kernel_S2, poly_g_reverse_, SXB_S2_M0_NUM_TERMS, T, C, stream_, T, C, A0_.ptr, element_.ptr + t0, m0_weights_.ptr, M0_adj_.ptr, A0_adj_.ptr, model_.a0_scaled ? dot0_.ptr + t0 : nullptr);
            launches_ += 1;
            span_end();
            span_begin("l0_reverse");
            {
                const int warp_grid = blocks_for(T, kWarpsPerBlock);
                if (C == 128)
                    l0_reverse_warp_kernel<4><<<warp_grid, warp_threads, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_adj_.ptr, fo, density0);
                else if (C == 64)
                    l0_reverse_warp_kernel<2><<<warp_grid, warp_threads, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_adj_.ptr, fo, density0);
                else if (C == 32)
                    l0_reverse_warp_kernel<1><<<warp_grid, warp_threads, 0, stream_>>>(T, t0, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_adj_.ptr, fo, density0);
                else
                    l0_reverse_kernel<0><<<T, C, 0, stream_>>>(T, t0, C, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, grid_, r0_table_.ptr, A0_adj_.ptr, fo, density0);
            }
            launches_ += 1;
            span_end();
        }
        if (model_.has_zbl) {
            span_begin("zbl");
            ZblParams zp;
            zp.pairs = reinterpret_cast<const ZblPair*>(zbl_pairs_.ptr);
            for (int q = 0; q < 4; ++q) zp.c[q] = static_cast<float>(model_.zbl_c[q]);
            zp.p = model_.zbl_p;
            zbl_kernel<<<blocks_for(static_cast<long>(R) * 32, 256), 256, 0, stream_>>>(
                R, first_.ptr, sources_.ptr, geom_.ptr, atype_.ptr, n_active, zp, node_energies_.ptr, energy_slots_.ptr, fo);
            launches_ += 1;
            span_end();
        }
        span_begin("finalize");
        if (deterministic_) {
            const long blocks = std::max<long>(blocks_for(std::max<long>(num_edges_, 1), kTotalsThreads), blocks_for(R, kTotalsThreads));
            reduce_node_forces_kernel<<<blocks_for(ALL, 128), 128, 0, stream_>>>(ALL, R, first_.ptr, source_offsets_.ptr, source_edges_.ptr,
                                                                                  edge_forces_.ptr, forces_.ptr);
            partial_totals_kernel<<<blocks, kTotalsThreads, 0, stream_>>>(num_edges_, R, geom_.ptr, edge_forces_.ptr, node_energies_.ptr,
                                                                          det_partials_.ptr);
            final_totals_kernel<<<1, 32, 0, stream_>>>(static_cast<int>(blocks), det_partials_.ptr, energy_slots_.ptr, virial_slots_.ptr);
            launches_ += 3;
        }
        publish_results_kernel<<<blocks_for(11 + static_cast<long>(R) + 3 * static_cast<long>(ALL), 256), 256, 0, stream_>>>(
            R, ALL, internal_of_.ptr, energy_slots_.ptr, virial_slots_.ptr, node_energies_.ptr, forces_.ptr, error_flag_.ptr, totals_.ptr,
            node_energies_out_.ptr, forces_out_.ptr, host_results_,
            // a decomposed run with a halo plan keeps energies and forces on the device: status and totals only
            (phases != 7 && halo_plan_.active) ? 11L : 11 + static_cast<long>(R) + 3 * static_cast<long>(ALL));
        launches_ += 1;
        if (phases != 7 && halo_plan_.active) {
            have_results_ = true;
            pack_ghost_forces(halo_plan_.world, halo_plan_.ghost_begin, num_nodes_ - num_receivers_, halo_plan_.force_send);
        }
        span_end();
    }
    SXB_CUDA(cudaGetLastError());
}

// Enqueues the geometry kernel (when `positions` is given) and the pipeline phases on the stream.
// Outside profiling the sequence is captured once per (phases, graph generation, position buffer)
// into a CUDA graph and replayed afterwards: every kernel argument is fixed for a prepared graph, so
// a step costs one graph launch instead of some twenty kernel launches.
void Evaluator::enqueue_phases(int phases, const double* positions, bool upload_staged)
{
    auto enqueue = [&] {
        if (upload_staged)
            SXB_CUDA(cudaMemcpyAsync(positions_.ptr, host_stage_, sizeof(double) * 3 * num_nodes_, cudaMemcpyHostToDevice, stream_));
        if (positions != nullptr) {
            SXB_CUDA(cudaMemsetAsync(error_flag_.ptr, 0, sizeof(int), stream_));
            const int grid = blocks_for(static_cast<long>(num_receivers_) * 32, 256);
            if (geometry_mode_ == 1)
                geometry_from_reference_kernel<false><<<grid, 256, 0, stream_>>>(
                    num_receivers_, first_.ptr, sources_.ptr, positions, original_.ptr, reference_positions_.ptr, reference_xyz_.ptr,
                    edge_map_.ptr, cell_.ptr, inv_cell_.ptr, pbc_mask_, geom_.ptr, error_flag_.ptr);
            else if (geometry_mode_ == 2)
                geometry_from_reference_kernel<true><<<grid, 256, 0, stream_>>>(
                    num_receivers_, first_.ptr, sources_.ptr, positions, original_.ptr, reference_positions_.ptr, reference_xyz_.ptr,
                    edge_map_.ptr, cell_.ptr, inv_cell_.ptr, pbc_mask_, geom_.ptr, error_flag_.ptr);
            else
                geometry_from_positions_kernel<<<grid, 256, 0, stream_>>>(
                    num_receivers_, first_.ptr, sources_.ptr, has_shifts_ ? shifts_.ptr : nullptr, positions, original_.ptr, cell_.ptr,
                    geom_.ptr, error_flag_.ptr);
            launches_ += 1;
        }
        run_pipeline(phases);
    };
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (stream_ != nullptr && cudaStreamIsCapturing(stream_, &capturing) != cudaSuccess) cudaGetLastError();
    if (!use_graphs_ || profiling_ || stream_ == nullptr || capturing != cudaStreamCaptureStatusNone) {
        enqueue();      // also when the caller is capturing this stream itself: the kernels then join its graph
        return;
    }
    StepGraph& slot = step_graphs_[phases];
    if (slot.exec == nullptr || slot.generation != generation_ || slot.positions != positions || slot.upload_staged != upload_staged
        || slot.keep_edge_forces != keep_edge_forces_) {
        if (slot.exec != nullptr) {
            cudaGraphExecDestroy(slot.exec);
            slot.exec = nullptr;
        }
        const long before = launches_;
        if (cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
            cudaGetLastError();        // this stream cannot be captured (e.g. the legacy default stream): launch directly
            use_graphs_ = false;
            enqueue();
            return;
        }
        cudaGraph_t graph = nullptr;
        try {
            enqueue();
        } catch (...) {
            cudaStreamEndCapture(stream_, &graph);
            if (graph != nullptr) cudaGraphDestroy(graph);
            launches_ = before;
            throw;
        }
        SXB_CUDA(cudaStreamEndCapture(stream_, &graph));
        const cudaError_t made = cudaGraphInstantiate(&slot.exec, graph, 0);
        cudaGraphDestroy(graph);
        slot.launches = launches_ - before;
        launches_ = before;
        if (made != cudaSuccess) {
            cudaGetLastError();
            slot.exec = nullptr;
            use_graphs_ = false;
            enqueue();
            return;
        }
        slot.generation = generation_;
        slot.positions = positions;
        slot.upload_staged = upload_staged;
        slot.keep_edge_forces = keep_edge_forces_;
    }
    SXB_CUDA(cudaGraphLaunch(slot.exec, stream_));
    launches_ += slot.launches;
}

void Evaluator::drop_step_graphs()
{
    for (auto& entry : step_graphs_)
        if (entry.second.exec != nullptr) cudaGraphExecDestroy(entry.second.exec);
    step_graphs_.clear();
}

void Evaluator::finish_compute()
{
    SXB_CUDA(cudaEventRecord(event_end_, stream_));
    int flag = 0;
    if (host_results_ != nullptr) {
        // the closing kernel has published status, totals, energies and forces into mapped host memory
        SXB_CUDA(cudaStreamSynchronize(stream_));
        flag = static_cast<int>(host_results_[0]);
        std::memcpy(host_totals_, host_results_ + 1, 10 * sizeof(double));
        mirror_valid_ = !halo_plan_.active;     // with a halo plan only status and totals were published
    } else {
        SXB_CUDA(cudaMemcpyAsync(&flag, error_flag_.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream_));
        SXB_CUDA(cudaMemcpyAsync(host_totals_, totals_.ptr, 10 * sizeof(double), cudaMemcpyDeviceToHost, stream_));
        SXB_CUDA(cudaStreamSynchronize(stream_));
        mirror_valid_ = false;
    }
    if (cudaEventElapsedTime(&last_ms_, event_begin_, event_end_) != cudaSuccess) {
        cudaGetLastError();       // the bracket was not recorded on this path (a caller-captured step): no device time
        last_ms_ = 0.0f;
    }
    profile_.clear();
    for (const auto& span : spans_) {
        float ms = 0.0f;
        SXB_CUDA(cudaEventElapsedTime(&ms, span.begin, span.end));
        profile_.push_back({span.name, ms, span.launches});
    }
    if (flag & 2) throw std::runtime_error("Tensor-core linear: a bounded wait expired; results are invalid.");
    if (flag != 0) throw std::invalid_argument("Edge geometry contains a zero-length or non-finite edge vector.");
    have_results_ = true;
}

void Evaluator::compute_positions(std::uint64_t generation, const double* positions, bool on_device)
{
    check_generation(generation);
    SXB_CUDA(cudaSetDevice(device_));
    have_results_ = false;
    mirror_valid_ = false;
    SXB_CUDA(cudaEventRecord(event_begin_, stream_));
    if (on_device) {
        enqueue_phases(7, positions, false);
    } else if (host_stage_ != nullptr) {
        // through the pinned staging copy: the upload is then a copy node of the captured step
        std::memcpy(host_stage_, positions, sizeof(double) * 3 * num_nodes_);
        enqueue_phases(7, positions_.ptr, true);
    } else {
        SXB_CUDA(cudaMemcpyAsync(positions_.ptr, positions, sizeof(double) * 3 * num_nodes_, cudaMemcpyHostToDevice, stream_));
        enqueue_phases(7, positions_.ptr, false);
    }
    finish_compute();
}

void Evaluator::compute_edge_vectors(std::uint64_t generation, const double* xyz)
{
    check_generation(generation);
    SXB_CUDA(cudaSetDevice(device_));
    have_results_ = false;
    mirror_valid_ = false;
    DeviceBuffer<double>& dxyz = edge_scratch_;      // kept between calls: the per-step call allocates nothing
    dxyz.reserve_with_slack(3 * static_cast<std::size_t>(num_edges_));
    SXB_CUDA(cudaEventRecord(event_begin_, stream_));
    SXB_CUDA(cudaMemcpyAsync(dxyz.ptr, xyz, sizeof(double) * 3 * num_edges_, cudaMemcpyHostToDevice, stream_));
    SXB_CUDA(cudaMemsetAsync(error_flag_.ptr, 0, sizeof(int), stream_));
    geometry_from_vectors_kernel<<<blocks_for(num_edges_, 256), 256, 0, stream_>>>(num_edges_, dxyz.ptr, edge_map_.ptr, geom_.ptr, error_flag_.ptr);
    launches_ += 1;
    enqueue_phases(7, nullptr, false);
    finish_compute();
}

// ---- three-phase evaluation for a domain-decomposed run (positions: device f64[3*num_nodes],
// receivers first, ghosts after them)
void Evaluator::distributed_begin(std::uint64_t generation, const double* device_positions)
{
    check_generation(generation);
    if (phase_ != 0) {
        phase_ = 0;
        throw std::logic_error("distributed evaluation: begin called while another evaluation is open.");
    }
    SXB_CUDA(cudaSetDevice(device_));
    have_results_ = false;
    mirror_valid_ = false;
    SXB_CUDA(cudaEventRecord(event_begin_, stream_));
    enqueue_phases(1, device_positions, false);
    phase_ = 1;
}

// The same first phase from caller-held edge vectors (device f64[3*num_edges], caller edge order), as
// the pair style passes them (begin_factorized_distributed_evaluation(..., xyz, r, generation),
// libsymmetrix/source/mace_kokkos.hpp:672-677; call site pair_symmetrix_mace_kokkos.cpp:1532-1568).
void Evaluator::distributed_begin_edge_vectors(std::uint64_t generation, const double* device_xyz)
{
    check_generation(generation);
    if (phase_ != 0) {
        phase_ = 0;
        throw std::logic_error("distributed evaluation: begin called while another evaluation is open.");
    }
    SXB_CUDA(cudaSetDevice(device_));
    have_results_ = false;
    mirror_valid_ = false;
    SXB_CUDA(cudaEventRecord(event_begin_, stream_));
    SXB_CUDA(cudaMemsetAsync(error_flag_.ptr, 0, sizeof(int), stream_));
    if (num_edges_ > 0)
        geometry_from_vectors_kernel<<<blocks_for(num_edges_, 256), 256, 0, stream_>>>(num_edges_, device_xyz, edge_map_.ptr, geom_.ptr,
                                                                                      error_flag_.ptr);
    launches_ += 1;
    enqueue_phases(1, nullptr, false);
    phase_ = 1;
}

void Evaluator::distributed_continue()
{
    if (phase_ != 1) {
        phase_ = 0;
        throw std::logic_error("distributed evaluation: continue must follow begin.");
    }
    SXB_CUDA(cudaSetDevice(device_));
    enqueue_phases(2, nullptr, false);
    phase_ = 2;
}

void Evaluator::distributed_finish()
{
    if (phase_ != 2) {
        phase_ = 0;
        throw std::logic_error("distributed evaluation: finish must follow continue.");
    }
    SXB_CUDA(cudaSetDevice(device_));
    phase_ = 0;
    enqueue_phases(4, nullptr, false);
    // no host synchronisation here: the caller still has ghost forces to exchange on this stream;
    // synchronize() fetches the totals and checks the device status word
    SXB_CUDA(cudaEventRecord(event_end_, stream_));
    pending_finish_ = true;
    have_results_ = true;
}

namespace {
// rows of a node tensor (row_floats per node) gathered into / scattered from a dense buffer;
// indices are caller-order node numbers
// (indices == nullptr: the caller-order rows first_row .. first_row + count - 1)
__global__ void pack_rows_kernel(long count, int row_floats, const int* __restrict__ indices, long first_row,
                                 const int* __restrict__ internal_of, const float* __restrict__ tensor, float* __restrict__ out)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int vec = row_floats >> 2;
    if (idx >= count * vec) return;
    const long r = idx / vec, q = idx % vec;
    const long node = internal_of[indices != nullptr ? indices[r] : first_row + r];
    reinterpret_cast<float4*>(out)[idx] = reinterpret_cast<const float4*>(tensor + node * row_floats)[q];
}

__global__ void unpack_rows_kernel(long count, int row_floats, const int* __restrict__ indices, long first_row,
                                   const int* __restrict__ internal_of, const float* __restrict__ in, float* __restrict__ tensor,
                                   int accumulate)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int vec = row_floats >> 2;
    if (idx >= count * vec) return;
    const long r = idx / vec, q = idx % vec;
    const long node = internal_of[indices != nullptr ? indices[r] : first_row + r];
    const float4 v = reinterpret_cast<const float4*>(in)[idx];
    float* dst = tensor + node * row_floats + 4 * q;
    if (accumulate) {
        // several images of one owned atom may be ghosts elsewhere: rows can repeat
        atomicAdd(reinterpret_cast<float4*>(dst), v);
    } else {
        *reinterpret_cast<float4*>(dst) = v;
    }
}

// out[k] = rows[indices[k]] (+ offsets[k]): three doubles per row
__global__ void gather_rows3_kernel(long count, const int* __restrict__ indices, const double* __restrict__ rows,
                                    const double* __restrict__ offsets, double* __restrict__ out)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= count * 3) return;
    const long k = idx / 3, q = idx % 3;
    double v = rows[3 * static_cast<long>(indices[k]) + q];
    if (offsets != nullptr) v += offsets[idx];
    out[idx] = v;
}

constexpr int kTotalsRows = 4;   // 10 totals (energy, 9 virial components) padded to four rows of three doubles

// Send buffer of the closing exchange.  Segment of peer p: the force rows of the ghosts that p owns
// (ghost_begin[p] .. ghost_begin[p+1], contiguous behind the receivers in caller order), then
// kTotalsRows rows holding this rank's energy and virial.
__global__ void pack_ghost_forces_kernel(int world, const int* __restrict__ ghost_begin, int num_receivers,
                                         const double* __restrict__ forces, const double* __restrict__ totals,
                                         double* __restrict__ out)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long rows = ghost_begin[world] + static_cast<long>(kTotalsRows) * world;
    if (idx >= rows * 3) return;
    const long row = idx / 3;
    const int q = static_cast<int>(idx % 3);
    int p = 0;
    while (p + 1 < world && row >= ghost_begin[p + 1] + static_cast<long>(kTotalsRows) * (p + 1)) ++p;
    const long local = row - (ghost_begin[p] + static_cast<long>(kTotalsRows) * p);
    const long ghosts = ghost_begin[p + 1] - ghost_begin[p];
    if (local < ghosts) {
        out[idx] = forces[3 * (num_receivers + ghost_begin[p] + local) + q];
    } else {
        const long slot = (local - ghosts) * 3 + q;
        out[idx] = slot < 10 ? totals[slot] : 0.0;
    }
}

// Receive buffer of the closing exchange: segment of peer p = force rows for my atoms send_begin[p] ..
// send_begin[p+1] of the send list, then p's totals.  Forces are added to the owners' rows; the totals
// of all ranks are summed in rank order (every rank obtains the same bits).
__global__ void unpack_ghost_forces_kernel(int world, const int* __restrict__ send_begin, const int* __restrict__ indices,
                                           const double* __restrict__ in, double* __restrict__ forces,
                                           double* __restrict__ totals_out)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx < 10) {
        double sum = 0.0;
        for (int p = 0; p < world; ++p) sum += in[3 * (send_begin[p + 1] + static_cast<long>(kTotalsRows) * p) + idx];
        totals_out[idx] = sum;
    }
    const long rows = send_begin[world] + static_cast<long>(kTotalsRows) * world;
    if (idx >= rows * 3) return;
    const long row = idx / 3;
    const int q = static_cast<int>(idx % 3);
    int p = 0;
    while (p + 1 < world && row >= send_begin[p + 1] + static_cast<long>(kTotalsRows) * (p + 1)) ++p;
    const long local = row - (send_begin[p] + static_cast<long>(kTotalsRows) * p);
    if (local < send_begin[p + 1] - send_begin[p])
        atomicAdd(forces + 3 * static_cast<long>(indices[send_begin[p] + local]) + q, in[idx]);
}

__global__ void add_force_rows_kernel(long count, const int* __restrict__ indices, const double* __restrict__ in,
                                      double* __restrict__ forces_caller_order)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= count * 3) return;
    const long r = idx / 3, q = idx % 3;
    atomicAdd(forces_caller_order + 3 * static_cast<long>(indices[r]) + q, in[idx]);
}
}  // namespace

float* Evaluator::halo_tensor(int which)
{
    if (which == 0) return H1_.ptr;
    if (which == 1) return H1_adj_.ptr;
    throw std::invalid_argument("Halo tensor selector must be 0 (H1) or 1 (H1_adj).");
}

void Evaluator::pack_rows(int which, const int* device_indices, long count, float* device_out)
{
    const int row = model_.num_hidden * model_.channels;
    if (count <= 0) return;
    pack_rows_kernel<<<blocks_for(count * (row / 4), 256), 256, 0, stream_>>>(count, row, device_indices, 0, internal_of_.ptr,
                                                                              halo_tensor(which), device_out);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
}

void Evaluator::unpack_rows(int which, const int* device_indices, long count, const float* device_in, bool accumulate)
{
    const int row = model_.num_hidden * model_.channels;
    if (count <= 0) return;
    unpack_rows_kernel<<<blocks_for(count * (row / 4), 256), 256, 0, stream_>>>(count, row, device_indices, 0, internal_of_.ptr,
                                                                                device_in, halo_tensor(which), accumulate ? 1 : 0);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
}

// Host-side access to a range of caller-order rows of H1 / H1_adj, for callers whose halo exchange
// runs through host buffers (a plain LAMMPS pair style's pack / unpack_forward_comm callbacks).
void Evaluator::get_halo_rows(int which, long first_row, long count, float* host_out)
{
    const int row = model_.num_hidden * model_.channels;
    if (first_row < 0 || count < 0 || first_row + count > num_nodes_) throw std::invalid_argument("Halo row range is out of bounds.");
    if (count == 0) return;
    halo_stage_.reserve_with_slack(static_cast<std::size_t>(count) * row);
    pack_rows_kernel<<<blocks_for(count * (row / 4), 256), 256, 0, stream_>>>(count, row, nullptr, first_row, internal_of_.ptr,
                                                                              halo_tensor(which), halo_stage_.ptr);
    launches_ += 1;
    SXB_CUDA(cudaMemcpyAsync(host_out, halo_stage_.ptr, sizeof(float) * count * row, cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::put_halo_rows(int which, long first_row, long count, const float* host_in, bool accumulate)
{
    const int row = model_.num_hidden * model_.channels;
    if (first_row < 0 || count < 0 || first_row + count > num_nodes_) throw std::invalid_argument("Halo row range is out of bounds.");
    if (count == 0) return;
    halo_stage_.reserve_with_slack(static_cast<std::size_t>(count) * row);
    SXB_CUDA(cudaMemcpyAsync(halo_stage_.ptr, host_in, sizeof(float) * count * row, cudaMemcpyHostToDevice, stream_));
    unpack_rows_kernel<<<blocks_for(count * (row / 4), 256), 256, 0, stream_>>>(count, row, nullptr, first_row, internal_of_.ptr,
                                                                                halo_stage_.ptr, halo_tensor(which), accumulate ? 1 : 0);
    launches_ += 1;
    SXB_CUDA(cudaStreamSynchronize(stream_));      // host_in may be reused by the caller right away
}

// First phase from host positions (f64[3*num_nodes], owned atoms first, ghosts after).
void Evaluator::distributed_begin_host(std::uint64_t generation, const double* host_positions)
{
    check_generation(generation);
    SXB_CUDA(cudaSetDevice(device_));
    SXB_CUDA(cudaMemcpyAsync(positions_.ptr, host_positions, sizeof(double) * 3 * num_nodes_, cudaMemcpyHostToDevice, stream_));
    distributed_begin(generation, positions_.ptr);
}

void Evaluator::add_force_rows(const int* device_indices, long count, const double* device_in)
{
    require_results();
    if (count <= 0) return;
    add_force_rows_kernel<<<blocks_for(count * 3, 256), 256, 0, stream_>>>(count, device_indices, device_in, forces_out_.ptr);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
}

namespace {
__global__ void internal_rows_kernel(long count, const int* __restrict__ indices, const int* __restrict__ internal_of, int num_nodes,
                                     int* __restrict__ out)
{
    const long k = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (k >= count) return;
    const int node = indices[k];
    out[k] = (node >= 0 && node < num_nodes) ? internal_of[node] : -1;
}
}  // namespace

void Evaluator::internal_rows(const int* device_indices, long count, int* device_out)
{
    if (count <= 0) return;
    internal_rows_kernel<<<blocks_for(count, 256), 256, 0, stream_>>>(count, device_indices, internal_of_.ptr, num_nodes_, device_out);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::gather_position_rows(const double* device_rows, const int* device_indices, long count,
                                     const double* device_offsets, double* device_out)
{
    if (count <= 0) return;
    gather_rows3_kernel<<<blocks_for(count * 3, 256), 256, 0, stream_>>>(count, device_indices, device_rows, device_offsets, device_out);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
}

void Evaluator::pack_ghost_forces(int world, const int* device_ghost_begin, long num_ghosts, double* device_out)
{
    require_results();
    if (world <= 0) throw std::invalid_argument("world size must be positive.");
    const long values = (num_ghosts + static_cast<long>(kTotalsRows) * world) * 3;
    pack_ghost_forces_kernel<<<blocks_for(values, 256), 256, 0, stream_>>>(world, device_ghost_begin, num_receivers_, forces_out_.ptr,
                                                                          totals_.ptr, device_out);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
}

void Evaluator::unpack_ghost_forces(int world, const int* device_send_begin, const int* device_indices, long num_rows,
                                    const double* device_in, double* device_totals_out)
{
    require_results();
    if (world <= 0) throw std::invalid_argument("world size must be positive.");
    const long values = std::max<long>((num_rows + static_cast<long>(kTotalsRows) * world) * 3, 10);
    unpack_ghost_forces_kernel<<<blocks_for(values, 256), 256, 0, stream_>>>(world, device_send_begin, device_indices, device_in,
                                                                            forces_out_.ptr, device_totals_out);
    launches_ += 1;
    SXB_CUDA(cudaGetLastError());
}

// Registers the buffers of a domain-decomposed run, so that the halo packing and unpacking become
// part of the (captured) phases instead of separate calls: the first phase ends by gathering the H1
// rows `send_indices` into `send_rows`; the third phase starts by adding `received_rows` (the adjoints
// peers collected for those same rows) into H1_adj and ends by packing the ghost forces and this
// rank's totals into `force_send` (layout of pack_ghost_forces).  All pointers are device memory that
// stays valid until the next graph preparation; NULL send_indices switches the plan off.
void Evaluator::set_halo_plan(const int* send_indices, long num_send, float* send_rows, const float* received_rows, int world,
                              const int* ghost_begin, double* force_send)
{
    drop_step_graphs();
    halo_plan_ = HaloPlan{};
    if (send_indices == nullptr && num_send > 0) return;
    // send_rows / received_rows may be NULL: the exchange then gathers from H1 and adds into H1_adj by itself
    if (world <= 0 || ghost_begin == nullptr || force_send == nullptr)
        throw std::invalid_argument("Halo plan needs the ghost offsets and the force buffer.");
    halo_plan_.active = true;
    halo_plan_.send_indices = send_indices;
    halo_plan_.num_send = num_send;
    halo_plan_.send_rows = send_rows;
    halo_plan_.received_rows = received_rows;
    halo_plan_.world = world;
    halo_plan_.ghost_begin = ghost_begin;
    halo_plan_.force_send = force_send;
}

// A caller that has captured begin / continue / finish (with its exchanges in between) into a CUDA
// graph of its own and replays that graph tells the evaluator so: the host-side state then is the one
// after distributed_finish, and synchronize() fetches status and totals as usual.
void Evaluator::mark_phases_replayed(std::uint64_t generation, long launches)
{
    check_generation(generation);
    phase_ = 0;
    pending_finish_ = true;
    have_results_ = true;
    mirror_valid_ = false;
    launches_ += launches;
}

void Evaluator::abort_phases()
{
    phase_ = 0;
    pending_finish_ = false;
    have_results_ = false;
    mirror_valid_ = false;
}

void Evaluator::set_stream(cudaStream_t stream)
{
    SXB_CUDA(cudaSetDevice(device_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    drop_step_graphs();
    if (owns_stream_ && stream_ != nullptr) SXB_CUDA(cudaStreamDestroy(stream_));
    stream_ = stream;
    owns_stream_ = false;
    if (const char* env = std::getenv("SXB_CUDA_GRAPHS")) use_graphs_ = env[0] != '0'; else use_graphs_ = true;
}

void Evaluator::synchronize()
{
    SXB_CUDA(cudaSetDevice(device_));
    if (pending_finish_) {
        pending_finish_ = false;
        have_results_ = false;
        finish_compute();
        mirror_valid_ = false;      // the published forces predate the ghost forces the caller has added since
        return;
    }
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::require_results() const
{
    if (!have_results_) throw std::runtime_error("No evaluation results are available; call a compute function first.");
}

void Evaluator::get_node_energies(double* out)
{
    require_results();
    if (mirror_valid_) {
        std::memcpy(out, host_results_ + 11, sizeof(double) * num_receivers_);
        return;
    }
    SXB_CUDA(cudaMemcpyAsync(out, node_energies_out_.ptr, sizeof(double) * num_receivers_, cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::get_atom_forces(double* out)
{
    require_results();
    if (mirror_valid_) {
        std::memcpy(out, host_results_ + 11 + num_receivers_, sizeof(double) * 3 * num_nodes_);
        return;
    }
    SXB_CUDA(cudaMemcpyAsync(out, forces_out_.ptr, sizeof(double) * 3 * num_nodes_, cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::get_edge_forces(double* out)
{
    require_results();
    if (!keep_edge_forces_) throw std::invalid_argument("Directed edge forces were not retained; enable them before compute.");
    DeviceBuffer<double>& tmp = edge_scratch_;
    tmp.reserve_with_slack(3 * static_cast<std::size_t>(num_edges_));
    unpermute_edges_kernel<<<blocks_for(num_edges_, 256), 256, 0, stream_>>>(num_edges_, edge_map_.ptr, edge_forces_.ptr, tmp.ptr);
    launches_ += 1;
    SXB_CUDA(cudaMemcpyAsync(out, tmp.ptr, sizeof(double) * 3 * num_edges_, cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
}

void Evaluator::set_keep_edge_forces(bool enabled)
{
    keep_edge_forces_ = enabled;
    if (enabled && num_edges_ > 0) edge_forces_.reserve(3 * static_cast<std::size_t>(num_edges_));
}

void Evaluator::get_stress(double volume, double* out9)
{
    require_results();
    if (pending_finish_) throw std::logic_error("Call synchronize() after distributed_finish before reading host results.");
    if (!std::isfinite(volume) || !(volume > 0.0)) throw std::invalid_argument("Stress reduction needs a finite positive volume.");
    for (int q = 0; q < 9; ++q) out9[q] = -host_totals_[1 + q] / volume;
}

double Evaluator::energy() const
{
    require_results();
    if (pending_finish_) throw std::logic_error("Call synchronize() after distributed_finish before reading host results.");
    return host_totals_[0];
}

int Evaluator::tile_capacity() const
{
    if (tile_size_ > 0 && tile_size_ < num_receivers_) return tile_size_;
    return std::max(num_receivers_, 1);
}

void Evaluator::set_deterministic(bool enabled)
{
    deterministic_ = enabled;
    drop_step_graphs();
    generation_ += 1;      // buffers and the source schedule are made at graph installation: prepare again
    have_results_ = false;
    mirror_valid_ = false;
}

void Evaluator::set_tile_size(int receivers_per_tile)
{
    if (receivers_per_tile < 0) throw std::invalid_argument("Tile size must be non-negative (0 switches tiling off).");
    tile_size_ = receivers_per_tile;
    generation_ += 1;      // buffers are sized at graph installation: the prepared graph becomes stale
    have_results_ = false;
    mirror_valid_ = false;
}

long Evaluator::get_stage(const std::string& name, double* out, long capacity)
{
    require_results();
    if (tile_capacity() < num_receivers_ && name != "H1" && name != "H1_adj" && name != "M0")
        throw std::invalid_argument("Stage tensors other than H1, H1_adj and M0 are not retained in tiled-streaming mode.");
    const long C = model_.channels, NH = model_.num_hidden, NE = model_.num_lme;
    long N = num_receivers_;
    const float* src = nullptr;
    long row = 0;
    if (name == "A0") { src = A0_.ptr; row = 16 * C; }
    else if (name == "A0_adj") { src = A0_adj_.ptr; row = 16 * C; }
    else if (name == "M0") { src = M0_.ptr; row = NH * C; }
    else if (name == "M0_adj") { src = M0_adj_.ptr; row = NH * C; }
    else if (name == "H1") { src = H1_.ptr; row = NH * C; N = num_nodes_; }
    else if (name == "H1_adj") { src = H1_adj_.ptr; row = NH * C; N = num_nodes_; }
    else if (name == "Phi1") { src = Phi1_.ptr; row = NE * C; }
    else if (name == "dPhi1") { src = dPhi1_.ptr; row = NE * C; }
    else if (name == "A1") { src = A1_.ptr; row = 16 * C; }
    else if (name == "A1_adj") { src = A1_adj_.ptr; row = 16 * C; }
    else if (name == "M1") { src = M1_.ptr; row = C; }
    else if (name == "H2") { src = H2_.ptr; row = C; }
    else if (name == "H2_adj") { src = H2_adj_.ptr; row = C; }
    else throw std::invalid_argument("Unknown stage tensor name: " + name);
    const long count = N * row;
    if (out == nullptr) return count;
    if (capacity < count) throw std::invalid_argument("Stage output buffer is too small.");
    DeviceBuffer<double> tmp;
    tmp.reserve(count);
    unpermute_stage_kernel<<<blocks_for(count, 256), 256, 0, stream_>>>(N, row, original_.ptr, src, tmp.ptr);
    launches_ += 1;
    SXB_CUDA(cudaMemcpyAsync(out, tmp.ptr, sizeof(double) * count, cudaMemcpyDeviceToHost, stream_));
    SXB_CUDA(cudaStreamSynchronize(stream_));
    return count;
}

}  // namespace sxb
