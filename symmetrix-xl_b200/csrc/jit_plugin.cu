// symmetrix_jit_cuda_plugin_query_v2 served by this library's layer-1 kernels
// (include/symmetrix_jit_cuda_plugin.h; reference interface symmetrix/source/symmetrix/jit_cuda_plugin_abi.h:
// 148-385).  The launch functions translate the plugin's argument blocks into what the kernels of
// edge_kernels.cuh consume -- a 16-byte geometry record per edge, a byte of active type per node, the
// coefficient table with the four cubic coefficients of a function adjacent -- and launch
// l1_forward_kernel_S1 / l1_reverse_kernel_S1 unchanged.  Scratch for the translation is device memory
// this file keeps between calls, per device.
#include "../../include/symmetrix_b200.h"
#include "../../include/symmetrix_jit_cuda_plugin.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

#include "edge_kernels.cuh"

namespace sxb {

void set_last_error(const std::string& message);   // c_api.cu

namespace {

constexpr int kChannels = 128;
constexpr int kPaths = SXB_S1_NUM_PATHS, kTerms = SXB_S1_NUM_TERMS;

struct Scratch {
    DeviceBuffer<EdgeGeom> geom;
    DeviceBuffer<unsigned char> atype;
    DeviceBuffer<int> first;
    DeviceBuffer<float> table;           // [pair][interval][function][4]
    const void* table_source = nullptr;  // address and extents the repacked copy was made from
    unsigned table_pairs = 0, table_intervals = 0, table_functions = 0;
};

std::mutex g_mutex;
Scratch g_scratch[16];
CouplingConstants g_coupling;
bool g_coupling_set = false;

const CouplingConstants& coupling()
{
    if (!g_coupling_set) {
        const float defaults[kTerms] = SXB_S1_DEFAULT_CG;
        std::memset(&g_coupling, 0, sizeof(g_coupling));
        for (int t = 0; t < kTerms; ++t) g_coupling.cg[t] = defaults[t];
        g_coupling_set = true;
    }
    return g_coupling;
}

// geometry records from per-edge radius and (optionally) edge vectors; without vectors only the length is set
__global__ void plugin_geometry_kernel(long num_edges, const double* __restrict__ radius, const void* __restrict__ xyz, int scalar_size,
                                       int is_unit, EdgeGeom* __restrict__ geom)
{
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= num_edges) return;
    const double r = radius[e];
    EdgeGeom g;
    g.r = static_cast<float>(r);
    g.ux = g.uy = g.uz = 0.0f;
    if (xyz != nullptr) {
        if (is_unit) {
            const float* u = static_cast<const float*>(xyz) + 3 * e;
            g.ux = u[0]; g.uy = u[1]; g.uz = u[2];
        } else if (scalar_size == 8) {
            const double* v = static_cast<const double*>(xyz) + 3 * e;
            g.ux = static_cast<float>(v[0] / r); g.uy = static_cast<float>(v[1] / r); g.uz = static_cast<float>(v[2] / r);
        } else {
            const float* v = static_cast<const float*>(xyz) + 3 * e;
            g.ux = static_cast<float>(v[0] / r); g.uy = static_cast<float>(v[1] / r); g.uz = static_cast<float>(v[2] / r);
        }
    }
    geom[e] = g;
}

__global__ void plugin_types_kernel(long num_nodes, const int* __restrict__ node_types, const int* __restrict__ type_to_active,
                                    unsigned char* __restrict__ atype)
{
    const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < num_nodes) atype[i] = static_cast<unsigned char>(type_to_active[node_types[i]]);
}

// first[i] for i <= n from first_neigh / num_neigh (the plugin's CSR has no closing entry)
__global__ void plugin_offsets_kernel(long num_nodes, const int* __restrict__ first_neigh, const int* __restrict__ num_neigh,
                                      int* __restrict__ first)
{
    const long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < num_nodes) first[i] = first_neigh[i];
    if (i == num_nodes - 1) first[num_nodes] = first_neigh[i] + num_neigh[i];
}

// receiver offsets from the receiver of every edge (edges are receiver-major): first[i] = first edge with receiver >= i
__global__ void plugin_offsets_from_receivers_kernel(long num_nodes, long num_edges, const int* __restrict__ edge_receivers,
                                                     int* __restrict__ first)
{
    const long e = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e > num_edges) return;
    const int here = e < num_edges ? edge_receivers[e] : static_cast<int>(num_nodes);
    const int before = e > 0 ? edge_receivers[e - 1] : -1;
    for (int i = before + 1; i <= here; ++i) first[i] = static_cast<int>(e);
}

// [pair][interval][4][F] -> [pair][interval][F][4]
__global__ void plugin_repack_kernel(long slabs, int functions, const float* __restrict__ in, float* __restrict__ out)
{
    const long idx = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= slabs * functions) return;
    const long slab = idx / functions, f = idx % functions;
    const float* src = in + slab * 4 * functions + f;
    reinterpret_cast<float4*>(out)[idx] = make_float4(src[0], src[functions], src[2 * static_cast<long>(functions)], src[3 * static_cast<long>(functions)]);
}

inline int blocks(long n) { return static_cast<int>((n + 255) / 256); }

bool radial_ok(const SymmetrixJitCudaRadialSplineV2& r)
{
    return r.struct_size >= sizeof(SymmetrixJitCudaRadialSplineV2) && r.functions == static_cast<unsigned>(kPaths * kChannels)
           && r.edge_types >= 1 && r.intervals >= 1 && r.coefficients != nullptr && r.h > 0.0;
}

// Common preparation; returns the scratch of the current device.
Scratch& prepare(const SymmetrixJitCudaRadialSplineV2& radial, long num_nodes, long num_edges, const int* node_types,
                 const int* type_to_active, const double* radius, const void* xyz, int scalar_size, int is_unit, cudaStream_t stream)
{
    int device = 0;
    SXB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 16) throw std::runtime_error("device ordinal out of range");
    Scratch& s = g_scratch[device];
    s.geom.reserve_with_slack(std::max<long>(num_edges, 1));
    s.atype.reserve_with_slack(std::max<long>(num_nodes, 1));
    s.first.reserve_with_slack(num_nodes + 1);
    if (num_edges > 0)
        plugin_geometry_kernel<<<blocks(num_edges), 256, 0, stream>>>(num_edges, radius, xyz, scalar_size, is_unit, s.geom.ptr);
    plugin_types_kernel<<<blocks(num_nodes), 256, 0, stream>>>(num_nodes, node_types, type_to_active, s.atype.ptr);
    const long slabs = static_cast<long>(radial.edge_types) * radial.intervals;
    if (s.table_source != radial.coefficients || s.table_pairs != radial.edge_types || s.table_intervals != radial.intervals
        || s.table_functions != radial.functions) {
        s.table.reserve(static_cast<std::size_t>(slabs) * radial.functions * 4);
        plugin_repack_kernel<<<blocks(slabs * radial.functions), 256, 0, stream>>>(slabs, static_cast<int>(radial.functions),
                                                                                 static_cast<const float*>(radial.coefficients), s.table.ptr);
        s.table_source = radial.coefficients;
        s.table_pairs = radial.edge_types;
        s.table_intervals = radial.intervals;
        s.table_functions = radial.functions;
    }
    return s;
}

SplineGrid grid_of(const SymmetrixJitCudaRadialSplineV2& radial, double cutoff)
{
    SplineGrid g;
    g.x0 = static_cast<float>(radial.x0);
    g.h = static_cast<float>(radial.h);
    g.r_cut = static_cast<float>(cutoff);
    g.intervals = static_cast<int>(radial.intervals);
    return g;
}

int32_t forward_launch(const SymmetrixJitCudaR1ForwardArgsV2* a, void* stream_pointer, int32_t persistent_blocks)
{
    if (a == nullptr || a->struct_size < sizeof(SymmetrixJitCudaR1ForwardArgsV2) || !radial_ok(a->radial) || a->num_nodes < 0
        || a->num_nodes > INT32_MAX || a->num_edges < 0 || a->num_edges > INT32_MAX || !std::isfinite(a->cutoff) || a->cutoff <= 0.0
        || a->active_type_count == 0 || a->active_type_count > 255 || persistent_blocks <= 0)
        return static_cast<int32_t>(cudaErrorInvalidValue);
    if (a->num_nodes == 0) return static_cast<int32_t>(cudaSuccess);
    try {
        std::lock_guard<std::mutex> lock(g_mutex);
        cudaStream_t stream = static_cast<cudaStream_t>(stream_pointer);
        Scratch& s = prepare(a->radial, a->num_nodes, a->num_edges, a->node_types, a->type_to_active, a->radius, nullptr, 0, 0, stream);
        plugin_offsets_kernel<<<blocks(a->num_nodes), 256, 0, stream>>>(a->num_nodes, a->first_neigh, a->num_neigh, s.first.ptr);
        const int pair_types = a->radial.edge_types > 1 ? static_cast<int>(a->active_type_count) : 1;
        l1_forward_kernel_S1<kChannels, true><<<static_cast<int>(a->num_nodes), kChannels, 0, stream>>>(
            static_cast<int>(a->num_nodes), 0, kChannels, s.first.ptr, a->neigh_indices, s.geom.ptr, s.atype.ptr, grid_of(a->radial, a->cutoff),
            reinterpret_cast<const float4*>(s.table.ptr), static_cast<const float*>(a->neighbor_features), coupling(),
            static_cast<float*>(a->output), nullptr, pair_types, static_cast<const float*>(a->harmonics_values));
        return static_cast<int32_t>(cudaPeekAtLastError());
    } catch (const std::exception&) {
        return static_cast<int32_t>(cudaErrorUnknown);
    }
}

int32_t reverse_launch(const SymmetrixJitCudaR1SourceArgsV2* sa, const SymmetrixJitCudaR1EdgeArgsV2* ea, void* stream_pointer,
                       int32_t persistent_blocks)
{
    if (sa == nullptr || ea == nullptr || sa->struct_size < sizeof(SymmetrixJitCudaR1SourceArgsV2)
        || ea->struct_size < sizeof(SymmetrixJitCudaR1EdgeArgsV2) || !radial_ok(sa->radial) || !radial_ok(ea->radial)
        || sa->num_nodes < 0 || sa->num_nodes > INT32_MAX || sa->num_edges < 0 || sa->num_edges > INT32_MAX
        || sa->num_edges != ea->num_edges || sa->active_type_count != ea->active_type_count || sa->cutoff != ea->cutoff
        || !std::isfinite(sa->cutoff) || sa->cutoff <= 0.0 || sa->active_type_count == 0 || sa->active_type_count > 255
        || persistent_blocks <= 0 || ea->xyz == nullptr || ea->edge_receivers == nullptr)
        return static_cast<int32_t>(cudaErrorInvalidValue);
    if (sa->num_nodes == 0 || sa->num_edges == 0) return static_cast<int32_t>(cudaSuccess);
    try {
        std::lock_guard<std::mutex> lock(g_mutex);
        cudaStream_t stream = static_cast<cudaStream_t>(stream_pointer);
        Scratch& s = prepare(ea->radial, sa->num_nodes, sa->num_edges, sa->node_types, sa->type_to_active, ea->radius, ea->xyz,
                             static_cast<int>(ea->coordinate_scalar_size), static_cast<int>(ea->coordinates_are_unit), stream);
        plugin_offsets_from_receivers_kernel<<<blocks(sa->num_edges + 1), 256, 0, stream>>>(sa->num_nodes, sa->num_edges, ea->edge_receivers,
                                                                                           s.first.ptr);
        const int pair_types = ea->radial.edge_types > 1 ? static_cast<int>(ea->active_type_count) : 1;
        ForceOutputs fo;
        fo.atom_forces = nullptr;            // only the directed forces of the edges are asked for
        fo.virial_slots = nullptr;
        fo.edge_forces = ea->directed_forces;
        fo.accumulate_edge = 1;              // the interface subtracts the edge's force from its entry
        fo.edge_source_adjoint = nullptr;    // source adjoint by atomics, added to source_adjoint
        const DensityScale none{nullptr, nullptr, nullptr, 1};
        l1_reverse_kernel_S1<kChannels><<<static_cast<int>(sa->num_nodes), kChannels, 0, stream>>>(
            static_cast<int>(sa->num_nodes), 0, kChannels, s.first.ptr, ea->neigh_indices, s.geom.ptr, s.atype.ptr, grid_of(ea->radial, ea->cutoff),
            reinterpret_cast<const float4*>(s.table.ptr), static_cast<const float*>(ea->neighbor_features),
            static_cast<const float*>(sa->output_adjoint), coupling(), static_cast<float*>(sa->source_adjoint), fo, none, pair_types);
        return static_cast<int32_t>(cudaPeekAtLastError());
    } catch (const std::exception&) {
        return static_cast<int32_t>(cudaErrorUnknown);
    }
}

const SymmetrixJitCudaPluginV2 g_plugin = {
    SXB_JIT_PLUGIN_ABI_VERSION_V2,
    static_cast<uint32_t>(sizeof(SymmetrixJitCudaPluginV2)),
    static_cast<uint32_t>(sizeof(void*)),
    SXB_JIT_PLUGIN_BYTE_ORDER,
    SXB_JIT_PLUGIN_CAN_FORWARD | SXB_JIT_PLUGIN_CAN_COORDINATE_REVERSE | SXB_JIT_PLUGIN_CAN_FUSED_REVERSE,
    SXB_JIT_PLUGIN_SCALAR_FLOAT32,
    static_cast<uint32_t>(sizeof(float)),
    0u,
    SXB_JIT_PLUGIN_ABI_TAG_V2,
    "symmetrix-xl-b200-r1-128-l3-L1",
    "",
    "",
    "",
    kChannels,
    64,
    3,
    1,
    100,
    kChannels,
    kChannels,
    kChannels,
    &forward_launch,
    &reverse_launch,
};

}  // namespace
}  // namespace sxb

extern "C" const SymmetrixJitCudaPluginV2* symmetrix_jit_cuda_plugin_query_v2(void) { return &sxb::g_plugin; }

extern "C" int sxb_jit_plugin_coupling(const float* coefficients, int32_t count, int32_t* terms_row, int32_t* terms_output)
{
    using namespace sxb;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (terms_row != nullptr || terms_output != nullptr) {
        int t = 0;
#define SXB_PLUGIN_TERM(term, row, lme)              \
        if (terms_row != nullptr) terms_row[t] = row;   \
        if (terms_output != nullptr) terms_output[t] = lme; \
        ++t;
        SXB_S1_TERMS(SXB_PLUGIN_TERM)
#undef SXB_PLUGIN_TERM
    }
    if (coefficients != nullptr) {
        if (count != kTerms) {
            set_last_error("sxb_jit_plugin_coupling expects one coefficient per sparse term (86).");
            return SXB_ERR_INVALID_ARGUMENT;
        }
        std::memset(&g_coupling, 0, sizeof(g_coupling));
        for (int t = 0; t < kTerms; ++t) g_coupling.cg[t] = coefficients[t];
        g_coupling_set = true;
    }
    return kTerms;
}
