/* Kernel-plugin boundary of the layer-1 edge tensor product, version 2, as this library exports it.
 *
 * The reference loads its layer-1 kernels from a shared library that exports one query symbol,
 * symmetrix_jit_cuda_plugin_query_v2, returning a table of metadata and two launch functions
 * (symmetrix/source/symmetrix/jit_cuda_plugin_abi.h:148-385; loader libsymmetrix/source/jit_cuda_plugin.hpp:
 * 31-106; call sites mace_kokkos_h1_phi1.cpp:1819-1834 and mace_kokkos_factorized_execution.cpp:844-919).
 * libsymmetrix_b200.so exports the same symbol over its own layer-1 kernels, so the two can be loaded side
 * by side and timed on identical device buffers.  The layouts below have to be binary-identical to the
 * reference's; the text is this library's own.  Only the parts this library implements are declared.
 *
 * Conventions (all tensors are contiguous row-major device memory; the argument blocks live on the host
 * and are read during the call only):
 *   graph        receiver-major CSR: first_neigh / num_neigh per receiver, neigh_indices (source node) and
 *                neigh_types (element slot of the source) per edge; node_types per node; type_to_active
 *                maps element slots to the dense index of the species present
 *   radius       f64 per edge; an edge with radius >= cutoff takes no part
 *   radial       cubic spline coefficients [edge_types][intervals][4][functions] in the scalar type,
 *                function = path * channels + channel, evaluated at x = radius - x0 - h * interval
 *   harmonics    Y_lm per edge [E][16] (forward); the reverse launch also receives the edge vectors
 *                (xyz: unit vectors in f32 when coordinates_are_unit, else Cartesian f64) and may receive
 *                gradients [E][3][16] (NULL: the kernel derives them)
 *   features     neighbor_features = H1 [nodes][4][C]; output = Phi1 [receivers][40][C];
 *                output_adjoint = dPhi1; source_adjoint = H1_adj (added to); directed_forces f64 [E][3]
 *                (the force of an edge is subtracted from its entry)
 * A launch function enqueues on `stream` (a cudaStream_t), returns a cudaError_t as int32 and keeps no
 * pointer it was given.  This library's implementation keeps device scratch of its own between calls
 * (edge records, a repacked copy of the coefficient table keyed by its address and extents).
 */
#ifndef SYMMETRIX_JIT_CUDA_PLUGIN_H
#define SYMMETRIX_JIT_CUDA_PLUGIN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SXB_JIT_PLUGIN_ABI_VERSION_V2 2u
#define SXB_JIT_PLUGIN_ABI_TAG_V2 "symmetrix.jit.cuda-plugin/2"
#define SXB_JIT_PLUGIN_BYTE_ORDER 0x01020304u
#define SXB_JIT_PLUGIN_SCALAR_FLOAT32 1u
#define SXB_JIT_PLUGIN_CAN_FORWARD (1u << 0)
#define SXB_JIT_PLUGIN_CAN_COORDINATE_REVERSE (1u << 1)
#define SXB_JIT_PLUGIN_CAN_FUSED_REVERSE (1u << 2)

typedef struct SymmetrixJitCudaRadialSplineV2 {
    uint32_t struct_size;
    uint32_t edge_types;
    uint32_t intervals;
    uint32_t functions;
    double h;
    double x0;
    const void* coefficients;
} SymmetrixJitCudaRadialSplineV2;

typedef struct SymmetrixJitCudaR1ForwardArgsV2 {
    uint32_t struct_size;
    uint32_t active_type_count;
    int64_t num_nodes;
    int64_t num_edges;
    const int32_t* node_types;
    const int32_t* num_neigh;
    const int32_t* first_neigh;
    const int32_t* neigh_indices;
    const int32_t* neigh_types;
    const int32_t* type_to_active;
    const double* radius;
    SymmetrixJitCudaRadialSplineV2 radial;
    const void* harmonics_values;
    const void* neighbor_features;
    void* output;
    double cutoff;
} SymmetrixJitCudaR1ForwardArgsV2;

typedef struct SymmetrixJitCudaR1SourceArgsV2 {
    uint32_t struct_size;
    uint32_t active_type_count;
    int64_t num_nodes;
    int64_t num_edges;
    const int32_t* node_types;
    const int32_t* neigh_types;
    const int32_t* source_offsets;
    const int32_t* source_edges;
    const int32_t* edge_receivers;
    const int32_t* type_to_active;
    const double* radius;
    SymmetrixJitCudaRadialSplineV2 radial;
    const void* harmonics_values;
    const void* output_adjoint;
    void* source_adjoint;
    double cutoff;
} SymmetrixJitCudaR1SourceArgsV2;

typedef struct SymmetrixJitCudaR1EdgeArgsV2 {
    uint32_t struct_size;
    uint32_t active_type_count;
    uint32_t coordinate_scalar_size;
    uint32_t coordinates_are_unit;
    int64_t num_nodes;
    int64_t num_edges;
    const int32_t* node_types;
    const int32_t* neigh_indices;
    const int32_t* neigh_types;
    const int32_t* edge_receivers;
    const int32_t* type_to_active;
    const void* xyz;
    const double* radius;
    SymmetrixJitCudaRadialSplineV2 radial;
    const void* harmonics_values;
    const void* harmonics_gradients;
    const void* neighbor_features;
    const void* output_adjoint;
    double* directed_forces;
    double cutoff;
} SymmetrixJitCudaR1EdgeArgsV2;

typedef int32_t (*SymmetrixJitCudaR1ForwardLaunchV2)(const SymmetrixJitCudaR1ForwardArgsV2*, void* stream, int32_t persistent_blocks);
typedef int32_t (*SymmetrixJitCudaR1CoordinateReverseLaunchV2)(const SymmetrixJitCudaR1SourceArgsV2*, const SymmetrixJitCudaR1EdgeArgsV2*,
                                                               void* stream, int32_t persistent_blocks);

typedef struct SymmetrixJitCudaPluginV2 {
    uint32_t abi_version;
    uint32_t struct_size;
    uint32_t pointer_size;
    uint32_t byte_order;
    uint32_t capabilities;
    uint32_t scalar_kind;
    uint32_t scalar_size;
    uint32_t reserved;
    const char* abi_tag;
    const char* artifact_id;
    const char* contract_fingerprint;
    const char* semantic_fingerprint;
    const char* structure_fingerprint;
    int32_t channels;
    int32_t embedding;
    int32_t edge_l_max;
    int32_t source_l_max;
    int32_t target_compute_capability;
    int32_t forward_threads_per_block;
    int32_t source_threads_per_block;
    int32_t edge_threads_per_block;
    SymmetrixJitCudaR1ForwardLaunchV2 r1_forward_launch;
    SymmetrixJitCudaR1CoordinateReverseLaunchV2 r1_coordinate_reverse_launch;
} SymmetrixJitCudaPluginV2;

/* The query symbol of the reference's plugins (jit_cuda_plugin_abi.h:354-385), served here by the layer-1
 * kernels of this library for the structure 128 channels, edge l <= 3, source l <= 1 (10 paths, 88 rows,
 * 40 outputs: the OMAT-0 / MPA-0 medium contract).  The fingerprint strings are empty: this library does
 * not derive the reference's SHA-256 fingerprints, so the reference's loader, which compares them, will
 * not accept it in place of a generated plugin; a harness that fills the argument blocks itself can. */
const SymmetrixJitCudaPluginV2* symmetrix_jit_cuda_plugin_query_v2(void);

/* The coupling coefficients of that structure are data in this library (one value per sparse term, in
 * the order of (row, output) pairs of its compiled term list).  A contract's own coefficients -- path
 * signs are a convention of whoever derived them -- are installed with this call before the first
 * launch; without it the library's own derivation is used.  Returns the number of terms (86), or a
 * negative SXB_ERR_* code.  terms_row / terms_output (int32[86], may be NULL) receive the compiled order. */
int sxb_jit_plugin_coupling(const float* coefficients, int32_t count, int32_t* terms_row, int32_t* terms_output);

#ifdef __cplusplus
}
#endif
#endif
