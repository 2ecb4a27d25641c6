// Channel-mixing linears on the 5th-generation tensor cores (sm_100a): a batched FP32 GEMM
//   C[row(g)][n] (+)= sum_k A[row(g)][k] * Bt[n][k]
// computed as three TF32 tcgen05.mma passes (a_hi*b_hi + a_hi*b_lo + a_lo*b_hi) accumulating in
// FP32 in tensor memory, which keeps the result within a few 1e-7 of an FP32 evaluation.  These
// linears are the only dense contractions of the force path (reference: cuBLAS SGEMM calls and
// KokkosBatched team GEMMs, libsymmetrix/source/mace_kokkos_second_interaction.cpp:385-522 and
// mace_kokkos_h1_phi1.cpp:425-440, 695-711).
//
// One CTA owns a 128-row x n_tile output tile and is warp-specialised:
//   * warps 0-3 load the A rows (structured node/component addressing, 128-bit loads, the next
//     K chunk prefetched in registers), split them into a TF32-exact high part and a residual, and
//     store both into shared memory in the K-major 128-byte-swizzled layout the tensor core reads;
//   * one control thread streams the pre-split weight tiles with TMA (cp.async.bulk.tensor, three
//     stages), issues the 12 tcgen05.mma of every 32-wide K chunk and commits them to an mbarrier;
//   * warps 0-3 finally read the accumulator with tcgen05.ld, transpose it through shared memory
//     and write whole rows with coalesced 128-bit stores.
// Every wait is bounded: on expiry the kernel raises an error flag, frees its tensor memory and
// returns.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "node_kernels.cuh"

namespace sxb {

constexpr int kTcRows = 128;                  // M tile
constexpr int kTcNTile = 64;                  // N tile (columns of the accumulator)
constexpr int kTcChunk = 32;                  // K elements per stage (128 bytes of TF32)
constexpr int kTcAStages = 2, kTcBStages = 3;
constexpr int kTcABytes = kTcRows * 128;      // one A operand buffer (hi or lo)
constexpr int kTcBBytes = kTcNTile * 128;     // one weight buffer (hi or lo)
constexpr int kTcBarrierBytes = 128;
constexpr int kTcSmemBytes = kTcAStages * 2 * kTcABytes + kTcBStages * 2 * kTcBBytes + kTcBarrierBytes;
constexpr int kTcThreads = 160;               // 4 loader/epilogue warps + 1 control warp
constexpr unsigned kTcWaitLimit = 200000u;    // tries of a wait that sleeps up to kTcSuspendHintNs each: under half a second
constexpr unsigned kTcSuspendHintNs = 2000u;

struct alignas(64) TcProblem {
    CUtensorMap map_hi;      // Bt_hi [N][K], box [n_tile][32], 128-byte swizzle
    CUtensorMap map_lo;      // residual
    const float* A;
    float* C;
    const float* bias;       // optional [N], added when not accumulating
    RowMap a_rows, c_rows;
    int first_node;
    int M, N, K;             // logical rows, outputs, contraction length (K % 32 == 0)
    int accumulate;
    int n_tile;              // columns per CTA: min(N, kTcNTile), multiple of 16, divides N
    int m_tiles, n_tiles;
    int tile_begin;          // first CTA of this problem
};

constexpr int kTcMaxProblems = 8;
struct TcBatch {
    TcProblem problem[kTcMaxProblems];
    int count;
    int total_tiles;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait on an mbarrier phase; gives up (returns false) when the limit expires or another
// thread of the CTA has already given up.  The wait uses mbarrier.try_wait with a suspend-time hint,
// so a waiting warp sleeps in hardware instead of polling: a polling warp takes issue slots and
// shared-memory queue entries from the single thread that issues the tensor-core instructions
// (measured: that thread ran three times slower next to eight polling warps).
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* failed)
{
    const unsigned addr = smem_u32(bar);
    for (unsigned spin = 0; spin < kTcWaitLimit; ++spin) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(kTcSuspendHintNs)
            : "memory");
        if (done) return true;
        if ((spin & 15u) == 15u && *failed) return false;
    }
    *failed = 1;
    return false;
}

// K-major, 128-byte swizzle: 8-row groups 1024 B apart, rows 128 B apart, 16-byte chunk c of row r
// stored at chunk position c ^ (r % 8).
__device__ __forceinline__ unsigned swizzled_offset(int row, int chunk)
{
    return static_cast<unsigned>((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr)
{
    // start address >> 4 | LBO (unused with swizzle) = 1 | SBO = 1024 B >> 4 | version 1 | SWIZZLE_128B
    unsigned long long desc = 0;
    desc |= static_cast<unsigned long long>((smem_addr & 0x3ffffu) >> 4);
    desc |= static_cast<unsigned long long>(1) << 16;
    desc |= static_cast<unsigned long long>(1024 >> 4) << 32;
    desc |= static_cast<unsigned long long>(1) << 46;
    desc |= static_cast<unsigned long long>(2) << 61;
    return desc;
}

__device__ __forceinline__ void umma_tf32(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b, unsigned idesc,
                                          unsigned accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One TMA tile load into this CTA only: box [n_tile rows][32 floats] at (k0, n0) of a [N][K] tensor.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, unsigned long long* bar, int k0, int n0)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)), "r"(k0), "r"(n0)
        : "memory");
}

__global__ void __launch_bounds__(kTcThreads, 2) tc_gemm_kernel(const __grid_constant__ TcBatch batch, int* __restrict__ error_flag)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    unsigned char* a_buf = smem;                                            // [stage][hi, lo]
    unsigned char* b_buf = smem + kTcAStages * 2 * kTcABytes;               // [stage][hi, lo]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(b_buf + kTcBStages * 2 * kTcBBytes);
    unsigned long long* a_ready = bars;            // [2], 128 arrivals
    unsigned long long* b_full = bars + 2;         // [3], TMA transaction barriers
    unsigned long long* mma_done = bars + 5;       // [2], tcgen05.commit
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 8);
    volatile int* failed = reinterpret_cast<volatile int*>(bars + 9);

    // locate the problem and the tile of this CTA
    int pi = 0;
    for (int q = 1; q < batch.count; ++q)
        if (static_cast<int>(blockIdx.x) >= batch.problem[q].tile_begin) pi = q;
    const TcProblem& P = batch.problem[pi];
    const int local = blockIdx.x - P.tile_begin;
    const int m_tile = local / P.n_tiles, n_tile_index = local % P.n_tiles;
    const int row0 = m_tile * kTcRows, col0 = n_tile_index * P.n_tile;
    const int NT = P.n_tile;
    const int chunks = P.K / kTcChunk;

    if (tid == 128) {
        mbar_init(&a_ready[0], 128);
        mbar_init(&a_ready[1], 128);
        for (int s = 0; s < kTcBStages; ++s) mbar_init(&b_full[s], 1);
        mbar_init(&mma_done[0], 1);
        mbar_init(&mma_done[1], 1);
        *failed = (smem_u32(smem) & 1023u) ? 1 : 0;   // the swizzled layout needs a 1 KB aligned base
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(static_cast<unsigned>(kTcNTile)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    if (warp < 4) {
        // ------------------------------------------------------------- A loaders / converters
        const int l_chunk = tid & 7, l_row = tid >> 3;   // 8 threads per row, 16 rows per pass
        const float* a_ptr[8];
#pragma unroll
        for (int pass = 0; pass < 8; ++pass) {
            const int g = row0 + pass * 16 + l_row;
            a_ptr[pass] = g < P.M ? P.A + row_address(P.a_rows, P.first_node, g) + l_chunk * 4 : nullptr;
        }
        float4 cur[8], nxt[8];
#pragma unroll
        for (int pass = 0; pass < 8; ++pass)
            cur[pass] = a_ptr[pass] != nullptr ? *reinterpret_cast<const float4*>(a_ptr[pass]) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int kc = 0; kc < chunks; ++kc) {
            const int stage = kc & 1;
            if (kc + 1 < chunks) {
#pragma unroll
                for (int pass = 0; pass < 8; ++pass)
                    nxt[pass] = a_ptr[pass] != nullptr ? *reinterpret_cast<const float4*>(a_ptr[pass] + (kc + 1) * kTcChunk)
                                                       : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            // the MMAs that read this stage (chunk kc - 2) must have completed
            if (kc >= 2 && !mbar_wait(&mma_done[stage], static_cast<unsigned>(((kc >> 1) - 1) & 1), failed)) break;
            unsigned char* a_hi = a_buf + (stage * 2) * kTcABytes;
            unsigned char* a_lo = a_hi + kTcABytes;
#pragma unroll
            for (int pass = 0; pass < 8; ++pass) {
                const float4 v = cur[pass];
                float4 hi, lo;
                hi.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); lo.x = v.x - hi.x;
                hi.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); lo.y = v.y - hi.y;
                hi.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); lo.z = v.z - hi.z;
                hi.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); lo.w = v.w - hi.w;
                const unsigned off = swizzled_offset(pass * 16 + l_row, l_chunk);
                *reinterpret_cast<float4*>(a_hi + off) = hi;
                *reinterpret_cast<float4*>(a_lo + off) = lo;
            }
            // generic-proxy writes -> visible to the tensor core, then signal the issuing thread
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(&a_ready[stage]);
#pragma unroll
            for (int pass = 0; pass < 8; ++pass) cur[pass] = nxt[pass];
        }
        // ------------------------------------------------------------- epilogue
        for (int s = 0; s < kTcAStages && !*failed; ++s) {
            const int uses = (chunks - s + 1) / 2;   // commits issued on stage s
            if (uses > 0) mbar_wait(&mma_done[s], static_cast<unsigned>((uses - 1) & 1), failed);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // every loader thread arrives, whatever happened
        const bool ok = !*failed;                         // uniform from here on
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            // accumulator rows -> shared staging [128][NT] (16-byte chunks XOR-swizzled by row), reusing the A buffers
            float* stage_out = reinterpret_cast<float*>(a_buf);
            const int my_row = warp * 32 + lane;
            for (int c0 = 0; c0 < NT; c0 += 32) {
                unsigned v[32];
                const unsigned taddr = tmem_base + (static_cast<unsigned>(warp * 32) << 16) + static_cast<unsigned>(c0);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                      "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                      "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                      "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int chunk = (c0 >> 2) + q;
                    const int phys = chunk ^ (my_row & 7);
                    *reinterpret_cast<float4*>(stage_out + my_row * NT + phys * 4) =
                        make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                    __uint_as_float(v[4 * q + 3]));
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ok) {
            float* stage_out = reinterpret_cast<float*>(a_buf);
            // coalesced row stores: NT/4 threads per row
            const int threads_per_row = NT >> 2, rows_per_pass = 128 / threads_per_row;
            const int c4 = tid % threads_per_row, r_in = tid / threads_per_row;
            for (int r = r_in; r < kTcRows; r += rows_per_pass) {
                const int g = row0 + r;
                if (g >= P.M) break;
                float4 o = *reinterpret_cast<const float4*>(stage_out + r * NT + ((c4 ^ (r & 7)) << 2));
                float4* dst = reinterpret_cast<float4*>(P.C + row_address(P.c_rows, P.first_node, g) + col0 + c4 * 4);
                if (P.accumulate) {
                    const float4 old = *dst;
                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                } else if (P.bias != nullptr) {
                    const float4 b = *reinterpret_cast<const float4*>(P.bias + col0 + c4 * 4);
                    o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
                }
                *dst = o;
            }
        }
    } else if (tid == 128) {
        // ------------------------------------------------------------- control thread: TMA + MMA issue
        // instruction descriptor: D = F32, A = B = TF32, both K-major, N = NT, M = 128
        const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<unsigned>(NT >> 3) << 17) |
                               (static_cast<unsigned>(kTcRows >> 4) << 24);
        const unsigned tile_bytes = static_cast<unsigned>(NT) * 128u;
        auto issue_b = [&](int q) {
            const int s = q % kTcBStages;
            unsigned char* hi = b_buf + (s * 2) * kTcBBytes;
            mbar_expect_tx(&b_full[s], 2u * tile_bytes);
            tma_load_2d(hi, &P.map_hi, &b_full[s], q * kTcChunk, col0);
            tma_load_2d(hi + kTcBBytes, &P.map_lo, &b_full[s], q * kTcChunk, col0);
        };
        int issued = 0, consumed = 0;
        if (!*failed) {
            for (int q = 0; q < kTcBStages && q < chunks; ++q) { issue_b(q); ++issued; }
            for (int kc = 0; kc < chunks; ++kc) {
                const int stage = kc & 1, bs = kc % kTcBStages;
                if (!mbar_wait(&b_full[bs], static_cast<unsigned>((kc / kTcBStages) & 1), failed)) break;
                ++consumed;
                if (!mbar_wait(&a_ready[stage], static_cast<unsigned>((kc >> 1) & 1), failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned a_hi_addr = smem_u32(a_buf + (stage * 2) * kTcABytes);
                const unsigned b_hi_addr = smem_u32(b_buf + (bs * 2) * kTcBBytes);
                const unsigned long long da_hi = umma_desc(a_hi_addr), da_lo = umma_desc(a_hi_addr + kTcABytes);
                const unsigned long long db_hi = umma_desc(b_hi_addr), db_lo = umma_desc(b_hi_addr + kTcBBytes);
#pragma unroll
                for (int ks = 0; ks < kTcChunk / 8; ++ks) {
                    // advancing K by 8 TF32 = 32 bytes = 2 units of the descriptor's 16-byte address field
                    const unsigned long long step = static_cast<unsigned long long>(ks * 2);
                    umma_tf32(tmem_base, da_hi + step, db_hi + step, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
                    umma_tf32(tmem_base, da_hi + step, db_lo + step, idesc, 1u);
                    umma_tf32(tmem_base, da_lo + step, db_hi + step, idesc, 1u);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&mma_done[stage])) : "memory");
                // refill the weight stage freed by the previous chunk's MMAs with chunk kc + 2
                const int q = kc + 2;
                if (kc >= 1 && q < chunks) {
                    if (!mbar_wait(&mma_done[(kc - 1) & 1], static_cast<unsigned>(((kc - 1) >> 1) & 1), failed)) break;
                    issue_b(q);
                    ++issued;
                }
            }
            // after a failure: let the weight copies still in flight land before the CTA exits
            for (int q = consumed; q < issued; ++q) {
                int never = 0;
                mbar_wait(&b_full[q % kTcBStages], static_cast<unsigned>((q / kTcBStages) & 1), &never);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *failed) atomicOr(error_flag, 2);
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(static_cast<unsigned>(kTcNTile)) : "memory");
    }
}

}  // namespace sxb
