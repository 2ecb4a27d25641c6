// Channel-mixing linears on the 5th-generation tensor cores, persistent operand-streaming form.
//   C[row(g)][n] (+)= sum_k A[row(g)][k] * Bt[n][k]         (three TF32 passes, FP32 accumulation)
// Same arithmetic as tc_gemm.cuh; what changes is how the work is fed:
//   * one CTA per SM walks a list of (row tile, column tile) work items, so barrier set-up, tensor
//     memory allocation and descriptor fetches are paid once, and the pipeline never drains between
//     tiles: operand stages and their mbarrier phases run on across tile boundaries;
//   * the A rows (node, component, channel-block addressing) are fetched by the TMA engine as boxes
//     of a rank-3 tensor [node][component][K] straight into the 128-byte-swizzled K-major layout,
//     four K chunks deep;
//   * the tensor core reads the raw FP32 tile as the TF32 high part (it uses the upper 19 bits of
//     every element, the same truncation the split uses); four warps only form the residual
//     a - trunc(a) from shared memory into a second buffer;
//   * the accumulator is double-buffered in tensor memory (2 x 128 columns): four epilogue warps
//     write tile i (tensor memory -> registers -> a small transposing tile in shared memory ->
//     whole 128-byte row segments) while the tensor core already works on tile i + 1.
// A row tile holds floor(128 / components) whole nodes (128, 126, 125 or 126 rows); the remaining
// accumulator lanes are never stored.  A column tile is min(N, 128) wide.
// Thread roles: warps 0-3 residual, warps 4-7 epilogue, warp 8 lane 0 tcgen05.mma issue (warp 8 also
// owns the tensor-memory allocation), warp 9 lane 0 weight TMA, warp 10 lane 0 activation TMA.  The
// issuing thread is the narrow point of such a pipeline (every mbarrier or tcgen05 instruction costs
// it 60-300 cycles of latency), so it does nothing else: per K chunk it waits on one barrier - the
// weight copy and the 128 residual writers arrive on the same one - issues the 12 MMAs and commits.
// Every wait is bounded: on expiry the kernel raises bit 1 of the status word, every role leaves
// its loop, the producers wait (bounded) for their own copies in flight, the tensor memory is
// freed and the CTA returns.
#pragma once

#include "tc_gemm.cuh"

namespace sxb {

constexpr int kT3AStages = 4;                 // raw activation tiles in flight
constexpr int kT3Stages = 3;                  // residual tiles and weight tiles (hi + lo)
constexpr int kT3OperandBytes = 128 * 128;    // 128 rows x 32 floats
constexpr int kT3StagingBytes = 4 * 32 * 128;  // epilogue: 32 rows x 128 bytes per warp
constexpr int kT3SmemBytes = (kT3AStages + 3 * kT3Stages) * kT3OperandBytes + kT3StagingBytes + 512;
constexpr int kT3Threads = 352;
constexpr int kT3AccColumns = 256;            // two accumulators of up to 128 columns

struct alignas(64) Tc3Problem {
    CUtensorMap map_a;       // activations [node][component][K], box [nodes_per_tile][components][32]
    CUtensorMap map_hi;      // Bt_hi [N][K], box [n_tile][32]
    CUtensorMap map_lo;
    float* C;
    const float* bias;       // optional [N], added when not accumulating
    RowMap c_rows;
    int first_node;
    int M, N, K;             // logical rows (nodes x components), outputs, K % 32 == 0
    int accumulate;
    int rows_per_tile, nodes_per_tile;
    int n_tile, n_tiles;     // min(N, 128) in {32, 64, 128}; N % n_tile == 0
    int m_tiles;
    int tile_begin;          // first work item of this problem (items are m-major: m_tile * n_tiles + n)
};

constexpr int kT3MaxProblems = 8;
struct Tc3Batch {
    Tc3Problem problem[kT3MaxProblems];
    int count;
    int total_tiles;
};

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void umma_commit(unsigned long long* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Work item -> problem, row tile, column tile.
struct Tc3Item {
    int problem, m_tile, n_index;
};
__device__ __forceinline__ Tc3Item tc3_locate(const Tc3Batch& batch, int item)
{
    int pi = 0;
    for (int q = 1; q < batch.count; ++q)
        if (item >= batch.problem[q].tile_begin) pi = q;
    const int local = item - batch.problem[pi].tile_begin;
    return {pi, local / batch.problem[pi].n_tiles, local % batch.problem[pi].n_tiles};
}

// Nearest TF32 value of x (ties away from zero), returned as a float whose low 13 mantissa bits are zero.
__device__ __forceinline__ float tf32_round(float x)
{
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__global__ void __launch_bounds__(kT3Threads, 1) tc_gemm_tma_kernel(const __grid_constant__ Tc3Batch batch, int* __restrict__ error_flag)
{
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5;

    unsigned char* a_raw = smem;                                                    // [kT3AStages]
    unsigned char* a_lo = a_raw + kT3AStages * kT3OperandBytes;                     // [kT3Stages]
    unsigned char* b_buf = a_lo + kT3Stages * kT3OperandBytes;                      // [kT3Stages][hi, lo]
    unsigned char* staging = b_buf + 2 * kT3Stages * kT3OperandBytes;               // [4 epilogue warps][32 rows][128 B]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(staging + kT3StagingBytes);
    unsigned long long* full_a = bars;                       // [4] activation TMA landed (transaction barrier)
    unsigned long long* free_a = full_a + kT3AStages;        // [4] tcgen05.commit: raw tile read
    unsigned long long* ready = free_a + kT3AStages;         // [3] weight TMA landed + 128 residual arrivals
    unsigned long long* free_s = ready + kT3Stages;          // [3] tcgen05.commit: residual and weight tiles read
    unsigned long long* acc_full = free_s + kT3Stages;       // [2] tcgen05.commit
    unsigned long long* acc_empty = acc_full + 2;            // [2] 128 arrivals
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
    volatile int* failed = reinterpret_cast<volatile int*>(acc_empty + 3);

    if (tid == 256) {
        for (int s = 0; s < kT3AStages; ++s) { mbar_init(&full_a[s], 1); mbar_init(&free_a[s], 1); }
        for (int s = 0; s < kT3Stages; ++s) { mbar_init(&ready[s], 129); mbar_init(&free_s[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 128); }
        *failed = (smem_u32(smem) & 1023u) ? 1 : 0;   // the swizzled layout needs a 1 KB aligned base
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(static_cast<unsigned>(kT3AccColumns)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    const int first_item = blockIdx.x, item_step = gridDim.x;

    if (warp < 4) {
        // ------------------------------------------------------------- residual a - trunc(a)
        int kc = 0;   // chunks seen by this CTA so far, over all of its work items
        for (int item = first_item; item < batch.total_tiles && !*failed; item += item_step) {
            const Tc3Item it = tc3_locate(batch, item);
            const int chunks = batch.problem[it.problem].K / kTcChunk;
            for (int c = 0; c < chunks; ++c, ++kc) {
                const int sa = kc % kT3AStages, s = kc % kT3Stages;
                if (!mbar_wait(&full_a[sa], static_cast<unsigned>((kc / kT3AStages) & 1), failed)) break;
                // residual tile s was last read by chunk kc - 3
                if (kc >= kT3Stages && !mbar_wait(&free_s[s], static_cast<unsigned>((kc / kT3Stages - 1) & 1), failed)) break;
                const float4* src = reinterpret_cast<const float4*>(a_raw + sa * kT3OperandBytes);
                float4* dst = reinterpret_cast<float4*>(a_lo + s * kT3OperandBytes);
#pragma unroll
                for (int p = 0; p < kT3OperandBytes / 16 / 128; ++p) {   // position-wise: the layouts are identical
                    const float4 v = src[p * 128 + tid];
                    float4 lo;
                    // the residual is itself read as TF32 by the tensor core, i.e. truncated; rounding it to nearest here
                    // keeps that last truncation from always pulling the product towards zero
                    lo.x = tf32_round(v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u));
                    lo.y = tf32_round(v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u));
                    lo.z = tf32_round(v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u));
                    lo.w = tf32_round(v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u));
                    dst[p * 128 + tid] = lo;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&ready[s]);
            }
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------- epilogue
        const int quarter = warp - 4, row = tid - 128;   // tensor-memory lanes 32*quarter .. +31
        int j = 0;                                        // work items handled so far
        for (int item = first_item; item < batch.total_tiles; item += item_step, ++j) {
            const Tc3Item it = tc3_locate(batch, item);
            const Tc3Problem& P = batch.problem[it.problem];
            const int b = j & 1;
            if (!mbar_wait(&acc_full[b], static_cast<unsigned>((j >> 1) & 1), failed)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int g = it.m_tile * P.rows_per_tile + row;
            const bool store = row < P.rows_per_tile && g < P.M;
            const int col0 = it.n_index * P.n_tile;
            // row pointer of this lane's accumulator row (0 when the row is not stored)
            const unsigned long long my_row_ptr =
                store ? reinterpret_cast<unsigned long long>(P.C + row_address(P.c_rows, P.first_node, g) + col0) : 0ull;
            const int n_tile = P.n_tile, accumulate = P.accumulate;
            const float* bias = P.bias;
            unsigned char* stage = staging + quarter * (32 * 128);
            const int lane = tid & 31, sub_row = lane >> 3, sub_chunk = lane & 7;
            for (int c0 = 0; c0 < n_tile; c0 += 32) {
                unsigned v[32];
                const unsigned taddr = tmem_base + (static_cast<unsigned>(quarter * 32) << 16) + static_cast<unsigned>(b * 128 + c0);
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
                // accumulating launches: fetch the old values of all eight passes first, so that their latency (the output
                // has usually left L2 by now) is paid once per column group and not once per pass
                float4 old[8];
                if (accumulate) {
#pragma unroll
                    for (int pass = 0; pass < 8; ++pass) {
                        const unsigned long long ptr = __shfl_sync(0xffffffffu, my_row_ptr, pass * 4 + sub_row);
                        old[pass] = ptr != 0ull ? *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(ptr) + c0 + 4 * sub_chunk)
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                // a lane holds 32 columns of one row; through the warp's staging tile (16-byte chunks XORed by
                // row, conflict-free both ways) the warp stores whole 128-byte row segments, four rows per pass
                __syncwarp();
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    *reinterpret_cast<float4*>(stage + lane * 128 + ((q ^ (lane & 7)) << 4)) =
                        make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                                    __uint_as_float(v[4 * q + 3]));
                __syncwarp();
#pragma unroll
                for (int pass = 0; pass < 8; ++pass) {
                    const int r = pass * 4 + sub_row;
                    const unsigned long long ptr = __shfl_sync(0xffffffffu, my_row_ptr, r);
                    if (ptr != 0ull) {
                        float4 o = *reinterpret_cast<const float4*>(stage + r * 128 + ((sub_chunk ^ (r & 7)) << 4));
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(ptr) + c0 + 4 * sub_chunk);
                        if (accumulate) {
                            o.x += old[pass].x; o.y += old[pass].y; o.z += old[pass].z; o.w += old[pass].w;
                        } else if (bias != nullptr) {
                            const float4 bv = *reinterpret_cast<const float4*>(bias + col0 + c0 + 4 * sub_chunk);
                            o.x += bv.x; o.y += bv.y; o.z += bv.z; o.w += bv.w;
                        }
                        *dst = o;
                    }
                }
            }
            // the accumulator has been read: hand it back to the issuing thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&acc_empty[b]);
        }
    } else if (tid == 256) {
        // ------------------------------------------------------------- tcgen05.mma issue: one wait and 12 MMAs per chunk
        const unsigned a_raw_addr = smem_u32(a_raw), a_lo_addr = smem_u32(a_lo), b_addr = smem_u32(b_buf);
        int kc = 0, j = 0;
        if (!*failed) {
            bool ok = true;
            for (int item = first_item; item < batch.total_tiles && ok; item += item_step, ++j) {
                const Tc3Item it = tc3_locate(batch, item);
                const int NT = batch.problem[it.problem].n_tile, chunks = batch.problem[it.problem].K / kTcChunk, b = j & 1;
                // instruction descriptor: D = F32, A = B = TF32, both K-major, N = NT, M = 128
                const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<unsigned>(NT >> 3) << 17) |
                                       (static_cast<unsigned>(kTcRows >> 4) << 24);
                // the epilogue must have drained this accumulator (work item j - 2)
                if (j >= 2 && !mbar_wait(&acc_empty[b], static_cast<unsigned>(((j >> 1) - 1) & 1), failed)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_d = tmem_base + static_cast<unsigned>(b * 128);
                for (int c = 0; c < chunks; ++c, ++kc) {
                    const int sa = kc % kT3AStages, s = kc % kT3Stages;
                    // weights landed and the residual is written (which implies the raw tile landed)
                    if (!mbar_wait(&ready[s], static_cast<unsigned>((kc / kT3Stages) & 1), failed)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned long long da_hi = umma_desc(a_raw_addr + sa * kT3OperandBytes);
                    const unsigned long long da_lo = umma_desc(a_lo_addr + s * kT3OperandBytes);
                    const unsigned long long db_hi = umma_desc(b_addr + (2 * s) * kT3OperandBytes);
                    const unsigned long long db_lo = umma_desc(b_addr + (2 * s + 1) * kT3OperandBytes);
#pragma unroll
                    for (int ks = 0; ks < kTcChunk / 8; ++ks) {
                        const unsigned long long step = static_cast<unsigned long long>(ks * 2);   // 32 bytes along K
                        umma_tf32(tmem_d, da_hi + step, db_hi + step, idesc, (c > 0 || ks > 0) ? 1u : 0u);
                        umma_tf32(tmem_d, da_hi + step, db_lo + step, idesc, 1u);
                        umma_tf32(tmem_d, da_lo + step, db_hi + step, idesc, 1u);
                    }
                    umma_commit(&free_a[sa]);
                    umma_commit(&free_s[s]);
                    if (c + 1 == chunks) umma_commit(&acc_full[b]);
                }
            }
        }
    } else if (tid == 288) {
        // ------------------------------------------------------------- weight TMA
        int issued = 0;
        if (!*failed) {
            bool ok = true;
            for (int item = first_item; item < batch.total_tiles && ok; item += item_step) {
                const Tc3Item it = tc3_locate(batch, item);
                const Tc3Problem& P = batch.problem[it.problem];
                const unsigned bytes = 2u * static_cast<unsigned>(P.n_tile) * 128u;
                const int chunks = P.K / kTcChunk, n0 = it.n_index * P.n_tile;
                for (int c = 0; c < chunks; ++c) {
                    const int s = issued % kT3Stages, use = issued / kT3Stages;
                    if (use > 0 && !mbar_wait(&free_s[s], static_cast<unsigned>((use - 1) & 1), failed)) { ok = false; break; }
                    unsigned char* hi = b_buf + (2 * s) * kT3OperandBytes;
                    const int k0 = c * kTcChunk;
                    mbar_expect_tx(&ready[s], bytes);
                    tma_load_2d(hi, &P.map_hi, &ready[s], k0, n0);
                    tma_load_2d(hi + kT3OperandBytes, &P.map_lo, &ready[s], k0, n0);
                    ++issued;
                }
            }
            // after a failure: let the copies still in flight land before the CTA exits
            if (*failed)
                for (int q = max(0, issued - kT3Stages); q < issued; ++q) {
                    int never = 0;
                    mbar_wait(&ready[q % kT3Stages], static_cast<unsigned>((q / kT3Stages) & 1), &never);
                }
        }
    } else if (tid == 320) {
        // ------------------------------------------------------------- activation TMA
        int issued = 0;
        if (!*failed) {
            bool ok = true;
            for (int item = first_item; item < batch.total_tiles && ok; item += item_step) {
                const Tc3Item it = tc3_locate(batch, item);
                const Tc3Problem& P = batch.problem[it.problem];
                const unsigned bytes = static_cast<unsigned>(P.rows_per_tile) * 128u;
                const int chunks = P.K / kTcChunk, node0 = it.m_tile * P.nodes_per_tile;
                for (int c = 0; c < chunks; ++c) {
                    const int s = issued % kT3AStages, use = issued / kT3AStages;
                    if (use > 0 && !mbar_wait(&free_a[s], static_cast<unsigned>((use - 1) & 1), failed)) { ok = false; break; }
                    mbar_expect_tx(&full_a[s], bytes);
                    tma_load_3d(a_raw + s * kT3OperandBytes, &P.map_a, &full_a[s], c * kTcChunk, 0, node0);
                    ++issued;
                }
            }
            if (*failed)
                for (int q = max(0, issued - kT3AStages); q < issued; ++q) {
                    int never = 0;
                    mbar_wait(&full_a[q % kT3AStages], static_cast<unsigned>((q / kT3AStages) & 1), &never);
                }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *failed) atomicOr(error_flag, 2);
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(static_cast<unsigned>(kT3AccColumns)) : "memory");
    }
}

}  // namespace sxb
