// Halo exchange over NVLink peer memory, one process per GPU.
//
// The reference moves ghost rows with LAMMPS' MPI brick swaps
// (pair_symmetrix/pair_symmetrix_mace_kokkos.cpp:737-1005, 1568-1705).  Here every rank maps the receive
// buffers of its peers (CUDA IPC handles of plain cudaMalloc allocations) and an exchange is two small
// steps on the evaluator's stream:
//   push: copies this rank's outgoing rows, segment by segment, straight into the peers' receive
//         buffers with 16-byte stores over NVLink, then raises this rank's arrival flag at each peer;
//   wait: spins, with a time limit, until every peer's flag shows the current step.  By default the
//         thread that raised the flag for a peer also waits for that peer's flag, inside the push
//         kernel (one launch per exchange); SXB_PEER_SPLIT_WAIT=1 runs the wait as a kernel of its own.
// There is no collective and no staging copy, and the kernels can be captured into a CUDA graph: the
// step number lives in device memory and is advanced by a kernel.  Every wait is bounded; when it
// expires the kernel records bit 32 in the status word and returns, so the context stays usable and the
// host raises after its next synchronisation.  Only plain peer loads and stores are used.
#include "../../include/symmetrix_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "common.cuh"

namespace sxb {

void set_last_error(const std::string& message);   // c_api.cu

namespace {

constexpr int kMaxPeers = 16;
constexpr int kPhases = 4;                       // positions, H1, H1_adj, forces
constexpr double kDefaultWaitSeconds = 10.0;      // limit of every wait unless sxb_peer_set_wait_limit says otherwise

struct PushPlan {
    int world;
    int row_bytes;                    // multiple of 8
    const unsigned char* send;        // local rows: ordered by destination rank, or gathered through row_source
    long long send_begin[kMaxPeers + 1];     // rows
    unsigned char* remote[kMaxPeers];        // my segment (or, with row_dest, the whole tensor) in each peer's memory
    unsigned long long* remote_flag[kMaxPeers];   // my slot of this phase in each peer's flag table
    const unsigned long long* step;   // device: number of the current step
    const int* row_source;            // optional [rows]: row of `send` to take for outgoing row r (gather while pushing)
    const int* row_dest;              // optional [rows]: row of the peer's tensor that outgoing row r goes to
    int accumulate;                   // add (FP32, 16 bytes at a time) instead of store: rows may repeat at the owner
};

// grid.y = destination rank; blocks of a rank stride over its segment.  The last block to finish a
// segment publishes the flag after a system-wide fence.
// Bounded spin until `flag` shows step `want`; records bit 32 in the status word when the limit runs out.
__device__ __forceinline__ void wait_for_flag(const unsigned long long* flag, unsigned long long want, int* status,
                                              long long limit_cycles)
{
    const long long start = clock64();
    for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(flag) : "memory");
        if (seen >= want) break;
        if (clock64() - start > limit_cycles) {
            *reinterpret_cast<volatile int*>(status) = 32;
            break;
        }
        __nanosleep(200);
    }
}

__global__ void __launch_bounds__(256) push_segments_kernel(PushPlan plan, unsigned int* __restrict__ done_counters,
                                                            const unsigned long long* __restrict__ incoming /*[world] or nullptr*/,
                                                            int* __restrict__ status, long long limit_cycles)
{
    const int peer = blockIdx.y;
    const long long first = plan.send_begin[peer], rows = plan.send_begin[peer + 1] - first;
    unsigned char* dst = plan.remote[peer];
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long start = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if ((plan.row_bytes & 15) == 0) {
        const int per_row = plan.row_bytes >> 4;
        const long long words = rows * per_row;
        for (long long i = start; i < words; i += stride) {
            const long long r = i / per_row, w = i - r * per_row;
            const long long from = plan.row_source != nullptr ? plan.row_source[first + r] : first + r;
            const long long to = plan.row_dest != nullptr ? plan.row_dest[first + r] : r;
            const float4 v = reinterpret_cast<const float4*>(plan.send + from * plan.row_bytes)[w];
            float4* out = reinterpret_cast<float4*>(dst + to * plan.row_bytes) + w;
            if (plan.accumulate) atomicAdd(out, v);
            else *out = v;
        }
    } else {
        const int per_row = plan.row_bytes >> 3;
        const long long words = rows * per_row;
        for (long long i = start; i < words; i += stride) {
            const long long r = i / per_row, w = i - r * per_row;
            const long long from = plan.row_source != nullptr ? plan.row_source[first + r] : first + r;
            const long long to = plan.row_dest != nullptr ? plan.row_dest[first + r] : r;
            reinterpret_cast<long long*>(dst + to * plan.row_bytes)[w] = reinterpret_cast<const long long*>(plan.send + from * plan.row_bytes)[w];
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int arrived = atomicAdd(done_counters + peer, 1u) + 1u;
        if (arrived == gridDim.x) {
            done_counters[peer] = 0;
            __threadfence_system();
            const unsigned long long step = *plan.step;
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(plan.remote_flag[peer]), "l"(step) : "memory");
            // this peer's rows for me: nothing of mine is pending any more, so the wait cannot block a push
            if (incoming != nullptr) wait_for_flag(incoming + peer, step, status, limit_cycles);
        }
    }
}

// One thread per peer waits until that peer's flag reaches the current step.
__global__ void wait_flags_kernel(int world, const unsigned long long* __restrict__ flags /*[world]*/,
                                  const unsigned long long* __restrict__ step, int* __restrict__ status, long long limit_cycles)
{
    const int peer = threadIdx.x;
    if (peer >= world) return;
    wait_for_flag(flags + peer, *step, status, limit_cycles);
}

__global__ void advance_step_kernel(unsigned long long* step) { *step += 1ull; }

}  // namespace

// State of one rank's side of the exchange.
struct PeerExchange {
    int device = 0, rank = 0, world = 1;
    unsigned long long* flags = nullptr;        // [kPhases][kMaxPeers], written by the peers
    unsigned long long* step = nullptr;         // current step, device
    unsigned int* counters = nullptr;           // [kPhases][kMaxPeers] block counters of the push kernel
    int* status = nullptr;                      // mapped pinned host word; bit 32: a wait expired
    std::vector<void*> opened;                  // mappings of peer memory to close
    PushPlan plans[kPhases];
    bool split_wait = false;                    // SXB_PEER_SPLIT_WAIT=1: the wait as a kernel of its own
    long long wait_cycles = 0;                  // limit of a wait in SM clock cycles
    double cycles_per_second = 0.0;
    bool planned[kPhases] = {false, false, false, false};
};

}  // namespace sxb

struct PeerExchange : sxb::PeerExchange {};

extern "C" {

int sxb_device_alloc(int32_t device_ordinal, int64_t bytes, void** out)
{
    try {
        if (out == nullptr || bytes <= 0) throw std::invalid_argument("sxb_device_alloc needs an output pointer and a positive size.");
        SXB_CUDA(cudaSetDevice(device_ordinal));
        SXB_CUDA(cudaMalloc(out, static_cast<size_t>(bytes)));
        SXB_CUDA(cudaMemset(*out, 0, static_cast<size_t>(bytes)));
        return SXB_OK;
    } catch (const std::invalid_argument& e) { sxb::set_last_error(e.what()); return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { sxb::set_last_error(e.what()); return SXB_ERR_RUNTIME; }
}

int sxb_device_free(void* pointer)
{
    if (pointer != nullptr && cudaFree(pointer) != cudaSuccess) {
        cudaGetLastError();
        sxb::set_last_error("cudaFree failed.");
        return SXB_ERR_RUNTIME;
    }
    return SXB_OK;
}

int sxb_ipc_export(const void* device_pointer, unsigned char* handle64)
{
    try {
        if (device_pointer == nullptr || handle64 == nullptr) throw std::invalid_argument("sxb_ipc_export needs a pointer and a handle buffer.");
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
        cudaIpcMemHandle_t handle;
        SXB_CUDA(cudaIpcGetMemHandle(&handle, const_cast<void*>(device_pointer)));
        std::memcpy(handle64, &handle, 64);
        return SXB_OK;
    } catch (const std::invalid_argument& e) { sxb::set_last_error(e.what()); return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { sxb::set_last_error(e.what()); return SXB_ERR_RUNTIME; }
}

int sxb_peer_create(int32_t device_ordinal, int32_t rank, int32_t world, PeerExchange** out)
{
    try {
        if (out == nullptr || world <= 0 || world > sxb::kMaxPeers || rank < 0 || rank >= world)
            throw std::invalid_argument("Peer exchange supports 1 to 16 ranks.");
        SXB_CUDA(cudaSetDevice(device_ordinal));
        auto* px = new PeerExchange();
        px->device = device_ordinal; px->rank = rank; px->world = world;
        if (const char* env = std::getenv("SXB_PEER_SPLIT_WAIT")) px->split_wait = env[0] == '1';
        int clock_khz = 0;
        SXB_CUDA(cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, device_ordinal));
        px->cycles_per_second = 1e3 * std::max(clock_khz, 1);
        px->wait_cycles = static_cast<long long>(sxb::kDefaultWaitSeconds * px->cycles_per_second);
        SXB_CUDA(cudaMalloc(reinterpret_cast<void**>(&px->flags), sizeof(unsigned long long) * sxb::kPhases * sxb::kMaxPeers));
        SXB_CUDA(cudaMemset(px->flags, 0, sizeof(unsigned long long) * sxb::kPhases * sxb::kMaxPeers));
        SXB_CUDA(cudaMalloc(reinterpret_cast<void**>(&px->step), sizeof(unsigned long long)));
        SXB_CUDA(cudaMemset(px->step, 0, sizeof(unsigned long long)));
        SXB_CUDA(cudaMalloc(reinterpret_cast<void**>(&px->counters), sizeof(unsigned int) * sxb::kPhases * sxb::kMaxPeers));
        SXB_CUDA(cudaMemset(px->counters, 0, sizeof(unsigned int) * sxb::kPhases * sxb::kMaxPeers));
        // the status word lives in mapped pinned host memory: the host reads it after a synchronisation without a copy
        SXB_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&px->status), sizeof(int), cudaHostAllocMapped));
        *px->status = 0;
        *out = px;
        return SXB_OK;
    } catch (const std::invalid_argument& e) { sxb::set_last_error(e.what()); return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { sxb::set_last_error(e.what()); return SXB_ERR_RUNTIME; }
}

// Reads and clears the status word (call after synchronising the stream): 0, or 32 when a wait expired.
int sxb_peer_status(PeerExchange* px, int32_t* out)
{
    if (px == nullptr || out == nullptr) { sxb::set_last_error("NULL argument."); return SXB_ERR_INVALID_ARGUMENT; }
    *out = *reinterpret_cast<volatile int*>(px->status);
    *reinterpret_cast<volatile int*>(px->status) = 0;
    return SXB_OK;
}

int sxb_peer_flags(PeerExchange* px, void** flags)
{
    if (px == nullptr || flags == nullptr) { sxb::set_last_error("NULL argument."); return SXB_ERR_INVALID_ARGUMENT; }
    *flags = px->flags;
    return SXB_OK;
}

// Maps a peer's allocation (handle from sxb_ipc_export in the peer's process); `same_process` handles
// (rank == own rank) are passed as plain pointers by the caller and never opened.
int sxb_peer_open(PeerExchange* px, const unsigned char* handle64, void** out)
{
    try {
        if (px == nullptr || handle64 == nullptr || out == nullptr) throw std::invalid_argument("NULL argument.");
        SXB_CUDA(cudaSetDevice(px->device));
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, handle64, 64);
        SXB_CUDA(cudaIpcOpenMemHandle(out, handle, cudaIpcMemLazyEnablePeerAccess));
        px->opened.push_back(*out);
        return SXB_OK;
    } catch (const std::invalid_argument& e) { sxb::set_last_error(e.what()); return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { sxb::set_last_error(e.what()); return SXB_ERR_RUNTIME; }
}

// Describes one of the four exchanges: my outgoing rows `send` (device, ordered by destination rank,
// send_begin[world+1] in rows of row_bytes bytes), where my segment starts in each peer's receive
// buffer (remote_pointers[world], already offset), and each peer's flag table (remote_flags[world],
// base addresses of the tables returned by sxb_peer_flags there).  Optional device arrays over all
// outgoing rows: row_source gathers the rows out of a larger local tensor while pushing (send is then
// that tensor), row_dest scatters them to rows of the peer's tensor (remote_pointers then name the
// tensors); accumulate adds instead of storing.
int sxb_peer_plan(PeerExchange* px, int32_t phase, const void* send, const int64_t* send_begin, int32_t row_bytes,
                  void* const* remote_pointers, void* const* remote_flags, const int32_t* device_row_source,
                  const int32_t* device_row_dest, int32_t accumulate)
{
    try {
        if (px == nullptr || phase < 0 || phase >= sxb::kPhases || send_begin == nullptr || remote_pointers == nullptr || remote_flags == nullptr)
            throw std::invalid_argument("Bad peer plan arguments.");
        if (row_bytes <= 0 || (row_bytes & 7) != 0) throw std::invalid_argument("Row size must be a positive multiple of 8 bytes.");
        sxb::PushPlan& plan = px->plans[phase];
        plan.world = px->world;
        plan.row_bytes = row_bytes;
        plan.send = static_cast<const unsigned char*>(send);
        plan.step = px->step;
        plan.row_source = device_row_source;
        plan.row_dest = device_row_dest;
        plan.accumulate = accumulate != 0 ? 1 : 0;
        if (plan.accumulate && (row_bytes & 15) != 0) throw std::invalid_argument("Accumulating pushes need rows that are multiples of 16 bytes.");
        for (int p = 0; p <= px->world; ++p) plan.send_begin[p] = send_begin[p];
        for (int p = 0; p < px->world; ++p) {
            plan.remote[p] = static_cast<unsigned char*>(remote_pointers[p]);
            if ((reinterpret_cast<uintptr_t>(plan.remote[p]) & 15) != 0 && (row_bytes & 15) == 0 && send_begin[p + 1] > send_begin[p])
                throw std::invalid_argument("Peer receive segments must start on 16-byte boundaries.");
            plan.remote_flag[p] = static_cast<unsigned long long*>(remote_flags[p]) + phase * sxb::kMaxPeers + px->rank;
        }
        if ((reinterpret_cast<uintptr_t>(plan.send) & 15) != 0 && send_begin[px->world] > 0)
            throw std::invalid_argument("The send buffer must start on a 16-byte boundary.");
        px->planned[phase] = true;
        return SXB_OK;
    } catch (const std::invalid_argument& e) { sxb::set_last_error(e.what()); return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { sxb::set_last_error(e.what()); return SXB_ERR_RUNTIME; }
}

// Enqueue on `stream`: advance the step counter (once per step, before the first exchange).
int sxb_peer_advance(PeerExchange* px, void* stream)
{
    if (px == nullptr) { sxb::set_last_error("NULL argument."); return SXB_ERR_INVALID_ARGUMENT; }
    sxb::advance_step_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(px->step);
    return cudaGetLastError() == cudaSuccess ? SXB_OK : SXB_ERR_RUNTIME;
}

// Enqueue on `stream`: push my rows of exchange `phase` to the peers, then wait for theirs.
int sxb_peer_exchange(PeerExchange* px, int32_t phase, void* stream)
{
    try {
        if (px == nullptr || phase < 0 || phase >= sxb::kPhases || !px->planned[phase]) throw std::invalid_argument("Peer exchange phase has no plan.");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const sxb::PushPlan& plan = px->plans[phase];
        long long largest = 0;
        for (int p = 0; p < px->world; ++p) largest = std::max(largest, (plan.send_begin[p + 1] - plan.send_begin[p]) * plan.row_bytes);
        // enough 16-byte stores in flight to fill the links: up to 128 blocks per destination
        int blocks = static_cast<int>(std::min<long long>(128, std::max<long long>(1, largest / (256 * 32))));
        dim3 grid(blocks, px->world);
        const unsigned long long* incoming = px->flags + phase * sxb::kMaxPeers;
        sxb::push_segments_kernel<<<grid, 256, 0, s>>>(plan, px->counters + phase * sxb::kMaxPeers, px->split_wait ? nullptr : incoming,
                                                       px->status, px->wait_cycles);
        if (px->split_wait) sxb::wait_flags_kernel<<<1, 32, 0, s>>>(px->world, incoming, px->step, px->status, px->wait_cycles);
        SXB_CUDA(cudaGetLastError());
        return SXB_OK;
    } catch (const std::invalid_argument& e) { sxb::set_last_error(e.what()); return SXB_ERR_INVALID_ARGUMENT;
    } catch (const std::exception& e) { sxb::set_last_error(e.what()); return SXB_ERR_RUNTIME; }
}

// Limit of every wait from now on (seconds of SM clock at the nominal rate; 10 by default).  Exchanges that are
// already captured in a CUDA graph keep the limit they were captured with.
int sxb_peer_set_wait_limit(PeerExchange* px, double seconds)
{
    if (px == nullptr || !(seconds > 0.0) || !(seconds <= 60.0)) {
        sxb::set_last_error("The wait limit must lie in (0, 60] seconds.");
        return SXB_ERR_INVALID_ARGUMENT;
    }
    px->wait_cycles = std::max(1ll, static_cast<long long>(seconds * px->cycles_per_second));
    return SXB_OK;
}

int sxb_peer_destroy(PeerExchange* px)
{
    if (px == nullptr) return SXB_OK;
    cudaSetDevice(px->device);
    cudaDeviceSynchronize();
    for (void* p : px->opened) cudaIpcCloseMemHandle(p);
    cudaFree(px->flags);
    cudaFree(px->step);
    cudaFree(px->counters);
    cudaFreeHost(px->status);
    cudaGetLastError();
    delete px;
    return SXB_OK;
}

}  // extern "C"
