// All-gather of a small per-rank buffer over NVLink peer memory, in ONE kernel launch per rank.
//
// The KV-sequence-sharded decode step exchanges two buffers of a few hundred KB per step (page candidates, then one
// (o, m, l) partial per head).  At that size a library all-gather is pure latency; here every rank's kernel stores
// its buffer straight into every peer's memory (plain 16-byte stores over NVLink: no multicast, no TMA, no loads
// from peer memory), publishes a per-step flag on every peer, waits - with a cycle budget - until the flags of all
// peers have arrived in its own memory, and copies the gathered rows to the caller's output.
//
// Memory: every rank owns one region (cudaMalloc'd by ta100_peer_exchange_create, opened by the peers through a
// CUDA IPC handle):
//   data   [2][world][slot_bytes]   gathered rows, double-buffered by step parity
//   flags  [2][world] u32           flags[parity][r] = step number of rank r's latest store into data[parity][r]
//   ctl    u32 step, u32 arrived, u32 left, i32 status
// Rank r writes data[parity][r] and flags[parity][r] of EVERY region (its own included).  Two parities suffice: a
// rank can enter step k + 1 only after every peer has stored its step-k rows, and it stores its step-(k + 1) rows
// only after its own step-k consumers ran (stream order), so nobody is ever more than one step ahead of a reader.
// The step counter lives in device memory and is advanced by the kernel itself, so the launch has the same
// arguments every step and can be replayed from a CUDA graph.
//
// One process per GPU.  The kernels of different ranks wait for each other, so they must run on different GPUs.
#include <cstdint>
#include <cstring>

#include "common.cuh"

namespace ta100 {

namespace {

constexpr int MAX_WORLD = 8;

struct ExchangeParams {
    const uint8_t* src;
    uint8_t* out;
    uint8_t* region[MAX_WORLD];    // every rank's region (index = rank), own included
    long long bytes;               // payload per rank, multiple of 16
    long long slot_bytes;          // stride between ranks inside a parity buffer
    int world, rank;
    long long budget;
};

__host__ __device__ inline long long flags_offset(int world, long long slot_bytes) { return 2LL * world * slot_bytes; }
__host__ __device__ inline long long ctl_offset(int world, long long slot_bytes) {
    return flags_offset(world, slot_bytes) + 2LL * world * 4;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) peer_all_gather_kernel(const ExchangeParams p) {
    __shared__ uint32_t s_step;
    __shared__ int s_ok;
    uint8_t* mine = p.region[p.rank];
    uint32_t* ctl = reinterpret_cast<uint32_t*>(mine + ctl_offset(p.world, p.slot_bytes));
    if (threadIdx.x == 0) { s_step = ctl[0] + 1u; s_ok = 1; }    // ctl[0] only changes when the last CTA of a launch leaves
    __syncthreads();
    const uint32_t step = s_step;
    const long long parity_off = static_cast<long long>(step & 1u) * p.world * p.slot_bytes;

    // ---- put: this rank's rows into slot `rank` of every region ----
    const long long vecs = p.bytes / 16;
    const uint4* src = reinterpret_cast<const uint4*>(p.src);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs * p.world;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int peer = static_cast<int>(i / vecs);
        const long long v = i - peer * vecs;
        reinterpret_cast<uint4*>(p.region[peer] + parity_off + p.rank * p.slot_bytes)[v] = __ldg(src + v);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t before = atomicAdd(&ctl[1], 1u);
        if (before == gridDim.x - 1) {
            // every CTA's stores are fenced: publish
            __threadfence_system();
            for (int peer = 0; peer < p.world; ++peer) {
                uint32_t* flags = reinterpret_cast<uint32_t*>(p.region[peer] + flags_offset(p.world, p.slot_bytes));
                st_release_sys(flags + (step & 1u) * p.world + p.rank, step);
            }
        }
    }

    // ---- wait (bounded) until every rank's rows of this step are in MY region ----
    if (threadIdx.x < p.world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + flags_offset(p.world, p.slot_bytes)) +
                               (step & 1u) * p.world + threadIdx.x;
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != step) {
            if (clock64() - t0 > p.budget) {
                s_ok = 0;
                atomicExch(reinterpret_cast<int*>(ctl + 3), 1);
                break;
            }
        }
    }
    __syncthreads();

    // ---- gathered rows to the caller's buffer [world, bytes] (zeros if a peer never arrived) ----
    const bool ok = s_ok != 0;
    uint4* out = reinterpret_cast<uint4*>(p.out);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < vecs * p.world;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / vecs);
        const long long v = i - r * vecs;
        out[i] = ok ? reinterpret_cast<const uint4*>(mine + parity_off + r * p.slot_bytes)[v] : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t before = atomicAdd(&ctl[2], 1u);
        if (before == gridDim.x - 1) {           // the last CTA out advances the step and re-arms the counters
            ctl[1] = 0u;
            ctl[2] = 0u;
            __threadfence();
            ctl[0] = step;
        }
    }
}

}  // namespace

size_t peer_exchange_region_bytes(int world, long long slot_bytes) {
    return static_cast<size_t>(ctl_offset(world, slot_bytes) + 64);
}

// Allocates this rank's region (zeroed) and returns its IPC handle (64 bytes).
int peer_exchange_create(int world, long long slot_bytes, void** region, unsigned char* handle64) {
    if (!region || !handle64) return TA100_ERR_NULL;
    if (world < 1 || world > MAX_WORLD || slot_bytes <= 0 || slot_bytes % 16 != 0) return TA100_ERR_SHAPE;
    void* ptr = nullptr;
    const size_t bytes = peer_exchange_region_bytes(world, slot_bytes);
    cudaError_t e = cudaMalloc(&ptr, bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemset(ptr, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) { cudaFree(ptr); return static_cast<int>(e); }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle64, &h, 64);
    *region = ptr;
    return TA100_OK;
}

int peer_exchange_open(const unsigned char* handle64, void** region) {
    if (!handle64 || !region) return TA100_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    return static_cast<int>(cudaIpcOpenMemHandle(region, h, cudaIpcMemLazyEnablePeerAccess));
}

int peer_exchange_close(void* region) { return region ? static_cast<int>(cudaIpcCloseMemHandle(region)) : TA100_OK; }

int peer_exchange_destroy(void* region) { return region ? static_cast<int>(cudaFree(region)) : TA100_OK; }

// regions: host array of `world` device pointers (index = rank; regions[rank] is this rank's own allocation).
int peer_all_gather_dispatch(const void* src, void* out, long long bytes, long long slot_bytes, int world, int rank,
                             void* const* regions, cudaStream_t stream) {
    if (!src || !out || !regions) return TA100_ERR_NULL;
    if (world < 1 || world > MAX_WORLD || rank < 0 || rank >= world) return TA100_ERR_SHAPE;
    if (bytes <= 0 || bytes % 16 != 0 || slot_bytes % 16 != 0 || bytes > slot_bytes) return TA100_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) return TA100_ERR_ALIGN;
    ExchangeParams p{};
    p.src = static_cast<const uint8_t*>(src);
    p.out = static_cast<uint8_t*>(out);
    for (int r = 0; r < world; ++r) {
        if (!regions[r]) return TA100_ERR_NULL;
        p.region[r] = static_cast<uint8_t*>(regions[r]);
    }
    p.bytes = bytes; p.slot_bytes = slot_bytes; p.world = world; p.rank = rank;
    p.budget = g_wait_budget_cycles;
    // few CTAs: they all have to be resident at once (every one of them waits for the flags), and the payload is small
    const long long vecs = bytes / 16 * world;
    int grid = static_cast<int>((vecs + 255) / 256);
    if (grid > 32) grid = 32;
    if (grid < 1) grid = 1;
    peer_all_gather_kernel<<<grid, 256, 0, stream>>>(p);
    return static_cast<int>(cudaGetLastError());
}

// 1 if a wait of an earlier all-gather on this region ran out (and clears the mark); synchronises the stream.
int peer_exchange_status(void* region, int world, long long slot_bytes, cudaStream_t stream) {
    if (!region) return TA100_ERR_NULL;
    int st = 0;
    uint8_t* at = static_cast<uint8_t*>(region) + ctl_offset(world, slot_bytes) + 12;
    cudaError_t e = cudaMemcpyAsync(&st, at, 4, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (st) {
        e = cudaMemsetAsync(at, 0, 4, stream);
        if (e != cudaSuccess) return static_cast<int>(e);
        return TA100_ERR_DEVICE_TIMEOUT;
    }
    return TA100_OK;
}

}  // namespace ta100
