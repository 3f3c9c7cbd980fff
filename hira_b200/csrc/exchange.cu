// Exchange of the softmax partials of sequence-sharded decode over NVLink peer memory, fused with
// their merge: one kernel per step and GPU, no library collective on the data path.
//
// Every rank owns one exchange buffer that its peers can write (mapped through CUDA IPC, plain
// peer stores over NVLink; no multicast of any kind):
//     rows  [2 parities][world sources][n_qheads][2 + vdim] floats   (m, l, normalised out)
//     flags [2 parities][world sources][n_qheads] uint32             the step number the row belongs to
// Block h of rank r's kernel (step number seq, parity seq & 1)
//   1. stores row h of this rank's partials into slot [parity][r][h] of EVERY rank's buffer (its own
//      included), fences, and stores seq into the matching flags;
//   2. waits (bounded) until the flags [parity][s][h] of its own buffer carry seq for every source s;
//   3. merges the world rows with the arithmetic of hira_merge_partials.
// A block pushes before it waits and waits only for pushes, so no rank's progress depends on another
// rank's waiting.  Two parities suffice: a rank can only push step s + 2 after it has merged step s + 1,
// for which every peer had pushed s + 1, which a peer does (stream order) after its merge of step s.
// If a wait runs out (a peer died or never launched) the block sets *status and leaves `out` untouched.
#include <atomic>
#include <cstring>

#include "common.cuh"
#include "merge_row.cuh"

namespace hira {

struct PeerBufs {
    float* p[HIRA_MAX_PEERS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// phases: bit 0 = push, bit 1 = wait + merge (both = the fused step; singly for one-GPU tests,
// where the kernels of several emulated ranks must not wait on one another)
__global__ void __launch_bounds__(128)
exchange_merge_kernel(const float* __restrict__ local, PeerBufs peers, int world, int rank, int n_qheads, int vdim,
                      uint32_t seq, int phases, unsigned long long wait_cycles, float* __restrict__ out,
                      float* __restrict__ out_ml, int* __restrict__ status) {
    const int h = blockIdx.x, tid = threadIdx.x;
    const int ps = vdim + 2;
    const int par = (int)(seq & 1u);
    const size_t n_rows = (size_t)2 * world * n_qheads;
    __shared__ int s_ok;
    if (tid == 0) s_ok = 1;
    if (phases & 1) {
        const size_t row = ((size_t)par * world + rank) * n_qheads + h;
        for (int p = 0; p < world; ++p) {
            float* dst = peers.p[p] + row * ps;
            for (int i = tid; i < ps; i += blockDim.x) dst[i] = local[(size_t)h * ps + i];
        }
        __threadfence_system();   // every thread's stores are out before the flags go
        __syncthreads();
        if (tid < world) st_release_sys(reinterpret_cast<uint32_t*>(peers.p[tid] + n_rows * ps) + row, seq);
    }
    if (!(phases & 2)) return;
    float* mine = peers.p[rank];
    if (tid < world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + n_rows * ps) + ((size_t)par * world + tid) * n_qheads + h;
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != seq) {
            if ((unsigned long long)(clock64() - t0) > wait_cycles) {
                s_ok = 0;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (!s_ok) {
        if (tid == 0) atomicExch(status, 1);
        return;
    }
    const float* rows = mine + ((size_t)par * world * n_qheads + h) * ps;   // source s: + s * n_qheads * ps
    merge_row(rows + 2, rows, (long long)n_qheads * ps, (long long)n_qheads * ps, world, vdim, 1, out + (size_t)h * vdim,
              out_ml ? out_ml + (size_t)h * 2 : nullptr);
}

}  // namespace hira

extern "C" int64_t hira_exchange_bytes(int32_t world, int32_t n_qheads, int32_t vdim) {
    if (world < 1 || n_qheads < 1 || vdim < 1) return 0;
    return (int64_t)2 * world * n_qheads * ((int64_t)(vdim + 2) * 4 + 4);
}

extern "C" int hira_peer_alloc(int64_t bytes, void** dev_ptr, unsigned char* handle) {
    HIRA_CHECK_ARG(bytes > 0 && dev_ptr != nullptr && handle != nullptr, HIRA_ERR_ARG, "hira_peer_alloc: bad argument");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t hnd;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&hnd, p);
    if (e != cudaSuccess) {
        hira::set_error("hira_peer_alloc(%lld bytes): %s", (long long)bytes, cudaGetErrorString(e));
        if (p) cudaFree(p);
        return HIRA_ERR_CUDA;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == HIRA_PEER_HANDLE_BYTES, "handle size");
    memcpy(handle, &hnd, sizeof(hnd));
    *dev_ptr = p;
    return HIRA_OK;
}

extern "C" int hira_peer_open(const unsigned char* handle, void** dev_ptr) {
    HIRA_CHECK_ARG(handle != nullptr && dev_ptr != nullptr, HIRA_ERR_ARG, "hira_peer_open: NULL argument");
    cudaIpcMemHandle_t hnd;
    memcpy(&hnd, handle, sizeof(hnd));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, hnd, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        hira::set_error("hira_peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
        return HIRA_ERR_CUDA;
    }
    *dev_ptr = p;
    return HIRA_OK;
}

extern "C" int hira_peer_close(void* dev_ptr) {
    if (dev_ptr == nullptr) return HIRA_OK;
    cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    if (e != cudaSuccess) {
        hira::set_error("hira_peer_close: %s", cudaGetErrorString(e));
        return HIRA_ERR_CUDA;
    }
    return HIRA_OK;
}

extern "C" int hira_peer_free(void* dev_ptr) {
    if (dev_ptr == nullptr) return HIRA_OK;
    cudaError_t e = cudaFree(dev_ptr);
    if (e != cudaSuccess) {
        hira::set_error("hira_peer_free: %s", cudaGetErrorString(e));
        return HIRA_ERR_CUDA;
    }
    return HIRA_OK;
}

extern "C" int hira_exchange_merge(const float* local_rows, void* const* peer_bufs, int32_t world, int32_t rank,
                                   int32_t n_qheads, int32_t vdim, uint32_t seq, int32_t phases, float wait_seconds,
                                   float* out, float* out_ml, int32_t* status, void* stream) {
    HIRA_CHECK_ARG(local_rows && peer_bufs && out && status, HIRA_ERR_ARG, "hira_exchange_merge: NULL argument");
    HIRA_CHECK_ARG(world >= 1 && world <= HIRA_MAX_PEERS && rank >= 0 && rank < world, HIRA_ERR_SHAPE,
                   "hira_exchange_merge: world=%d (at most %d) rank=%d", world, HIRA_MAX_PEERS, rank);
    HIRA_CHECK_ARG(n_qheads >= 1 && vdim >= 1, HIRA_ERR_SHAPE, "hira_exchange_merge: n_qheads=%d vdim=%d", n_qheads, vdim);
    HIRA_CHECK_ARG(seq != 0 && (phases & 3) != 0 && (phases & ~3) == 0, HIRA_ERR_ARG,
                   "hira_exchange_merge: seq must be non-zero (buffers start zeroed), phases in 1..3 (got %d)", phases);
    hira::PeerBufs pb;
    for (int i = 0; i < HIRA_MAX_PEERS; ++i) pb.p[i] = nullptr;
    for (int i = 0; i < world; ++i) {
        HIRA_CHECK_ARG(peer_bufs[i] != nullptr, HIRA_ERR_ARG, "hira_exchange_merge: peer buffer %d is NULL", i);
        pb.p[i] = reinterpret_cast<float*>(peer_bufs[i]);
    }
    // SM clock of the current device, asked for once (the query is slow): turns the bound into cycles
    static std::atomic<int> g_khz[64];
    int dev = 0;
    cudaGetDevice(&dev);
    int khz = (dev >= 0 && dev < 64) ? g_khz[dev].load(std::memory_order_relaxed) : 0;
    if (khz == 0) {
        cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev);
        if (khz <= 0) khz = 1500000;
        if (dev >= 0 && dev < 64) g_khz[dev].store(khz, std::memory_order_relaxed);
    }
    if (!(wait_seconds > 0.f)) wait_seconds = 2.0f;
    const unsigned long long cycles = (unsigned long long)((double)wait_seconds * khz * 1e3);
    hira::exchange_merge_kernel<<<n_qheads, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        local_rows, pb, world, rank, n_qheads, vdim, seq, phases, cycles, out, out_ml, status);
    HIRA_CHECK_LAUNCH("hira_exchange_merge launch");
    return HIRA_OK;
}
