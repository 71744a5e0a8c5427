// Peer memory for the column-sharded multi-GPU decode: one process per GPU, each allocates one
// region of device memory (activation buffers and arrival words at the same offsets on every
// rank), exports it as a CUDA IPC handle and maps the other ranks' regions.  The matmul kernels
// then store into the peers' regions directly (mm8_cluster.cuh, Exchange).  No multicast, no
// collective library on the data path.
#include "common.cuh"

namespace {

constexpr unsigned kWaitSpinLimit = 1u << 21;

// One warp: lane r waits (bounded) until arrival word r has reached `seq`.
__global__ void peer_wait_kernel(const unsigned* arrived, int world, unsigned seq, const unsigned* seq_base, unsigned* error) {
    const int r = threadIdx.x;
    if (r < world) {
        if (seq_base != nullptr) seq += __ldcg(seq_base);
        unsigned it = 0;
        while (true) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(arrived + r) : "memory");
            if (int(v - seq) >= 0) break;
            if (++it >= kWaitSpinLimit) { atomicExch(error, 1u); break; }
            __nanosleep(64);
        }
    }
}

__global__ void peer_advance_kernel(unsigned* seq_base, unsigned add) { *seq_base += add; }

}  // namespace

extern "C" int rwkv_peer_alloc(size_t bytes, void** ptr_out) {
    RWKV_CHECK_ARG(bytes > 0 && ptr_out != nullptr);
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaGetLastError(); cudaFree(p); return RWKV_ERR_LAUNCH; }
    *ptr_out = p;
    return RWKV_OK;
}

extern "C" int rwkv_peer_free(void* ptr) {
    if (ptr != nullptr && cudaFree(ptr) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}

// handle_out: RWKV_PEER_HANDLE_BYTES (64) bytes that another process passes to rwkv_peer_open.
extern "C" int rwkv_peer_export(const void* ptr, void* handle_out) {
    RWKV_CHECK_ARG(ptr != nullptr && handle_out != nullptr);
    static_assert(sizeof(cudaIpcMemHandle_t) == RWKV_PEER_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    memcpy(handle_out, &h, sizeof(h));
    return RWKV_OK;
}

extern "C" int rwkv_peer_open(const void* handle, void** ptr_out) {
    RWKV_CHECK_ARG(handle != nullptr && ptr_out != nullptr);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    *ptr_out = p;
    return RWKV_OK;
}

extern "C" int rwkv_peer_close(void* ptr) {
    if (ptr != nullptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) { cudaGetLastError(); return RWKV_ERR_LAUNCH; }
    return RWKV_OK;
}

// Enqueue a wait (bounded; sets *error on giving up) until every rank's arrival word has reached
// seq (+ *seq_base when given).
extern "C" int rwkv_peer_wait(const uint32_t* arrived, int world, uint32_t seq, const uint32_t* seq_base, uint32_t* error,
                              void* stream) {
    RWKV_CHECK_ARG(arrived != nullptr && error != nullptr && world >= 1 && world <= 32);
    peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(arrived, world, seq, seq_base, error);
    return rwkv_launch_status();
}

// *seq_base += add, in stream order (one per token of a replayed graph).
extern "C" int rwkv_peer_advance(uint32_t* seq_base, uint32_t add, void* stream) {
    RWKV_CHECK_ARG(seq_base != nullptr);
    peer_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(seq_base, add);
    return rwkv_launch_status();
}
