// Multi-GPU glue for the N-sharded matmul (one process per GPU): a bounded flag barrier over
// peer-mapped memory.  The data path itself is in the streaming kernel, whose epilogue stores
// each output value into every peer's gather buffer with plain stores over NVLink -- no
// multimem, no TMA, no loads from peer memory.
#include "kernels.h"

namespace bpq4k {

namespace {

struct BarrierArgs {
    uint32_t* flags[8];  // flags[p]: peer p's flag array (flags[rank] is this GPU's own array)
    uint32_t n_peers, rank, epoch;
    uint64_t timeout_cycles;
    int* status;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const __grid_constant__ BarrierArgs a) {
    const uint32_t p = threadIdx.x;
    // epoch 0 = "next": the count lives in word 63 of this GPU's own flag array, so a barrier
    // replayed from a CUDA graph advances by itself (every rank replays the same barriers)
    uint32_t epoch = a.epoch;
    if (epoch == 0) {
        if (p == 0) {
            epoch = a.flags[a.rank][63] + 1u;
            a.flags[a.rank][63] = epoch;
        }
        epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);
    }
    if (p >= a.n_peers) return;
    // everything this GPU stored to peer memory earlier in the stream is ordered before the flag
    __threadfence_system();
    volatile uint32_t* remote = a.flags[p] + a.rank;
    *remote = epoch;
    __threadfence_system();
    // wait for peer p's flag in this GPU's own array; flags only grow, so >= tolerates a fast peer
    volatile uint32_t* mine = a.flags[a.rank] + p;
    const long long t0 = clock64();
    while ((int32_t)(*mine - epoch) < 0) {
        if ((uint64_t)(clock64() - t0) > a.timeout_cycles) {
            if (a.status) atomicExch(a.status, kDeviceTimeout);
            return;
        }
        __nanosleep(200);
    }
    __threadfence_system();
}

}  // namespace

cudaError_t launch_peer_barrier(uint32_t* const* flag_ptrs_host, uint32_t n_peers, uint32_t rank, uint32_t epoch,
                                uint64_t timeout_cycles, int* status_dev, cudaStream_t stream) {
    if (n_peers == 0 || n_peers > 8 || rank >= n_peers) return cudaErrorInvalidValue;
    BarrierArgs a{};
    for (uint32_t p = 0; p < n_peers; p++) a.flags[p] = flag_ptrs_host[p];
    a.n_peers = n_peers;
    a.rank = rank;
    a.epoch = epoch;
    a.timeout_cycles = timeout_cycles;
    a.status = status_dev;
    peer_barrier_kernel<<<1, 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace bpq4k
