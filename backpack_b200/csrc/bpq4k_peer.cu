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
    // Programmatic dependent launch on both sides: this kernel becomes resident while the matmul before it
    // still runs, and the kernel after it may start its own prologue (weight prefetch) at once.  Nothing
    // below the wait runs before the preceding kernel has completed, so all its stores to peer memory are
    // ordered before the flag.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // epoch 0 = "next": the count lives in word 63 of this GPU's own flag array, so a barrier
    // replayed from a CUDA graph advances by itself (every rank replays the same barriers)
    uint32_t epoch = a.epoch;
    if (epoch == 0) {
        if (p == 0) epoch = a.flags[a.rank][63] + 1u;
        epoch = __shfl_sync(0xFFFFFFFFu, epoch, 0);
    }
    if (p < a.n_peers) {
        // release: everything this GPU stored to peer memory earlier in the stream is ordered before the flag
        uint32_t* remote = a.flags[p] + a.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
        // acquire-poll peer p's flag in this GPU's own array; flags only grow, so >= tolerates a fast peer
        const uint32_t* mine = a.flags[a.rank] + p;
        const long long t0 = clock64();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - epoch) >= 0) break;
            if ((uint64_t)(clock64() - t0) > a.timeout_cycles) {   // give up: report it, never hang
                if (a.status) atomicExch(a.status, kDeviceTimeout);
                break;
            }
        }
    }
    // the step count advances once every peer's flag has been seen (kernels of the next step read it to
    // pick their half of the double-buffered gather slots)
    __syncwarp();
    if (p == 0 && a.epoch == 0) a.flags[a.rank][63] = epoch;
}

}  // namespace

cudaError_t launch_peer_barrier(uint32_t* const* flag_ptrs_host, uint32_t n_peers, uint32_t rank, uint32_t epoch,
                                uint64_t timeout_cycles, int* status_dev, cudaStream_t stream, bool pdl) {
    if (n_peers == 0 || n_peers > 8 || rank >= n_peers) return cudaErrorInvalidValue;
    BarrierArgs a{};
    for (uint32_t p = 0; p < n_peers; p++) a.flags[p] = flag_ptrs_host[p];
    a.n_peers = n_peers;
    a.rank = rank;
    a.epoch = epoch;
    a.timeout_cycles = timeout_cycles;
    a.status = status_dev;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, peer_barrier_kernel, a);
}

}  // namespace bpq4k
