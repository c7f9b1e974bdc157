// Several host <-> device segment copies in ONE launch, for host buffers the GPU can address
// (pinned / registered memory).  Used by the host-buffer batch entry point in place of one
// asynchronous copy per activation vector and per output vector: the copies of a decode step are
// many and small (16 KB in, up to 513 KB out), so their number costs more than their bytes.
#include "kernels.h"

namespace bpq4k {

namespace {

__global__ void __launch_bounds__(256) copy_segments_kernel(const __grid_constant__ CopySegments segs) {
    // a streaming matmul launched behind this kernel may start prefetching its weights now; it reads
    // the gathered activations only after this grid has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t s = blockIdx.y;
    if (s >= segs.count) return;
    const uint4* __restrict__ src = static_cast<const uint4*>(segs.src[s]);
    uint4* __restrict__ dst = static_cast<uint4*>(segs.dst[s]);
    const uint32_t n16 = segs.bytes[s] / 16u;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += gridDim.x * blockDim.x) dst[i] = src[i];
    // tail (sizes are multiples of 4 bytes)
    const uint32_t done = n16 * 16u, rest = (segs.bytes[s] - done) / 4u;
    if (blockIdx.x == 0 && threadIdx.x < rest)
        reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(dst) + done)[threadIdx.x] =
            reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(src) + done)[threadIdx.x];
}

}  // namespace

cudaError_t launch_copy_segments(const CopySegments& segs, cudaStream_t stream) {
    if (segs.count == 0) return cudaSuccess;
    uint32_t max_bytes = 0;
    for (uint32_t i = 0; i < segs.count; i++) max_bytes = segs.bytes[i] > max_bytes ? segs.bytes[i] : max_bytes;
    uint32_t gx = (max_bytes / 16u + 1023u) / 1024u;  // four 16-byte words per thread
    if (gx == 0) gx = 1;
    if (gx > 64) gx = 64;
    copy_segments_kernel<<<dim3(gx, segs.count), 256, 0, stream>>>(segs);
    return cudaGetLastError();
}

}  // namespace bpq4k
