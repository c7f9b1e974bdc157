// Greedy sampling step after the output head: index of the largest logit, in one launch.
//
// Replaces the reference's two dispatches argmax + argmax_reduce (runtime/kernels/shape/argmax.wgsl,
// argmax_reduce.wgsl; runtime/model_runner.cpp:2246, 2441-2452).  Same answer wherever the maximum is
// unique: strict comparison against a start value of -1e30 (so values <= -1e30 and NaNs never win, and
// the result is 0 when nothing does).  Where the reference's answer on ties depends on its scan order,
// this kernel returns the lowest index.
//
// Each thread scans a strided part, warps and the block reduce a packed 64-bit key
// (order-preserving bits of the value << 32 | ~index), blocks combine with one atomicMax; the last
// block to finish writes the result and clears the two scratch words for the next call.
#include "kernels.h"

namespace bpq4k {

namespace {

__device__ __forceinline__ unsigned long long pack_key(float v, uint32_t idx) {
    if (!(v > -1e30f)) return 0ull;  // also false for NaN
    const uint32_t b = __float_as_uint(v);
    const uint32_t key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}

__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, uint32_t n, int32_t* __restrict__ result,
                                                      unsigned long long* __restrict__ best, uint32_t* __restrict__ arrived) {
    unsigned long long k = 0ull;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const unsigned long long c = pack_key(__ldg(logits + i), i);
        k = c > k ? c : k;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long c = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        k = c > k ? c : k;
    }
    __shared__ unsigned long long wbest[8];
    __shared__ uint32_t last;
    if ((threadIdx.x & 31u) == 0) wbest[threadIdx.x >> 5] = k;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) k = wbest[w] > k ? wbest[w] : k;
        if (k) atomicMax(best, k);
        __threadfence();
        last = atomicAdd(arrived, 1u) == gridDim.x - 1u;
        if (last) {
            __threadfence();
            const unsigned long long b = atomicExch(best, 0ull);  // read and clear for the next call
            *result = b ? (int32_t)(0xFFFFFFFFu - (uint32_t)(b & 0xFFFFFFFFull)) : 0;
            *arrived = 0u;
        }
    }
}

}  // namespace

// `scratch` : 16 zeroed bytes owned by the caller (8-byte aligned); the kernel leaves them zeroed.
cudaError_t launch_argmax(const float* logits, uint32_t n, int32_t* result, void* scratch, int sm_count, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    uint32_t grid = (n + 1023u) / 1024u;
    if (grid > (uint32_t)sm_count * 2u) grid = (uint32_t)sm_count * 2u;
    auto* best = static_cast<unsigned long long*>(scratch);
    argmax_kernel<<<grid, 256, 0, stream>>>(logits, n, result, best, reinterpret_cast<uint32_t*>(best + 1));
    return cudaGetLastError();
}

}  // namespace bpq4k
