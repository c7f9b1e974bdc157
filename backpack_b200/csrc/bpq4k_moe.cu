// The last step of a routed-expert feed-forward layer: every token's output row gains the weighted sum
// of its slots' expert outputs.  The reference runs one dispatch per slot
// (runtime/kernels/moe/weighted_accumulate_decode.wgsl, out[c] = out[c] + weights[k] * src[c]; issued from
// runtime/model_runner.cpp:3643-3651); one launch here walks the slots of a token in the same ascending
// order, so the float sums are formed in the reference's order.
#include "kernels.h"

namespace bpq4k {

namespace {

__global__ void __launch_bounds__(256) moe_accumulate_kernel(float* __restrict__ Y, const float* __restrict__ O,
                                                             const float* __restrict__ route_w, uint32_t T, uint32_t topk,
                                                             uint32_t N) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");  // O comes from the kernel before this one
    const uint32_t nv = N / 4u;                          // N is a multiple of 4 (checked by the caller)
    const uint64_t total = (uint64_t)T * nv;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / nv), c = (uint32_t)(i - (uint64_t)t * nv);
        float4 acc = reinterpret_cast<const float4*>(Y + (uint64_t)t * N)[c];
        for (uint32_t k = 0; k < topk; k++) {
            const float w = __ldg(route_w + (uint64_t)t * topk + k);
            const float4 o = __ldg(reinterpret_cast<const float4*>(O + ((uint64_t)t * topk + k) * N) + c);
            acc.x = acc.x + w * o.x;
            acc.y = acc.y + w * o.y;
            acc.z = acc.z + w * o.z;
            acc.w = acc.w + w * o.w;
        }
        reinterpret_cast<float4*>(Y + (uint64_t)t * N)[c] = acc;
    }
}

}  // namespace

cudaError_t launch_moe_accumulate(float* Y, const float* O, const float* route_w, uint32_t T, uint32_t topk, uint32_t N,
                                  int sm_count, cudaStream_t stream) {
    if (T == 0 || N == 0 || topk == 0) return cudaSuccess;
    const uint64_t total = (uint64_t)T * (N / 4u);
    uint64_t blocks = (total + 255) / 256;
    if (blocks > (uint64_t)sm_count * 8) blocks = (uint64_t)sm_count * 8;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, moe_accumulate_kernel, Y, O, route_w, T, topk, N);
}

}  // namespace bpq4k
