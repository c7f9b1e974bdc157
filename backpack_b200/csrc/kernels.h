// Internal launch interface between the C ABI (bpq4k_capi.cu) and the kernel
// translation units.  Every function enqueues on `stream` and returns the
// cudaError_t of the launch; none of them allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bpq4k {

// One matmul problem as the kernels see it.  Rows of W are `w_row_bytes`
// apart.  For the indirect (expert) form `offsets`/`x_rows` are non-null and
// `n_slots` problems of M = 1 are solved by one launch.
struct MatmulArgs {
    const float* X;
    const uint8_t* W;
    const float* bias;   // may be null
    float* Y;            // already advanced by yOffset
    uint32_t M, N, K;
    uint64_t w_row_bytes;
    const uint32_t* offsets;  // null for the direct form
    const uint32_t* x_rows;   // null: slot s reads row s
    uint32_t n_slots;         // 0 for the direct form
};

cudaError_t launch_dequant_f32(const uint8_t* W, uint32_t N, uint32_t K, uint64_t w_row_bytes, float* out,
                               cudaStream_t stream);

// One warp per output row, float FMAs in the reference shader's arithmetic.
cudaError_t launch_gemv_fp32(const MatmulArgs& a, cudaStream_t stream, int* launches);

}  // namespace bpq4k
