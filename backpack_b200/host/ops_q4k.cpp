// The Q4_K operators, registered the way the reference registers its ONNX ops
// (REGISTER_OP at the end of runtime/ops/matmul.cpp:582-585).  The reference has no
// ONNX op for Q4_K -- its Q4_K kernels are driven by ModelRunner -- so the op carries
// a custom name and follows MatMulNBits' conventions (runtime/ops/matmul.cpp:205-335):
// attributes K and N, M = product of the leading dims of X, the op allocates its output,
// and on bad input it returns early leaving the output invalid.
//
//   MatMulQ4K   inputs  X float32[..., K], W uint8[N, K/256*144] (raw GGUF super-blocks),
//                       optional Bias float32[N];  attrs K, N;  output Y float32[..., N]
//   DequantQ4K  input   W uint8[N, K/256*144];  attrs K, N;  output float32[N, K]
//               (dequant_kquant, runtime/gguf_loader.cpp:455-496)
#include <cstdio>

#include <cuda_runtime.h>

#include "bp_runtime.h"

static bool weight_ok(const GpuTensor* W, uint32_t N, uint32_t K) {
    return W && W->IsValid() && W->dtype == TensorDtype::UInt8 && K % 256 == 0 &&
           (uint64_t)W->ElementCount() >= (uint64_t)N * (K / 256) * 144;
}

static void opMatMulQ4K(OpContext& ex, const OnnxGraphNode& n, const std::vector<GpuTensor*>& in,
                        std::vector<GpuTensor*>& out) {
    if (in.size() < 2 || out.empty()) return;
    GpuTensor* X = in[0];
    GpuTensor* W = in[1];
    GpuTensor* B = in.size() > 2 && in[2] && in[2]->IsValid() ? in[2] : nullptr;
    if (!X || !X->IsValid() || X->dtype != TensorDtype::Float32 || X->shape.empty()) return;
    const uint32_t N = (uint32_t)n.GetInt("N"), K = (uint32_t)n.GetInt("K");
    if (!N || !K || X->shape.back() != (int64_t)K || !weight_ok(W, N, K)) {
        fprintf(stderr, "[MatMulQ4K] %s: bad shapes (N=%u K=%u)\n", n.name.c_str(), N, K);
        return;
    }
    if (B && (B->dtype != TensorDtype::Float32 || B->ElementCount() < (int64_t)N)) return;
    ex.EnsureGpu(*X);
    ex.EnsureGpu(*W);
    if (B) ex.EnsureGpu(*B);
    int64_t M = 1;
    for (size_t i = 0; i + 1 < X->shape.size(); i++) M *= X->shape[i];
    auto outShape = X->shape;
    outShape.back() = N;
    GpuTensor y = ex.AllocTensor(outShape, TensorDtype::Float32);
    if (!y.buffer.handle) return;
    GPUContext* gpu = ex.getGpu();
    const int st = bpq4k_matmul_f32(gpu->q4k(), static_cast<const float*>(X->buffer.handle), W->buffer.handle,
                                    B ? static_cast<const float*>(B->buffer.handle) : nullptr,
                                    static_cast<float*>(y.buffer.handle), (uint32_t)M, N, K,
                                    bpq4k_row_stride_words(K), 0, gpu->stream());
    if (st != BPQ4K_OK) {
        fprintf(stderr, "[MatMulQ4K] %s: %s\n", n.name.c_str(), bpq4k_last_error_string(gpu->q4k()));
        gpu->releaseBuffer(y.buffer);
        return;  // output stays invalid
    }
    *out[0] = std::move(y);
}

static void opDequantQ4K(OpContext& ex, const OnnxGraphNode& n, const std::vector<GpuTensor*>& in,
                         std::vector<GpuTensor*>& out) {
    if (in.empty() || out.empty()) return;
    GpuTensor* W = in[0];
    const uint32_t N = (uint32_t)n.GetInt("N"), K = (uint32_t)n.GetInt("K");
    if (!N || !K || !weight_ok(W, N, K)) return;
    ex.EnsureGpu(*W);
    GpuTensor y = ex.AllocTensor({(int64_t)N, (int64_t)K}, TensorDtype::Float32);
    if (!y.buffer.handle) return;
    GPUContext* gpu = ex.getGpu();
    const int st = bpq4k_dequant_f32(gpu->q4k(), W->buffer.handle, N, K, bpq4k_row_stride_words(K),
                                     static_cast<float*>(y.buffer.handle), gpu->stream());
    if (st != BPQ4K_OK) {
        fprintf(stderr, "[DequantQ4K] %s: %s\n", n.name.c_str(), bpq4k_last_error_string(gpu->q4k()));
        gpu->releaseBuffer(y.buffer);
        return;
    }
    *out[0] = std::move(y);
}

// ---- Q5_K / Q6_K: the same op contract with W in the file format of its type -----------------------
//   MatMulQ5K   W uint8[N, K/256*176]      MatMulQ6K   W uint8[N, K/256*210]
// Q6_K blocks are re-spaced on the device into the padded layout of the streaming kernel on every
// call (a model runner would do that once, at load time, with bpq4k_kq_pack_host or
// bpq4k_gguf_upload_tensor).
template <int QTYPE>
static void opMatMulKQ(OpContext& ex, const OnnxGraphNode& n, const std::vector<GpuTensor*>& in, std::vector<GpuTensor*>& out) {
    const char* opname = QTYPE == BPQ4K_TYPE_Q5_K ? "MatMulQ5K" : "MatMulQ6K";
    if (in.size() < 2 || out.empty()) return;
    GpuTensor* X = in[0];
    GpuTensor* W = in[1];
    GpuTensor* B = in.size() > 2 && in[2] && in[2]->IsValid() ? in[2] : nullptr;
    if (!X || !X->IsValid() || X->dtype != TensorDtype::Float32 || X->shape.empty()) return;
    const uint32_t N = (uint32_t)n.GetInt("N"), K = (uint32_t)n.GetInt("K");
    const uint32_t bb = bpq4k_kq_block_bytes(QTYPE);
    if (!N || !K || K % 256 || X->shape.back() != (int64_t)K || !W || !W->IsValid() || W->dtype != TensorDtype::UInt8 ||
        (uint64_t)W->ElementCount() < (uint64_t)N * (K / 256) * bb) {
        fprintf(stderr, "[%s] %s: bad shapes (N=%u K=%u)\n", opname, n.name.c_str(), N, K);
        return;
    }
    if (B && (B->dtype != TensorDtype::Float32 || B->ElementCount() < (int64_t)N)) return;
    ex.EnsureGpu(*X);
    ex.EnsureGpu(*W);
    if (B) ex.EnsureGpu(*B);
    int64_t M = 1;
    for (size_t i = 0; i + 1 < X->shape.size(); i++) M *= X->shape[i];
    auto outShape = X->shape;
    outShape.back() = N;
    GpuTensor y = ex.AllocTensor(outShape, TensorDtype::Float32);
    if (!y.buffer.handle) return;
    GPUContext* gpu = ex.getGpu();
    int layout = QTYPE;
    const void* wdev = W->buffer.handle;
    GPUBuffer padded{};
    if (QTYPE == BPQ4K_TYPE_Q6_K) {
        layout = BPQ4K_TYPE_Q6_K_PADDED;
        padded = gpu->createBuffer("q6k_padded", (uint64_t)N * bpq4k_kq_row_stride_words(layout, K) * 4u);
        if (!padded.handle || bpq4k_kq_respace_device(gpu->q4k(), layout, W->buffer.handle, N, K, padded.handle, gpu->stream()) != BPQ4K_OK) {
            fprintf(stderr, "[%s] %s: cannot re-space the weights\n", opname, n.name.c_str());
            if (padded.handle) gpu->releaseBuffer(padded);
            gpu->releaseBuffer(y.buffer);
            return;
        }
        wdev = padded.handle;
    }
    const int st = bpq4k_kq_matmul_f32(gpu->q4k(), layout, static_cast<const float*>(X->buffer.handle), wdev,
                                       B ? static_cast<const float*>(B->buffer.handle) : nullptr,
                                       static_cast<float*>(y.buffer.handle), (uint32_t)M, N, K,
                                       bpq4k_kq_row_stride_words(layout, K), 0, gpu->stream());
    if (padded.handle) {
        cudaStreamSynchronize(static_cast<cudaStream_t>(gpu->stream()));  // the kernel reads the temporary
        gpu->releaseBuffer(padded);
    }
    if (st != BPQ4K_OK) {
        fprintf(stderr, "[%s] %s: %s\n", opname, n.name.c_str(), bpq4k_last_error_string(gpu->q4k()));
        gpu->releaseBuffer(y.buffer);
        return;  // output stays invalid
    }
    *out[0] = std::move(y);
}

static void opMatMulQ5K(OpContext& ex, const OnnxGraphNode& n, const std::vector<GpuTensor*>& in, std::vector<GpuTensor*>& out) {
    opMatMulKQ<BPQ4K_TYPE_Q5_K>(ex, n, in, out);
}
static void opMatMulQ6K(OpContext& ex, const OnnxGraphNode& n, const std::vector<GpuTensor*>& in, std::vector<GpuTensor*>& out) {
    opMatMulKQ<BPQ4K_TYPE_Q6_K>(ex, n, in, out);
}

REGISTER_OP(MatMulQ4K, opMatMulQ4K)
REGISTER_OP(DequantQ4K, opDequantQ4K)
REGISTER_OP(MatMulQ5K, opMatMulQ5K)
REGISTER_OP(MatMulQ6K, opMatMulQ6K)
