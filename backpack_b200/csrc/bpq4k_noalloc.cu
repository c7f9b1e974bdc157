// bpq4k_matmul_noalloc_f32: the small-M Q4_K matmul for callers that must not allocate.
//
// Who cannot allocate: a serving process that has already handed all free device memory to
// its own pool (a cudaMalloc from a library would fail, or punch a hole into the pool's
// budget), and any path where the device-wide synchronisation hidden inside
// cudaMalloc/cudaFree is not acceptable -- a decode loop with other streams in flight.  Such
// callers also cannot create a bpq4k handle, because bpq4k_create allocates a status word
// and a scratch slab.  This entry point therefore takes no handle.
//
// It runs the same two kernels as bpq4k_matmul_f32 on its scratch path (the activations are
// quantised to base-128 digits in global memory by one kernel, the streaming kernel reads them
// from there), with the scratch placed in the fixed-size __device__ array below instead of
// allocated memory.  Every device that loads this library carries the array until the
// process exits.
//
// Rules that follow from the shared, fixed scratch:
//   * M <= 8 and R * K <= kNoAllocMaxMK, where R = 1 for M = 1 and M rounded up to a multiple of 4
//     otherwise; else BPQ4K_ERR_UNSUPPORTED.
//   * The array keeps the previous call's contents.  Nothing in it has to start at zero for
//     the next call: the quantising kernel rewrites the zero region, the digits and the
//     per-sub-block sums of every activation row it is given, and rows beyond M are written as
//     zeros, before the streaming kernel (ordered behind it on the same stream) reads them.
//   * All calls on a device share the one array.  Calls that may overlap on the GPU -- issued
//     on different streams without an ordering between them, or from different threads --
//     race on it; serialise them.
//   * The first call on each device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and configures the kernels.  Make that
//     first call before any stream capture begins.
#include <cstdio>
#include <mutex>

#include "../../include/bpq4k.h"
#include "kernels.h"

namespace {

constexpr uint32_t kNoAllocMaxMK = BPQ4K_NOALLOC_MAX_MK;
// zero region + digits (4 B per activation) + two floats per 32 activations + slack
constexpr size_t kScratchBytes = 1024 + (size_t)kNoAllocMaxMK * 4 + (size_t)kNoAllocMaxMK / 32 * 8 + 256;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {};  // device address of g_noalloc_scratch, per device
int g_sm_count[kMaxDevices] = {};

thread_local char g_error[256] = "no error";

int fail(int status, const char* msg) {
    snprintf(g_error, sizeof(g_error), "%s", msg);
    return status;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

const char* bpq4k_noalloc_last_error(void) { return g_error; }

int bpq4k_matmul_noalloc_f32(const float* X, const void* W, const float* bias, float* Y, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t rowStrideWords, uint32_t yOffset, void* stream) {
    if (M == 0 || N == 0) return BPQ4K_OK;
    if (!X || !W || !Y) return fail(BPQ4K_ERR_INVALID_ARG, "X, W or Y is null");
    if (K == 0 || K % BPQ4K_QK_K != 0) return fail(BPQ4K_ERR_UNSUPPORTED, "K is not a positive multiple of 256");
    if (rowStrideWords < (K / BPQ4K_QK_K) * BPQ4K_BLOCK_WORDS) return fail(BPQ4K_ERR_INVALID_ARG, "rowStrideWords is smaller than a row");
    if (rowStrideWords % 4u) return fail(BPQ4K_ERR_MISALIGNED, "rowStrideWords is not a multiple of 4 words");
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (reinterpret_cast<uintptr_t>(W) & 15u))
        return fail(BPQ4K_ERR_MISALIGNED, "X or W is not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 3u) return fail(BPQ4K_ERR_MISALIGNED, "Y is not 4-byte aligned");
    const uint64_t rows_padded = M <= 1 ? 1 : (uint64_t)(M + 3) / 4 * 4;  // the kernel works on 4-row slots
    if (M > 8 || rows_padded * K > kNoAllocMaxMK) {
        snprintf(g_error, sizeof(g_error),
                 "M=%u, K=%u is beyond the fixed scratch: need M <= 8 and (M rounded up to a multiple of 4, or 1)*K <= %u", M, K,
                 kNoAllocMaxMK);
        return BPQ4K_ERR_UNSUPPORTED;
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(BPQ4K_ERR_NO_DEVICE, "no current CUDA device");
    void* scratch = nullptr;
    int sms = 0;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_scratch_ptr[dev]) {
            // once per device, with that device current: the array's name is only a host-side stand-in,
            // the kernels need its address on THIS device
            int major = 0;
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (major != 10) return fail(BPQ4K_ERR_NO_DEVICE, "the current device is not compute capability 10.x");
            void* p = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p) {
                cudaGetLastError();
                snprintf(g_error, sizeof(g_error), "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
                return BPQ4K_ERR_CUDA;
            }
            cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
            g_scratch_ptr[dev] = p;
        }
        scratch = g_scratch_ptr[dev];
        sms = g_sm_count[dev];
    }
    bpq4k::MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = Y + yOffset;
    a.M = M;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    bpq4k::StreamTuning tune;
    tune.force_scratch = 1;  // activations go through the (static) global scratch
    const cudaError_t e = bpq4k::launch_gemv_stream(a, tune, scratch, kScratchBytes, /*status*/ nullptr, sms,
                                                    /*tensor-map cache*/ nullptr, static_cast<cudaStream_t>(stream), nullptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        snprintf(g_error, sizeof(g_error), "launch failed: %s", cudaGetErrorString(e));
        return BPQ4K_ERR_CUDA;
    }
    return BPQ4K_OK;
}

}  // extern "C"
#pragma GCC visibility pop
