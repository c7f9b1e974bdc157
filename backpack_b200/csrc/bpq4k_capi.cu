// C ABI of libbpq4k.so (declared in include/bpq4k.h): handle, argument
// validation, kernel selection.  No kernel code lives here.
#include "../../include/bpq4k.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "kernels.h"

using namespace bpq4k;

struct bpq4k_context {
    int device = 0;
    int sm_count = 0;
    int cc_major = 0;
    int clock_khz = 0;  // SM clock for cycle-counted time-outs; queried once (the query takes about a millisecond)
    char err[512] = "no error";
    int gemv_variant = BPQ4K_GEMV_AUTO;
    int prefill_mode = BPQ4K_PREFILL_F16X3;
    int prefill_variant = 0;  // BPQ4K_OPT_PREFILL_VARIANT
    int prefill_arg() const { return prefill_mode | (prefill_variant << 4); }  // what the launcher takes
    int prefill_min_m = 25;  // four 8-row slabs of the streaming kernel cost as much as one tensor-core pass
    uint64_t launches = 0;
    // staging for the *_host entry point
    float* stage_x = nullptr;
    size_t stage_x_bytes = 0;
    float* stage_y = nullptr;
    size_t stage_y_bytes = 0;
    // scratch for kernels that need it (split activations)
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // device status word written by kernels whose bounded waits run out
    int* dev_status = nullptr;
    StreamTuning tune;
    TmapCache tmaps;
    // the host-buffer batch call replays its dispatch list from a CUDA graph once it has seen the
    // same list twice (the reference records its decode dispatch list once and replays it too)
    uint64_t batch_key = 0;
    uint32_t batch_seen = 0;
    uint64_t batch_launches = 0;
    cudaGraphExec_t batch_exec = nullptr;
    cudaStream_t batch_stream = nullptr;
    cudaEvent_t batch_event = nullptr;
    // double-buffered gather slots of the fused all-gather (bpq4k_peer_double_buffer)
    const uint32_t* peer_parity = nullptr;
    uint64_t peer_parity_stride = 0;
    uint32_t stamp_next = 0;     // launches stamped so far (BPQ4K_OPT_STREAM_STAMPS); tune.stamp_next points here
    uint32_t batch_records = 0;  // how many times a list was captured into a graph (BPQ4K_OPT_BATCH_RECORDS)
    // device blocks that were outgrown; freed at destroy (see ensure_bytes)
    static constexpr uint32_t kMaxRetired = 48;
    void* retired[kMaxRetired] = {};
    uint32_t n_retired = 0;
};

namespace {

int fail(bpq4k_context* h, int status, const char* fmt, ...) {
    if (h) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(h->err, sizeof(h->err), fmt, ap);
        va_end(ap);
    }
    return status;
}

int cuda_fail(bpq4k_context* h, cudaError_t e, const char* what) {
    return fail(h, BPQ4K_ERR_CUDA, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Shape and layout checks shared by every matmul-like entry point.
int check_weights(bpq4k_context* h, const void* W, uint32_t N, uint32_t K, uint32_t rowStrideWords) {
    (void)N;
    if (K == 0 || K % BPQ4K_QK_K != 0)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "K=%u is not a positive multiple of 256", K);
    if (!W) return fail(h, BPQ4K_ERR_INVALID_ARG, "W is null");
    const uint32_t need = (K / BPQ4K_QK_K) * BPQ4K_BLOCK_WORDS;
    if (rowStrideWords < need)
        return fail(h, BPQ4K_ERR_INVALID_ARG, "rowStrideWords=%u is smaller than (K/256)*36=%u", rowStrideWords, need);
    if (rowStrideWords % 4u != 0)
        return fail(h, BPQ4K_ERR_MISALIGNED, "rowStrideWords=%u is not a multiple of 4 words (16 bytes)", rowStrideWords);
    if (!aligned16(W)) return fail(h, BPQ4K_ERR_MISALIGNED, "W is not 16-byte aligned");
    return BPQ4K_OK;
}

// Forget the recorded dispatch list of the host-batch call (its graph holds raw buffer addresses).
void drop_batch_graph(bpq4k_context* h) {
    if (h->batch_exec) cudaGraphExecDestroy(h->batch_exec);
    h->batch_exec = nullptr;
    h->batch_key = 0;
    h->batch_seen = 0;
}

// Grow one of the handle's device buffers.  The old block is NOT freed here: a CUDA graph (the
// handle's own replay graph of the host-batch call, or one the caller captured around a matmul
// that uses the scratch) may still hold its address, and a replay would then touch freed memory.
// Old blocks are retired and freed at bpq4k_destroy; sizes at least double, so the retired blocks
// together stay below the live one.  The handle's own replay graph is dropped and re-recorded.
int ensure_bytes(bpq4k_context* h, void** p, size_t* have, size_t need) {
    if (*have >= need) return BPQ4K_OK;
    size_t want = need < (1u << 20) ? (1u << 20) : need;
    if (want < 2 * *have) want = 2 * *have;
    void* fresh = nullptr;
    cudaError_t e = cudaMalloc(&fresh, want);
    if (e != cudaSuccess && want > need) {
        cudaGetLastError();
        want = need;
        e = cudaMalloc(&fresh, want);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, BPQ4K_ERR_ALLOC, "cudaMalloc(%zu) failed: %s", want, cudaGetErrorString(e));
    }
    if (*p) {
        if (h->n_retired < bpq4k_context::kMaxRetired) {
            h->retired[h->n_retired++] = *p;
        } else {
            // cannot happen with doubling sizes (48 doublings exceed any device); wait for all work, then free
            cudaDeviceSynchronize();
            cudaFree(*p);
        }
    }
    *p = fresh;
    *have = want;
    drop_batch_graph(h);
    return BPQ4K_OK;
}

constexpr uint32_t kStreamMaxM = 16;  // rows of X one streaming launch can cover
// Rows per launch when X is walked in slabs: 16 while the digits of 16 rows (4 bytes per value) still sit in
// shared memory next to the weight rings, else 8 (16 rows read from the global scratch measured slower than
// two slabs of 8 read from shared memory: 304 against 199 us on 128256 x 4096).
inline uint32_t stream_slab_rows(uint32_t K) { return (uint64_t)K * 16u * 4u <= 132u * 1024u ? 16u : 8u; }

// Kernel selection.  FP32: always the float kernel.  STREAM / AUTO: the streaming
// kernel, X walked in slabs of 8 rows (each slab re-reads the weights, as the
// reference's batched8 shader does per 8 rows).
int run_matmul(bpq4k_context* h, const MatmulArgs& a, cudaStream_t st) {
    int launches = 0;
    cudaError_t e = cudaSuccess;
    if (h->gemv_variant == BPQ4K_GEMV_FP32) {
        e = launch_gemv_fp32(a, st, &launches);
    } else if (!a.n_slots && a.M >= (uint32_t)h->prefill_min_m && h->gemv_variant == BPQ4K_GEMV_AUTO) {
        // prefill: tensor-core kernel; its 16-bit copy of the activations lives in the handle's scratch
        const size_t need = prefill_scratch_bytes(a.M, a.N, a.K, h->prefill_arg(), h->sm_count);
        if (need > h->scratch_bytes) {
            if (int s = ensure_bytes(h, &h->scratch, &h->scratch_bytes, need)) return s;
        }
        e = launch_prefill_tc(a, h->prefill_arg(), h->scratch, h->scratch_bytes, h->dev_status, h->sm_count, st, &launches);
    } else {
        const uint32_t Mtot = a.n_slots ? 1 : a.M;
        const size_t need = a.n_slots ? 0 : gemv_stream_scratch_bytes(Mtot < kStreamMaxM ? Mtot : kStreamMaxM, a.K);
        if (need > h->scratch_bytes) {
            if (int s = ensure_bytes(h, &h->scratch, &h->scratch_bytes, need)) return s;
        }
        MatmulArgs c = a;
        const uint32_t slab = stream_slab_rows(a.K);
        for (uint32_t m0 = 0; m0 < Mtot && e == cudaSuccess; m0 += slab) {
            if (!a.n_slots) {
                c.M = Mtot - m0 < slab ? Mtot - m0 : slab;
                c.X = a.X + (uint64_t)m0 * a.K;
                c.Y = a.Y + (uint64_t)m0 * a.N;
            }
            e = launch_gemv_stream(c, h->tune, h->scratch, h->scratch_bytes, h->dev_status, h->sm_count, &h->tmaps, st, &launches);
        }
    }
    h->launches += (uint64_t)launches;
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "matmul launch");
    }
    return BPQ4K_OK;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int bpq4k_version(void) { return BPQ4K_VERSION; }

const char* bpq4k_status_string(int s) {
    switch (s) {
        case BPQ4K_OK: return "ok";
        case BPQ4K_ERR_INVALID_ARG: return "invalid argument";
        case BPQ4K_ERR_UNSUPPORTED: return "unsupported shape";
        case BPQ4K_ERR_MISALIGNED: return "misaligned pointer or stride";
        case BPQ4K_ERR_CUDA: return "CUDA error";
        case BPQ4K_ERR_NCCL: return "NCCL error";
        case BPQ4K_ERR_TIMEOUT: return "device-side wait timed out";
        case BPQ4K_ERR_NO_DEVICE: return "no usable device";
        case BPQ4K_ERR_ALLOC: return "allocation failed";
        case BPQ4K_ERR_DEVICE_ASSERT: return "a kernel's index check failed (debug build)";
        default: return "unknown status";
    }
}

int bpq4k_create(int device, bpq4k_handle_t* out) {
    if (!out) return BPQ4K_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return BPQ4K_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= count) return BPQ4K_ERR_INVALID_ARG;
    bpq4k_context* h = new (std::nothrow) bpq4k_context();
    if (!h) return BPQ4K_ERR_ALLOC;
    h->device = device;
    cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&h->cc_major, cudaDevAttrComputeCapabilityMajor, device);
    if (h->cc_major != 10) {
        // The kernels are built for sm_100a only; there is no other code path.
        delete h;
        return BPQ4K_ERR_NO_DEVICE;
    }
    {
        DeviceGuard g(device);
        // status word and a first scratch slab are allocated here so that later calls
        // with common shapes allocate nothing (and can be captured into CUDA graphs)
        cudaError_t e2 = cudaMalloc(reinterpret_cast<void**>(&h->dev_status), 256);
        if (e2 == cudaSuccess) e2 = cudaMemset(h->dev_status, 0, 256);
        if (e2 == cudaSuccess) {
            e2 = cudaMalloc(&h->scratch, 4u << 20);
            if (e2 == cudaSuccess) h->scratch_bytes = 4u << 20;
        }
        if (e2 != cudaSuccess) {
            cudaGetLastError();
            if (h->dev_status) cudaFree(h->dev_status);
            delete h;
            return BPQ4K_ERR_ALLOC;
        }
    }
    *out = h;
    return BPQ4K_OK;
}

int bpq4k_destroy(bpq4k_handle_t h) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    {
        DeviceGuard g(h->device);
        if (h->stage_x) cudaFree(h->stage_x);
        if (h->stage_y) cudaFree(h->stage_y);
        if (h->scratch) cudaFree(h->scratch);
        if (h->dev_status) cudaFree(h->dev_status);
        if (h->tune.stamps) cudaFree(h->tune.stamps);
        for (uint32_t i = 0; i < h->n_retired; i++) cudaFree(h->retired[i]);
        if (h->batch_exec) cudaGraphExecDestroy(h->batch_exec);
        if (h->batch_stream) cudaStreamDestroy(h->batch_stream);
        if (h->batch_event) cudaEventDestroy(h->batch_event);
    }
    delete h;
    return BPQ4K_OK;
}

const char* bpq4k_last_error_string(bpq4k_handle_t h) { return h ? h->err : "null handle"; }

int bpq4k_device_index(bpq4k_handle_t h) { return h ? h->device : -1; }

int bpq4k_set_option(bpq4k_handle_t h, int option, int value) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    switch (option) {
        case BPQ4K_OPT_GEMV_VARIANT:
            if (value < BPQ4K_GEMV_AUTO || value > BPQ4K_GEMV_STREAM)
                return fail(h, BPQ4K_ERR_INVALID_ARG, "gemv variant %d out of range", value);
            h->gemv_variant = value;
            return BPQ4K_OK;
        case BPQ4K_OPT_PREFILL_MODE:
            if (value < BPQ4K_PREFILL_F16X3 || value > BPQ4K_PREFILL_BF16)
                return fail(h, BPQ4K_ERR_INVALID_ARG, "prefill mode %d out of range", value);
            h->prefill_mode = value;
            return BPQ4K_OK;
        case BPQ4K_OPT_PREFILL_MIN_M:
            if (value < 1) return fail(h, BPQ4K_ERR_INVALID_ARG, "prefill_min_m must be >= 1");
            h->prefill_min_m = value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_WARPS:
            if (value < 0 || value > 16) return fail(h, BPQ4K_ERR_INVALID_ARG, "stream warps must be 0..16");
            h->tune.warps = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_KSPLIT:
            if (value < 0 || value > 16) return fail(h, BPQ4K_ERR_INVALID_ARG, "stream k-split must be 0..16");
            h->tune.wk = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAGE_BLOCKS:
            if (value < 0 || value > 8) return fail(h, BPQ4K_ERR_INVALID_ARG, "stage blocks must be 0..8");
            h->tune.cb = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAGES:
            if (value < 0 || value > 8) return fail(h, BPQ4K_ERR_INVALID_ARG, "stages must be 0..8");
            h->tune.stages = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_CTAS_PER_SM:
            if (value < 0 || value > 32) return fail(h, BPQ4K_ERR_INVALID_ARG, "ctas per sm must be 0..32");
            h->tune.ctas_per_sm = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_FORCE_SCRATCH:
            h->tune.force_scratch = value ? 1u : 0u;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_NO_PDL:
            h->tune.no_pdl = value ? 1u : 0u;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_NO_UNIT_LIST:
            h->tune.no_unit_list = value == 2 ? 2u : value ? 1u : 0u;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_UNIT_ROWS:
            if (value != 0 && value != 16 && value != 32) return fail(h, BPQ4K_ERR_INVALID_ARG, "unit rows must be 0, 16 or 32");
            h->tune.rows_per_unit = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_CLUSTER:
            if (value != 0 && value != 1 && value != 2 && value != 4) return fail(h, BPQ4K_ERR_INVALID_ARG, "cluster size must be 0, 1, 2 or 4");
            h->tune.cluster = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAGING_WARPS:
            if (value < 0 || value > 16) return fail(h, BPQ4K_ERR_INVALID_ARG, "staging warps must be 0..16");
            h->tune.staging_warps = (uint32_t)value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAMPS: {
            if (value < 0 || value > 4096) return fail(h, BPQ4K_ERR_INVALID_ARG, "stamp slots must be 0..4096");
            if (value > 0 && !gemv_stream_stamps_built())
                return fail(h, BPQ4K_ERR_INVALID_ARG, "this build has no time stamps: load libbpq4k_stamps.so (make -C csrc stamps)");
            DeviceGuard g(h->device);
            drop_batch_graph(h);  // (a recorded list carries the old buffer and slots)
            if (h->tune.stamps) {
                cudaDeviceSynchronize();
                cudaFree(h->tune.stamps);
            }
            h->tune.stamps = nullptr;
            h->tune.stamp_next = nullptr;
            h->tune.stamp_launches = 0;
            h->stamp_next = 0;
            if (value > 0) {
                const size_t bytes = (size_t)value * kStreamStampCtas * 8u * sizeof(unsigned long long);
                if (cudaMalloc(reinterpret_cast<void**>(&h->tune.stamps), bytes) != cudaSuccess || cudaMemset(h->tune.stamps, 0, bytes) != cudaSuccess) {
                    h->tune.stamps = nullptr;
                    return fail(h, BPQ4K_ERR_CUDA, "stamp buffer: %s", cudaGetErrorString(cudaGetLastError()));
                }
                h->tune.stamp_next = &h->stamp_next;
                h->tune.stamp_launches = (uint32_t)value;
            }
            return BPQ4K_OK;
        }
        case BPQ4K_OPT_PREFILL_VARIANT:
            if (value < 0 || value > 2) return fail(h, BPQ4K_ERR_INVALID_ARG, "prefill variant must be 0, 1 or 2");
            h->prefill_variant = value;
            return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_PREWAIT_STAGES:
            if (value < 0 || value > 9) return fail(h, BPQ4K_ERR_INVALID_ARG, "pre-wait stages must be 0..9");
            h->tune.pre_wait = (uint32_t)value;
            return BPQ4K_OK;
        default: return fail(h, BPQ4K_ERR_INVALID_ARG, "unknown option %d", option);
    }
}

int bpq4k_get_option(bpq4k_handle_t h, int option, int* value) {
    if (!h || !value) return BPQ4K_ERR_INVALID_ARG;
    switch (option) {
        case BPQ4K_OPT_GEMV_VARIANT: *value = h->gemv_variant; return BPQ4K_OK;
        case BPQ4K_OPT_PREFILL_MODE: *value = h->prefill_mode; return BPQ4K_OK;
        case BPQ4K_OPT_PREFILL_VARIANT: *value = h->prefill_variant; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAMPS: *value = (int)h->tune.stamp_launches; return BPQ4K_OK;
        case BPQ4K_OPT_PREFILL_MIN_M: *value = h->prefill_min_m; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_WARPS: *value = (int)h->tune.warps; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_KSPLIT: *value = (int)h->tune.wk; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAGE_BLOCKS: *value = (int)h->tune.cb; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAGES: *value = (int)h->tune.stages; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_CTAS_PER_SM: *value = (int)h->tune.ctas_per_sm; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_FORCE_SCRATCH: *value = (int)h->tune.force_scratch; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_NO_PDL: *value = (int)h->tune.no_pdl; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_NO_UNIT_LIST: *value = (int)h->tune.no_unit_list; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_UNIT_ROWS: *value = (int)h->tune.rows_per_unit; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_CLUSTER: *value = (int)h->tune.cluster; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_STAGING_WARPS: *value = (int)h->tune.staging_warps; return BPQ4K_OK;
        case BPQ4K_OPT_STREAM_PREWAIT_STAGES: *value = (int)h->tune.pre_wait; return BPQ4K_OK;
        case BPQ4K_OPT_BATCH_RECORDS: *value = (int)h->batch_records; return BPQ4K_OK;
        default: return fail(h, BPQ4K_ERR_INVALID_ARG, "unknown option %d", option);
    }
}

int bpq4k_read_stream_stamps(bpq4k_handle_t h, unsigned long long* dst, size_t words, uint32_t* launches_stamped) {
    if (!h || !dst) return BPQ4K_ERR_INVALID_ARG;
    if (!h->tune.stamps) return fail(h, BPQ4K_ERR_INVALID_ARG, "time stamps are off (BPQ4K_OPT_STREAM_STAMPS)");
    const size_t have = (size_t)h->tune.stamp_launches * kStreamStampCtas * 8u;
    if (words > have) words = have;
    DeviceGuard g(h->device);
    if (cudaDeviceSynchronize() != cudaSuccess || cudaMemcpy(dst, h->tune.stamps, words * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess)
        return fail(h, BPQ4K_ERR_CUDA, "stamp read: %s", cudaGetErrorString(cudaGetLastError()));
    if (launches_stamped) *launches_stamped = h->stamp_next;
    return BPQ4K_OK;
}

uint64_t bpq4k_launch_count(bpq4k_handle_t h, int reset) {
    if (!h) return 0;
    const uint64_t v = h->launches;
    if (reset) h->launches = 0;
    return v;
}

int bpq4k_device_status(bpq4k_handle_t h, void* stream, int* status_out) {
    if (!h || !status_out) return BPQ4K_ERR_INVALID_ARG;
    DeviceGuard g(h->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, h->dev_status, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(h, e, "status read-back");
    *status_out = v;
    if (v != 0) {
        cudaMemsetAsync(h->dev_status, 0, sizeof(int), st);
        return fail(h, v, "a kernel reported status %d (%s)", v, bpq4k_status_string(v));
    }
    return BPQ4K_OK;
}

uint32_t bpq4k_n_blocks(uint32_t K) { return (K + BPQ4K_QK_K - 1u) / BPQ4K_QK_K; }
uint32_t bpq4k_row_stride_words(uint32_t K) { return bpq4k_n_blocks(K) * BPQ4K_BLOCK_WORDS; }

int bpq4k_pack_q4k_host(const void* raw_host, uint32_t N, uint32_t K, uint32_t* words_host) {
    if ((!raw_host || !words_host) && N != 0 && K != 0) return BPQ4K_ERR_INVALID_ARG;
    const uint64_t row_bytes = (uint64_t)bpq4k_n_blocks(K) * BPQ4K_BLOCK_BYTES;
    const uint64_t stride = bpq4k_row_stride_words(K);
    const uint8_t* src = static_cast<const uint8_t*>(raw_host);
    for (uint32_t r = 0; r < N; r++) std::memcpy(words_host + r * stride, src + r * row_bytes, row_bytes);
    return BPQ4K_OK;
}

int bpq4k_upload_weights(bpq4k_handle_t h, const uint32_t* words_host, uint64_t n_words, void** w_dev) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (!w_dev || (!words_host && n_words)) return fail(h, BPQ4K_ERR_INVALID_ARG, "null pointer");
    DeviceGuard g(h->device);
    *w_dev = nullptr;
    const size_t bytes = n_words ? (size_t)n_words * 4u : 16u;
    cudaError_t e = cudaMalloc(w_dev, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, BPQ4K_ERR_ALLOC, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    if (n_words) {
        e = cudaMemcpy(*w_dev, words_host, (size_t)n_words * 4u, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            cudaFree(*w_dev);
            *w_dev = nullptr;
            return cuda_fail(h, e, "weight upload");
        }
    }
    return BPQ4K_OK;
}

int bpq4k_free_device(bpq4k_handle_t h, void* p) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (!p) return BPQ4K_OK;
    DeviceGuard g(h->device);
    cudaError_t e = cudaFree(p);
    if (e != cudaSuccess) return cuda_fail(h, e, "cudaFree");
    return BPQ4K_OK;
}

int bpq4k_dequant_f32(bpq4k_handle_t h, const void* W, uint32_t N, uint32_t K, uint32_t rowStrideWords, float* out,
                      void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (N == 0) return BPQ4K_OK;
    if (int s = check_weights(h, W, N, K, rowStrideWords)) return s;
    if (!out) return fail(h, BPQ4K_ERR_INVALID_ARG, "out is null");
    if (!aligned16(out)) return fail(h, BPQ4K_ERR_MISALIGNED, "out is not 16-byte aligned");
    DeviceGuard g(h->device);
    cudaError_t e = launch_dequant_f32(static_cast<const uint8_t*>(W), N, K, (uint64_t)rowStrideWords * 4u, out,
                                       static_cast<cudaStream_t>(stream));
    h->launches += 1;
    if (e != cudaSuccess) return cuda_fail(h, e, "dequant launch");
    return BPQ4K_OK;
}

int bpq4k_matmul_f32(bpq4k_handle_t h, const float* X, const void* W, const float* bias, float* Y, uint32_t M,
                     uint32_t N, uint32_t K, uint32_t rowStrideWords, uint32_t yOffset, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return BPQ4K_OK;
    if (int s = check_weights(h, W, N, K, rowStrideWords)) return s;
    if (!X || !Y) return fail(h, BPQ4K_ERR_INVALID_ARG, "X or Y is null");
    if (!aligned16(X)) return fail(h, BPQ4K_ERR_MISALIGNED, "X is not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "Y is not 4-byte aligned");
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = Y + yOffset;
    a.M = M;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    return run_matmul(h, a, static_cast<cudaStream_t>(stream));
}

// ---- Q5_K / Q6_K siblings ----------------------------------------------------

uint32_t bpq4k_kq_block_bytes(int qtype) {
    return qtype == BPQ4K_TYPE_Q4_K ? 144u : qtype == BPQ4K_TYPE_Q5_K ? 176u : qtype == BPQ4K_TYPE_Q6_K ? 210u
         : qtype == BPQ4K_TYPE_Q6_K_PADDED ? 224u : 0u;
}

uint32_t bpq4k_kq_row_stride_words(int qtype, uint32_t K) {
    return (bpq4k_n_blocks(K) * bpq4k_kq_block_bytes(qtype) + 3u) / 4u;
}

int bpq4k_kq_pack_host(int qtype, const void* raw_host, uint32_t N, uint32_t K, uint32_t* words_host) {
    const uint32_t bb = bpq4k_kq_block_bytes(qtype);
    if (!bb) return BPQ4K_ERR_UNSUPPORTED;
    if ((!raw_host || !words_host) && N != 0 && K != 0) return BPQ4K_ERR_INVALID_ARG;
    const uint32_t nb = bpq4k_n_blocks(K);
    const uint64_t stride = bpq4k_kq_row_stride_words(qtype, K);
    const uint8_t* src = static_cast<const uint8_t*>(raw_host);
    if (qtype == BPQ4K_TYPE_Q6_K_PADDED) {  // file-format blocks in, one padded block out for each
        for (uint64_t r = 0; r < N; r++)
            for (uint32_t b = 0; b < nb; b++) {
                uint8_t* dst = reinterpret_cast<uint8_t*>(words_host + r * stride) + (uint64_t)b * 224u;
                std::memcpy(dst, src + (r * nb + b) * 210u, 210u);
                std::memset(dst + 210, 0, 14);
            }
        return BPQ4K_OK;
    }
    const uint64_t row_bytes = (uint64_t)nb * bb;
    for (uint32_t r = 0; r < N; r++) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(words_host + r * stride);
        std::memcpy(dst, src + r * row_bytes, row_bytes);
        std::memset(dst + row_bytes, 0, stride * 4u - row_bytes);
    }
    return BPQ4K_OK;
}

namespace {
int check_kq_weights(bpq4k_context* h, int qtype, const void* W, uint32_t K, uint32_t rowStrideWords) {
    const uint32_t bb = bpq4k_kq_block_bytes(qtype);
    if (!bb) return fail(h, BPQ4K_ERR_UNSUPPORTED, "quantisation type %d is not Q4_K (12), Q5_K (13), Q6_K (14) or padded Q6_K (270)", qtype);
    if (K == 0 || K % BPQ4K_QK_K != 0)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "K=%u is not a positive multiple of 256", K);
    if (!W) return fail(h, BPQ4K_ERR_INVALID_ARG, "W is null");
    const uint32_t need = bpq4k_kq_row_stride_words(qtype, K);
    if (rowStrideWords < need)
        return fail(h, BPQ4K_ERR_INVALID_ARG, "rowStrideWords=%u is smaller than the %u words a row of K=%u needs", rowStrideWords, need, K);
    if (qtype == BPQ4K_TYPE_Q6_K) {
        if (reinterpret_cast<uintptr_t>(W) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "W is not 4-byte aligned");
    } else {
        if (rowStrideWords % 4u != 0)
            return fail(h, BPQ4K_ERR_MISALIGNED, "rowStrideWords=%u is not a multiple of 4 words (16 bytes)", rowStrideWords);
        if (!aligned16(W)) return fail(h, BPQ4K_ERR_MISALIGNED, "W is not 16-byte aligned");
    }
    return BPQ4K_OK;
}
}  // namespace

int bpq4k_kq_dequant_f32(bpq4k_handle_t h, int qtype, const void* W, uint32_t N, uint32_t K, uint32_t rowStrideWords,
                         float* out, void* stream) {
    if (qtype == BPQ4K_TYPE_Q4_K) return bpq4k_dequant_f32(h, W, N, K, rowStrideWords, out, stream);
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (N == 0) return BPQ4K_OK;
    if (int s = check_kq_weights(h, qtype, W, K, rowStrideWords)) return s;
    if (!out) return fail(h, BPQ4K_ERR_INVALID_ARG, "out is null");
    if (!aligned16(out)) return fail(h, BPQ4K_ERR_MISALIGNED, "out is not 16-byte aligned");
    DeviceGuard g(h->device);
    cudaError_t e = launch_kq_dequant_f32(qtype, static_cast<const uint8_t*>(W), nullptr, N, N, K, (uint64_t)rowStrideWords * 4u,
                                          out, static_cast<cudaStream_t>(stream));
    h->launches += 1;
    if (e != cudaSuccess) return cuda_fail(h, e, "dequant launch");
    return BPQ4K_OK;
}

int bpq4k_kq_gather_f32(bpq4k_handle_t h, int qtype, const void* W, uint32_t nRows, uint32_t K, uint32_t rowStrideWords,
                        const uint32_t* tokens, uint32_t nTokens, float* out, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (nTokens == 0) return BPQ4K_OK;
    if (qtype == BPQ4K_TYPE_Q4_K) return fail(h, BPQ4K_ERR_UNSUPPORTED, "the embedding gather covers Q5_K and Q6_K tables");
    if (int s = check_kq_weights(h, qtype, W, K, rowStrideWords)) return s;
    if (!out || !tokens) return fail(h, BPQ4K_ERR_INVALID_ARG, "out or tokens is null");
    if (!aligned16(out)) return fail(h, BPQ4K_ERR_MISALIGNED, "out is not 16-byte aligned");
    DeviceGuard g(h->device);
    cudaError_t e = launch_kq_dequant_f32(qtype, static_cast<const uint8_t*>(W), tokens, nRows, nTokens, K,
                                          (uint64_t)rowStrideWords * 4u, out, static_cast<cudaStream_t>(stream));
    h->launches += 1;
    if (e != cudaSuccess) return cuda_fail(h, e, "gather launch");
    return BPQ4K_OK;
}

int bpq4k_kq_matmul_f32(bpq4k_handle_t h, int qtype, const float* X, const void* W, const float* bias, float* Y,
                        uint32_t M, uint32_t N, uint32_t K, uint32_t rowStrideWords, uint32_t yOffset, void* stream) {
    if (qtype == BPQ4K_TYPE_Q4_K) return bpq4k_matmul_f32(h, X, W, bias, Y, M, N, K, rowStrideWords, yOffset, stream);
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return BPQ4K_OK;
    if (int s = check_kq_weights(h, qtype, W, K, rowStrideWords)) return s;
    if (!X || !Y) return fail(h, BPQ4K_ERR_INVALID_ARG, "X or Y is null");
    if (reinterpret_cast<uintptr_t>(X) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "X is not 4-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "Y is not 4-byte aligned");
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = Y + yOffset;
    a.M = M;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    int launches = 0;
    cudaError_t e = cudaErrorInvalidValue;
    // many rows of Q5_K or padded Q6_K: the tensor-core kernel, as for Q4_K
    const bool tensor_cores = (qtype == BPQ4K_TYPE_Q5_K || qtype == BPQ4K_TYPE_Q6_K_PADDED) && h->gemv_variant == BPQ4K_GEMV_AUTO &&
                              aligned16(X) && M >= (uint32_t)h->prefill_min_m;
    // padded Q6_K: the streaming kernel in slabs of up to 8 rows; a slab whose rows do not fit in shared
    // memory together (long K) is halved (8 -> 4 -> 2 -> 1 rows), which still beats the plain kernel
    if (!tensor_cores && qtype == BPQ4K_TYPE_Q6_K_PADDED && h->gemv_variant != BPQ4K_GEMV_FP32 && aligned16(X) && K % 4u == 0) {
        const cudaStream_t st = static_cast<cudaStream_t>(stream);
        MatmulArgs c = a;
        e = cudaSuccess;
        uint32_t slab = 8;
        for (uint32_t m0 = 0; m0 < M && e == cudaSuccess;) {
            c.M = M - m0 < slab ? M - m0 : slab;
            c.X = a.X + (uint64_t)m0 * K;
            c.Y = a.Y + (uint64_t)m0 * N;
            e = launch_q6k_stream(c, h->tune, h->dev_status, h->sm_count, &h->tmaps, st, &launches);
            if (e == cudaErrorInvalidValue && c.M > 1) {  // does not fit: smaller slabs from here on
                slab = c.M > 4 ? 4 : c.M > 2 ? 2 : 1;
                e = cudaSuccess;
                continue;
            }
            m0 += c.M;
        }
        if (e == cudaErrorInvalidValue) launches = 0;  // not even one row fits: the plain kernel below
    }
    if (tensor_cores) {
        const size_t need = prefill_scratch_bytes(M, N, K, h->prefill_arg(), h->sm_count);
        if (need > h->scratch_bytes) {
            if (int s = ensure_bytes(h, &h->scratch, &h->scratch_bytes, need)) return s;
        }
        e = launch_prefill_tc(a, h->prefill_arg(), h->scratch, h->scratch_bytes, h->dev_status, h->sm_count,
                              static_cast<cudaStream_t>(stream), &launches, qtype);
    } else
    // Q5_K: the streaming kernel in slabs of 8 rows (each slab re-reads the weights)
    if (qtype == BPQ4K_TYPE_Q5_K && h->gemv_variant != BPQ4K_GEMV_FP32 && aligned16(X)) {
        const size_t need = gemv_stream_scratch_bytes(M < kStreamMaxM ? M : kStreamMaxM, K);
        if (need > h->scratch_bytes) {
            if (int s = ensure_bytes(h, &h->scratch, &h->scratch_bytes, need)) return s;
        }
        MatmulArgs c = a;
        e = cudaSuccess;
        const uint32_t slab = stream_slab_rows(K);
        for (uint32_t m0 = 0; m0 < M && e == cudaSuccess; m0 += slab) {
            c.M = M - m0 < slab ? M - m0 : slab;
            c.X = a.X + (uint64_t)m0 * K;
            c.Y = a.Y + (uint64_t)m0 * N;
            e = launch_gemv_stream(c, h->tune, h->scratch, h->scratch_bytes, h->dev_status, h->sm_count, &h->tmaps,
                                   static_cast<cudaStream_t>(stream), &launches, 13);
        }
    }
    if (e == cudaErrorInvalidValue) e = launch_kq_gemv_fp32(qtype, a, static_cast<cudaStream_t>(stream), &launches);
    h->launches += (uint64_t)launches;
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "matmul launch");
    }
    return BPQ4K_OK;
}

int bpq4k_matmul_fused_f32(bpq4k_handle_t h, int qtype, int prologue, const float* X, const float* aux, float eps,
                           const void* W, const float* bias, const float* residual, float* Y, uint32_t N, uint32_t K,
                           uint32_t rowStrideWords, uint32_t yOffset, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (N == 0) return BPQ4K_OK;
    if (qtype != BPQ4K_TYPE_Q4_K && qtype != BPQ4K_TYPE_Q5_K && qtype != BPQ4K_TYPE_Q6_K_PADDED)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "the fused forms cover Q4_K (12), Q5_K (13) and padded Q6_K (270), not type %d", qtype);
    if (prologue < BPQ4K_PROLOGUE_NONE || prologue > BPQ4K_PROLOGUE_SILU_MUL)
        return fail(h, BPQ4K_ERR_INVALID_ARG, "unknown prologue %d", prologue);
    if (int s = check_kq_weights(h, qtype, W, K, rowStrideWords)) return s;
    if (!X || !Y) return fail(h, BPQ4K_ERR_INVALID_ARG, "X or Y is null");
    if (prologue != BPQ4K_PROLOGUE_NONE && !aux) return fail(h, BPQ4K_ERR_INVALID_ARG, "aux is null");
    if (!aligned16(X) || (aux && !aligned16(aux))) return fail(h, BPQ4K_ERR_MISALIGNED, "X or aux is not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "Y is not 4-byte aligned");
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = Y + yOffset;
    a.M = 1;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    a.prologue = (uint32_t)prologue;
    a.aux = aux;
    a.eps = eps;
    a.residual = residual;
    int launches = 0;
    const cudaError_t e = qtype == BPQ4K_TYPE_Q6_K_PADDED
                              ? launch_q6k_stream(a, h->tune, h->dev_status, h->sm_count, &h->tmaps, static_cast<cudaStream_t>(stream), &launches)
                              : launch_gemv_stream(a, h->tune, h->scratch, h->scratch_bytes, h->dev_status, h->sm_count, &h->tmaps,
                                                   static_cast<cudaStream_t>(stream), &launches, qtype);
    h->launches += (uint64_t)launches;
    if (e == cudaErrorInvalidValue) {
        cudaGetLastError();
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "K=%u is too long for the fused single-row kernel", K);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "matmul launch");
    }
    return BPQ4K_OK;
}

int bpq4k_argmax_f32(bpq4k_handle_t h, const float* logits, uint32_t n, int32_t* result, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (!logits || !result || n == 0) return fail(h, BPQ4K_ERR_INVALID_ARG, "logits or result is null, or n is 0");
    if (reinterpret_cast<uintptr_t>(logits) & 3u || reinterpret_cast<uintptr_t>(result) & 3u)
        return fail(h, BPQ4K_ERR_MISALIGNED, "logits or result is not 4-byte aligned");
    DeviceGuard g(h->device);
    // bytes 64..79 of the status allocation are this kernel's two scratch words (zeroed at creation)
    const cudaError_t e = launch_argmax(logits, n, result, reinterpret_cast<char*>(h->dev_status) + 64, h->sm_count,
                                        static_cast<cudaStream_t>(stream));
    h->launches += 1;
    if (e != cudaSuccess) return cuda_fail(h, e, "argmax launch");
    return BPQ4K_OK;
}

int bpq4k_matmul_moe_f32(bpq4k_handle_t h, const float* X, const void* W, const float* bias, float* Y,
                         const uint32_t* offsets, const uint32_t* x_rows, uint32_t nSlots, uint32_t N, uint32_t K,
                         uint32_t rowStrideWords, uint32_t wRows, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (nSlots == 0 || N == 0) return BPQ4K_OK;
    if (int s = check_weights(h, W, N, K, rowStrideWords)) return s;
    if (!X || !Y || !offsets) return fail(h, BPQ4K_ERR_INVALID_ARG, "X, Y or offsets is null");
    if (wRows < N) return fail(h, BPQ4K_ERR_INVALID_ARG, "wRows=%u is smaller than N=%u", wRows, N);
    if (!aligned16(X)) return fail(h, BPQ4K_ERR_MISALIGNED, "X is not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "Y is not 4-byte aligned");
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = Y;
    a.M = 1;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    a.offsets = offsets;
    a.x_rows = x_rows;
    a.n_slots = nSlots;
    a.w_total_rows = wRows;
    return run_matmul(h, a, static_cast<cudaStream_t>(stream));
}

int bpq4k_kq_matmul_moe_f32(bpq4k_handle_t h, int qtype, const float* X, const void* W, const float* bias, float* Y,
                            const uint32_t* offsets, const uint32_t* x_rows, uint32_t nSlots, uint32_t N, uint32_t K,
                            uint32_t rowStrideWords, uint32_t wRows, void* stream) {
    if (qtype == BPQ4K_TYPE_Q4_K) return bpq4k_matmul_moe_f32(h, X, W, bias, Y, offsets, x_rows, nSlots, N, K, rowStrideWords, wRows, stream);
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (nSlots == 0 || N == 0) return BPQ4K_OK;
    if (qtype != BPQ4K_TYPE_Q5_K && qtype != BPQ4K_TYPE_Q6_K_PADDED)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "the expert-indexed form covers Q4_K, Q5_K and padded Q6_K, not type %d", qtype);
    if (int s = check_kq_weights(h, qtype, W, K, rowStrideWords)) return s;
    if (!X || !Y || !offsets) return fail(h, BPQ4K_ERR_INVALID_ARG, "X, Y or offsets is null");
    if (wRows < N) return fail(h, BPQ4K_ERR_INVALID_ARG, "wRows=%u is smaller than N=%u", wRows, N);
    if (!aligned16(X)) return fail(h, BPQ4K_ERR_MISALIGNED, "X is not 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 3u) return fail(h, BPQ4K_ERR_MISALIGNED, "Y is not 4-byte aligned");
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = Y;
    a.M = 1;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    a.offsets = offsets;
    a.x_rows = x_rows;
    a.n_slots = nSlots;
    a.w_total_rows = wRows;
    int launches = 0;
    const cudaError_t e = qtype == BPQ4K_TYPE_Q6_K_PADDED
                              ? launch_q6k_stream(a, h->tune, h->dev_status, h->sm_count, &h->tmaps, static_cast<cudaStream_t>(stream), &launches)
                              : launch_gemv_stream(a, h->tune, nullptr, 0, h->dev_status, h->sm_count, &h->tmaps,
                                                   static_cast<cudaStream_t>(stream), &launches, 13);
    h->launches += (uint64_t)launches;
    if (e == cudaErrorInvalidValue) {
        cudaGetLastError();
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "K=%u is too long (or there are too many slots) for the expert-indexed kernel", K);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "matmul launch");
    }
    return BPQ4K_OK;
}

uint64_t bpq4k_moe_ffn_work_floats(uint32_t T, uint32_t topk, uint32_t H, uint32_t F) {
    return (uint64_t)T * topk * (2ull * F + H);
}

int bpq4k_moe_ffn_f32(bpq4k_handle_t h, int qtype, const float* X, const void* Wgate, const void* Wup, const void* Wdown,
                      const uint32_t* expert_ids, const float* route_w, float* Y, uint32_t T, uint32_t topk,
                      uint32_t nExperts, uint32_t H, uint32_t F, float* work, uint64_t work_floats, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (T == 0 || topk == 0) return BPQ4K_OK;
    if (qtype != BPQ4K_TYPE_Q4_K && qtype != BPQ4K_TYPE_Q5_K && qtype != BPQ4K_TYPE_Q6_K_PADDED)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "the routed-expert layer covers Q4_K (12), Q5_K (13) and padded Q6_K (270), not type %d", qtype);
    if (nExperts == 0 || H == 0 || F == 0) return fail(h, BPQ4K_ERR_INVALID_ARG, "nExperts, H or F is 0");
    if (H % 256u || F % 256u) return fail(h, BPQ4K_ERR_UNSUPPORTED, "H=%u and F=%u must be multiples of 256", H, F);
    const uint64_t pairs = (uint64_t)T * topk;
    if (pairs > 0x7FFFFFFFull || (uint64_t)nExperts * F > 0xFFFFFFFFull || (uint64_t)nExperts * H > 0xFFFFFFFFull)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "the expert stacks have more than 2^32 rows");
    const uint32_t rs_h = bpq4k_kq_row_stride_words(qtype, H), rs_f = bpq4k_kq_row_stride_words(qtype, F);
    if (int s = check_kq_weights(h, qtype, Wgate, H, rs_h)) return s;
    if (int s = check_kq_weights(h, qtype, Wup, H, rs_h)) return s;
    if (int s = check_kq_weights(h, qtype, Wdown, F, rs_f)) return s;
    if (!X || !Y || !expert_ids || !route_w || !work) return fail(h, BPQ4K_ERR_INVALID_ARG, "a pointer argument is null");
    if (work_floats < bpq4k_moe_ffn_work_floats(T, topk, H, F))
        return fail(h, BPQ4K_ERR_INVALID_ARG, "work holds %llu floats, the call needs %llu", (unsigned long long)work_floats,
                    (unsigned long long)bpq4k_moe_ffn_work_floats(T, topk, H, F));
    if (!aligned16(X) || !aligned16(Y) || !aligned16(work)) return fail(h, BPQ4K_ERR_MISALIGNED, "X, Y or work is not 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(expert_ids) | reinterpret_cast<uintptr_t>(route_w)) & 3u)
        return fail(h, BPQ4K_ERR_MISALIGNED, "expert_ids or route_w is not 4-byte aligned");
    DeviceGuard g(h->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* gate_out = work;
    float* up_out = work + pairs * F;
    float* down_out = work + 2 * pairs * F;
    int launches = 0;
    cudaError_t e = cudaSuccess;
    auto expert_matmul = [&](const float* x, const void* W, float* y, uint32_t N, uint32_t K, uint32_t rs, uint32_t x_div,
                             const float* aux, const void* W2, float* y2) {
        MatmulArgs a{};
        a.X = x;
        a.W = static_cast<const uint8_t*>(W);
        a.Y = y;
        a.M = 1;
        a.N = N;
        a.K = K;
        a.w_row_bytes = (uint64_t)rs * 4u;
        a.offsets = expert_ids;
        a.offset_mul = N;  // expert e starts at row e*N of its stack
        a.x_row_div = x_div;
        a.n_slots = (uint32_t)pairs;
        a.w_total_rows = (uint64_t)nExperts * N;
        a.W2 = static_cast<const uint8_t*>(W2);
        a.Y2 = y2;
        if (aux) {
            a.prologue = BPQ4K_PROLOGUE_SILU_MUL;
            a.aux = aux;
        }
        if (qtype == BPQ4K_TYPE_Q6_K_PADDED) {
            if (W2 || pairs > 65535u) return cudaErrorInvalidValue;  // one grid row per slot, one stack per launch
            return launch_q6k_stream(a, h->tune, h->dev_status, h->sm_count, &h->tmaps, st, &launches);
        }
        return launch_gemv_stream(a, h->tune, nullptr, 0, h->dev_status, h->sm_count, &h->tmaps, st, &launches, qtype);
    };
    // gate and up in one launch (same activations and experts) when the unit list allows it
    e = expert_matmul(X, Wgate, gate_out, F, H, rs_h, topk, nullptr, Wup, up_out);
    if (e == cudaErrorInvalidValue) {
        cudaGetLastError();
        e = expert_matmul(X, Wgate, gate_out, F, H, rs_h, topk, nullptr, nullptr, nullptr);
        if (e == cudaSuccess) e = expert_matmul(X, Wup, up_out, F, H, rs_h, topk, nullptr, nullptr, nullptr);
    }
    if (e == cudaSuccess) e = expert_matmul(gate_out, Wdown, down_out, H, F, rs_f, 0, up_out, nullptr, nullptr);
    if (e == cudaSuccess) {
        e = launch_moe_accumulate(Y, down_out, route_w, T, topk, H, h->sm_count, st);
        launches++;
    }
    h->launches += (uint64_t)launches;
    if (e == cudaErrorInvalidValue) {
        cudaGetLastError();
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "H=%u or F=%u is too long for the expert-indexed kernel", H, F);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "routed-expert layer launch");
    }
    return BPQ4K_OK;
}

int bpq4k_matmul_host_f32(bpq4k_handle_t h, const float* X_host, const void* W_dev, const float* bias_dev,
                          float* Y_host, uint32_t M, uint32_t N, uint32_t K, uint32_t rowStrideWords,
                          void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return BPQ4K_OK;
    if (!X_host || !Y_host) return fail(h, BPQ4K_ERR_INVALID_ARG, "X_host or Y_host is null");
    if (int s = check_weights(h, W_dev, N, K, rowStrideWords)) return s;
    DeviceGuard g(h->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t xb = (size_t)M * K * 4u, yb = (size_t)M * N * 4u;
    if (int s = ensure_bytes(h, reinterpret_cast<void**>(&h->stage_x), &h->stage_x_bytes, xb)) return s;
    if (int s = ensure_bytes(h, reinterpret_cast<void**>(&h->stage_y), &h->stage_y_bytes, yb)) return s;
    cudaError_t e = cudaMemcpyAsync(h->stage_x, X_host, xb, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_fail(h, e, "activation upload");
    MatmulArgs a{};
    a.X = h->stage_x;
    a.W = static_cast<const uint8_t*>(W_dev);
    a.bias = bias_dev;
    a.Y = h->stage_y;
    a.M = M;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    if (int s = run_matmul(h, a, st)) return s;
    e = cudaMemcpyAsync(Y_host, h->stage_y, yb, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return cuda_fail(h, e, "result read-back");
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(h, e, "stream synchronize");
    return BPQ4K_OK;
}

int bpq4k_matmul_allgather_f32(bpq4k_handle_t h, const float* X, const void* W, const float* bias, float* const* slot_ptrs,
                               uint32_t nPeers, uint32_t M, uint32_t N, uint32_t K, uint32_t rowStrideWords, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return BPQ4K_OK;
    if (int s = check_weights(h, W, N, K, rowStrideWords)) return s;
    if (!X || !slot_ptrs) return fail(h, BPQ4K_ERR_INVALID_ARG, "X or slot_ptrs is null");
    if (nPeers == 0 || nPeers > 8) return fail(h, BPQ4K_ERR_UNSUPPORTED, "nPeers=%u: 1..8 GPUs are supported", nPeers);
    if (M > 8u) return fail(h, BPQ4K_ERR_UNSUPPORTED, "the fused gather covers M <= 8 (M=%u)", M);
    if (!aligned16(X)) return fail(h, BPQ4K_ERR_MISALIGNED, "X is not 16-byte aligned");
    for (uint32_t p = 0; p < nPeers; p++)
        if (!slot_ptrs[p] || (reinterpret_cast<uintptr_t>(slot_ptrs[p]) & 3u))
            return fail(h, BPQ4K_ERR_INVALID_ARG, "slot_ptrs[%u] is null or misaligned", p);
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = slot_ptrs[0];
    a.M = M;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    a.n_peers = nPeers - 1;
    for (uint32_t p = 1; p < nPeers; p++) a.peer_Y[p - 1] = slot_ptrs[p];
    a.slot_parity = h->peer_parity;
    a.slot_parity_stride = h->peer_parity_stride;
    const size_t need = gemv_stream_scratch_bytes(M, K);
    if (need > h->scratch_bytes) {
        if (int s = ensure_bytes(h, &h->scratch, &h->scratch_bytes, need)) return s;
    }
    int launches = 0;
    const cudaError_t e = launch_gemv_stream(a, h->tune, h->scratch, h->scratch_bytes, h->dev_status, h->sm_count, &h->tmaps,
                                             static_cast<cudaStream_t>(stream), &launches);
    h->launches += (uint64_t)launches;
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "matmul launch");
    }
    return BPQ4K_OK;
}

int bpq4k_kq_matmul_allgather_f32(bpq4k_handle_t h, int qtype, const float* X, const void* W, const float* bias,
                                  float* const* slot_ptrs, uint32_t nPeers, uint32_t M, uint32_t N, uint32_t K,
                                  uint32_t rowStrideWords, void* stream) {
    if (qtype == BPQ4K_TYPE_Q4_K) return bpq4k_matmul_allgather_f32(h, X, W, bias, slot_ptrs, nPeers, M, N, K, rowStrideWords, stream);
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return BPQ4K_OK;
    if (qtype != BPQ4K_TYPE_Q5_K && qtype != BPQ4K_TYPE_Q6_K_PADDED)
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "the fused gather covers Q4_K, Q5_K and padded Q6_K, not type %d", qtype);
    if (int s = check_kq_weights(h, qtype, W, K, rowStrideWords)) return s;
    if (!X || !slot_ptrs) return fail(h, BPQ4K_ERR_INVALID_ARG, "X or slot_ptrs is null");
    if (nPeers == 0 || nPeers > 8) return fail(h, BPQ4K_ERR_UNSUPPORTED, "nPeers=%u: 1..8 GPUs are supported", nPeers);
    const uint32_t max_m = qtype == BPQ4K_TYPE_Q6_K_PADDED ? 1u : 8u;
    if (M > max_m) return fail(h, BPQ4K_ERR_UNSUPPORTED, "the fused gather covers M <= %u for this type (M=%u)", max_m, M);
    if (!aligned16(X)) return fail(h, BPQ4K_ERR_MISALIGNED, "X is not 16-byte aligned");
    for (uint32_t p = 0; p < nPeers; p++)
        if (!slot_ptrs[p] || (reinterpret_cast<uintptr_t>(slot_ptrs[p]) & 3u))
            return fail(h, BPQ4K_ERR_INVALID_ARG, "slot_ptrs[%u] is null or misaligned", p);
    DeviceGuard g(h->device);
    MatmulArgs a{};
    a.X = X;
    a.W = static_cast<const uint8_t*>(W);
    a.bias = bias;
    a.Y = slot_ptrs[0];
    a.M = M;
    a.N = N;
    a.K = K;
    a.w_row_bytes = (uint64_t)rowStrideWords * 4u;
    a.n_peers = nPeers - 1;
    for (uint32_t p = 1; p < nPeers; p++) a.peer_Y[p - 1] = slot_ptrs[p];
    a.slot_parity = h->peer_parity;
    a.slot_parity_stride = h->peer_parity_stride;
    int launches = 0;
    cudaError_t e;
    if (qtype == BPQ4K_TYPE_Q5_K) {
        const size_t need = gemv_stream_scratch_bytes(M, K);
        if (need > h->scratch_bytes) {
            if (int s = ensure_bytes(h, &h->scratch, &h->scratch_bytes, need)) return s;
        }
        e = launch_gemv_stream(a, h->tune, h->scratch, h->scratch_bytes, h->dev_status, h->sm_count, &h->tmaps,
                               static_cast<cudaStream_t>(stream), &launches, 13);
    } else {
        e = launch_q6k_stream(a, h->tune, h->dev_status, h->sm_count, &h->tmaps, static_cast<cudaStream_t>(stream), &launches);
    }
    h->launches += (uint64_t)launches;
    if (e == cudaErrorInvalidValue) {
        cudaGetLastError();
        return fail(h, BPQ4K_ERR_UNSUPPORTED, "K=%u is too long for the fused single-row kernel", K);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(h, e, "matmul launch");
    }
    return BPQ4K_OK;
}

int bpq4k_peer_double_buffer(bpq4k_handle_t h, const uint32_t* step_word, uint64_t stride_floats) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (step_word && (reinterpret_cast<uintptr_t>(step_word) & 3u)) return fail(h, BPQ4K_ERR_MISALIGNED, "step_word is not 4-byte aligned");
    h->peer_parity = step_word;
    h->peer_parity_stride = step_word ? stride_floats : 0;
    return BPQ4K_OK;
}

int bpq4k_peer_barrier(bpq4k_handle_t h, uint32_t* const* flag_ptrs, uint32_t nPeers, uint32_t rank, uint32_t epoch,
                       uint32_t timeout_ms, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (!flag_ptrs || nPeers == 0 || nPeers > 8 || rank >= nPeers) return fail(h, BPQ4K_ERR_INVALID_ARG, "bad peer arguments");
    for (uint32_t p = 0; p < nPeers; p++)
        if (!flag_ptrs[p]) return fail(h, BPQ4K_ERR_INVALID_ARG, "flag_ptrs[%u] is null", p);
    DeviceGuard g(h->device);
    if (h->clock_khz <= 0) {
        cudaDeviceGetAttribute(&h->clock_khz, cudaDevAttrClockRate, h->device);
        if (h->clock_khz <= 0) h->clock_khz = 1900000;
    }
    const int khz = h->clock_khz;
    const uint64_t cycles = (uint64_t)(timeout_ms ? timeout_ms : 1000u) * (uint64_t)khz;
    const cudaError_t e = launch_peer_barrier(flag_ptrs, nPeers, rank, epoch, cycles, h->dev_status, static_cast<cudaStream_t>(stream));
    h->launches += 1;
    if (e != cudaSuccess) return cuda_fail(h, e, "barrier launch");
    return BPQ4K_OK;
}

namespace {

// A host pointer the GPU can address directly (pinned or registered memory): its device alias, else null.
void* device_alias(const void* host_ptr) {
    cudaPointerAttributes pa{};
    if (cudaPointerGetAttributes(&pa, host_ptr) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return pa.type == cudaMemoryTypeHost ? pa.devicePointer : nullptr;
}

uint64_t fnv1a(uint64_t hsh, const void* p, size_t n) {
    const unsigned char* b = static_cast<const unsigned char*>(p);
    for (size_t i = 0; i < n; i++) hsh = (hsh ^ b[i]) * 1099511628211ull;
    return hsh;
}

}  // namespace

int bpq4k_matmul_host_batch_f32(bpq4k_handle_t h, const bpq4k_host_matmul* items, uint32_t count, void* stream) {
    if (!h) return BPQ4K_ERR_INVALID_ARG;
    if (count == 0) return BPQ4K_OK;
    if (!items) return fail(h, BPQ4K_ERR_INVALID_ARG, "items is null");
    size_t xb = 0, yb = 0;
    uint32_t live = 0;
    for (uint32_t i = 0; i < count; i++) {
        const bpq4k_host_matmul& it = items[i];
        if (it.M == 0 || it.N == 0) continue;
        if (!it.X_host || !it.Y_host) return fail(h, BPQ4K_ERR_INVALID_ARG, "item %u: X_host or Y_host is null", i);
        if (int s = check_weights(h, it.W_dev, it.N, it.K, it.rowStrideWords)) return s;
        xb += ((size_t)it.M * it.K * 4u + 255u) & ~(size_t)255u;  // keep every slice 256-byte aligned
        yb += ((size_t)it.M * it.N * 4u + 255u) & ~(size_t)255u;
        live++;
    }
    if (live == 0) return BPQ4K_OK;
    DeviceGuard g(h->device);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int s = ensure_bytes(h, reinterpret_cast<void**>(&h->stage_x), &h->stage_x_bytes, xb)) return s;
    if (int s = ensure_bytes(h, reinterpret_cast<void**>(&h->stage_y), &h->stage_y_bytes, yb)) return s;

    // Host buffers the GPU can address (pinned memory) are gathered and scattered by one kernel each
    // instead of one asynchronous copy per vector; other host memory takes the copy path.
    // Outputs of items the streaming kernel serves (every value stored exactly once, by the tile's
    // epilogue) go straight to the pinned host buffer: the stores cross PCIe while the kernel still
    // streams weights, and only the tensor-core items (split-K partial sums) are staged and scattered.
    CopySegments gin{}, gout{};
    bool direct = live <= CopySegments::kMax;
    float* y_direct[CopySegments::kMax] = {};
    auto stores_once = [&](const bpq4k_host_matmul& it) {
        return !(h->gemv_variant == BPQ4K_GEMV_AUTO && it.M >= (uint32_t)h->prefill_min_m);
    };
    {
        size_t xo = 0, yo = 0;
        for (uint32_t i = 0; i < count && direct; i++) {
            const bpq4k_host_matmul& it = items[i];
            if (it.M == 0 || it.N == 0) continue;
            const size_t xbytes = (size_t)it.M * it.K * 4u, ybytes = (size_t)it.M * it.N * 4u;
            void* xa = device_alias(it.X_host);
            void* ya = device_alias(it.Y_host);
            if (!xa || !ya || !aligned16(xa) || !aligned16(ya) || xbytes > 0xFFFFFFFFull || ybytes > 0xFFFFFFFFull) {
                direct = false;
                break;
            }
            if (stores_once(it)) {
                y_direct[gin.count] = static_cast<float*>(ya);
            } else {
                gout.src[gout.count] = reinterpret_cast<uint8_t*>(h->stage_y) + yo;
                gout.dst[gout.count] = ya;
                gout.bytes[gout.count++] = (uint32_t)ybytes;
            }
            gin.src[gin.count] = xa;
            gin.dst[gin.count] = reinterpret_cast<uint8_t*>(h->stage_x) + xo;
            gin.bytes[gin.count++] = (uint32_t)xbytes;
            xo += (xbytes + 255u) & ~(size_t)255u;
            yo += (ybytes + 255u) & ~(size_t)255u;
        }
    }

    // the whole dispatch list on one stream: inputs in, matmuls, outputs out
    auto enqueue = [&](cudaStream_t s_) -> int {
        cudaError_t e = cudaSuccess;
        if (direct) {
            e = launch_copy_segments(gin, s_);
            h->launches += 1;
        } else {
            size_t xo = 0;
            for (uint32_t i = 0; i < count && e == cudaSuccess; i++) {
                const bpq4k_host_matmul& it = items[i];
                if (it.M == 0 || it.N == 0) continue;
                const size_t bytes = (size_t)it.M * it.K * 4u;
                e = cudaMemcpyAsync(reinterpret_cast<uint8_t*>(h->stage_x) + xo, it.X_host, bytes, cudaMemcpyHostToDevice, s_);
                xo += (bytes + 255u) & ~(size_t)255u;
            }
        }
        if (e != cudaSuccess) return cuda_fail(h, e, "activation upload");
        size_t xo = 0, yo = 0;
        uint32_t li = 0;  // index among the live items
        for (uint32_t i = 0; i < count; i++) {
            const bpq4k_host_matmul& it = items[i];
            if (it.M == 0 || it.N == 0) continue;
            MatmulArgs a{};
            a.X = reinterpret_cast<const float*>(reinterpret_cast<uint8_t*>(h->stage_x) + xo);
            a.W = static_cast<const uint8_t*>(it.W_dev);
            a.bias = it.bias_dev;
            a.Y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(h->stage_y) + yo);
            if (direct && y_direct[li]) a.Y = y_direct[li];
            li++;
            a.M = it.M;
            a.N = it.N;
            a.K = it.K;
            a.w_row_bytes = (uint64_t)it.rowStrideWords * 4u;
            if (int s = run_matmul(h, a, s_)) return s;
            xo += ((size_t)it.M * it.K * 4u + 255u) & ~(size_t)255u;
            yo += ((size_t)it.M * it.N * 4u + 255u) & ~(size_t)255u;
        }
        if (direct) {
            if (gout.count) {
                e = launch_copy_segments(gout, s_);
                h->launches += 1;
            }
        } else {
            yo = 0;
            for (uint32_t i = 0; i < count && e == cudaSuccess; i++) {
                const bpq4k_host_matmul& it = items[i];
                if (it.M == 0 || it.N == 0) continue;
                const size_t bytes = (size_t)it.M * it.N * 4u;
                e = cudaMemcpyAsync(it.Y_host, reinterpret_cast<uint8_t*>(h->stage_y) + yo, bytes, cudaMemcpyDeviceToHost, s_);
                yo += (bytes + 255u) & ~(size_t)255u;
            }
        }
        if (e != cudaSuccess) return cuda_fail(h, e, "result read-back");
        return BPQ4K_OK;
    };

    // Replay: the same list (same buffers, shapes and options) seen before is captured into a CUDA
    // graph on the handle's own stream the second time and launched from it from then on.
    uint64_t key = 1469598103934665603ull;
    key = fnv1a(key, items, sizeof(bpq4k_host_matmul) * count);
    key = fnv1a(key, &h->tune, sizeof(h->tune));
    const int opts[3] = {h->gemv_variant, h->prefill_arg(), h->prefill_min_m};
    key = fnv1a(key, opts, sizeof(opts));
    const void* bufs[3] = {h->stage_x, h->stage_y, h->scratch};  // the graph holds these addresses
    key = fnv1a(key, bufs, sizeof(bufs));
    if (direct && h->batch_key == key && h->batch_seen >= 1) {
        cudaError_t e = cudaSuccess;
        if (!h->batch_stream) e = cudaStreamCreateWithFlags(&h->batch_stream, cudaStreamNonBlocking);
        if (e == cudaSuccess && !h->batch_event) e = cudaEventCreateWithFlags(&h->batch_event, cudaEventDisableTiming);
        if (e == cudaSuccess && !h->batch_exec) {
            cudaGraph_t graph = nullptr;
            const uint64_t before = h->launches;
            e = cudaStreamBeginCapture(h->batch_stream, cudaStreamCaptureModeThreadLocal);
            if (e == cudaSuccess) {
                const int s = enqueue(h->batch_stream);
                const cudaError_t e2 = cudaStreamEndCapture(h->batch_stream, &graph);
                e = s != BPQ4K_OK ? cudaErrorUnknown : e2;
            }
            if (e == cudaSuccess) e = cudaGraphInstantiate(&h->batch_exec, graph, 0);
            if (e == cudaSuccess) h->batch_records++;
            if (graph) cudaGraphDestroy(graph);
            h->batch_launches = h->launches - before;
            h->launches = before;  // nothing ran yet
            if (e != cudaSuccess) {
                cudaGetLastError();
                h->batch_exec = nullptr;
                h->batch_seen = 0;  // do not try again for this list
                h->batch_key = 0;
            }
        }
        if (e == cudaSuccess && h->batch_exec) {
            e = cudaEventRecord(h->batch_event, st);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(h->batch_stream, h->batch_event, 0);
            if (e == cudaSuccess) e = cudaGraphLaunch(h->batch_exec, h->batch_stream);
            if (e == cudaSuccess) e = cudaStreamSynchronize(h->batch_stream);
            if (e != cudaSuccess) return cuda_fail(h, e, "graph replay of the dispatch list");
            h->launches += h->batch_launches;
            return BPQ4K_OK;
        }
    } else if (h->batch_key != key) {
        if (h->batch_exec) cudaGraphExecDestroy(h->batch_exec);
        h->batch_exec = nullptr;
        h->batch_key = key;
        h->batch_seen = 0;
    }
    if (int s = enqueue(st)) return s;
    const cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_fail(h, e, "stream synchronize");
    if (h->batch_key == key) h->batch_seen++;
    return BPQ4K_OK;
}

}  // extern "C"
#pragma GCC visibility pop
