// Internal launch interface between the C ABI (bpq4k_capi.cu) and the kernel
// translation units.  Every function enqueues on `stream` and returns the
// cudaError_t of the launch; none of them allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

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
    uint64_t w_total_rows;    // indirect form: rows of the whole expert stack (bounds the copies)
    uint32_t offset_mul;      // 0: offsets[s] is a weight row; else offsets[s] is an expert id and the row is offsets[s]*offset_mul
    uint32_t x_row_div;       // x_rows null and this non-zero: slot s reads activation row s / x_row_div
    // indirect form, optional second stack of the same shape served by the same launch with the same
    // activations and offsets (an expert layer's gate and up stacks): results to Y2[s*N + n]
    const uint8_t* W2;
    float* Y2;
    // fused all-gather: every output is also stored to these buffers (other GPUs' memory, plain stores)
    float* peer_Y[8];
    uint32_t n_peers;
    // fused all-gather, double-buffered slots: when slot_parity is set, Y and every peer_Y are advanced by
    // (*slot_parity & 1) * slot_parity_stride floats (read after the dependency wait; the word is the step count
    // that the peer barrier keeps in this GPU's own flag array)
    const uint32_t* slot_parity;
    uint64_t slot_parity_stride;
    // fused prologue on the activation row (single row only) and residual epilogue:
    //   1: x = X * rsqrt(mean(X^2) + eps) * aux      (aux = RMSNorm weight[K])
    //   2: x = gelu_tanh(X) * aux,  3: x = silu(X) * aux   (aux = the "up" vector[K])
    // indirect form: slot s transforms its own row with row s of aux ([n_slots][K]); no residual there
    uint32_t prologue;
    const float* aux;
    float eps;
    const float* residual;  // null or float[N]: added to every output
};

cudaError_t launch_dequant_f32(const uint8_t* W, uint32_t N, uint32_t K, uint64_t w_row_bytes, float* out,
                               cudaStream_t stream);

// Value a kernel stores in the handle's device status word when a bounded wait runs out.
constexpr int kDeviceTimeout = 6;
// Value stored by a kernel of the debug build whose index check failed (the C ABI's BPQ4K_ERR_DEVICE_ASSERT).
constexpr int kDeviceAssert = 9;

// Tuning knobs of the streaming kernel; 0 = choose automatically.
constexpr uint32_t kStreamStampCtas = 160;
struct StreamTuning {
    uint32_t warps = 0;        // warps per CTA (<= 16)
    uint32_t wk = 0;           // warps that split K of one 16-row tile
    uint32_t cb = 0;           // super-blocks per ring stage
    uint32_t stages = 0;       // ring depth per warp
    uint32_t ctas_per_sm = 0;  // cap on resident CTAs per SM
    uint32_t force_scratch = 0;  // 1: always split activations into global scratch first
    uint32_t no_pdl = 0;       // 1: launch without programmatic dependent launch
    uint32_t no_unit_list = 0; // 1: indirect form always as one grid row per slot
    uint32_t rows_per_unit = 0; // several activation rows: weight rows a warp takes at a time, 0 automatic, 16 or 32
    uint32_t pre_wait = 0;     // ring stages issued before the dependency wait: 0 automatic, 1..8, 9 = none
    uint32_t cluster = 0;      // CTAs per cluster sharing the staging of a single activation row: 0 automatic, 1, 2, 4
    uint32_t staging_warps = 0;  // single row: warps that stage the activation row (helpers leave before the main loop): 0 automatic (16), 1..16
    // time stamps of the single-row streaming kernel (BPQ4K_OPT_STREAM_STAMPS): device buffer of stamp_launches slots of
    // kStreamStampCtas CTAs x 8 words, the handle's running launch counter
    unsigned long long* stamps = nullptr;
    uint32_t* stamp_next = nullptr;
    uint32_t stamp_launches = 0;
};

// Launch configuration of ONE kernel instantiation per device: the opt-in dynamic shared-memory size
// (a per-device function attribute) and the occupancy of the last (threads, smem) pair asked for.
// The launchers keep one of these in a function-local static per instantiation; handles on different
// devices and threads share it, hence the mutex and the per-device slots.
struct KernelConfig {
    static constexpr int kMaxDevices = 64;
    struct Entry {
        size_t smem_cfg = 0;
        uint32_t threads = 0;
        size_t smem = 0;
        int occ = 0;
    };
    std::mutex mu;
    Entry per_dev[kMaxDevices];

    // Make `func` launchable with `smem` bytes of dynamic shared memory on the current device and, when
    // occ_out is given, report how many CTAs of `threads` threads fit one SM.
    cudaError_t prepare(const void* func, uint32_t threads, size_t smem, int* occ_out) {
        int dev = 0;
        if (cudaError_t e = cudaGetDevice(&dev)) return e;
        if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu);
        Entry& en = per_dev[dev];
        if (smem > en.smem_cfg) {
            if (cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) return e;
            en.smem_cfg = smem;
            en.threads = 0;
        }
        if (occ_out) {
            if (en.threads != threads || en.smem != smem) {
                int occ = 0;
                if (cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, func, (int)threads, smem)) return e;
                en.threads = threads;
                en.smem = smem;
                en.occ = occ > 0 ? occ : 1;
            }
            *occ_out = en.occ;
        }
        return cudaSuccess;
    }
};

// Encoded tensor maps of recently used weight matrices (encoding one costs ~15 us of host time;
// a decode loop calls with the same few weights over and over).
struct TmapCache {
    static constexpr uint32_t kEntries = 64;
    struct Entry {
        const void* W = nullptr;
        uint64_t rows = 0, row_bytes = 0;
        uint32_t nb = 0, cb = 0;
        alignas(64) unsigned char map[128];
    };
    Entry entries[kEntries];
    uint32_t next = 0;
};

// Bytes of scratch launch_gemv_stream needs when the activations do not fit in shared memory.
size_t gemv_stream_scratch_bytes(uint32_t M, uint32_t K);

// Streaming tensor-core matmul for M <= 8 (or the indirect form).  `scratch` may be null
// when the activations fit in shared memory.  qtype 12: Q4_K (144-byte blocks), 13: Q5_K (176-byte).
cudaError_t launch_gemv_stream(const MatmulArgs& a, const StreamTuning& tune, void* scratch, size_t scratch_bytes,
                               int* status_dev, int sm_count, TmapCache* tmaps, cudaStream_t stream, int* launches,
                               int qtype = 12);

// Tensor-core prefill matmul (tcgen05 + TMEM).  mode follows bpq4k_prefill_mode: 0 three-pass half
// split, 1 one pass half, 2 one pass bfloat16.  `scratch` holds the 16-bit activations.
bool gemv_stream_stamps_built();  // true in libbpq4k_stamps.so
size_t prefill_scratch_bytes(uint32_t M, uint32_t N, uint32_t K, int mode, int sm_count);
cudaError_t launch_prefill_tc(const MatmulArgs& a, int mode, void* scratch, size_t scratch_bytes, int* status_dev,
                              int sm_count, cudaStream_t stream, int* launches, int qtype = 12);  // 12 Q4_K, 13 Q5_K, 0x10E padded Q6_K

// Cross-GPU barrier on flag words in peer memory (one process per GPU): store `epoch` into slot
// `rank` of every peer's flag array, then wait -- at most timeout_cycles -- until every slot of the
// own array has reached `epoch`.  On a time-out the kernel stores kDeviceTimeout to *status.
cudaError_t launch_peer_barrier(uint32_t* const* flag_ptrs_host, uint32_t n_peers, uint32_t rank, uint32_t epoch,
                                uint64_t timeout_cycles, int* status_dev, cudaStream_t stream, bool pdl = true);

// Index of the largest of n floats (lowest index on ties; 0 when nothing exceeds -1e30) into *result.
// `scratch`: 16 zeroed, 8-byte aligned device bytes that the kernel leaves zeroed.
cudaError_t launch_argmax(const float* logits, uint32_t n, int32_t* result, void* scratch, int sm_count, cudaStream_t stream);

// Up to kMax segment copies in one launch; every pointer must be addressable by the GPU and 16-byte
// aligned, every size a multiple of 4 bytes.
struct CopySegments {
    static constexpr uint32_t kMax = 32;
    const void* src[kMax];
    void* dst[kMax];
    uint32_t bytes[kMax];
    uint32_t count;
};
cudaError_t launch_copy_segments(const CopySegments& segs, cudaStream_t stream);

// Y[t][n] += sum over k ascending of route_w[t*topk + k] * O[(t*topk + k)*N + n]; N a multiple of 4, rows 16-byte aligned.
cudaError_t launch_moe_accumulate(float* Y, const float* O, const float* route_w, uint32_t T, uint32_t topk, uint32_t N,
                                  int sm_count, cudaStream_t stream);

// One warp per output row, float FMAs in the reference shader's arithmetic.
cudaError_t launch_gemv_fp32(const MatmulArgs& a, cudaStream_t stream, int* launches);

// Q5_K (qtype 13) and Q6_K (qtype 14) on the reference's packed layout: bit-exact dequantiser
// (source row r = rows[r] when `rows` is given, zeros for ids >= n_src_rows) and float-FMA matmul.
cudaError_t launch_kq_dequant_f32(int qtype, const uint8_t* W, const uint32_t* rows, uint32_t n_src_rows, uint32_t N,
                                  uint32_t K, uint64_t w_row_bytes, float* out, cudaStream_t stream);
cudaError_t launch_kq_gemv_fp32(int qtype, const MatmulArgs& a, cudaStream_t stream, int* launches);

// Q6_K with every block padded to 224 bytes (type number of the C ABI's BPQ4K_TYPE_Q6_K_PADDED).
constexpr int kQ6PaddedType = 0x10E;
constexpr uint32_t kQ6PaddedBytes = 224;

// Streaming tensor-core matmul for M <= 8 activation rows of Q6_K weights in the padded layout.
// cudaErrorInvalidValue: the shape does not fit the kernel (several rows of a long K; go row by row).
cudaError_t launch_q6k_stream(const MatmulArgs& a, const StreamTuning& tune, int* status_dev, int sm_count, TmapCache* tmaps,
                              cudaStream_t stream, int* launches);

}  // namespace bpq4k
