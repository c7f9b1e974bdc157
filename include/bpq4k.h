/*
 * bpq4k.h -- C ABI of libbpq4k.so: the GGUF Q4_K dequantize-fused matrix
 * multiply for NVIDIA B200 (sm_100a).
 *
 * The library replaces, for this one operator, what the Backpack runtime does
 * through Dawn/WGSL: its six `q4k_*` compute shaders, the host-side packer and
 * the CPU decode.  Every entry point below names the reference interface it
 * stands in for (file:line relative to the reference tree).
 *
 * Conventions
 *  - Plain C: pointers, sizes, an opaque handle.  No C++ or framework types.
 *  - Unless a name ends in `_host`, every data pointer is a DEVICE pointer on
 *    the handle's device, owned by the caller.  The library owns only the
 *    scratch memory inside the handle.  That scratch grows on demand (a call with a
 *    larger M*K than any before); an outgrown block stays allocated until
 *    bpq4k_destroy, so a CUDA graph the caller captured around an earlier call keeps
 *    pointing at valid memory.
 *  - `stream` is a cudaStream_t / CUstream passed as void*; NULL is the
 *    default stream.  Calls are asynchronous with respect to the host and
 *    ordered on that stream, like dispatches on the reference's single WebGPU
 *    queue (runtime/model_runner.h:27-30).
 *  - A handle is bound to one device and is not thread-safe, like the
 *    reference's GPUContext/ExecutionContext.
 *  - Every call returns a bpq4k_status; nothing aborts, traps or throws.  The
 *    reference's ops return void and leave the output invalid on bad input
 *    (runtime/ops/matmul.cpp:212,333); callers here map a non-zero status to
 *    that behaviour.
 *  - Weights are the raw GGUF Q4_K bytes, exactly what the reference uploads
 *    (runtime/gguf_loader.cpp:359-379, runtime/model_runner.cpp:958-963):
 *    row-major [N][K/256] super-blocks of 144 bytes; `rowStrideWords` is the
 *    distance between rows in 32-bit words (KQuantPacked::rowStrideWords,
 *    runtime/gguf_loader.h:108-117) and must be a multiple of 4 (16 bytes) and
 *    at least (K/256)*36.  K must be a multiple of 256.
 */
#ifndef BPQ4K_H
#define BPQ4K_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BPQ4K_VERSION 100
#define BPQ4K_QK_K 256u
#define BPQ4K_BLOCK_BYTES 144u
#define BPQ4K_BLOCK_WORDS 36u

typedef struct bpq4k_context* bpq4k_handle_t;

typedef enum bpq4k_status {
    BPQ4K_OK = 0,
    BPQ4K_ERR_INVALID_ARG = 1,   /* null pointer, zero handle, bad enum */
    BPQ4K_ERR_UNSUPPORTED = 2,   /* K not a multiple of 256, size beyond a stated limit */
    BPQ4K_ERR_MISALIGNED = 3,    /* pointer or stride not aligned as documented */
    BPQ4K_ERR_CUDA = 4,          /* a CUDA runtime call failed; see last_error_string */
    BPQ4K_ERR_NCCL = 5,          /* reserved for callers that layer a collective on top */
    BPQ4K_ERR_TIMEOUT = 6,       /* a bounded device-side wait ran out */
    BPQ4K_ERR_NO_DEVICE = 7,     /* no usable sm_100 device */
    BPQ4K_ERR_ALLOC = 8,         /* device or host allocation failed */
    BPQ4K_ERR_DEVICE_ASSERT = 9  /* debug build only: a kernel's index check failed (the access was skipped) */
} bpq4k_status;

/* Options (bpq4k_set_option).  The reference selects kernels with environment
 * switches such as BP_Q4K_DECODE_256 (runtime/model_runner.cpp:2045-2053);
 * here the choice is an explicit per-handle option. */
typedef enum bpq4k_option {
    BPQ4K_OPT_GEMV_VARIANT = 1,  /* bpq4k_gemv_variant; default AUTO */
    BPQ4K_OPT_PREFILL_MODE = 2,  /* bpq4k_prefill_mode; default F16X3 */
    BPQ4K_OPT_PREFILL_MIN_M = 3, /* smallest M routed to the tensor-core prefill kernel; default 25 */
    /* Tuning of the streaming kernel; 0 = automatic.  The reference tunes its decode
     * kernels through an autotune cache (runtime/model_runner.cpp:5113-5199). */
    BPQ4K_OPT_STREAM_WARPS = 10,         /* warps per CTA, <= 16 */
    BPQ4K_OPT_STREAM_KSPLIT = 11,        /* warps that share the K range of one 16-row tile */
    BPQ4K_OPT_STREAM_STAGE_BLOCKS = 12,  /* super-blocks per ring stage */
    BPQ4K_OPT_STREAM_STAGES = 13,        /* ring depth per warp, <= 8 */
    BPQ4K_OPT_STREAM_CTAS_PER_SM = 14,   /* cap on resident CTAs per SM */
    BPQ4K_OPT_STREAM_FORCE_SCRATCH = 15, /* 1: split activations into global scratch even if they fit on chip */
    /* The streaming kernel is launched with programmatic dependent launch: it prefetches
     * WEIGHTS while the preceding kernel of the stream drains, and reads X / writes Y only
     * after that kernel has completed.  The expert-indexed forms also read their slot tables
     * (offsets / expert ids, x_rows) in that early phase.  A kernel that does not itself trigger
     * dependent launches early is always complete before this one starts; set to 1 if a
     * preceding kernel that does trigger early writes the weights or the slot tables. */
    BPQ4K_OPT_STREAM_NO_PDL = 16,
    /* 1: the expert-indexed form always runs one grid row per slot (default 0: one list of
     * (slot, tile) units over a persistent 1-D grid when there are more slots than SMs or two stacks share
     * the launch, and each CTA's share spans at most four slots); 2: the unit list whenever it is possible. */
    BPQ4K_OPT_STREAM_NO_UNIT_LIST = 17,
    /* Ring stages whose copies are issued BEFORE the dependency wait (the weight prefetch that overlaps the
     * preceding kernel); the remaining stages are issued right after the loads of the activations.  0: automatic
     * (the whole ring while it is small, ~64 KB per SM of a deep one), 1..8: that many, 9: none. */
    BPQ4K_OPT_STREAM_PREWAIT_STAGES = 18,
    /* Several activation rows (M = 2..16): weight rows a warp takes through its ring at a time.  32 halves the
     * reads of the activation digits per weight byte; 0: automatic (32 from 8192 weight rows on), 16, 32. */
    BPQ4K_OPT_STREAM_UNIT_ROWS = 19,
    /* One activation row: CTAs per thread-block cluster that quantise the row together (each a share, written into
     * every member's shared memory).  0: automatic (pairs from K = 14336 on), 1: none, 2, 4. */
    BPQ4K_OPT_STREAM_CLUSTER = 20,
    /* One activation row: warps per CTA that quantise the row; those beyond the plan's warps (BPQ4K_OPT_STREAM_WARPS)
     * leave before the main loop.  0: automatic (16), 1..16 (values below the plan's warp count change nothing). */
    BPQ4K_OPT_STREAM_STAGING_WARPS = 21,
    /* Single-pass precision modes of the tensor-core kernel, Q4_K: how a weight tile meets the activations.
     * 0 (default): one CTA per 256 weight rows x 256 activation rows, dequantised weights through shared memory.
     * 1: two CTAs of a cluster share tcgen05.mma.cta_group::2 (2 x 128 weight rows x 512 activation rows; M > 256).
     * 2: dequantised weights go to tensor memory (tcgen05.st) and the mma takes its A operand from there
     *    (256 weight rows x 128 activation rows per CTA).
     * All three give identical bits; 1 and 2 measured slower on B200 and exist for comparison. */
    BPQ4K_OPT_PREFILL_VARIANT = 23,
    /* Time stamps of the single-row streaming kernel, for attributing a launch's microseconds.  n > 0: keep the
     * stamps of the last n launches (a device buffer of n x 160 CTAs x 8 words; launch i writes slot i mod n;
     * launches captured into a graph keep the slot they were given at capture); 0: off (default, no cost).
     * Read with bpq4k_read_stream_stamps.  Only libbpq4k_stamps.so (make -C backpack_b200/csrc stamps: the product
     * library with the streaming kernel compiled again) has the stamps; the product library answers n > 0 with
     * BPQ4K_ERR_INVALID_ARG (even untaken, the six branches cost its decode step 2 %).  No counterpart in the reference. */
    BPQ4K_OPT_STREAM_STAMPS = 24,
    /* Read-only (bpq4k_get_option): how many times bpq4k_matmul_host_batch_f32 has recorded a dispatch
     * list into a replay graph on this handle.  A list is recorded again after any of the handle's
     * buffers had to grow. */
    BPQ4K_OPT_BATCH_RECORDS = 30
} bpq4k_option;

typedef enum bpq4k_gemv_variant {
    BPQ4K_GEMV_AUTO = 0,
    BPQ4K_GEMV_FP32 = 1,   /* one warp per output row, float FMAs (the reference shader's arithmetic) */
    BPQ4K_GEMV_STREAM = 2  /* bulk-copy ring + tensor-core dot products, split-precision activations */
} bpq4k_gemv_variant;

typedef enum bpq4k_prefill_mode {
    BPQ4K_PREFILL_F16X3 = 0,  /* three-term half split of W and X: meets the float tolerance */
    BPQ4K_PREFILL_F16 = 1,    /* single half-precision pass */
    BPQ4K_PREFILL_BF16 = 2    /* single bfloat16 pass */
} bpq4k_prefill_mode;

/* ---- library and handle ------------------------------------------------ */

int bpq4k_version(void);
const char* bpq4k_status_string(int status);

/* Create a handle on CUDA device `device`.  Stands in for GPUContext::init +
 * pipeline creation (runtime/gpu_context.h:151-220): after this call no entry
 * point below compiles, loads or allocates anything except where it says so. */
int bpq4k_create(int device, bpq4k_handle_t* out);
int bpq4k_destroy(bpq4k_handle_t h);

/* Text of the last failure on this handle (never NULL).  Stands in for the
 * stderr reporting of Dawn's error callbacks (runtime/gpu_context.cpp:212-237). */
const char* bpq4k_last_error_string(bpq4k_handle_t h);

/* CUDA device the handle was created on (-1 for a null handle). */
int bpq4k_device_index(bpq4k_handle_t h);

int bpq4k_set_option(bpq4k_handle_t h, int option, int value);
int bpq4k_get_option(bpq4k_handle_t h, int option, int* value);

/* Copies the time-stamp buffer to the host (after a device synchronisation): per stamped launch slot 160 CTAs x 8 words
 * of the GPU's nanosecond timer: [0] kernel start, [1] before the dependency wait, [2] released by the preceding
 * kernel, [3] activation row staged, [4] thread 0's last tile done, [5] kernel end, [7] SM id | grid size << 32
 * (zero for CTAs the launch did not have).  `words` is clipped to the buffer; *launches_stamped (may be NULL)
 * receives how many launches have been stamped since the option was set.  No counterpart in the reference. */
int bpq4k_read_stream_stamps(bpq4k_handle_t h, unsigned long long* dst, size_t words, uint32_t* launches_stamped);

/* Number of kernels this handle has launched since creation (or since the
 * counter was last reset with reset != 0).  The reference counts dispatches in
 * GPUContext::timing (runtime/gpu_context.h:223-231). */
uint64_t bpq4k_launch_count(bpq4k_handle_t h, int reset);

/* Read (and clear) the device status word that kernels set when one of their
 * bounded waits runs out; waits for `stream`.  Returns BPQ4K_OK and *status_out = 0
 * when nothing was reported, else that status (BPQ4K_ERR_TIMEOUT).  Stands in for
 * GPUContext's deviceLost / lastAllocFailed flags (runtime/gpu_context.cpp:212-237). */
int bpq4k_device_status(bpq4k_handle_t h, void* stream, int* status_out);

/* ---- host-side packing -------------------------------------------------- */

/* nBlocks and rowStrideWords of KQuantPacked for a given K
 * (runtime/gguf_loader.cpp:366-367). */
uint32_t bpq4k_n_blocks(uint32_t K);
uint32_t bpq4k_row_stride_words(uint32_t K);

/* pack_q4k (runtime/gguf_loader.cpp:359-379): copy N rows of raw blocks into
 * `words_host` (N * bpq4k_row_stride_words(K) words).  Host memory only. */
int bpq4k_pack_q4k_host(const void* raw_host, uint32_t N, uint32_t K, uint32_t* words_host);

/* uploadKQWeight (runtime/model_runner.cpp:958-963): allocate a device buffer
 * and copy packed words into it.  The copy is synchronous.  Free with
 * bpq4k_free_device. */
int bpq4k_upload_weights(bpq4k_handle_t h, const uint32_t* words_host, uint64_t n_words, void** w_dev);
int bpq4k_free_device(bpq4k_handle_t h, void* dev_ptr);

/* ---- device operators ---------------------------------------------------- */

/* dequant_kquant(raw, out, N, K, GGUF_TYPE_Q4_K) (runtime/gguf_loader.cpp:455-496)
 * on the device: out[n*K + k] = (d*sc)*q - dmin*mn, bit-identical to the
 * reference's float arithmetic.  `out` is float[N*K]. */
int bpq4k_dequant_f32(bpq4k_handle_t h, const void* W, uint32_t N, uint32_t K,
                      uint32_t rowStrideWords, float* out, void* stream);

/* The Q4_K matmul dispatch: Y[yOffset + m*N + n] = sum_k X[m*K+k]*deq(W)[n][k] + bias[n].
 * One call covers every shader variant the reference picks by M
 * (runtime/model_runner.cpp:2032-2054, 5841-5845): q4k_matmul.wgsl:20-95,
 * q4k_matmul_128.wgsl:8-17 (yOffset), q4k_matmul_batched4/8.wgsl:9-23; bindings
 * X, W, Bias, Y and params {K, N, nBlocks, rowStrideWords, yOffset}
 * (runtime/model_runner.cpp:2404-2413).  Grid and tile choices are internal.
 * `bias` may be NULL (the reference always binds a zero buffer).  X and W must be
 * 16-byte aligned; Y (outputs are written one float at a time) 4-byte aligned.
 * M >= the PREFILL_MIN_M option goes to the tensor-core kernel in the PREFILL_MODE
 * option's precision; smaller M runs the streaming kernel in slabs of 8 rows. */
int bpq4k_matmul_f32(bpq4k_handle_t h, const float* X, const void* W, const float* bias, float* Y,
                     uint32_t M, uint32_t N, uint32_t K, uint32_t rowStrideWords,
                     uint32_t yOffset, void* stream);

/* Indirect (expert-stacked) form, the ABI of the reference's `*_matmul_moe`
 * shaders (runtime/kernels/quant_kq/iq4xs_matmul_moe.wgsl:5-10,55-66,96-99) with
 * every routed slot served by ONE launch instead of one dispatch per slot
 * (runtime/model_runner.cpp:3584-3651).  W stacks all experts row-wise
 * ([nExperts*N][K], runtime/model_runner.cpp:1520-1562); offsets[s] is the first
 * weight row of slot s's expert (compute_offsets.wgsl:26-36: expert*N).  Slot s
 * reads activation row x_rows[s] of X (x_rows NULL: row s) and writes
 * Y[s*N + n] = sum_k X[x_rows[s]*K + k]*deq(W)[offsets[s]+n][k] + bias[n].
 * `wRows` is the number of rows of the whole stack (nExperts*N): the size of the
 * reference's weight binding, which bounds what the kernel may read. */
int bpq4k_matmul_moe_f32(bpq4k_handle_t h, const float* X, const void* W, const float* bias, float* Y,
                         const uint32_t* offsets, const uint32_t* x_rows, uint32_t nSlots,
                         uint32_t N, uint32_t K, uint32_t rowStrideWords, uint32_t wRows, void* stream);

/* Same operator with HOST activations and HOST outputs: copies X_host to the
 * handle's staging buffer, runs the matmul on the resident device weights and
 * copies Y back, then waits.  This is the per-token host<->device traffic of
 * the reference's decode loop (one input write, one result read-back:
 * runtime/model_runner.cpp:5725-5764).  Allocates staging on first use and
 * when sizes grow. */
int bpq4k_matmul_host_f32(bpq4k_handle_t h, const float* X_host, const void* W_dev,
                          const float* bias_dev, float* Y_host, uint32_t M, uint32_t N, uint32_t K,
                          uint32_t rowStrideWords, void* stream);

/* ---- several GPUs, one process per GPU ------------------------------------ */

/* N-sharded matmul with the all-gather of the output slices fused into the kernel.  The
 * reference is single-GPU; this is what the multi-GPU configurations add.  This rank owns N
 * rows of the global matrix (W is its shard) and computes Y_slice[M][N]; the epilogue stores
 * every value to slot_ptrs[0] (normally the rank's slot in its own gather buffer) and to
 * slot_ptrs[1..nPeers-1] (the same slot in the other ranks' gather buffers, peer-mapped
 * memory: plain stores over NVLink, nothing is loaded from a peer).  M <= 8.  The data is
 * visible to a peer after that peer's next bpq4k_peer_barrier with this rank. */
int bpq4k_matmul_allgather_f32(bpq4k_handle_t h, const float* X, const void* W, const float* bias,
                               float* const* slot_ptrs, uint32_t nPeers, uint32_t M, uint32_t N, uint32_t K,
                               uint32_t rowStrideWords, void* stream);

/* Double-buffered gather slots.  With one gather buffer, a rank that runs ahead could store the slices of step
 * t+1 into a peer's buffer while that peer still reads step t; with two halves used in turn, one barrier per
 * step is enough (a rank that has passed barrier t+1 knows every peer has queued its reads of step t's half
 * ahead of it).  step_word is the step counter that bpq4k_peer_barrier keeps in word 63 of this rank's own
 * flag array (epoch 0 form); the bpq4k_*_allgather_f32 calls that follow store to slot_ptrs[p] +
 * (*step_word & 1) * stride_floats, read on the device when the kernel runs, so a CUDA graph of a step
 * alternates by itself.  The slices of the last completed step are in half ((*step_word - 1) & 1).
 * step_word NULL switches back to single slots.  No counterpart in the reference (single GPU). */
int bpq4k_peer_double_buffer(bpq4k_handle_t h, const uint32_t* step_word, uint64_t stride_floats);

/* Barrier between the ranks' streams over flag words in peer-mapped memory: writes `epoch` to
 * flag_ptrs[p][rank] for every p, then waits until flag_ptrs[rank][p] >= epoch for every p.
 * flag_ptrs[p] is rank p's flag array (64 words, zero-initialised); epochs must grow.  epoch 0
 * means "the next one": the count is kept in word 63 of the rank's own array, which lets a
 * barrier that is replayed from a CUDA graph advance by itself (the word is advanced when the barrier
 * completes).  The kernel is launched with programmatic dependent launch on both sides: it is resident
 * before the kernel ahead of it has drained, and the kernel behind it may prefetch its weights meanwhile.  The
 * wait is bounded: after timeout_ms (0: one second) the kernel gives up and sets the device
 * status word (bpq4k_device_status then reports BPQ4K_ERR_TIMEOUT); it never traps. */
int bpq4k_peer_barrier(bpq4k_handle_t h, uint32_t* const* flag_ptrs, uint32_t nPeers, uint32_t rank,
                       uint32_t epoch, uint32_t timeout_ms, void* stream);

/* A list of matmuls on host buffers served by ONE call: all activations go up, all kernels
 * run, all outputs come back, one wait.  This is how the reference runs a decode step -- a
 * pre-recorded list of Dispatch structs replayed by one queue submit, one small write before
 * and one read-back after (runtime/gpu_context.h:36-44, runtime/model_runner.cpp:4839,
 * 5725-5764).  Entries are independent of each other (no entry reads another's output).
 * With pinned (GPU-addressable) host buffers one kernel gathers all inputs, the streaming kernel
 * stores its outputs straight into the host buffers (they cross the bus while the kernel still
 * streams weights; entries served by the tensor-core kernel are staged and scattered by one kernel),
 * and a list seen twice (same buffers, shapes and options) is replayed from a CUDA graph
 * on a stream of the handle's, ordered after the work already queued on `stream`; other host
 * memory takes one copy per vector.  The call returns when the outputs are in host memory. */
typedef struct bpq4k_host_matmul {
    const float* X_host;      /* M*K floats; pinned host memory makes the copies asynchronous */
    const void* W_dev;        /* resident weights */
    const float* bias_dev;    /* may be NULL */
    float* Y_host;            /* M*N floats */
    uint32_t M, N, K, rowStrideWords;
} bpq4k_host_matmul;

int bpq4k_matmul_host_batch_f32(bpq4k_handle_t h, const bpq4k_host_matmul* items, uint32_t count, void* stream);

/* ---- the Q5_K and Q6_K siblings -------------------------------------------
 * Real "Q4_K_M" files mix Q4_K with Q5_K / Q6_K tensors (token embedding and output
 * head are usually Q6_K).  These entry points take the reference's GGUFType number
 * (runtime/gguf_loader.h:27-30) and accept all three types; for Q4_K they are the
 * entry points above.  Weights are the reference's packed words: raw GGUF blocks
 * (176 B for Q5_K, 210 B for Q6_K), rows rowStrideWords words apart, Q6_K rows
 * padded with zeros to a whole word (pack_q5k / pack_q6k, runtime/gguf_loader.cpp:381-424). */
enum bpq4k_qtype {
    BPQ4K_TYPE_Q4_K = 12,
    BPQ4K_TYPE_Q5_K = 13,
    BPQ4K_TYPE_Q6_K = 14,
    /* Q6_K with every 210-byte block followed by 14 zero bytes (224 bytes, rows 16-byte
     * aligned).  Not a file format: bpq4k_kq_pack_host writes it from raw GGUF blocks, and it
     * is the layout the fast single-row Q6_K kernel (bulk copies, tensor cores) reads; the
     * unpadded type always runs the plain kernel.  It has no counterpart in the reference. */
    BPQ4K_TYPE_Q6_K_PADDED = 0x10E
};

/* Bytes per 256-weight block as stored (144, 176, 210; 224 for the padded type); 0 for an unknown type. */
uint32_t bpq4k_kq_block_bytes(int qtype);
/* rowStrideWords of KQuantPacked: ceil(ceil(K/256) * block bytes / 4). */
uint32_t bpq4k_kq_row_stride_words(int qtype, uint32_t K);
/* pack_q4k / pack_q5k / pack_q6k: N rows of raw GGUF blocks (always the file format: 210-byte
 * blocks for both Q6_K types) into N * rowStrideWords words (host). */
int bpq4k_kq_pack_host(int qtype, const void* raw_host, uint32_t N, uint32_t K, uint32_t* words_host);

/* Q6_K blocks in the file format that are already on the device (N rows of K/256 blocks of 210
 * bytes, no padding) into the layout of `layout_qtype` (BPQ4K_TYPE_Q6_K: the word-padded rows of
 * pack_q6k; BPQ4K_TYPE_Q6_K_PADDED: 224-byte blocks).  out_dev: N * row stride words of that layout.
 * The device-side twin of bpq4k_kq_pack_host for callers that hold raw tensor bytes on the GPU. */
int bpq4k_kq_respace_device(bpq4k_handle_t h, int layout_qtype, const void* raw_dev, uint32_t N, uint32_t K,
                            void* out_dev, void* stream);

/* dequant_kquant(raw, out, N, K, type) (runtime/gguf_loader.cpp:455-573) on the device,
 * bit-identical to the reference's float arithmetic.  W needs 4-byte alignment for Q6_K,
 * 16-byte for the other two. */
int bpq4k_kq_dequant_f32(bpq4k_handle_t h, int qtype, const void* W, uint32_t N, uint32_t K,
                         uint32_t rowStrideWords, float* out, void* stream);

/* Embedding lookup: out[t*K + k] = deq(W)[tokens[t]][k].  Replaces q6k_gather.wgsl (one token)
 * and q6k_gather_batched.wgsl; Q5_K and Q6_K tables.  `tokens` is a device array; a token id
 * >= nRows yields a row of zeros.  The values are those of bpq4k_kq_dequant_f32. */
int bpq4k_kq_gather_f32(bpq4k_handle_t h, int qtype, const void* W, uint32_t nRows, uint32_t K,
                        uint32_t rowStrideWords, const uint32_t* tokens, uint32_t nTokens,
                        float* out, void* stream);

/* The matmul dispatch for any of the three types: q5k_matmul.wgsl, q6k_matmul.wgsl,
 * q6k_matmul_wide.wgsl, q5k/q6k_matmul_batched4.wgsl and the kernel selection at
 * runtime/model_runner.cpp:2032-2054, 4124-4135, 5841-5845.  Arguments as bpq4k_matmul_f32. */
int bpq4k_kq_matmul_f32(bpq4k_handle_t h, int qtype, const float* X, const void* W, const float* bias,
                        float* Y, uint32_t M, uint32_t N, uint32_t K, uint32_t rowStrideWords,
                        uint32_t yOffset, void* stream);

/* The routed-expert feed-forward step of one layer, for T tokens, in three launches (four when the
 * shapes do not allow gate and up to share one).  The reference
 * issues six dispatches per routed slot -- gate, up, silu, mul, down, weighted accumulate
 * (runtime/model_runner.cpp:3584-3651; offsets from compute_offsets.wgsl:26-36; the accumulate step
 * is runtime/kernels/moe/weighted_accumulate_decode.wgsl).  For pair p = t*topk + k with expert
 * e = expert_ids[p]:
 *     g = X[t] . Wgate[e]^T,  u = X[t] . Wup[e]^T          expert-indexed matmuls, F values each
 *     o = (silu(g) * u) . Wdown[e]^T                        silu*up staged by the down matmul itself
 *     Y[t] = Y[t] + route_w[p] * o                          k ascending, as the reference accumulates
 * X and Y are [T][H] (Y is read and written: the caller leaves the residual stream or zeros there),
 * Wgate / Wup stack the experts' [F][H] matrices row-wise, Wdown the [H][F] matrices, all of type
 * `qtype` (Q4_K, Q5_K or padded Q6_K; Q6_K runs gate and up as two launches) with the packed row stride of their K.  expert_ids and route_w are device
 * arrays of T*topk entries; an id >= nExperts reads zeros.  `work` is caller-owned device scratch of
 * at least bpq4k_moe_ffn_work_floats() floats (the call allocates nothing). */
uint64_t bpq4k_moe_ffn_work_floats(uint32_t T, uint32_t topk, uint32_t H, uint32_t F);
int bpq4k_moe_ffn_f32(bpq4k_handle_t h, int qtype, const float* X, const void* Wgate, const void* Wup, const void* Wdown,
                      const uint32_t* expert_ids, const float* route_w, float* Y, uint32_t T, uint32_t topk,
                      uint32_t nExperts, uint32_t H, uint32_t F, float* work, uint64_t work_floats, void* stream);

/* bpq4k_matmul_moe_f32 with the weight type given: Q4_K, Q5_K or padded Q6_K (BPQ4K_TYPE_Q6_K_PADDED,
 * at most 65535 slots) expert stacks. */
int bpq4k_kq_matmul_moe_f32(bpq4k_handle_t h, int qtype, const float* X, const void* W, const float* bias, float* Y,
                            const uint32_t* offsets, const uint32_t* x_rows, uint32_t nSlots, uint32_t N, uint32_t K,
                            uint32_t rowStrideWords, uint32_t wRows, void* stream);

/* bpq4k_matmul_allgather_f32 for the sibling types: Q5_K (M <= 8) and padded Q6_K (M = 1). */
int bpq4k_kq_matmul_allgather_f32(bpq4k_handle_t h, int qtype, const float* X, const void* W, const float* bias,
                                  float* const* slot_ptrs, uint32_t nPeers, uint32_t M, uint32_t N, uint32_t K,
                                  uint32_t rowStrideWords, void* stream);

/* ---- decode matmul with a fused prologue / epilogue -------------------------
 * The single-row (M = 1) matmul with the element-wise step that precedes it computed
 * while the activation row is staged, and an optional residual added to the output:
 *   BPQ4K_PROLOGUE_RMSNORM   x = X * (1/sqrt(mean(X^2) + eps)) * aux,  aux = norm weight[K]
 *                            (q4k_matmul_norm.wgsl:47-92, q5k_matmul_norm.wgsl)
 *   BPQ4K_PROLOGUE_GELU_MUL  x = 0.5*g*(1 + tanh(0.7978845608*(g + 0.044715*g^3))) * aux,
 *                            g = X, aux = the "up" vector[K]  (q4k_down_gelu.wgsl:47-62; the
 *                            reference passes gate and up as one buffer: aux = X + K)
 *   BPQ4K_PROLOGUE_SILU_MUL  x = g/(1 + exp(-g)) * aux   (silu_mul_fused followed by the down
 *                            projection, runtime/model_runner.cpp:3755-3766)
 *   Y[yOffset + n] = sum_k x[k]*deq(W)[n][k] + bias[n] + residual[n]   (bias, residual may be NULL;
 *   the residual add is the dispatch at runtime/model_runner.cpp:3774)
 * Q4_K, Q5_K and padded Q6_K weights.  Each removes one small launch and one round trip of the activation
 * row through memory per projection.  X and aux must be 16-byte aligned. */
enum bpq4k_prologue {
    BPQ4K_PROLOGUE_NONE = 0,
    BPQ4K_PROLOGUE_RMSNORM = 1,
    BPQ4K_PROLOGUE_GELU_MUL = 2,
    BPQ4K_PROLOGUE_SILU_MUL = 3
};
int bpq4k_matmul_fused_f32(bpq4k_handle_t h, int qtype, int prologue, const float* X, const float* aux,
                           float eps, const void* W, const float* bias, const float* residual, float* Y,
                           uint32_t N, uint32_t K, uint32_t rowStrideWords, uint32_t yOffset, void* stream);

/* ---- greedy sampling step ----------------------------------------------------
 * *result = index of the largest of the n logits, in one launch.  Replaces the reference's
 * argmax + argmax_reduce dispatches after the output head (runtime/kernels/shape/argmax.wgsl,
 * argmax_reduce.wgsl; runtime/model_runner.cpp:2246, 2441-2452): same strict comparison against a
 * start value of -1e30 (NaNs and values <= -1e30 never win; 0 when nothing does); on ties, where the
 * reference's answer depends on its scan order, the lowest index.  `logits` and `result` are device
 * pointers.  Calls on one handle that may overlap on the GPU must be serialised by the caller. */
int bpq4k_argmax_f32(bpq4k_handle_t h, const float* logits, uint32_t n, int32_t* result, void* stream);

/* ---- GGUF files ------------------------------------------------------------
 * Reader for the file format the weights come in, and the tensor -> device step.  Stands in for
 * GGUFFile::open and its accessors (runtime/gguf_loader.h:46-91, runtime/gguf_loader.cpp:14-182)
 * and for pack_q*k + uploadKQWeight (runtime/model_runner.cpp:958-963, 1054-1061).  The parser
 * needs no GPU.  Differences from the reference's reader: every length is checked against the
 * file size (a corrupt file is an error, not an allocation), general.alignment is honoured when
 * present (the reference always aligns the tensor data to 32 bytes), and arrays of every scalar
 * type are kept. */
typedef struct bpq4k_gguf* bpq4k_gguf_t;
int bpq4k_gguf_open(const char* path, bpq4k_gguf_t* out); /* UNSUPPORTED: not a GGUF v2+ file or corrupt */
int bpq4k_gguf_close(bpq4k_gguf_t g);
const char* bpq4k_gguf_last_error(bpq4k_gguf_t g);
uint32_t bpq4k_gguf_version(bpq4k_gguf_t g);
uint64_t bpq4k_gguf_n_tensors(bpq4k_gguf_t g);
uint64_t bpq4k_gguf_data_offset(bpq4k_gguf_t g);
/* hasKey / getU32 / getFloat / getBool / getString of the reference, same coercions
 * (getU32: any integer scalar, or the maximum of an int32 array). */
int bpq4k_gguf_has_key(bpq4k_gguf_t g, const char* key);
uint32_t bpq4k_gguf_get_u32(bpq4k_gguf_t g, const char* key, uint32_t def);
float bpq4k_gguf_get_f32(bpq4k_gguf_t g, const char* key, float def);
int bpq4k_gguf_get_bool(bpq4k_gguf_t g, const char* key, int def);
/* String value (index < 0) or element `index` of a string array, copied NUL-terminated into buf
 * (cap bytes; may be NULL to query).  Returns the string's length, -1 if absent or not a string. */
int64_t bpq4k_gguf_get_string(bpq4k_gguf_t g, const char* key, int64_t index, char* buf, uint64_t cap);
int64_t bpq4k_gguf_array_length(bpq4k_gguf_t g, const char* key); /* -1: absent or not an array */
int bpq4k_gguf_get_i32_array(bpq4k_gguf_t g, const char* key, uint64_t first, uint64_t n, int32_t* out);
int bpq4k_gguf_find_tensor(bpq4k_gguf_t g, const char* name, uint64_t* index);
/* name, dims (shape[0] is the contiguous one, K of a weight matrix), GGML type, offset from the
 * start of the tensor data, size in bytes (0 for a type this reader cannot size).  Any output
 * pointer may be NULL. */
int bpq4k_gguf_tensor_info(bpq4k_gguf_t g, uint64_t index, const char** name, uint32_t* n_dims, uint64_t shape[4],
                           uint32_t* type, uint64_t* offset, uint64_t* n_bytes);
int bpq4k_gguf_read_tensor(bpq4k_gguf_t g, uint64_t index, uint64_t first, uint64_t n, void* dst_host);
/* A Q4_K / Q5_K / Q6_K tensor from the file into device memory on the handle's device, in the layout
 * the matmul entry points take (layout_qtype 0: the packed layout of the tensor's type;
 * BPQ4K_TYPE_Q6_K_PADDED for a Q6_K tensor: the padded one).  N = product of the dims after the
 * first.  Free *w_dev with bpq4k_free_device.  Synchronous. */
int bpq4k_gguf_upload_tensor(bpq4k_handle_t h, bpq4k_gguf_t g, uint64_t index, int layout_qtype, void** w_dev,
                             int* qtype_out, uint32_t* N_out, uint32_t* K_out, uint32_t* rowStrideWords_out);

/* Several tensors of one K-quant type and one row length, concatenated by rows into ONE device allocation:
 * fuseKQ + uploadKQWeight (runtime/model_runner.cpp:1002-1012, 958-963) without the host-side copy.  Arguments
 * as bpq4k_gguf_upload_tensor, with `count` tensor indices; N_out is the sum of the rows. */
int bpq4k_gguf_upload_fused(bpq4k_handle_t h, bpq4k_gguf_t g, const uint64_t* indices, uint32_t count, int layout_qtype,
                            void** w_dev, int* qtype_out, uint32_t* N_out, uint32_t* K_out, uint32_t* rowStrideWords_out);

/* ModelConfig as extractModelConfig fills it (runtime/gguf_loader.h:164-224, runtime/gguf_loader.cpp:184-317):
 * same fields, same keys, same defaults.  activation: 0 SiLU, 1 GELU (the Gemma family).  The per-layer
 * attention types (0 global, 1 sliding window; present only when slidingWindow > 0) are written to
 * layer_attn_types[0 .. min(cap, nLayerAttnTypes)) when that pointer is given. */
typedef struct bpq4k_model_config {
    char arch[64];
    uint32_t nLayer, nHead, nKvHeads, nEmbd, intermediateSize, nVocab, headDim, kvHeadDim;
    float rmsNormEps, ropeTheta;
    int32_t tieWordEmbeddings, hasQkNorm;
    int32_t activation;
    float embeddingScale, logitSoftcap;
    uint32_t slidingWindow, nLayerAttnTypes;
    int32_t hasSandwichNorm;
    uint32_t pleSize, sharedKvLayers;
    int32_t hasMtp;
    uint32_t mtpNumLayers;
    uint32_t numExperts, numExpertsPerTok, moeIntermediateSize, moeSharedIntermediateSize;
    uint32_t ssmInnerSize, ssmStateSize, ssmConvKernel, ssmGroupCount, ssmTimeStepRank, fullAttentionInterval;
    int32_t ropeSections[4];
} bpq4k_model_config;
int bpq4k_gguf_model_config(bpq4k_gguf_t g, bpq4k_model_config* out, uint8_t* layer_attn_types, uint32_t cap);

/* The loader's quantisation probe (runtime/model_runner.cpp:1014-1049): *qtype = GGML type of the first of
 * blk.0.attn_q / attn_qkv / ffn_gate / ffn_down that exists (-1: none), *uniform_kquant = 1 when attn_q, ffn_gate
 * and ffn_down of layer 0 all carry that one K-quant type (the reference's `isKQuant`). */
int bpq4k_gguf_weight_format(bpq4k_gguf_t g, int* qtype, int* uniform_kquant);

/* A layer's projection weights on the device, with the loader's fusion rules (runtime/model_runner.cpp:1223-1370):
 * Q+K+V by rows into `qkv` (n_fused = 3; a file's pre-fused attn_qkv: n_fused = 1, qkv_prefused = 1), attn_output
 * into `o`, gate+up into `gate_up` (n_fused = 2), ffn_down into `down`.  A group is fused when all members are
 * K-quant tensors of one type and one row length; otherwise each K-quant member is uploaded on its own (q, k, v,
 * gate, up) -- the reference sends such layers through its Q8 re-quantisation, which this library does not have,
 * and its fuseKQ would give a mixed-type group the first member's row stride.  Absent or non-K-quant members:
 * w = NULL, qtype = the file's GGML type or -1.  q6_layout = BPQ4K_TYPE_Q6_K_PADDED stores Q6_K tensors in the
 * padded layout of the fast kernels.  Free with bpq4k_free_layer. */
typedef struct bpq4k_kq_tensor {
    void* w;
    int32_t qtype;
    uint32_t N, K, rowStrideWords, n_fused;
} bpq4k_kq_tensor;
typedef struct bpq4k_layer_weights {
    bpq4k_kq_tensor qkv, q, k, v, o, gate_up, gate, up, down;
    int32_t qkv_prefused;
} bpq4k_layer_weights;
int bpq4k_gguf_load_layer(bpq4k_handle_t h, bpq4k_gguf_t g, uint32_t layer, int q6_layout, bpq4k_layer_weights* out);
int bpq4k_free_layer(bpq4k_handle_t h, bpq4k_layer_weights* lw);

/* The small-M matmul for callers that must not allocate device memory.  It has no counterpart
 * in the reference.
 *
 * Such callers exist: a serving process that has handed all free device memory to its own pool
 * (an allocation made by a library would fail or eat into that pool's budget), and any path
 * that cannot afford the device-wide synchronisation inside cudaMalloc/cudaFree, such as a
 * decode loop with other streams in flight.  They cannot create a handle either (bpq4k_create
 * allocates), so this entry point takes none.
 *
 * Same arguments and result as bpq4k_matmul_f32 for M <= 8.  Its working memory (the
 * activations re-coded for the tensor cores) is a fixed array inside the library, present on
 * every device that loads it, so:
 *   - sizes are limited: M <= 8 and R * K <= BPQ4K_NOALLOC_MAX_MK with R = 1 for M = 1, else M rounded
 *     up to a multiple of 4,
 *     otherwise BPQ4K_ERR_UNSUPPORTED and a message in bpq4k_noalloc_last_error();
 *   - all calls on a device share that array: calls that may overlap on the GPU (different
 *     streams without an ordering between them, or different threads) race and must be
 *     serialised by the caller; the array keeps the last call's contents, and each call
 *     rewrites everything it will read, so no clearing is needed between calls;
 *   - the first call on each device looks up the array's address on that device and should be
 *     made before any stream capture begins.
 * No cudaMalloc, cudaFree or allocating library routine is called.  Errors are reported per
 * thread by bpq4k_noalloc_last_error(). */
#define BPQ4K_NOALLOC_MAX_MK 131072u
int bpq4k_matmul_noalloc_f32(const float* X, const void* W, const float* bias, float* Y,
                             uint32_t M, uint32_t N, uint32_t K, uint32_t rowStrideWords,
                             uint32_t yOffset, void* stream);
const char* bpq4k_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* BPQ4K_H */
