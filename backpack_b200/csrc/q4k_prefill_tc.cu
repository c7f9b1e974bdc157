// Prefill Q4_K matmul (M >= 25 by default) on the 5th-generation tensor cores: weights are dequantised
// on chip into 16-bit tiles, multiplied with tcgen05.mma, accumulated in TMEM.
//
// The reference has no tensor-core path for Q4_K: its "prefill" is q4k_matmul_batched8
// (runtime/kernels/quant_kq/q4k_matmul_batched8.wgsl:9-23, picked at
// runtime/model_runner.cpp:5841-5845), scalar FMAs that re-read the weights M/8 times, or
// serial decode (runtime/model_runner.cpp:4447-4471).  This kernel reads each weight once per
// 256 activation rows.
//
//   Y[m][n] = sum_k X[m][k] * deq(W)[n][k] + bias[n]
//
// MMA orientation: D[weight row][activation row] = A[weight row][k] * B[activation row][k]^T, so
// the 128 TMEM lanes are weight rows and the accumulator columns are activation rows (N_mma = 256).
// A CTA owns ROWS weight rows (ROWS/128 accumulators of 256 columns) x 256 activation rows and
// walks K in steps of 64 (one 64-weight group of a super-block = one 128-byte swizzle row).
//
// Roles (warp-specialised, all hand-offs through mbarriers):
//   warp 0        one lane issues the TMA loads of the activation tile (16-bit, K-major,
//                 SWIZZLE_128B; plain loads, no multicast)
//   warp 1        allocates TMEM; one lane issues tcgen05.mma and tcgen05.commit
//   warps 2..     thread r dequantises weight row r: raw super-block (144 B, prefetched into
//                 registers one block ahead) -> w = (d*sc)*q - dmin*mn in float -> 16-bit ->
//                 the K-major 128-byte-swizzled A tile; afterwards the same warps drain TMEM
//                 (tcgen05.ld), add the bias and store Y.
//
// Precision modes: one pass in half or bfloat16 (weights and activations rounded to 16 bits), or
// three passes with W = Wh + Wl, X = Xh + Xl in half (Wh*Xh + Wh*Xl + Wl*Xh, all into the same
// accumulator), which meets the float tolerance of the path.
//
// Every wait is bounded: on a time-out the role raises the CTA's abort flag and the device status
// word, every role leaves its loop, TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>

#include "kernels.h"
#include "q4k_common.cuh"

namespace bpq4k {

namespace {

constexpr uint32_t kTokTile = 256;   // activation rows per CTA tile (= mma N)
constexpr uint32_t kKStep = 64;      // k per pipeline stage
constexpr uint32_t kWaitLimit = 1u << 24;

struct PrefillArgs {
    CUtensorMap tmap_x[2];  // [0]: X (or its high part), [1]: low part (three-pass mode)
    const uint8_t* W;
    const float* bias;
    float* Y;
    uint32_t M, N, K;
    uint64_t w_row_bytes;
    int* status;
    // split-K: blockIdx.z takes super-blocks [z*bps, (z+1)*bps) and writes Ypart[z] (no bias);
    // splitk_reduce_kernel adds the slices in a fixed order.  ksplit == 1: the kernel writes Y.
    uint32_t ksplit, bps;
    float* Ypart;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait.  Returns false if the CTA is aborting (this wait or another role's timed out).
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicExch(status, kDeviceTimeout);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 B apart, 8-row groups
// 1024 B apart (SBO), version 1 (sm_100), LBO unused (1).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: D = f32, A/B = f16 (0) or bf16 (1), both K-major, M = 128, N = 256.
__device__ __forceinline__ constexpr uint32_t umma_idesc(bool bf16) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((kTokTile >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if constexpr (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    } else {
        const __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
}
// low part of a half split: half(x - float(half(x)))
__device__ __forceinline__ uint32_t pack2_lo(float a, float b, uint32_t hi_bits) {
    const __half2 hi = *reinterpret_cast<const __half2*>(&hi_bits);
    const float2 hf = __half22float2(hi);
    const __half2 v = __floats2half2_rn(a - hf.x, b - hf.y);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Single-pass modes: dequantise one code word (four code bytes = four weights of the even and four
// of the odd sub-block) entirely in packed 16-bit arithmetic.  The nibbles are dropped into the
// mantissa of a constant (half: 0x6400 = 1024, bfloat16: 0x4300 = 128), one packed subtract or
// fma recovers the integer q exactly, one packed fma applies w = dsc*q - dmn.  About 1.75
// instructions per weight instead of 4.5 through float; the scales are rounded to 16 bits first,
// which these modes round the weights to anyway.
//   out[0] = even (w0, w1), out[1] = even (w2, w3), out[2] = odd (w0, w1), out[3] = odd (w2, w3)
template <bool BF16>
__device__ __forceinline__ void dequant_word_16(uint32_t w, uint32_t dsc_e2, uint32_t ndmn_e2, uint32_t dsc_o2,
                                                uint32_t ndmn_o2, uint32_t (&out)[4]) {
    // bytes (0, x, 1, x) and (2, x, 3, x) in the low bytes of the two halves: neighbours land in one packed pair
    // and no further shift is needed for the low nibbles
    const uint32_t t = __byte_perm(w, 0u, 0x3120u), t2 = __byte_perm(w, 0u, 0x1302u);
    if constexpr (BF16) {
        const uint32_t u = t >> 4, u2 = t2 >> 4;
        const uint32_t e0 = (t & 0x000F000Fu) | 0x43004300u, e1 = (t2 & 0x000F000Fu) | 0x43004300u;  // 128 + q
        const uint32_t o0 = (u & 0x000F000Fu) | 0x43004300u, o1 = (u2 & 0x000F000Fu) | 0x43004300u;
        auto conv = [](uint32_t x, uint32_t dsc2, uint32_t ndmn2) -> uint32_t {
            const __nv_bfloat162 k128 = __float2bfloat162_rn(128.f);
            const __nv_bfloat162 q = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&x), k128);
            const __nv_bfloat162 r = __hfma2(q, *reinterpret_cast<const __nv_bfloat162*>(&dsc2),
                                             *reinterpret_cast<const __nv_bfloat162*>(&ndmn2));
            return *reinterpret_cast<const uint32_t*>(&r);
        };
        out[0] = conv(e0, dsc_e2, ndmn_e2);
        out[1] = conv(e1, dsc_e2, ndmn_e2);
        out[2] = conv(o0, dsc_o2, ndmn_o2);
        out[3] = conv(o1, dsc_o2, ndmn_o2);
    } else {
        const uint32_t e0 = (t & 0x000F000Fu) | 0x64006400u, e1 = (t2 & 0x000F000Fu) | 0x64006400u;  // 1024 + q
        const uint32_t o0 = (t & 0x00F000F0u) | 0x64006400u, o1 = (t2 & 0x00F000F0u) | 0x64006400u;  // 1024 + 16 q
        const __half2 k1024 = __float2half2_rn(1024.f), k16th = __float2half2_rn(0.0625f), k64 = __float2half2_rn(64.f);
        auto fin = [](const __half2 q, uint32_t dsc2, uint32_t ndmn2) -> uint32_t {
            const __half2 r = __hfma2(q, *reinterpret_cast<const __half2*>(&dsc2), *reinterpret_cast<const __half2*>(&ndmn2));
            return *reinterpret_cast<const uint32_t*>(&r);
        };
        out[0] = fin(__hsub2(*reinterpret_cast<const __half2*>(&e0), k1024), dsc_e2, ndmn_e2);
        out[1] = fin(__hsub2(*reinterpret_cast<const __half2*>(&e1), k1024), dsc_e2, ndmn_e2);
        out[2] = fin(__hfma2(*reinterpret_cast<const __half2*>(&o0), k16th, __hneg2(k64)), dsc_o2, ndmn_o2);
        out[3] = fin(__hfma2(*reinterpret_cast<const __half2*>(&o1), k16th, __hneg2(k64)), dsc_o2, ndmn_o2);
    }
}

// Shared-memory plan (all tiles 1024-byte aligned for the 128-byte swizzle):
//   per stage: NV versions (1, or hi+lo) of the A tile [ROWS x 128 B] and of the B tile [256 x 128 B]
// SPLIT: dequantising threads per weight row of a stage.  Three-pass mode of Q4_K and Q5_K: two, each takes 32 of the
// stage's 64 weights through float (128256 x 4096, M = 512: 484 against 440 TFLOP/s with one thread per row -- twice
// the warps hide each other's latencies).  The single-pass modes keep one thread per row: two threads sharing every
// stage measured 892 against 985 TFLOP/s over the eight projections (scale preparation and barrier traffic double
// while the packed 16-bit dequantisation itself is short), two threads taking alternate stages 1158 against 1209
// on the largest one.  Q6_K keeps one thread per row.
template <int ROWS, int PASSES, int QT = 0>
struct Plan {
    static constexpr uint32_t SPLIT = (QT == 2 || PASSES == 1) ? 1 : 2;
    static constexpr uint32_t NV = PASSES == 3 ? 2 : 1;
    static constexpr uint32_t A_BYTES = ROWS * 128u, B_BYTES = kTokTile * 128u;
    static constexpr uint32_t STAGE_BYTES = NV * (A_BYTES + B_BYTES);
    static constexpr uint32_t STAGES = (200u * 1024u) / STAGE_BYTES;
    static constexpr uint32_t ROW_WARPS = ROWS / 32;
    static constexpr uint32_t DEQ_WARPS = ROW_WARPS * SPLIT;
    static constexpr uint32_t THREADS = (2 + DEQ_WARPS) * 32;
    // three-pass mode: a second accumulator takes the two small cross terms (see the mma issuer)
    static constexpr uint32_t TMEM_COLS = (PASSES == 3 ? 2 : ROWS / 128) * kTokTile;
    static constexpr uint32_t SMEM_BYTES = 1024 /*align slack*/ + STAGES * STAGE_BYTES + 256 /*barriers*/;
};

// Q5: Q5_K weights (176-byte blocks: the Q4_K header, 32 bytes of fifth bits, 128 nibble bytes); the
// fifth bit is merged into the code before the float dequantisation (the packed 16-bit shortcut of the
// single-pass modes is Q4_K only).
// QT = 2: Q6_K weights in the padded layout (224-byte blocks: 128 nibble bytes, 64 bit-pair bytes, 16 signed
// scales, half d, padding); w = d*sc*(code - 32) with one scale per 16 weights.
template <int ROWS, int PASSES, bool BF16, int QT = 0>
__global__ void __launch_bounds__(Plan<ROWS, PASSES, QT>::THREADS, 1) prefill_tc_kernel(const __grid_constant__ PrefillArgs a) {
    constexpr bool Q5 = QT == 1, Q6 = QT == 2;
    constexpr int BU = Q6 ? 14 : Q5 ? 11 : 9;   // 16-byte units per super-block
    constexpr int CU = Q5 ? 3 : 1;              // first unit of the nibble bytes (Q4_K, Q5_K)
    using P = Plan<ROWS, PASSES, QT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_base = base + P::STAGES * P::STAGE_BYTES;
    // barriers: full[s] (dequant warps + TMA producer), empty[s] (mma commit), acc_full
    auto full_bar = [&](uint32_t s) { return bar_base + s * 8u; };
    auto empty_bar = [&](uint32_t s) { return bar_base + (P::STAGES + s) * 8u; };
    const uint32_t acc_bar = bar_base + 2u * P::STAGES * 8u;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + P::STAGES * P::STAGE_BYTES + 2u * P::STAGES * 8u + 16u);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + P::STAGES * P::STAGE_BYTES + 2u * P::STAGES * 8u + 32u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n0 = blockIdx.x * ROWS, tok0 = blockIdx.y * kTokTile;
    const uint32_t blk0 = blockIdx.z * a.bps;                          // first super-block of this K slice
    const uint32_t blk1 = min(a.K / kQK, blk0 + a.bps);
    const uint32_t nkb = (blk1 - blk0) * 4u;                           // pipeline iterations (64 k each)
    const uint32_t kbase = blk0 * kQK;                                 // first k of the slice

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < P::STAGES; s++) {
            mbar_init(full_bar(s), P::DEQ_WARPS + 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // TMEM allocation by one whole warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(P::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    auto a_tile = [&](uint32_t s, uint32_t v) { return base + s * P::STAGE_BYTES + v * P::A_BYTES; };
    auto b_tile = [&](uint32_t s, uint32_t v) { return base + s * P::STAGE_BYTES + P::NV * P::A_BYTES + v * P::B_BYTES; };

    if (warp == 0) {
        // ---------------- TMA producer: activation tiles ----------------
        if (lane == 0) {
            for (uint32_t kb = 0; kb < nkb; kb++) {
                const uint32_t s = kb % P::STAGES, it = kb / P::STAGES;
                if (it > 0 && !wait_bar(empty_bar(s), (it - 1) & 1u, abort_flag, a.status)) break;
                mbar_expect_tx(full_bar(s), P::NV * P::B_BYTES);
                for (uint32_t v = 0; v < P::NV; v++) tma_load_2d(b_tile(s, v), &a.tmap_x[v], kbase + kb * kKStep, tok0, full_bar(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(BF16);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; kb++) {
                const uint32_t s = kb % P::STAGES, it = kb / P::STAGES;
                ok = wait_bar(full_bar(s), it & 1u, abort_flag, a.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t ks = 0; ks < kKStep / 16; ks++) {
                    const uint32_t acc = (kb | ks) ? 1u : 0u;
#pragma unroll
                    for (uint32_t r = 0; r < (uint32_t)ROWS / 128; r++) {
                        // a 128-row half of the A tile is 16 KiB further on; a k-step of 16 is 32 B inside the swizzle row
                        const uint64_t da_h = umma_desc(a_tile(s, 0) + r * 16384u + ks * 32u);
                        const uint64_t db_h = umma_desc(b_tile(s, 0) + ks * 32u);
                        const uint32_t d = tmem_base + r * kTokTile;
                        umma_f16(d, da_h, db_h, idesc, acc);
                        if constexpr (PASSES == 3) {
                            // The tensor core truncates when it adds into a float accumulator, so the error
                            // of a long K grows with the number of accumulations times the accumulator's
                            // magnitude.  The cross terms Wh*Xl + Wl*Xh are 2^-11 of the main term: they get
                            // an accumulator of their own (columns 256..511) and are added in the epilogue,
                            // which leaves the large accumulator with a third of the accumulations.
                            const uint64_t da_l = umma_desc(a_tile(s, 1) + r * 16384u + ks * 32u);
                            const uint64_t db_l = umma_desc(b_tile(s, 1) + ks * 32u);
                            umma_f16(d + kTokTile, da_h, db_l, idesc, acc);
                            umma_f16(d + kTokTile, da_l, db_h, idesc, 1u);
                        }
                    }
                }
                umma_commit(empty_bar(s));  // the stage's smem may be overwritten once these mmas retire
            }
            if (ok) umma_commit(acc_bar);
        }
    } else {
        // ---------------- dequantise (thread = weight row), then drain TMEM ----------------
        const uint32_t dw = warp - 2;              // 0 .. DEQ_WARPS-1
        const uint32_t r = (dw % P::ROW_WARPS) * 32u + lane;  // row inside the tile
        [[maybe_unused]] const uint32_t part = dw / P::ROW_WARPS;  // which 32 of a stage's 64 weights (SPLIT = 2)
        const uint32_t n = n0 + r;
        const bool row_ok = n < a.N;
        // rows past N read the last row: their accumulator lanes are never stored
        const uint4* wrow = reinterpret_cast<const uint4*>(a.W + (uint64_t)(row_ok ? n : (Q6 ? 0u : a.N - 1u)) * a.w_row_bytes);
        const uint32_t nblocks = blk1 - blk0;
        wrow += (uint64_t)blk0 * BU;
        bool ok = true;
        // swizzled address of 16-byte chunk c of row r: 8-row group base + row*128 + ((c ^ (r&7)) * 16)
        const uint32_t row_off = (r >> 3) * 1024u + (r & 7u) * 128u;
        const uint32_t sw = r & 7u;
        if constexpr (Q6) {
            // Per half of 128 weights six units (64 nibble bytes, 32 bit-pair bytes) serve two k-steps of 64:
            // the low nibbles first, then the high ones.  The next half is fetched while this one is used.
            const uint4 zero4 = make_uint4(0, 0, 0, 0);
            uint4 cur[6], nx[6], scu = zero4, dun = zero4, scn = zero4, dnn = zero4;
            auto load_half = [&](uint32_t b, uint32_t h, uint4 (&dst)[6]) {
                const uint4* p = wrow + (uint64_t)b * 14u;
#pragma unroll
                for (int i = 0; i < 4; i++) dst[i] = __ldg(p + h * 4u + i);
                dst[4] = __ldg(p + 8u + h * 2u);
                dst[5] = __ldg(p + 9u + h * 2u);
            };
#pragma unroll
            for (int i = 0; i < 6; i++) nx[i] = zero4;
            if (row_ok && nblocks) {
                load_half(0, 0, nx);
                scn = __ldg(wrow + 12);
                dnn = __ldg(wrow + 13);
            }
            for (uint32_t b = 0; b < nblocks && ok; b++) {
                scu = scn;
                dun = dnn;
                const float d = half_bits_to_float(dun.x);
#pragma unroll
                for (uint32_t h = 0; h < 2; h++) {
#pragma unroll
                    for (int i = 0; i < 6; i++) cur[i] = nx[i];
                    if (row_ok) {
                        if (h == 0) {
                            load_half(b, 1, nx);
                        } else if (b + 1 < nblocks) {
                            load_half(b + 1, 0, nx);
                            scn = __ldg(wrow + (uint64_t)(b + 1) * 14u + 12);
                            dnn = __ldg(wrow + (uint64_t)(b + 1) * 14u + 13);
                        }
                    }
                    const uint32_t wa[8] = {cur[0].x, cur[0].y, cur[0].z, cur[0].w, cur[1].x, cur[1].y, cur[1].z, cur[1].w};
                    const uint32_t wb[8] = {cur[2].x, cur[2].y, cur[2].z, cur[2].w, cur[3].x, cur[3].y, cur[3].z, cur[3].w};
                    const uint32_t wq[8] = {cur[4].x, cur[4].y, cur[4].z, cur[4].w, cur[5].x, cur[5].y, cur[5].z, cur[5].w};
#pragma unroll
                    for (uint32_t gl = 0; gl < 2 && ok; gl++) {
                        const uint32_t g = 2u * h + gl, kb = b * 4u + g;
                        const uint32_t s = kb % P::STAGES, it = kb / P::STAGES;
                        if (it > 0 && !wait_bar(empty_bar(s), (it - 1) & 1u, abort_flag, a.status)) {
                            ok = false;
                            break;
                        }
                        // the k-step's four scales: first group of 32 (weights < 16, >= 16), second group (same)
                        const uint32_t scw = h ? (gl ? scu.w : scu.z) : (gl ? scu.y : scu.x);
                        float ds[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) ds[i] = d * (float)(int)(int8_t)((scw >> (8 * i)) & 0xFFu);
                        const uint32_t ta = a_tile(s, 0) + row_off;
#pragma unroll
                        for (uint32_t c = 0; c < 4; c++) {
                            uint32_t lo_bits[4], hi_bits[4], lo_l[4], hi_l[4];
                            const float dsa = ds[c >> 1], dsb = ds[2 + (c >> 1)];
#pragma unroll
                            for (uint32_t j = 0; j < 2; j++) {
                                const uint32_t va = wa[2 * c + j] >> (4 * gl), vb = wb[2 * c + j] >> (4 * gl), vq = wq[2 * c + j] >> (4 * gl);
                                float e[4], o[4];
#pragma unroll
                                for (uint32_t q = 0; q < 4; q++) {
                                    const uint32_t ca = ((va >> (8 * q)) & 15u) | (((vq >> (8 * q)) & 3u) << 4);
                                    const uint32_t cb2 = ((vb >> (8 * q)) & 15u) | (((vq >> (8 * q + 2)) & 3u) << 4);
                                    const float qa = __uint_as_float(ca | 0x4B000000u) - 8388640.f;   // code - 32
                                    const float qb = __uint_as_float(cb2 | 0x4B000000u) - 8388640.f;
                                    e[q] = dsa * qa;
                                    o[q] = dsb * qb;
                                }
                                lo_bits[2 * j] = pack2<BF16>(e[0], e[1]);
                                lo_bits[2 * j + 1] = pack2<BF16>(e[2], e[3]);
                                hi_bits[2 * j] = pack2<BF16>(o[0], o[1]);
                                hi_bits[2 * j + 1] = pack2<BF16>(o[2], o[3]);
                                if constexpr (PASSES == 3) {
                                    lo_l[2 * j] = pack2_lo(e[0], e[1], lo_bits[2 * j]);
                                    lo_l[2 * j + 1] = pack2_lo(e[2], e[3], lo_bits[2 * j + 1]);
                                    hi_l[2 * j] = pack2_lo(o[0], o[1], hi_bits[2 * j]);
                                    hi_l[2 * j + 1] = pack2_lo(o[2], o[3], hi_bits[2 * j + 1]);
                                }
                            }
                            if (!row_ok) {
#pragma unroll
                                for (int q = 0; q < 4; q++) lo_bits[q] = hi_bits[q] = lo_l[q] = hi_l[q] = 0u;
                            }
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ta + ((c ^ sw) << 4)), "r"(lo_bits[0]),
                                         "r"(lo_bits[1]), "r"(lo_bits[2]), "r"(lo_bits[3])
                                         : "memory");
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ta + (((c + 4u) ^ sw) << 4)), "r"(hi_bits[0]),
                                         "r"(hi_bits[1]), "r"(hi_bits[2]), "r"(hi_bits[3])
                                         : "memory");
                            if constexpr (PASSES == 3) {
                                const uint32_t tl = a_tile(s, 1) + row_off;
                                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tl + ((c ^ sw) << 4)), "r"(lo_l[0]),
                                             "r"(lo_l[1]), "r"(lo_l[2]), "r"(lo_l[3])
                                             : "memory");
                                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tl + (((c + 4u) ^ sw) << 4)), "r"(hi_l[0]),
                                             "r"(hi_l[1]), "r"(hi_l[2]), "r"(hi_l[3])
                                             : "memory");
                            }
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full_bar(s));
                    }
                    if (!ok) break;
                }
            }
        } else {
        // This thread's share of a super-block: the header, (Q5_K) one unit of fifth bits and, of each 64-weight
        // group, the 16 code bytes `part` (weights 16*part .. 16*part+15 of the even and of the odd sub-block).
        constexpr bool HALF_ROW = P::SPLIT == 2;
        constexpr int PARTS = HALF_ROW ? 1 : 2;           // 16-byte code units per group this thread handles
        constexpr int GH = 4;                             // 64-weight groups of a super-block
        constexpr int RU = 1 + GH * PARTS + (Q5 ? PARTS : 0);
        const uint32_t upart = HALF_ROW ? part : 0u;      // which half of a group's code bytes
        uint4 raw[RU], nxt[RU];
        auto load_block = [&](uint32_t b, uint4 (&dst)[RU]) {
            const uint4* p = wrow + (uint64_t)b * BU;
            dst[0] = __ldg(p);
#pragma unroll
            for (int gi = 0; gi < GH; gi++)
#pragma unroll
                for (int q = 0; q < PARTS; q++) dst[1 + gi * PARTS + q] = __ldg(p + CU + 2 * gi + upart * PARTS + q);
            if constexpr (Q5)
#pragma unroll
                for (int q = 0; q < PARTS; q++) dst[1 + GH * PARTS + q] = __ldg(p + 1 + upart * PARTS + q);
        };
        if (nblocks) load_block(0, nxt);
        // running pipeline position (stage, parity of the stage's previous use) instead of a division per stage
        uint32_t st_s = 0, st_it = 0;   // stage and how often the ring has wrapped before it
        // swizzled byte offsets of this thread's chunks inside an A tile (loop-invariant)
        uint32_t choff[2 * PARTS][2];
#pragma unroll
        for (uint32_t cl = 0; cl < 2u * PARTS; cl++) {
            const uint32_t c = 2u * PARTS * upart + cl;
            choff[cl][0] = row_off + ((c ^ sw) << 4);
            choff[cl][1] = row_off + (((c + 4u) ^ sw) << 4);
        }
        for (uint32_t b = 0; b < nblocks && ok; b++) {
#pragma unroll
            for (int i = 0; i < RU; i++) raw[i] = nxt[i];
            if (b + 1 < nblocks) load_block(b + 1, nxt);
            // Q5_K: the four words of fifth bits of this part (word w: weights 16*part + 4w..4w+3 of every sub-block)
            [[maybe_unused]] uint32_t qhw[4 * PARTS];
            if constexpr (Q5) {
#pragma unroll
                for (int q = 0; q < PARTS; q++) {
                    const uint4 u = raw[1 + GH * PARTS + q];
                    qhw[4 * q] = u.x, qhw[4 * q + 1] = u.y, qhw[4 * q + 2] = u.z, qhw[4 * q + 3] = u.w;
                }
            }
            const BlockHeader h{raw[0].x, raw[0].y, raw[0].z, raw[0].w};
            const float d = half_bits_to_float(h.w0), dmin = half_bits_to_float(h.w0 >> 16);
            uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
            unpack_scales_packed(h, sc_lo, sc_hi, mn_lo, mn_hi);
#pragma unroll
            for (uint32_t gi = 0; gi < (uint32_t)GH; gi++) {
                const uint32_t g = gi;
                // The stage's 16-bit values are computed BEFORE its buffer is waited for: in steady state the buffer
                // is what the warp waits on, and only the stores, the fence and the arrival are left on the path
                // between "buffer free" and "tile ready" (no measurable change by itself: the stores and the fence
                // are the long part of that path).
                // w = (d*sc)*q - dmin*mn in float, rounded to 16 bits afterwards
                const float dsc_e = d * (float)byte_of(sc_lo, sc_hi, 2 * g), dmn_e = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g);
                const float dsc_o = d * (float)byte_of(sc_lo, sc_hi, 2 * g + 1), dmn_o = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g + 1);
                uint32_t words[4 * PARTS];  // this thread's code bytes of the group
#pragma unroll
                for (int q = 0; q < PARTS; q++) {
                    const uint4 u = raw[1 + gi * PARTS + q];
                    words[4 * q] = u.x, words[4 * q + 1] = u.y, words[4 * q + 2] = u.z, words[4 * q + 3] = u.w;
                }
                [[maybe_unused]] uint32_t dsc_e2 = 0, ndmn_e2 = 0, dsc_o2 = 0, ndmn_o2 = 0;
                if constexpr (PASSES == 1 && !Q5) {
                    dsc_e2 = pack2<BF16>(dsc_e, dsc_e), ndmn_e2 = pack2<BF16>(-dmn_e, -dmn_e);
                    dsc_o2 = pack2<BF16>(dsc_o, dsc_o), ndmn_o2 = pack2<BF16>(-dmn_o, -dmn_o);
                }
                uint32_t lo_bits[2 * PARTS][4], hi_bits[2 * PARTS][4];
                [[maybe_unused]] uint32_t lo_l[2 * PARTS][4], hi_l[2 * PARTS][4];
#pragma unroll
                for (uint32_t cl = 0; cl < 2u * PARTS; cl++) {  // chunk c: weights 8c..8c+7 of the even sub-block, chunk c+4: of the odd one
                    if constexpr (PASSES == 1 && !Q5) {
#pragma unroll
                        for (uint32_t j = 0; j < 2; j++) {
                            uint32_t o4[4];
                            dequant_word_16<BF16>(words[2 * cl + j], dsc_e2, ndmn_e2, dsc_o2, ndmn_o2, o4);
                            lo_bits[cl][2 * j] = o4[0];
                            lo_bits[cl][2 * j + 1] = o4[1];
                            hi_bits[cl][2 * j] = o4[2];
                            hi_bits[cl][2 * j + 1] = o4[3];
                        }
                    } else {
#pragma unroll
                    for (uint32_t j = 0; j < 2; j++) {
                        const uint32_t w = words[2 * cl + j];
                        float e[4], o[4];
#pragma unroll
                        for (uint32_t q = 0; q < 4; q++) {
                            // 0x4B000000 | q is the float 2^23 + q: one subtraction gives q without the
                            // (slow) integer-to-float unit; w = dsc*q - dmn as one fma (the rounding to
                            // 16 bits that follows is 2^13 times coarser than the fma/mul+sub difference)
                            uint32_t ce = (w >> (8 * q)) & 15u, co = (w >> (8 * q + 4)) & 15u;
                            if constexpr (Q5) {
                                const uint32_t hq = qhw[2 * cl + j] >> (8 * q + 2 * g);  // bits 2g, 2g+1 of the weight's byte
                                ce |= (hq & 1u) << 4;
                                co |= (hq & 2u) << 3;
                            }
                            const float qe = __uint_as_float(ce | 0x4B000000u) - 8388608.f;
                            const float qo = __uint_as_float(co | 0x4B000000u) - 8388608.f;
                            e[q] = fmaf(dsc_e, qe, -dmn_e);
                            o[q] = fmaf(dsc_o, qo, -dmn_o);
                        }
                        lo_bits[cl][2 * j] = pack2<BF16>(e[0], e[1]);
                        lo_bits[cl][2 * j + 1] = pack2<BF16>(e[2], e[3]);
                        hi_bits[cl][2 * j] = pack2<BF16>(o[0], o[1]);
                        hi_bits[cl][2 * j + 1] = pack2<BF16>(o[2], o[3]);
                        if constexpr (PASSES == 3) {
                            lo_l[cl][2 * j] = pack2_lo(e[0], e[1], lo_bits[cl][2 * j]);
                            lo_l[cl][2 * j + 1] = pack2_lo(e[2], e[3], lo_bits[cl][2 * j + 1]);
                            hi_l[cl][2 * j] = pack2_lo(o[0], o[1], hi_bits[cl][2 * j]);
                            hi_l[cl][2 * j + 1] = pack2_lo(o[2], o[3], hi_bits[cl][2 * j + 1]);
                        }
                    }
                    }
                }
                const uint32_t s = st_s;
                if (st_it > 0 && !wait_bar(empty_bar(s), (st_it - 1u) & 1u, abort_flag, a.status)) {
                    ok = false;
                    break;
                }
                if (++st_s == P::STAGES) st_s = 0, st_it++;
                const uint32_t ta = a_tile(s, 0);
#pragma unroll
                for (uint32_t cl = 0; cl < 2u * PARTS; cl++) {
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ta + choff[cl][0]), "r"(lo_bits[cl][0]),
                                 "r"(lo_bits[cl][1]), "r"(lo_bits[cl][2]), "r"(lo_bits[cl][3])
                                 : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ta + choff[cl][1]), "r"(hi_bits[cl][0]),
                                 "r"(hi_bits[cl][1]), "r"(hi_bits[cl][2]), "r"(hi_bits[cl][3])
                                 : "memory");
                    if constexpr (PASSES == 3) {
                        const uint32_t tl = a_tile(s, 1);
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tl + choff[cl][0]), "r"(lo_l[cl][0]),
                                     "r"(lo_l[cl][1]), "r"(lo_l[cl][2]), "r"(lo_l[cl][3])
                                     : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tl + choff[cl][1]), "r"(hi_l[cl][0]),
                                     "r"(hi_l[cl][1]), "r"(hi_l[cl][2]), "r"(hi_l[cl][3])
                                     : "memory");
                    }
                }
                // make the generic-proxy stores visible to the tensor core, then one arrival per warp
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(full_bar(s));
            }
        }
        }
        // ---------------- epilogue: TMEM -> registers -> Y ----------------
        if (ok && wait_bar(acc_bar, 0, abort_flag, a.status)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t quad = warp & 3u;               // the TMEM lanes this warp may read
            // the warps of one quadrant share the accumulators and, when there are more warps than accumulators, the columns
            constexpr uint32_t NACC = (uint32_t)ROWS / 128u, NCP = P::DEQ_WARPS / 4u / NACC;
            const uint32_t accum = (dw / 4u) % NACC;        // which 128-row accumulator
            const uint32_t cpart = (dw / 4u) / NACC;        // which run of kTokTile / NCP columns
            const uint32_t row = n0 + accum * 128u + quad * 32u + lane;
            const float bias = (a.ksplit == 1 && a.bias && row < a.N) ? a.bias[row] : 0.f;
            float* Yout = a.ksplit == 1 ? a.Y : a.Ypart + (uint64_t)blockIdx.z * a.M * a.N;
            for (uint32_t c0 = cpart * (kTokTile / NCP); c0 < (cpart + 1u) * (kTokTile / NCP); c0 += 32) {
                if (tok0 + c0 >= a.M) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((quad * 32u) << 16) + accum * kTokTile + c0, v);
                if constexpr (PASSES == 3) {  // add the cross-term accumulator
                    uint32_t v2[32];
                    tmem_ld32(tmem_base + ((quad * 32u) << 16) + kTokTile + c0, v2);
#pragma unroll
                    for (uint32_t t = 0; t < 32; t++) v[t] = __float_as_uint(__uint_as_float(v[t]) + __uint_as_float(v2[t]));
                }
                if (row < a.N) {
#pragma unroll
                    for (uint32_t t = 0; t < 32; t++) {
                        const uint32_t tok = tok0 + c0 + t;
                        if (tok < a.M) Yout[(uint64_t)tok * a.N + row] = __uint_as_float(v[t]) + bias;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P::TMEM_COLS) : "memory");
    }
}


// ---------------------------------------------------------------------------
// Single-pass modes, Q4_K, with the dequantised weights in TENSOR MEMORY instead of shared memory
// (BPQ4K_OPT_PREFILL_VARIANT = 2).  tcgen05.mma can take its A operand from TMEM (lane = row, a 32-bit column = two
// consecutive k).  The dequantising thread of a weight row writes its 64 values of a k-step straight into its TMEM
// lane (tcgen05.st, 32 columns), so the weights never pass through shared memory and the activation tiles get a ring
// of their own, eight deep.
//   TMEM (512 columns): accumulators of the two 128-row halves at columns 0 and 128 (128 activation rows each),
//   four A stages at 256 + 64*s (32 columns per half).  Shared memory: a ring of eight 16 KB activation tiles.
// A CTA owns 256 weight rows x 128 activation rows; the CTAs that share a weight tile are neighbours in the grid.
// The accumulators and the A stages share the 512 columns, which caps the activation tile at 128 rows: every
// dequantised weight then serves half as many rows as in the kernel above, and the dequantisation becomes the bound
// (128256 x 4096, M = 512, bfloat16: 825 against 1207 TFLOP/s; same bits).  Not the default.
struct PlanTS {
    static constexpr uint32_t TOK = 128, SA = 4, SB = 8;
    static constexpr uint32_t B_BYTES = TOK * 128u;
    static constexpr uint32_t THREADS = 10 * 32;
    static constexpr uint32_t TMEM_COLS = 512, A_COL0 = 256;
    static constexpr uint32_t SMEM_BYTES = 1024 + SB * B_BYTES + 512;
};
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

template <bool BF16>
__global__ void __launch_bounds__(PlanTS::THREADS, 1) prefill_tc_ts_kernel(const __grid_constant__ PrefillArgs a) {
    using P = PlanTS;
    constexpr int BU = 9;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_base = base + P::SB * P::B_BYTES;
    auto a_full = [&](uint32_t s) { return bar_base + s * 8u; };
    auto a_empty = [&](uint32_t s) { return bar_base + (P::SA + s) * 8u; };
    auto b_full = [&](uint32_t s) { return bar_base + (2u * P::SA + s) * 8u; };
    auto b_empty = [&](uint32_t s) { return bar_base + (2u * P::SA + P::SB + s) * 8u; };
    const uint32_t acc_bar = bar_base + (2u * P::SA + 2u * P::SB) * 8u;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + P::SB * P::B_BYTES + (2u * P::SA + 2u * P::SB) * 8u + 16u);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + P::SB * P::B_BYTES + (2u * P::SA + 2u * P::SB) * 8u + 32u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tok0 = blockIdx.x * P::TOK, n0 = blockIdx.y * 256u;
    const uint32_t blk0 = blockIdx.z * a.bps;
    const uint32_t blk1 = min(a.K / kQK, blk0 + a.bps);
    const uint32_t nkb = (blk1 - blk0) * 4u;
    const uint32_t kbase = blk0 * kQK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < P::SA; s++) {
            mbar_init(a_full(s), 8);
            mbar_init(a_empty(s), 1);
        }
        for (uint32_t s = 0; s < P::SB; s++) {
            mbar_init(b_full(s), 1);
            mbar_init(b_empty(s), 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(P::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    auto b_tile = [&](uint32_t s) { return base + s * P::B_BYTES; };

    if (warp == 0) {
        // ---------------- TMA producer: activation tiles, eight deep ----------------
        if (lane == 0) {
            for (uint32_t kb = 0; kb < nkb; kb++) {
                const uint32_t s = kb % P::SB, it = kb / P::SB;
                if (it > 0 && !wait_bar(b_empty(s), (it - 1) & 1u, abort_flag, a.status)) break;
                mbar_expect_tx(b_full(s), P::B_BYTES);
                tma_load_2d(b_tile(s), &a.tmap_x[0], kbase + kb * kKStep, tok0, b_full(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: A from tensor memory, B from shared memory ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) | ((P::TOK >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; kb++) {
                const uint32_t sa = kb % P::SA, sb = kb % P::SB;
                ok = wait_bar(a_full(sa), (kb / P::SA) & 1u, abort_flag, a.status) && wait_bar(b_full(sb), (kb / P::SB) & 1u, abort_flag, a.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t ks = 0; ks < kKStep / 16; ks++) {
                    const uint32_t acc = (kb | ks) ? 1u : 0u;
                    const uint64_t db = umma_desc(b_tile(sb) + ks * 32u);
#pragma unroll
                    for (uint32_t h = 0; h < 2; h++)
                        umma_f16_ts(tmem_base + h * P::TOK, tmem_base + P::A_COL0 + sa * 64u + h * 32u + ks * 8u, db, idesc, acc);
                }
                umma_commit(a_empty(sa));
                umma_commit(b_empty(sb));
            }
            if (ok) umma_commit(acc_bar);
        }
    } else {
        // ---------------- dequantise into this thread's TMEM lane, then drain the accumulators ----------------
        const uint32_t dw = warp - 2;
        const uint32_t h = dw >> 2, quad = warp & 3u;  // row half; the TMEM lane quarter this warp may access
        const uint32_t r = h * 128u + quad * 32u + lane;
        const uint32_t n = n0 + r;
        const uint4* wrow = reinterpret_cast<const uint4*>(a.W + (uint64_t)(n < a.N ? n : a.N - 1u) * a.w_row_bytes);
        const uint32_t nblocks = blk1 - blk0;
        wrow += (uint64_t)blk0 * BU;
        const uint32_t lane_addr = tmem_base + ((quad * 32u) << 16);
        bool ok = true;
        uint4 raw[BU], nxt[BU];
        auto load_block = [&](uint32_t b, uint4 (&dst)[BU]) {
            const uint4* p = wrow + (uint64_t)b * BU;
#pragma unroll
            for (int i = 0; i < BU; i++) dst[i] = __ldg(p + i);
        };
        if (nblocks) load_block(0, nxt);
        uint32_t st_s = 0, st_it = 0;
        for (uint32_t b = 0; b < nblocks && ok; b++) {
#pragma unroll
            for (int i = 0; i < BU; i++) raw[i] = nxt[i];
            if (b + 1 < nblocks) load_block(b + 1, nxt);
            const BlockHeader hd{raw[0].x, raw[0].y, raw[0].z, raw[0].w};
            const float d = half_bits_to_float(hd.w0), dmin = half_bits_to_float(hd.w0 >> 16);
            uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
            unpack_scales_packed(hd, sc_lo, sc_hi, mn_lo, mn_hi);
#pragma unroll
            for (uint32_t g = 0; g < 4; g++) {
                const float dsc_e = d * (float)byte_of(sc_lo, sc_hi, 2 * g), dmn_e = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g);
                const float dsc_o = d * (float)byte_of(sc_lo, sc_hi, 2 * g + 1), dmn_o = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g + 1);
                const uint32_t dsc_e2 = pack2<BF16>(dsc_e, dsc_e), ndmn_e2 = pack2<BF16>(-dmn_e, -dmn_e);
                const uint32_t dsc_o2 = pack2<BF16>(dsc_o, dsc_o), ndmn_o2 = pack2<BF16>(-dmn_o, -dmn_o);
                const uint4 u0 = raw[1 + 2 * g], u1 = raw[2 + 2 * g];
                const uint32_t words[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
                // column j of the stage holds k = 2j, 2j+1: the even sub-block's 32 weights, then the odd one's
                uint32_t v[32];
#pragma unroll
                for (uint32_t wv = 0; wv < 8; wv++) {
                    uint32_t o4[4];
                    dequant_word_16<BF16>(words[wv], dsc_e2, ndmn_e2, dsc_o2, ndmn_o2, o4);
                    v[2 * wv] = o4[0];
                    v[2 * wv + 1] = o4[1];
                    v[16 + 2 * wv] = o4[2];
                    v[16 + 2 * wv + 1] = o4[3];
                }
                const uint32_t s = st_s;
                if (st_it > 0 && !wait_bar(a_empty(s), (st_it - 1u) & 1u, abort_flag, a.status)) ok = false;
                ok = __all_sync(0xFFFFFFFFu, ok);  // the tensor-memory store below is a whole-warp instruction
                if (!ok) break;
                if (++st_s == P::SA) st_s = 0, st_it++;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                tmem_st32(lane_addr + P::A_COL0 + s * 64u + h * 32u, v);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full(s));
            }
        }
        if (ok) ok = wait_bar(acc_bar, 0, abort_flag, a.status);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float bias = (a.ksplit == 1 && a.bias && n < a.N) ? a.bias[n] : 0.f;
            float* Yout = a.ksplit == 1 ? a.Y : a.Ypart + (uint64_t)blockIdx.z * a.M * a.N;
            for (uint32_t c0 = 0; c0 < P::TOK; c0 += 32) {
                if (tok0 + c0 >= a.M) break;
                uint32_t v[32];
                tmem_ld32(lane_addr + h * P::TOK + c0, v);
                if (n < a.N) {
#pragma unroll
                    for (uint32_t t = 0; t < 32; t++)
                        if (tok0 + c0 + t < a.M) Yout[(uint64_t)(tok0 + c0 + t) * a.N + n] = __uint_as_float(v[t]) + bias;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P::TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Pair kernel (single-pass modes, Q4_K, M > 256; BPQ4K_OPT_PREFILL_VARIANT = 1): two CTAs of a cluster share one
// tcgen05.mma.cta_group::2.  The pair owns 256 weight rows x 512 activation rows.  Each CTA dequantises ITS 128 weight
// rows (the A operand of its half of M = 256) and loads HALF of each 256-row activation tile (the B operand is read
// from both CTAs' shared memory); its TMEM holds the 128 x 512 accumulators of its weight rows.  Against two
// independent CTAs of 256 x 256 this halves the dequantisation per flop and reads every weight byte once per 512
// activation rows.  Same bits as the one-CTA kernel; measured slower on B200 (128256 x 4096, M = 512, bfloat16:
// 990 against 1207 TFLOP/s, whether the second CTA's activation loads complete on the leader's barrier directly or
// are forwarded by a thread, with one or two dequantising threads per row), so it is not the default.
//
// Roles.  warp 0: TMA loads of this CTA's activation halves (cp.async.bulk.tensor with .cta_group::2 and NO multicast:
// the bytes land in the issuing CTA, the completion is counted on the LEADER's full barrier).  warp 1 of the leader
// (cluster rank 0): issues the mmas of the pair and the commits (to the barriers of both CTAs).  warps 2-9: two threads
// per weight row dequantise and arrive on the leader's full barrier (a remote arrive from the second CTA), then all
// eight drain the accumulators.  Every wait is bounded; the two cluster barriers are reached by every thread on every path.
struct PlanPair {
    static constexpr uint32_t A_BYTES = 128u * 128u, B_BYTES = 128u * 128u;  // 128 rows x 64 k x 2 B
    static constexpr uint32_t STAGE_BYTES = A_BYTES + 2u * B_BYTES;          // two activation tiles of 256 rows, half each
    static constexpr uint32_t STAGES = 4;
    static constexpr uint32_t DEQ_WARPS = 8, EPI_WARPS = 8;
    static constexpr uint32_t THREADS = (2 + EPI_WARPS) * 32;
    static constexpr uint32_t TMEM_COLS = 512;
    static constexpr uint32_t SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;
};
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ bool wait_bar_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
    for (uint32_t i = 0; i < kWaitLimit; i++) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicExch(status, kDeviceTimeout);
    return false;
}
// arrive on a barrier of another CTA of the cluster (address from mapa)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load whose completion is counted on a barrier of the pair's leader CTA (cluster address); no multicast:
// the bytes land in the issuing CTA's shared memory only
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tmap, uint32_t x, uint32_t y, uint32_t leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(leader_bar)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// commit of the pair's mmas: arrives on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(mask)
                 : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <bool BF16>
__global__ void __launch_bounds__(PlanPair::THREADS, 1) prefill_tc_pair_kernel(const __grid_constant__ PrefillArgs a) {
    using P = PlanPair;
    constexpr int BU = 9;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_base = base + P::STAGES * P::STAGE_BYTES;
    auto full_bar = [&](uint32_t s) { return bar_base + s * 8u; };                       // leader's: 4 + 4 dequant warps, 2 tile arrivals
    auto empty_bar = [&](uint32_t s) { return bar_base + (P::STAGES + s) * 8u; };        // both CTAs: the pair's commit
    const uint32_t acc_bar = bar_base + 3u * P::STAGES * 8u;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + P::STAGES * P::STAGE_BYTES + 3u * P::STAGES * 8u + 16u);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + P::STAGES * P::STAGE_BYTES + 3u * P::STAGES * 8u + 32u);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    uint32_t crank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    const bool leader = crank == 0;
    const uint32_t n0 = (blockIdx.x >> 1) * 256u + crank * 128u, tok0 = blockIdx.y * 512u;
    const uint32_t blk0 = blockIdx.z * a.bps;
    const uint32_t blk1 = min(a.K / kQK, blk0 + a.bps);
    const uint32_t nkb = (blk1 - blk0) * 4u;
    const uint32_t kbase = blk0 * kQK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < P::STAGES; s++) {
            mbar_init(full_bar(s), 2u * P::DEQ_WARPS + 1u);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both CTAs allocates the pair's TMEM
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(P::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // both CTAs' barriers initialised and TMEM allocated before anything crosses over
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    auto a_tile = [&](uint32_t s) { return base + s * P::STAGE_BYTES; };
    auto b_tile = [&](uint32_t s, uint32_t j) { return base + s * P::STAGE_BYTES + P::A_BYTES + j * P::B_BYTES; };
    auto leader_full = [&](uint32_t s) {
        uint32_t r;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(full_bar(s)), "r"(0u));
        return r;
    };

    if (warp == 0) {
        // ---------------- TMA producer: this CTA's 128 rows of each of the two activation tiles ----------------
        if (lane == 0) {
            const uint32_t lfull_tma = leader_full(0);
            for (uint32_t kb = 0; kb < nkb; kb++) {
                const uint32_t s = kb % P::STAGES, it = kb / P::STAGES;
                if (it > 0 && !wait_bar(empty_bar(s), (it - 1) & 1u, abort_flag, a.status)) break;
                if (leader) mbar_expect_tx(full_bar(s), 4u * P::B_BYTES);  // both CTAs' halves of both tiles
                const uint32_t lbar = lfull_tma + s * 8u;
                for (uint32_t j = 0; j < 2; j++)
                    tma_load_2d_pair(b_tile(s, j), &a.tmap_x[0], kbase + kb * kKStep, tok0 + j * 256u + crank * 128u, lbar);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            // ---------------- MMA issuer of the pair ----------------
            constexpr uint32_t idesc = (1u << 4) | ((BF16 ? 1u : 0u) << 7) | ((BF16 ? 1u : 0u) << 10) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; kb++) {
                const uint32_t s = kb % P::STAGES, it = kb / P::STAGES;
                ok = wait_bar_cluster(full_bar(s), it & 1u, abort_flag, a.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t ks = 0; ks < kKStep / 16; ks++) {
                    const uint32_t acc = (kb | ks) ? 1u : 0u;
                    const uint64_t da = umma_desc(a_tile(s) + ks * 32u);
#pragma unroll
                    for (uint32_t j = 0; j < 2; j++) umma_f16_pair(tmem_base + j * 256u, da, umma_desc(b_tile(s, j) + ks * 32u), idesc, acc);
                }
                umma_commit_pair(empty_bar(s));
            }
            if (ok) umma_commit_pair(acc_bar);
        }
    } else {
        const uint32_t dw = warp - 2;  // 0..7
        bool ok = true;
        {
            // ---------------- dequantise (two threads per weight row of this CTA's 128) ----------------
            const uint32_t r = (dw & 3u) * 32u + lane;
            const uint32_t part = dw >> 2;  // which 16 of a sub-block's 32 weights (two threads per row)
            const uint32_t n = n0 + r;
            const uint4* wrow = reinterpret_cast<const uint4*>(a.W + (uint64_t)(n < a.N ? n : a.N - 1u) * a.w_row_bytes);
            const uint32_t nblocks = blk1 - blk0;
            wrow += (uint64_t)blk0 * BU;
            const uint32_t row_off = (r >> 3) * 1024u + (r & 7u) * 128u;
            const uint32_t sw = r & 7u;
            const uint32_t lfull0 = leader_full(0);  // the leader's full barriers follow each other, 8 bytes apart
            constexpr int RU2 = 5;  // header + one code unit per 64-weight group
            uint4 raw[RU2], nxt[RU2];
            auto load_block = [&](uint32_t b, uint4 (&dst)[RU2]) {
                const uint4* p = wrow + (uint64_t)b * BU;
                dst[0] = __ldg(p);
#pragma unroll
                for (int g = 0; g < 4; g++) dst[1 + g] = __ldg(p + 1 + 2 * g + part);
            };
            if (nblocks) load_block(0, nxt);
            uint32_t st_s = 0, st_it = 0;
            uint32_t choff[2][2];
#pragma unroll
            for (uint32_t cl = 0; cl < 2; cl++) {
                const uint32_t c = 2u * part + cl;
                choff[cl][0] = row_off + ((c ^ sw) << 4);
                choff[cl][1] = row_off + (((c + 4u) ^ sw) << 4);
            }
            for (uint32_t b = 0; b < nblocks && ok; b++) {
#pragma unroll
                for (int i = 0; i < RU2; i++) raw[i] = nxt[i];
                if (b + 1 < nblocks) load_block(b + 1, nxt);
                const BlockHeader h{raw[0].x, raw[0].y, raw[0].z, raw[0].w};
                const float d = half_bits_to_float(h.w0), dmin = half_bits_to_float(h.w0 >> 16);
                uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
                unpack_scales_packed(h, sc_lo, sc_hi, mn_lo, mn_hi);
#pragma unroll
                for (uint32_t g = 0; g < 4; g++) {
                    const uint32_t s = st_s;
                    if (st_it > 0 && !wait_bar(empty_bar(s), (st_it - 1u) & 1u, abort_flag, a.status)) {
                        ok = false;
                        break;
                    }
                    if (++st_s == P::STAGES) st_s = 0, st_it++;
                    const float dsc_e = d * (float)byte_of(sc_lo, sc_hi, 2 * g), dmn_e = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g);
                    const float dsc_o = d * (float)byte_of(sc_lo, sc_hi, 2 * g + 1), dmn_o = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g + 1);
                    const uint32_t dsc_e2 = pack2<BF16>(dsc_e, dsc_e), ndmn_e2 = pack2<BF16>(-dmn_e, -dmn_e);
                    const uint32_t dsc_o2 = pack2<BF16>(dsc_o, dsc_o), ndmn_o2 = pack2<BF16>(-dmn_o, -dmn_o);
                    const uint4 u0 = raw[1 + g];
                    const uint32_t words[4] = {u0.x, u0.y, u0.z, u0.w};
                    const uint32_t ta = a_tile(s);
#pragma unroll
                    for (uint32_t c = 0; c < 2; c++) {
                        uint32_t lo_bits[4], hi_bits[4];
#pragma unroll
                        for (uint32_t j = 0; j < 2; j++) {
                            uint32_t o4[4];
                            dequant_word_16<BF16>(words[2 * c + j], dsc_e2, ndmn_e2, dsc_o2, ndmn_o2, o4);
                            lo_bits[2 * j] = o4[0];
                            lo_bits[2 * j + 1] = o4[1];
                            hi_bits[2 * j] = o4[2];
                            hi_bits[2 * j + 1] = o4[3];
                        }
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ta + choff[c][0]), "r"(lo_bits[0]),
                                     "r"(lo_bits[1]), "r"(lo_bits[2]), "r"(lo_bits[3])
                                     : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(ta + choff[c][1]), "r"(hi_bits[0]),
                                     "r"(hi_bits[1]), "r"(hi_bits[2]), "r"(hi_bits[3])
                                     : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(full_bar(s));
                        else mbar_arrive_remote(lfull0 + s * 8u);
                    }
                }
            }
        }
        // ---------------- epilogue: this CTA's 128 x 512 accumulators -> Y ----------------
        if (ok && wait_bar(acc_bar, 0, abort_flag, a.status)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t quad = warp & 3u;   // the TMEM lanes this warp may read
            const uint32_t jt = dw >> 2;       // which 256-row activation tile
            const uint32_t row = n0 + quad * 32u + lane;
            const float bias = (a.ksplit == 1 && a.bias && row < a.N) ? a.bias[row] : 0.f;
            float* Yout = a.ksplit == 1 ? a.Y : a.Ypart + (uint64_t)blockIdx.z * a.M * a.N;
            for (uint32_t c0 = 0; c0 < 256u; c0 += 32) {
                const uint32_t t0 = tok0 + jt * 256u + c0;
                if (t0 >= a.M) break;
                uint32_t v[32];
                tmem_ld32(tmem_base + ((quad * 32u) << 16) + jt * 256u + c0, v);
                if (row < a.N) {
#pragma unroll
                    for (uint32_t t = 0; t < 32; t++)
                        if (t0 + t < a.M) Yout[(uint64_t)(t0 + t) * a.N + row] = __uint_as_float(v[t]) + bias;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // both CTAs have drained their accumulators; nothing crosses over any more
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(P::TMEM_COLS) : "memory");
    }
}

// X float32 [M][K] -> 16-bit [M][K] (and, for the three-pass mode, the low part of the half split)
template <bool BF16, bool SPLIT>
__global__ void __launch_bounds__(256) cast_activations_kernel(const float* __restrict__ X, uint64_t count4,
                                                               uint2* __restrict__ hi, uint2* __restrict__ lo) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (uint64_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(X) + i);
        uint2 h;
        h.x = pack2<BF16>(v.x, v.y);
        h.y = pack2<BF16>(v.z, v.w);
        hi[i] = h;
        if constexpr (SPLIT) {
            uint2 l;
            l.x = pack2_lo(v.x, v.y, h.x);
            l.y = pack2_lo(v.z, v.w, h.y);
            lo[i] = l;
        }
    }
}

// Y = bias + sum_z Ypart[z], slices added in ascending z (deterministic)
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, uint32_t Z, uint64_t MN, uint32_t N,
                                                            const float* __restrict__ bias, float* __restrict__ Y) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < MN; i += (uint64_t)gridDim.x * blockDim.x) {
        float s = bias ? bias[i % N] : 0.f;
        for (uint32_t z = 0; z < Z; z++) s += part[(uint64_t)z * MN + i];
        Y[i] = s;
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

template <int ROWS, int PASSES, bool BF16, int QT = 0>
cudaError_t launch_tc(const PrefillArgs& pa, cudaStream_t stream) {
    using P = Plan<ROWS, PASSES, QT>;
    static KernelConfig kcfg;  // per-device slots inside
    if (cudaError_t e = kcfg.prepare(reinterpret_cast<const void*>(prefill_tc_kernel<ROWS, PASSES, BF16, QT>), P::THREADS,
                                     P::SMEM_BYTES, nullptr))
        return e;
    const dim3 grid((pa.N + ROWS - 1) / ROWS, (pa.M + kTokTile - 1) / kTokTile, pa.ksplit);
    prefill_tc_kernel<ROWS, PASSES, BF16, QT><<<grid, P::THREADS, P::SMEM_BYTES, stream>>>(pa);
    return cudaGetLastError();
}


template <bool BF16>
cudaError_t launch_tc_ts(const PrefillArgs& pa, cudaStream_t stream) {
    using P = PlanTS;
    static KernelConfig kcfg;
    if (cudaError_t e = kcfg.prepare(reinterpret_cast<const void*>(prefill_tc_ts_kernel<BF16>), P::THREADS, P::SMEM_BYTES, nullptr))
        return e;
    const dim3 grid((pa.M + P::TOK - 1) / P::TOK, (pa.N + 255u) / 256u, pa.ksplit);
    prefill_tc_ts_kernel<BF16><<<grid, P::THREADS, P::SMEM_BYTES, stream>>>(pa);
    return cudaGetLastError();
}

template <bool BF16>
cudaError_t launch_tc_pair(const PrefillArgs& pa, cudaStream_t stream) {
    using P = PlanPair;
    static KernelConfig kcfg;
    if (cudaError_t e = kcfg.prepare(reinterpret_cast<const void*>(prefill_tc_pair_kernel<BF16>), P::THREADS, P::SMEM_BYTES, nullptr))
        return e;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2u * ((pa.N + 255u) / 256u), (pa.M + 511u) / 512u, pa.ksplit);
    cfg.blockDim = dim3(P::THREADS);
    cfg.dynamicSmemBytes = P::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, prefill_tc_pair_kernel<BF16>, pa);
}

}  // namespace

// K slices per problem: enough CTAs to occupy the machine when there are few output tiles, slices
// of at least 1024 k, and (three-pass mode) at most 4096 k per slice so that the accumulation
// error of the tensor core stays inside the tolerance of the path.
// `mode` carries the precision mode in its low four bits and the single-pass variant above them (0: one CTA per tile,
// weights through shared memory; 1: CTA pairs; 2: weights through tensor memory).
static int variant_of(int mode, uint32_t M) {
    const int v = (mode & 15) == 0 ? 0 : mode >> 4;
    return (v == 1 && M <= kTokTile) ? 0 : v;  // a pair's tile is 512 activation rows: nothing to share below 257
}
static uint32_t choose_ksplit(uint32_t M, uint32_t N, uint32_t K, int mode_v, int sm_count) {
    const int mode = mode_v & 15, variant = variant_of(mode_v, M);
    const uint32_t rows = mode == 0 ? 128u : 256u;
    const uint32_t tiles = variant == 1   ? 2u * ((N + 255u) / 256u) * ((M + 511u) / 512u)
                           : variant == 2 ? ((N + 255u) / 256u) * ((M + 127u) / 128u)
                                          : ((N + rows - 1) / rows) * ((M + kTokTile - 1) / kTokTile);
    const uint32_t nblk = K / kQK;
    uint32_t z = tiles >= (uint32_t)sm_count ? 1u : (uint32_t)sm_count / tiles;  // stay within one wave of CTAs
    const uint32_t zmax = nblk / 4u ? nblk / 4u : 1u;  // >= 1024 k per slice
    if (z > zmax) z = zmax;
    if (mode == 0 && nblk > 16u * z) z = (nblk + 15u) / 16u;
    if (z > 16u) z = 16u;
    if (z < 1u) z = 1u;
    const uint32_t bps = (nblk + z - 1) / z;  // super-blocks per slice
    return (nblk + bps - 1) / bps;            // no empty slice
}

size_t prefill_scratch_bytes(uint32_t M, uint32_t N, uint32_t K, int mode_v, int sm_count) {
    const int mode = mode_v & 15;
    const size_t one = ((size_t)M * K * 2u + 255u) & ~(size_t)255u;
    const uint32_t z = choose_ksplit(M, N, K, mode_v, sm_count);
    return (mode == 0 ? 2 * one : one) + (z > 1 ? (size_t)z * M * N * 4u : 0);
}

// mode: 0 = three-pass half split, 1 = one pass half, 2 = one pass bfloat16 (the values of bpq4k_prefill_mode)
cudaError_t launch_prefill_tc(const MatmulArgs& m, int mode_v, void* scratch, size_t scratch_bytes, int* status_dev,
                              int sm_count, cudaStream_t stream, int* launches, int qtype) {
    if (m.M == 0 || m.N == 0) return cudaSuccess;
    if (qtype != 12 && qtype != 13 && qtype != kQ6PaddedType) return cudaErrorInvalidValue;
    const bool q5 = qtype == 13, q6 = qtype == kQ6PaddedType;
    if (m.n_slots) return cudaErrorInvalidValue;
    if (q5 || q6) mode_v &= 15;  // the variants exist for Q4_K
    const int mode = mode_v & 15, variant = variant_of(mode_v, m.M);
    if (!scratch || scratch_bytes < prefill_scratch_bytes(m.M, m.N, m.K, mode_v, sm_count)) return cudaErrorInvalidValue;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    uint8_t* hi = static_cast<uint8_t*>(scratch);
    uint8_t* lo = hi + (((size_t)m.M * m.K * 2u + 255u) & ~(size_t)255u);
    const uint64_t count4 = (uint64_t)m.M * m.K / 4u;
    const unsigned cgrid = (unsigned)((count4 + 255) / 256 < 148u * 16u ? (count4 + 255) / 256 : 148u * 16u);
    if (mode == 0)
        cast_activations_kernel<false, true><<<cgrid, 256, 0, stream>>>(m.X, count4, reinterpret_cast<uint2*>(hi), reinterpret_cast<uint2*>(lo));
    else if (mode == 1)
        cast_activations_kernel<false, false><<<cgrid, 256, 0, stream>>>(m.X, count4, reinterpret_cast<uint2*>(hi), nullptr);
    else
        cast_activations_kernel<true, false><<<cgrid, 256, 0, stream>>>(m.X, count4, reinterpret_cast<uint2*>(hi), nullptr);
    if (launches) ++*launches;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;

    PrefillArgs pa{};
    pa.W = m.W;
    pa.bias = m.bias;
    pa.Y = m.Y;
    pa.M = m.M;
    pa.N = m.N;
    pa.K = m.K;
    pa.w_row_bytes = m.w_row_bytes;
    pa.status = status_dev;
    pa.ksplit = choose_ksplit(m.M, m.N, m.K, mode_v, sm_count);
    pa.bps = (m.K / kQK + pa.ksplit - 1) / pa.ksplit;
    pa.Ypart = reinterpret_cast<float*>(lo + (mode == 0 ? (((size_t)m.M * m.K * 2u + 255u) & ~(size_t)255u) : 0));
    for (int v = 0; v < (mode == 0 ? 2 : 1); v++) {
        const cuuint64_t gdim[2] = {(cuuint64_t)m.K, (cuuint64_t)m.M};
        const cuuint64_t gstride[1] = {(cuuint64_t)m.K * 2u};
        const cuuint32_t box[2] = {kKStep, variant ? 128u : kTokTile};  // pairs and the tensor-memory form load 128 activation rows per copy
        const cuuint32_t estr[2] = {1u, 1u};
        const CUresult r = enc(&pa.tmap_x[v], CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, v == 0 ? hi : lo, gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    if (mode != 0) pa.tmap_x[1] = pa.tmap_x[0];
    if (variant == 2) e = mode == 1 ? launch_tc_ts<false>(pa, stream) : launch_tc_ts<true>(pa, stream);
    else if (variant == 1) e = mode == 1 ? launch_tc_pair<false>(pa, stream) : launch_tc_pair<true>(pa, stream);
    else if (mode == 0) e = q6 ? launch_tc<128, 3, false, 2>(pa, stream) : q5 ? launch_tc<128, 3, false, 1>(pa, stream) : launch_tc<128, 3, false>(pa, stream);
    else if (mode == 1) e = q6 ? launch_tc<256, 1, false, 2>(pa, stream) : q5 ? launch_tc<256, 1, false, 1>(pa, stream) : launch_tc<256, 1, false>(pa, stream);
    else e = q6 ? launch_tc<256, 1, true, 2>(pa, stream) : q5 ? launch_tc<256, 1, true, 1>(pa, stream) : launch_tc<256, 1, true>(pa, stream);
    if (launches) ++*launches;
    if (e != cudaSuccess) return e;
    if (pa.ksplit > 1) {
        const uint64_t MN = (uint64_t)m.M * m.N;
        const unsigned rgrid = (unsigned)((MN + 255) / 256 < (uint64_t)sm_count * 8u ? (MN + 255) / 256 : (uint64_t)sm_count * 8u);
        splitk_reduce_kernel<<<rgrid, 256, 0, stream>>>(pa.Ypart, pa.ksplit, MN, m.N, m.bias, m.Y);
        if (launches) ++*launches;
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace bpq4k
