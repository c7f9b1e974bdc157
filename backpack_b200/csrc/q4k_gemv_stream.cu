// Bandwidth-bound Q4_K matmul for small M (decode): a persistent kernel that
// streams raw 144-byte super-blocks from HBM into per-warp shared-memory rings
// with bulk asynchronous copies (cp.async.bulk + mbarrier), decodes the 4-bit
// codes in registers and takes the dot products on the tensor cores.
//
// Replaces the reference's q4k_matmul / q4k_matmul_128 / q4k_matmul_batched4/8
// shaders (runtime/kernels/quant_kq/q4k_matmul.wgsl:20-95 and siblings) and the
// per-slot `*_matmul_moe` dispatch form (iq4xs_matmul_moe.wgsl:55-99).
//
// Arithmetic.  For sub-block sb of row n:  w = dsc*q - dmn  with dsc = d*sc,
// dmn = dmin*mn, so
//     sum_k x_k w_k = dsc * sum_k x_k q_k  -  dmn * sum_k x_k .
// sum_k x_k q_k is taken EXACTLY in integers on the tensor cores (mma.sync m16n8k32,
// u8 x s8 -> s32): the activation row is scaled so that max|x| maps to 2080000 (< 2^21),
// rounded to an integer xi and written as three signed base-128 digits
// xi = d0*2^14 + d1*2^7 + d2 (|d| <= 64).  The 4-bit codes need almost no decoding: a
// code word masked with 0x0F0F0F0F is four u8 weights of the even sub-block, masked with
// 0xF0F0F0F0 it is four weights of the odd sub-block times 16 (the 1/16 goes into dsc).
// Per sub-block   T = 2^14*sum(q d0) + 2^7*sum(q d1) + sum(q d2)   (exact: the two low
// digit sums are combined in int32, the top one joins in float where it is exact), then
//     contribution = dsc*float(T) - dmn*float(sum xi)
// in float.  x keeps 22 bits relative to its row maximum; everything else is float, so the
// result differs from the float reference by ~1e-6 relative.
//
// Work decomposition.  A tile is 16 output rows.  The warps of a CTA are arranged
// as WT tile slots x WK slices of K; a warp streams its slice of its tile through
// a private ring of `stages` buffers of `cb` blocks x 16 rows (one bulk copy per
// row), so the only CTA-wide synchronisation is the staging of the activations.
// The K slices of a tile are combined through shared memory in a fixed order, so
// results are deterministic.  CTAs are persistent and walk tiles with stride
// gridDim.x*WT.
//
// mma operand mapping (one mma = 16 rows x the 32 weights of one sub-block).  ldmatrix hands
// thread (r = lane/4, t = lane%4) word t of a 16-byte run of code bytes of rows r and r+8:
// exactly the A fragment of m16n8k32 (a0: row r, k = 4t..4t+3; a1: row r+8; a2, a3: k+16),
// in natural k order, so the activation digits are stored in natural order too.
// The 8 mma columns are 4 pairs; a pair's two columns carry digits (d0, d1) in the first
// mma of a sub-block and (d2, 0) in the second.  Pair j carries digits only in the mmas of
// sub-block parity j%2 and zeros in the others, so after the four mmas of a 64-weight group
// thread t holds the sums of sub-block parity t%2 -- the per-sub-block scaling work is
// spread over the four threads of a quad without any shuffles; pairs 2,3 repeat pairs 0,1 and
// threads t>=2 take row r+8.  That is the single-row kernel (M1).  With several activation rows
// the four pairs are four activation rows instead: every mma is one sub-block x four rows of X,
// no zero columns, and thread t finishes activation row t for rows r and r+8 of the tile.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "kernels.h"
#include "q4k_common.cuh"
#include "stream_common.cuh"

namespace bpq4k {

namespace {

constexpr uint32_t kMaxWarps = 16;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kRingBarBytes = kMaxWarps * kMaxStages * 8;  // 1 KiB of ring mbarriers
constexpr uint32_t kBarBytes = kRingBarBytes + 64;              // + the barrier of the activation copy (XC)
constexpr uint32_t kWaitPolls = 1u << 22;                    // bounded mbarrier wait

constexpr uint32_t kZeroBytes = 1024;  // zero region the "other parity" lanes read their B operand from

struct StreamArgs {
    CUtensorMap tmap;      // W as a 2-D tensor [rows][row words], box = 16 rows x cb blocks
    CUtensorMap tmap_rem;  // same tensor, box = 16 rows x rem blocks (tail of a warp's K range)
    CUtensorMap tmap_b, tmap_b_rem;  // IND with two matrices: the same two boxes over m.W2
    MatmulArgs m;
    uint32_t wk, wt, cb, rem, bpw, stages, stage_bytes, ntiles, tokens;  // bpw: blocks per warp per tile
    uint32_t off_zero, off_S, off_x, off_part, off_ring;
    int* status;
    // activations prepared by quantize_activations_kernel (XG mode)
    const uint8_t* xfrag_g;
    const float* S_g;
    uint32_t nvslots;  // IND: slots times matrices (virtual slot vs: matrix vs / n_slots, slot vs % n_slots)
    uint32_t u_base, u_extra;  // IND / contig: CTA c takes u_base units (+1 for c < u_extra) of the unit list, in order
    uint32_t pre_wait;         // ring stages issued before the dependency wait (the rest after the activation loads)
    uint32_t contig;           // direct form with a balanced contiguous tile range per CTA (units = tiles)
    uint32_t csize;            // CTAs per cluster that share the staging of the activation row (1: none)
    // optional time stamps (BPQ4K_OPT_STREAM_STAMPS): eight words per CTA of this launch's slot, written by thread 0
    unsigned long long* stamps;
    uint32_t stamp_slot;
};

// Largest |xi|: its top base-128 digit still fits a signed byte.
constexpr float kXiMax = 2080000.f;

// Quantise the activations.  Work item c8 of row `tok` belongs to 32-float sub-block c8/4 and is piece
// t = c8%4 of it: the floats k = 4t..4t+3 and 16+4t..16+4t+3 of the sub-block (item_offset), i.e. exactly
// the values of the two 16-byte chunks (c, t) below, so a thread writes whole chunks and nothing has to
// move between lanes.  The four items of a sub-block sit in four adjacent lanes, which agree on the
// sub-block's max|x| with two shuffles.  Each sub-block gets its own scale kXiMax/max|x| (block floating
// point), xi = rint(x*scale), and the three base-128 digits of xi are stored in the mma B layout:
//   per (token, 64-weight group G, parity): 128 B = [c: 0,1][t: 0..3][16 B]
//   16 B of (c, t): c = 0: d0[4t..4t+3], d0[16+4t..], d2[4t..], d2[16+4t..]
//                   c = 1: d1[4t..4t+3], d1[16+4t..], 0, 0
// and per sub-block the two floats the kernel needs: inv = max|x|/kXiMax and sum(xi)*inv,
//   SI[((tok*nb + blk)*2 + parity)*8 + {0: sum*inv, 4: inv} + g].
// All 32 lanes of a warp must call this together (idle lanes pass valid = false).
__device__ __forceinline__ uint32_t item_offset(uint32_t c8) { return (c8 >> 2) * 32u + (c8 & 3u) * 4u; }  // first float4; the second is 16 floats on
// `rows`: the several-row kernels keep the two floats elsewhere, four activation rows side by side, so that
// the four threads of a quad (one activation row each) read one 64-byte run without bank conflicts:
//   SI[((((tok/4)*nb + blk)*4 + g)*4 + tok%4)*4 + parity*2 + {0: sum*inv, 1: inv}].
struct QuantItem {
    uint4 c0, c1;    // the item's two 16-byte chunks (c = 0: top and low digits, c = 1: middle digits)
    float sinv, inv;  // sum(xi)*inv and inv of the item's sub-block
};
// The arithmetic of an item, no memory access: several items of a thread are computed side by side
// (independent dependency chains; a warp per scheduler or two has little else to hide latency with).
__device__ __forceinline__ QuantItem quantize_compute(float4 v0, float4 v1) {
    float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                       fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    float scale = 1.f, inv = 1.f;
    if (amax > 1e-30f && amax < 3e38f) {  // zero, tiny, inf or nan: leave unscaled
        // (approximate reciprocal and a multiplication instead of two divisions on the kernel's one serial path: scale*inv
        //  is 1 within 3e-7, a common factor of the sub-block far inside the digits' 2^-21; the clamp below catches the ulps)
        scale = amax < 1e37f ? __fdividef(kXiMax, amax) : kXiMax / amax;  // (the fast form returns 0 for divisors above 2^126)
        inv = amax * (1.f / kXiMax);
    }
    const float xs[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    int d0[8], d1[8], d2[8];
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float vc = fminf(fmaxf(xs[i] * scale, -kXiMax), kXiMax);  // x*scale may overshoot by an ulp
        const int xi = __float2int_rn(vc);
        d2[i] = (xi << 25) >> 25;  // signed low seven bits
        const int r1 = (xi - d2[i]) >> 7;
        d1[i] = (r1 << 25) >> 25;
        d0[i] = (r1 - d1[i]) >> 7;
        sum += xi;
    }
    auto pack4 = [](const int* d) {  // the low bytes of four digits
        return __byte_perm(__byte_perm((uint32_t)d[0], (uint32_t)d[1], 0x0040), __byte_perm((uint32_t)d[2], (uint32_t)d[3], 0x0040), 0x5410);
    };
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    QuantItem q;
    q.c0 = make_uint4(pack4(d0), pack4(d0 + 4), pack4(d2), pack4(d2 + 4));
    q.c1 = make_uint4(pack4(d1), pack4(d1 + 4), 0u, 0u);
    q.sinv = (float)sum * inv;
    q.inv = inv;
    return q;
}
__device__ __forceinline__ void quantize_store(const QuantItem& q, uint32_t K, uint32_t tok, uint32_t c8, bool valid,
                                               uint8_t* frag, float* SI, bool rows) {
    if (!valid) return;
    const uint32_t nb = K / kQK, NG = K / 64u;
    const uint32_t sbg = c8 >> 2, t = c8 & 3u;  // sub-block in the row, piece of the sub-block
    const uint32_t G = sbg >> 1, par = sbg & 1u;
    uint8_t* base = frag + ((uint64_t)(tok * NG + G) * 2u + par) * 128u + t * 16u;
    // Two 16-byte stores per thread.  The lanes of even sub-blocks write their c = 0 chunk first, those of odd
    // sub-blocks their c = 1 chunk: the eight lanes that share a shared-memory wavefront then cover all 32 banks.
    *reinterpret_cast<uint4*>(base + (par ? 64u : 0u)) = par ? q.c1 : q.c0;
    *reinterpret_cast<uint4*>(base + (par ? 0u : 64u)) = par ? q.c0 : q.c1;
    if (t == 0) {
        if (rows) {
            float* si = SI + (((uint64_t)((tok >> 2) * nb + (sbg >> 3)) * 4u + ((sbg >> 1) & 3u)) * 4u + (tok & 3u)) * 4u + par * 2u;
            si[0] = q.sinv;
            si[1] = q.inv;
        } else {
            float* si = SI + ((uint64_t)(tok * nb + (sbg >> 3)) * 2u + par) * 8u + ((sbg >> 1) & 3u);
            si[0] = q.sinv;
            si[4] = q.inv;
        }
    }
}
__device__ __forceinline__ void quantize_loaded(float4 v0, float4 v1, uint32_t K, uint32_t tok, uint32_t c8, bool valid,
                                                uint8_t* frag, float* SI, bool rows = false) {
    const QuantItem q = quantize_compute(v0, v1);
    quantize_store(q, K, tok, c8, valid, frag, SI, rows);
}
// Single activation row staged by a cluster: the item goes to the same place in the shared memory of every CTA of
// the cluster (xr[r], sr[r]: shared::cluster addresses of CTA r's digit and scale arrays).
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint4 v) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void quantize_store_cluster(const QuantItem& q, uint32_t c8, bool valid, const uint32_t (&xr)[4],
                                                       const uint32_t (&sr)[4], uint32_t cs) {
    if (!valid) return;
    const uint32_t sbg = c8 >> 2, t = c8 & 3u;
    const uint32_t G = sbg >> 1, par = sbg & 1u;
    const uint32_t off = (G * 2u + par) * 128u + t * 16u;
    const uint32_t so = (((sbg >> 3) * 2u + par) * 8u + ((sbg >> 1) & 3u)) * 4u;
#pragma unroll
    for (uint32_t r = 0; r < 4; r++) {
        if (r >= cs) break;
        st_cluster_v4(xr[r] + off + (par ? 64u : 0u), par ? q.c1 : q.c0);
        st_cluster_v4(xr[r] + off + (par ? 0u : 64u), par ? q.c0 : q.c1);
        if (t == 0) {
            st_cluster_f32(sr[r] + so, q.sinv);
            st_cluster_f32(sr[r] + so + 16u, q.inv);
        }
    }
}
// Load the 8 floats of an item (zeros for rows past M or an idle lane), then quantise them.
__device__ __forceinline__ void quantize_item(const float* __restrict__ X, uint32_t M, uint32_t K, uint32_t tok,
                                              uint32_t c8, bool valid, uint8_t* frag, float* SI, bool rows) {
    float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
    if (valid && tok < M) {
        const float4* xp = reinterpret_cast<const float4*>(X + (uint64_t)tok * K + item_offset(c8));
        v0 = __ldg(xp);
        v1 = __ldg(xp + 4);
    }
    quantize_loaded(v0, v1, K, tok, c8, valid, frag, SI, rows);
}

// Q5_K: code bytes of sub-blocks 2g (low nibbles) and 2g+1 (high nibbles) of one code word, each
// with its fifth bit (bits 2g and 2g+1 of the matching byte of `qh`) merged in at bit 4.
template <int g>
__device__ __forceinline__ void merge_fifth_bit(uint32_t codes, uint32_t qh, uint32_t& even, uint32_t& odd) {
    constexpr uint32_t kLo = 0x0F0F0F0Fu, kBit = 0x10101010u;
    const uint32_t be = g == 0 ? (qh << 4) : g == 1 ? (qh << 2) : g == 2 ? qh : (qh >> 2);
    const uint32_t bo = g == 0 ? (qh << 3) : g == 1 ? (qh << 1) : g == 2 ? (qh >> 1) : (qh >> 3);
    even = (codes & kLo) | (be & kBit);
    odd = ((codes >> 4) & kLo) | (bo & kBit);
}

// Q5: the weights are Q5_K super-blocks (176 bytes: the Q4_K header, 32 bytes of fifth bits, 128
// nibble bytes); the fifth bit is merged into each code byte, so odd sub-blocks reach the mma as
// q (not 16*q) and carry no 1/16 in their scale.
// XC (with XG false): the digits live in shared memory as usual, but they were quantised once per call by
// quantize_activations_kernel and every CTA only copies them in (bulk copies from the scratch) instead of
// quantising all rows itself -- with eight rows that is ~1 us instead of ~8 us per CTA.
// FP (single row only): the call has a fused prologue and/or a residual; kept out of the plain kernel, whose
// code it would otherwise slow down by ~1 %.
// IND (single row only): the indirect form as ONE list of (slot, tile) units over a 1-D grid.  CTA c takes the
// units [U*c/G, U*(c+1)/G), which lie in at most kMaxLocalSlots consecutive slots; it stages those slots'
// activation rows side by side and every tile picks its slot's row.  All SMs carry the same load whatever the
// number of slots (with blockIdx.y = slot, 64 slots occupy 128 of 148 SMs).  With a second matrix (m.W2, same
// shape, activations and offsets: the gate and up stacks of an expert layer) the list simply continues
// over it, results to m.Y2.
constexpr uint32_t kMaxLocalSlots = 4;
[[maybe_unused]] constexpr uint32_t kStampCtas = kStreamStampCtas;  // CTAs per launch that leave time stamps
template <int NT, bool M1, bool XG, bool Q5 = false, bool XC = false, bool FP = false, bool IND = false, int RT = 1, bool PEER = false>
__global__ void __launch_bounds__(RT == 2 ? 256 : (M1 || NT == 1) ? 512 : 384, 1) gemv_stream_kernel(const __grid_constant__ StreamArgs a) {
    static_assert(!FP || (M1 && !XG && !XC), "the fused forms are single-row and stage the row themselves");
    static_assert(!IND || (M1 && !XG && !XC), "the unit-list form is single-row and stages its rows itself");
    static_assert(!(XG && XC), "digits are read from the scratch directly (XG) or copied into shared memory (XC)");
    static_assert(RT == 1 || (RT == 2 && !M1), "32-row units (two mma row tiles per warp and stage) exist for several activation rows only");
    constexpr uint32_t TR = 16u * RT;  // weight rows of one tile: what a warp takes through its ring at a time
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t BB = Q5 ? 176u : kBlockBytes, BW = BB / 4u;  // bytes and words per super-block
    constexpr uint32_t QS = Q5 ? 48u : 16u;                          // offset of the nibble bytes
    constexpr int TOK = M1 ? 1 : NT * 4;  // activation-row slots (four per 8-column mma tile)

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    // Time stamps for the attribution of a launch's microseconds: 0 start, 1 before the dependency wait, 2 released,
    // 3 activations staged, 4 last tile slot of thread 0 done, 5 end; word 7 = SM id and grid size.  Compiled into
    // libbpq4k_stamps.so only (make stamps): in the product library even the six untaken branches cost the
    // eight-launch decode step 1.9 us.
#ifdef BPQ4K_STAMPS
    auto stamp = [&](uint32_t i) {
        if (a.stamps && tid == 0 && blockIdx.y == 0 && blockIdx.x < kStampCtas) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            a.stamps[((uint64_t)a.stamp_slot * kStampCtas + blockIdx.x) * 8u + i] = t;
        }
    };
#else
    auto stamp = [](uint32_t) {};
#endif
    stamp(0);
    // Warps beyond the plan's wk x wt are helpers: they take part in the staging of the activations (the one serial
    // step of the kernel, faster with one item per thread) and leave before the main loop.
    const uint32_t swarps = blockDim.x >> 5;
    const uint32_t nwarps = a.wk * a.wt;
    const bool helper = warp >= nwarps;
    const uint32_t wk = warp % a.wk, wt = warp / a.wk;
    const uint32_t K = a.m.K, N = a.m.N, nb = K / kQK;
    // every warp of a tile takes the same number of blocks: full stages of cb, then one of rem
    const uint32_t b0 = wk * a.bpw;
    const uint32_t nfull = a.bpw / a.cb;
    const uint32_t nchunks = nfull + (a.rem ? 1u : 0u);

    // problem selection (indirect form: blockIdx.y is the slot)
    const float* X = a.m.X;
    float* Y = a.m.Y;
    uint32_t wrow0 = 0;
    uint32_t M = a.m.M;
    const float* AUX = FP ? a.m.aux : nullptr;
    uint32_t tstride = gridDim.x * a.wt;
    uint32_t tile0 = blockIdx.x * a.wt + wt;   // IND: a unit index, not a tile
    uint32_t my_tiles = tile0 < a.ntiles ? (a.ntiles - tile0 + tstride - 1) / tstride : 0;
    // IND: this CTA's first virtual slot, how many it touches, and their first weight rows
    [[maybe_unused]] uint32_t s_first = 0, nloc = 1;
    [[maybe_unused]] uint32_t offs[kMaxLocalSlots] = {0u, 0u, 0u, 0u};
    [[maybe_unused]] const float* xrow[kMaxLocalSlots] = {a.m.X, a.m.X, a.m.X, a.m.X};
    [[maybe_unused]] const float* arow[kMaxLocalSlots] = {a.m.aux, a.m.aux, a.m.aux, a.m.aux};
    auto slot_of = [&](uint32_t vs) { return vs >= a.m.n_slots ? vs - a.m.n_slots : vs; };
    auto x_row_of = [&](uint32_t s) { return a.m.x_rows ? a.m.x_rows[s] : a.m.x_row_div ? s / a.m.x_row_div : s; };
    if constexpr (!IND) {
        if (a.contig) {
            // direct form: CTA c owns the contiguous tile range [u_begin, u_end), its tile slots stride through it
            const uint32_t u_begin = blockIdx.x * a.u_base + min(blockIdx.x, a.u_extra);
            const uint32_t u_end = u_begin + a.u_base + (blockIdx.x < a.u_extra ? 1u : 0u);
            tstride = a.wt;
            tile0 = u_begin + wt;
            my_tiles = tile0 < u_end ? (u_end - tile0 + tstride - 1u) / tstride : 0u;
        }
    }
    if constexpr (IND) {
        const uint32_t u_begin = blockIdx.x * a.u_base + min(blockIdx.x, a.u_extra);
        const uint32_t u_end = u_begin + a.u_base + (blockIdx.x < a.u_extra ? 1u : 0u);
        s_first = u_begin / a.ntiles;  // the only division; everything else advances by subtraction
        tstride = a.wt;
        tile0 = u_begin + wt;
        my_tiles = tile0 < u_end ? (u_end - tile0 + tstride - 1u) / tstride : 0u;  // tstride is a small power of two or close: cheap
        nloc = u_end > u_begin ? 1u : 0u;
        for (uint32_t r = u_end - 1u - s_first * a.ntiles; nloc && r >= a.ntiles && nloc <= kMaxLocalSlots; r -= a.ntiles) nloc++;
        if (nloc > kMaxLocalSlots) nloc = 0, my_tiles = 0;  // the host sizes the grid so that this never happens
#pragma unroll
        for (uint32_t l = 0; l < kMaxLocalSlots; l++)
            if (l < nloc) {
                const uint32_t s = slot_of(s_first + l);
                const uint32_t o = a.m.offsets[s];
                offs[l] = a.m.offset_mul ? o * a.m.offset_mul : o;
                xrow[l] = a.m.X + (uint64_t)x_row_of(s) * K;  // addresses only; the rows are read after the dependency wait
                if (FP && a.m.aux) arow[l] = a.m.aux + (uint64_t)s * K;
            }
        M = 1;
    } else if (a.m.n_slots) {
        const uint32_t s = blockIdx.y;
        wrow0 = a.m.offsets[s];
        if (a.m.offset_mul) wrow0 *= a.m.offset_mul;
        X += (uint64_t)x_row_of(s) * K;
        Y += (uint64_t)s * N;
        if (FP && AUX) AUX += (uint64_t)s * K;
        M = 1;
    }
    if (helper) my_tiles = 0;
    const uint32_t total_units = my_tiles * nchunks;

    const uint32_t bar0 = smem_u32(smem) + warp * kMaxStages * 8u;
    const uint32_t ring = smem_u32(smem + a.off_ring) + warp * a.stages * a.stage_bytes;

    const uint32_t xbar = smem_u32(smem) + kRingBarBytes;  // XC: completion of the activation copy
    if (lane == 0) {
        for (uint32_t s = 0; s < a.stages; s++) mbar_init(bar0 + s * 8u, 1);
        if (XC && warp == 0) mbar_init(xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    __syncwarp();
    // Cluster staging (single row, plain form): the CTAs of a cluster quantise a share of the row each and write it
    // into every member's shared memory.  First cluster phase: every member is running (its shared memory exists).
    constexpr bool CL = M1 && !XG && !XC && !IND;
    [[maybe_unused]] uint32_t crank = 0;
    const uint32_t cs = CL ? a.csize : 1u;
    if constexpr (CL) {
        if (cs > 1u) {
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
            asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
        }
    }

    // ---- producer side: lane 0 issues one tensor copy per unit ------------------
    uint32_t iss_tile = tile0, iss_c = 0, iss_st = 0;
    // IND: the unit as (local slot, tile of that slot), advanced without divisions
    [[maybe_unused]] uint32_t iss_l = 0, iss_tl = 0;
    if constexpr (IND) {
        iss_tl = tile0 - s_first * a.ntiles;
        while (iss_tl >= a.ntiles) iss_tl -= a.ntiles, iss_l++;
    }
    auto issue_next = [&]() {
        if (lane == 0) {
            const uint32_t bar = bar0 + iss_st * 8u;
            const bool full = iss_c < nfull;
            mbar_expect_tx(bar, TR * BB * (full ? a.cb : a.rem));
            if constexpr (IND) {
                const uint32_t l = iss_l;
                const uint32_t row = (l == 0 ? offs[0] : l == 1 ? offs[1] : l == 2 ? offs[2] : offs[3]) + iss_tl * TR;
                const CUtensorMap* map = s_first + l >= a.m.n_slots ? (full ? &a.tmap_b : &a.tmap_b_rem) : (full ? &a.tmap : &a.tmap_rem);
                tma_load_2d(ring + iss_st * a.stage_bytes, map, (b0 + iss_c * a.cb) * BW, row, bar);
            } else {
            if (BPQ4K_CHECK((b0 + iss_c * a.cb + (full ? a.cb : a.rem)) <= nb && iss_tile < a.ntiles && iss_st < a.stages &&
                                (full ? a.cb : a.rem) * TR * BB <= a.stage_bytes, a.status))
            tma_load_2d(ring + iss_st * a.stage_bytes, full ? &a.tmap : &a.tmap_rem, (b0 + iss_c * a.cb) * BW,
                        (uint32_t)wrow0 + iss_tile * TR, bar);
            }
        }
        if (++iss_st == a.stages) iss_st = 0;
        if (++iss_c == nchunks) {
            iss_c = 0;
            iss_tile += tstride;
            if constexpr (IND) {
                iss_tl += tstride;
                while (iss_tl >= a.ntiles) iss_tl -= a.ntiles, iss_l++;  // at most tstride (<= 16) rounds
            }
        }
    };
    // Ring prefetch in two parts.  `pre_wait` stages go out now; the rest of the ring follows once the loads of
    // the activations have been issued (issue_rest).  A deep ring issued in one go just before the dependency
    // wait ends puts ~180 KB per SM in front of those loads in the memory system, and the activation staging
    // -- the one serial step of the kernel -- then waits 1.5-2.5 us for data that is sitting in L2.
    const uint32_t pre_total = min(a.stages, total_units);
    const uint32_t pre_early = min(a.pre_wait, pre_total);
    for (uint32_t i = 0; i < pre_early; i++) issue_next();
    auto issue_rest = [&]() {
        for (uint32_t i = pre_early; i < pre_total; i++) issue_next();
    };
    // Bring the activation rows into L2 (and their page into the TLBs) while waiting.  A prefetch is not a read:
    // if the preceding kernel still writes X, its stores land in the same L2 lines.
    if constexpr (!IND) {
        if (!a.m.n_slots && !XG && !XC) {
            const uint32_t lines = (M * K + 31u) / 32u;
            for (uint32_t i = tid; i < lines; i += blockDim.x) asm volatile("prefetch.global.L2 [%0];" ::"l"(X + (uint64_t)i * 32u));
        }
    }
    // Programmatic dependent launch: everything above touches only this CTA's shared memory
    // and READS the weights, so it may overlap the tail of the preceding kernel in the stream.
    // Let the next kernel start its own prologue, then wait for the preceding kernel (which may
    // have produced X, or may still read Y) before reading X or writing anything.
    stamp(1);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(2);
    if constexpr (XG) issue_rest();  // nothing is staged per CTA in this mode

    // ---- activations: quantise to base-128 digits, once per CTA ---------------------
    const uint32_t NG = K / 64u;
    if constexpr (XC) {
        // digits and scales of all rows, quantised by the kernel that precedes this one in the stream:
        // warp 0 copies them in (one bulk copy per row for each), everybody waits for the bytes
        for (uint32_t i = tid; i < kZeroBytes / 4u; i += blockDim.x) reinterpret_cast<uint32_t*>(smem + a.off_zero)[i] = 0u;
        if (warp == 0) {
            const uint32_t seg = K * 4u, sseg = nb * 256u;  // digits of one row; scales of four interleaved rows
            if (lane == 0) mbar_expect_tx(xbar, (uint32_t)TOK * seg + (uint32_t)(TOK / 4) * sseg);
            __syncwarp();
            for (uint32_t tok = lane; tok < (uint32_t)TOK; tok += 32u) {
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smem_u32(smem + a.off_x) + tok * seg),
                             "l"(a.xfrag_g + kZeroBytes + (uint64_t)tok * seg), "r"(seg), "r"(xbar)
                             : "memory");
                if (tok < (uint32_t)(TOK / 4))
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     smem_u32(smem + a.off_S) + tok * sseg),
                                 "l"(reinterpret_cast<const uint8_t*>(a.S_g) + (uint64_t)tok * sseg), "r"(sseg), "r"(xbar)
                                 : "memory");
            }
        }
        issue_rest();
        uint32_t polls = 0;
        while (!mbar_try_wait(xbar, 0)) {
            if (++polls > kWaitPolls) {  // give up: flag it and carry on with whatever is there
                if (tid == 0 && a.status) atomicExch(a.status, kDeviceTimeout);
                break;
            }
        }
        __syncthreads();  // zero region written
    } else if constexpr (!XG) {
        // one pass: every thread quantises 8-float items straight from global memory
        for (uint32_t i = tid; i < kZeroBytes / 4u; i += blockDim.x) reinterpret_cast<uint32_t*>(smem + a.off_zero)[i] = 0u;
        const uint32_t per_row = K / 8u;
        uint8_t* frag = smem + a.off_x;
        float* SI = reinterpret_cast<float*>(smem + a.off_S);
        // rows past M carry zeros: clear their digits and scales instead of quantising zeros
        const uint32_t mrows = M1 ? 1u : min(M, (uint32_t)TOK);
        if constexpr (!M1) {
            for (uint32_t i = mrows * K + tid; i < (uint32_t)TOK * K; i += blockDim.x) reinterpret_cast<uint32_t*>(frag)[i] = 0u;
            // (scales of four rows are interleaved: float i belongs to row (i / (nb*64))*4 + (i % 16)/4)
            if (mrows < (uint32_t)TOK)
                for (uint32_t i = tid; i < (uint32_t)TOK * nb * 16u; i += blockDim.x)
                    if ((i / (nb * 64u)) * 4u + ((i & 15u) >> 2) >= mrows) SI[i] = 0.f;
        }
        // IND: the rows of all local slots in one pass, slot l staged as "row l" of the shared-memory layout
        const uint32_t items = (IND ? nloc : mrows) * per_row;
        [[maybe_unused]] auto pick = [&](const float* const* rows, uint32_t l) {
            return l == 0 ? rows[0] : l == 1 ? rows[1] : l == 2 ? rows[2] : rows[3];
        };
        // Fused prologue on the single activation row (the reference's q4k_matmul_norm.wgsl:47-92
        // and q4k_down_gelu.wgsl:47-62, plus the silu form of silu_mul_fused): transform while staging.
        [[maybe_unused]] auto prologue_item = [&](float4 (&v)[2], const float4 (&w)[2], float rstd) {
            float* vf = reinterpret_cast<float*>(v);
            const float* wf = reinterpret_cast<const float*>(w);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float g = vf[i];
                if (a.m.prologue == 1u) {
                    vf[i] = g * rstd * wf[i];
                } else if (a.m.prologue == 2u) {
                    const float inner = 0.7978845608f * (g + 0.044715f * g * g * g);
                    vf[i] = 0.5f * g * (1.f + tanhf(inner)) * wf[i];
                } else {
                    vf[i] = __fdividef(g, 1.f + __expf(-g)) * wf[i];  // relative error ~1e-6: far inside the digits' 2^-22
                }
            }
        };
        if (FP && a.m.prologue && !(CL && cs > 1u)) {
            float rstd = 1.f;
            bool rest_issued = false;
            constexpr int UP = 4;  // items per thread and round, loads of x and aux issued together
            // RMSNorm of a row that fits one round: the values stay in registers between the sum of squares and the
            // transform (one pass over X instead of two)
            const bool one_round = !IND && items <= blockDim.x * UP;
            if (a.m.prologue == 1u && !one_round) {
                float ss = 0.f;
                for (uint32_t i = tid; i < K / 4u; i += blockDim.x) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(X) + i);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                issue_rest();
                rest_issued = true;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                float* red = reinterpret_cast<float*>(smem + a.off_part);
                if (lane == 0) red[warp] = ss;
                __syncthreads();
                float tot = 0.f;
                for (uint32_t w2 = 0; w2 < swarps; w2++) tot += red[w2];
                rstd = 1.f / sqrtf(tot / (float)K + a.m.eps);
                __syncthreads();  // red is the partial-sum buffer of the main loop
            }
            for (uint32_t base = 0; base < items; base += blockDim.x * UP) {
                const uint32_t nj = min((uint32_t)UP, (items - base + blockDim.x - 1) / blockDim.x);  // uniform over the CTA
                float4 v[UP][2], w[UP][2];
#pragma unroll
                for (int j = 0; j < UP; j++) {
                    const uint32_t it = base + j * blockDim.x + tid;
                    v[j][0] = v[j][1] = w[j][0] = w[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if ((uint32_t)j < nj && it < items) {
                        const uint32_t l = IND ? it / per_row : 0u, c = it - l * per_row;
                        const float4* xp = reinterpret_cast<const float4*>((IND ? pick(xrow, l) : X) + item_offset(c));
                        const float4* ap = reinterpret_cast<const float4*>((IND ? pick(arow, l) : AUX) + item_offset(c));
                        v[j][0] = __ldg(xp);
                        v[j][1] = __ldg(xp + 4);
                        w[j][0] = __ldg(ap);
                        w[j][1] = __ldg(ap + 4);
                    }
                }
                if (!rest_issued) issue_rest(), rest_issued = true;
                if (a.m.prologue == 1u && one_round) {  // (one_round: this is the loop's only iteration, for every thread)
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < UP; j++) {  // items that were not loaded are zeros
                        const float* vf = reinterpret_cast<const float*>(v[j]);
#pragma unroll
                        for (int i = 0; i < 8; i++) ss = fmaf(vf[i], vf[i], ss);
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                    float* red = reinterpret_cast<float*>(smem + a.off_part);
                    if (lane == 0) red[warp] = ss;
                    __syncthreads();
                    float tot = 0.f;
                    for (uint32_t w2 = 0; w2 < swarps; w2++) tot += red[w2];
                    rstd = 1.f / sqrtf(tot / (float)K + a.m.eps);
                    __syncthreads();  // red is the partial-sum buffer of the main loop
                }
                // two items side by side
#pragma unroll
                for (int j = 0; j < UP; j += 2) {
                    if ((uint32_t)j >= nj) break;
                    const uint32_t it0 = base + j * blockDim.x + tid, it1 = it0 + blockDim.x;
                    const bool two = (uint32_t)(j + 1) < nj;
                    const uint32_t l0 = (IND && it0 < items) ? it0 / per_row : 0u;
                    prologue_item(v[j], w[j], rstd);
                    if (two) {
                        const uint32_t l1 = (IND && it1 < items) ? it1 / per_row : 0u;
                        prologue_item(v[j + 1], w[j + 1], rstd);
                        const QuantItem q0 = quantize_compute(v[j][0], v[j][1]), q1 = quantize_compute(v[j + 1][0], v[j + 1][1]);
                        quantize_store(q0, K, l0, it0 < items ? it0 - l0 * per_row : 0u, it0 < items, frag, SI, false);
                        quantize_store(q1, K, l1, it1 < items ? it1 - l1 * per_row : 0u, it1 < items, frag, SI, false);
                    } else {
                        quantize_loaded(v[j][0], v[j][1], K, l0, it0 < items ? it0 - l0 * per_row : 0u, it0 < items, frag, SI);
                    }
                }
            }
        } else if (CL && cs > 1u) {
            if constexpr (CL) {
            // this CTA's share of the row: a run of whole sub-blocks (four items each)
            const uint32_t ipc = (((items + cs - 1u) / cs) + 3u) & ~3u;
            const uint32_t it0 = crank * ipc;
            const uint32_t mine = it0 < items ? min(ipc, items - it0) : 0u;
            uint32_t xr[4], sr[4];
#pragma unroll
            for (uint32_t r = 0; r < 4; r++) {
                const uint32_t rr = r < cs ? r : 0u;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(xr[r]) : "r"(smem_u32(frag)), "r"(rr));
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(sr[r]) : "r"(smem_u32(SI)), "r"(rr));
            }
            constexpr int U = 2;
            bool started = false;
            for (uint32_t base = 0; base < mine || !started; base += blockDim.x * U) {
                float4 v[U][2];
                [[maybe_unused]] float4 w[U][2];
                uint32_t c8[U];
                bool valid[U];
#pragma unroll
                for (int j = 0; j < U; j++) {
                    const uint32_t li = base + j * blockDim.x + tid;
                    valid[j] = li < mine;
                    c8[j] = valid[j] ? it0 + li : 0u;
                    v[j][0] = v[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if constexpr (FP) w[j][0] = w[j][1] = v[j][0];
                    if (valid[j]) {
                        const float4* xp = reinterpret_cast<const float4*>(X + item_offset(c8[j]));
                        v[j][0] = __ldg(xp);
                        v[j][1] = __ldg(xp + 4);
                        if (FP && a.m.prologue) {  // (element-wise prologues only: the host keeps RMSNorm rows unclustered)
                            const float4* ap = reinterpret_cast<const float4*>(AUX + item_offset(c8[j]));
                            w[j][0] = __ldg(ap);
                            w[j][1] = __ldg(ap + 4);
                        }
                    }
                }
                if (!started) issue_rest();
                if constexpr (FP) {
                    if (a.m.prologue) {
                        prologue_item(v[0], w[0], 1.f);
                        prologue_item(v[1], w[1], 1.f);
                    }
                }
                const QuantItem q0 = quantize_compute(v[0][0], v[0][1]), q1 = quantize_compute(v[1][0], v[1][1]);
                if (!started) {  // every member runs: its shared memory may be written
                    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                    started = true;
                }
                quantize_store_cluster(q0, c8[0], valid[0] && BPQ4K_CHECK(c8[0] < per_row, a.status), xr, sr, cs);
                quantize_store_cluster(q1, c8[1], valid[1] && BPQ4K_CHECK(c8[1] < per_row, a.status), xr, sr, cs);
            }
            }
        } else {
        // up to four items per thread and round, all loads issued before the first use (a round
        // trip to L2 or HBM per item would otherwise be paid one after the other)
        constexpr int U = 4;
        for (uint32_t base = 0; base < items; base += blockDim.x * U) {
            const uint32_t nj = min((uint32_t)U, (items - base + blockDim.x - 1) / blockDim.x);  // uniform over the CTA
            float4 v[U][2];
            uint32_t tok[U], c8[U];
            bool valid[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const uint32_t it = base + j * blockDim.x + tid;
                valid[j] = (uint32_t)j < nj && it < items;
                tok[j] = valid[j] ? it / per_row : 0u;
                c8[j] = valid[j] ? it - tok[j] * per_row : 0u;
                v[j][0] = v[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (valid[j]) {
                    const float4* xp = reinterpret_cast<const float4*>((IND ? pick(xrow, tok[j]) : X + (uint64_t)tok[j] * K) + item_offset(c8[j]));
                    v[j][0] = __ldg(xp);
                    v[j][1] = __ldg(xp + 4);
                }
            }
            if (base == 0) issue_rest();
            // two items side by side (nj is uniform over the CTA, so every lane takes the same branch)
#pragma unroll
            for (int j = 0; j < U; j += 2) {
                if ((uint32_t)j >= nj) break;
                const bool two = (uint32_t)(j + 1) < nj;
                const bool ok0 = valid[j] && BPQ4K_CHECK(tok[j] < (IND ? kMaxLocalSlots : (uint32_t)TOK) && c8[j] < per_row, a.status);
                if (two) {
                    const bool ok1 = valid[j + 1] && BPQ4K_CHECK(tok[j + 1] < (IND ? kMaxLocalSlots : (uint32_t)TOK) && c8[j + 1] < per_row, a.status);
                    const QuantItem q0 = quantize_compute(v[j][0], v[j][1]), q1 = quantize_compute(v[j + 1][0], v[j + 1][1]);
                    quantize_store(q0, K, tok[j], c8[j], ok0, frag, SI, !M1);
                    quantize_store(q1, K, tok[j + 1], c8[j + 1], ok1, frag, SI, !M1);
                } else {
                    quantize_loaded(v[j][0], v[j][1], K, tok[j], c8[j], ok0, frag, SI, !M1);
                }
            }
        }
        }
        if (items == 0) issue_rest();  // (never with a valid launch: every CTA stages at least one row)
        if (CL && cs > 1u) {
            // second cluster phase: every member's share has been written everywhere (also orders this CTA's threads)
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        } else {
            __syncthreads();
        }
    }

    stamp(3);
    if (helper) return;  // (no CTA-wide barrier follows: the tile epilogues use named barriers over the plan's warps)

    // ---- per-lane constants ----------------------------------------------------
    // ldmatrix row addresses: lanes 0-7 rows 0-7 bytes [0,16), 8-15 rows 8-15 bytes [0,16),
    // 16-23 rows 0-7 bytes [16,32), 24-31 rows 8-15 bytes [16,32)
    // (row pitch = bytes of the stage's box row: cb or rem blocks)
    const uint32_t lm_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u, lm_col = QS + (lane >> 4) * 16u;
    // B operand: column n = lane/4 -> pair n/2 (parity n/2%2), part n%2; t = lane%4
    const uint32_t bn = lane >> 2, bt = lane & 3u;
    const uint32_t b_par = (bn >> 1) & 1u;
    // C / post-processing role: column pair t.  M1: sub-block parity t%2 of row r (t < 2) or r+8.
    // Otherwise: activation row t of the mma tile, both rows r and r+8, both parities.
    const uint32_t c_par = lane & 1u;
    const uint32_t row_a = M1 ? (lane >> 2) + ((bt >> 1) << 3) : (lane >> 2);
    const uint32_t sel0 = 0x7440u + c_par, sel1 = 0x7442u + c_par;
    const float par_scale = (c_par && !Q5) ? 0.0625f : 1.f;  // Q4_K: odd sub-blocks arrive as 16*q

    // This lane's B data lives at  xbase + ((tok*NG + G)*2 + parity)*128 + c*64 + t*16  (c = n%2).
    // In the mmas of the other parity the lane feeds zeros: it reads the zero block with
    // stride 0 instead.  AddrT is a shared-memory offset, or a global address in XG mode.
    using AddrT = typename std::conditional<XG, uint64_t, uint32_t>::type;
    AddrT xdata, xzero, s_addr;
    if constexpr (XG) {
        xdata = reinterpret_cast<uint64_t>(a.xfrag_g) + kZeroBytes;  // the scratch starts with the zero region
        xzero = reinterpret_cast<uint64_t>(a.xfrag_g);
        s_addr = reinterpret_cast<uint64_t>(a.S_g);
    } else {
        xdata = smem_u32(smem + a.off_x);
        xzero = smem_u32(smem + a.off_zero);
        s_addr = smem_u32(smem + a.off_S);
    }
    // M1: the lane's own parity block, or the zero region for the mmas of the other parity.
    const AddrT mine = xdata + b_par * 128u + (bn & 1u) * 64u + bt * 16u;
    const AddrT pa0 = b_par == 0 ? mine : xzero;       // source for the even-sub-block mmas
    const AddrT pb0 = b_par == 1 ? mine : xzero;       // source for the odd-sub-block mmas
    const uint32_t stride_a = b_par == 0 ? 256u : 0u;  // per 64-weight group
    const uint32_t stride_b = b_par == 1 ? 256u : 0u;
    const AddrT s0_addr = s_addr + c_par * 32u;        // + blk*64
    // several rows: column n carries activation row n/2 of the mma tile (digit column n%2); the even
    // and the odd sub-block's 128-byte blocks follow each other
    const AddrT gx_addr = xdata + (AddrT)((bn >> 1) * NG) * 256u + (bn & 1u) * 64u + bt * 16u;  // + nt*4*NG*256 + G*256 (+128)
    const AddrT gs_addr = s_addr + (AddrT)bt * 16u;                                                // + (nt*nb + blk)*256 + g*64
    // 16-byte load at addr + OFF (OFF is folded into the instruction)
    auto load16 = [&](AddrT addr, auto off_tag) -> uint4 {
        constexpr int OFF = decltype(off_tag)::value;
        if constexpr (XG) return __ldg(reinterpret_cast<const uint4*>(addr + OFF));
        else return lds128<OFF>(addr);
    };

    float* part = reinterpret_cast<float*>(smem + a.off_part);
    // double-buffered gather slots: which half this step writes (the word was last written by the barrier
    // kernel that closed the previous step, which precedes this kernel in the stream)
    // (PEER: the fused all-gather's instantiations.  Left in the plain ones, the peer stores and this word cost the
    //  single-GPU decode step 1.4 us although they never ran.)
    const uint64_t par_off = (PEER && a.m.slot_parity) ? (uint64_t)(*reinterpret_cast<const volatile uint32_t*>(a.m.slot_parity) & 1u) * a.m.slot_parity_stride : 0ull;
    uint32_t st = 0, ph = 0, u = 0, failed = 0;
    [[maybe_unused]] uint32_t cur_l = 0, cur_tl = 0;
    if constexpr (IND) {
        cur_tl = tile0 - s_first * a.ntiles;
        while (cur_tl >= a.ntiles) cur_tl -= a.ntiles, cur_l++;
    }

    // One super-block of a 16-row tile against the single activation row (M1): boff = the block in the ring, hdr_off /
    // lm_off = this lane's header and ldmatrix offsets for the stage's row pitch, blk = the block's index in the row.
    [[maybe_unused]] auto m1_block = [&](uint32_t boff, uint32_t hdr_off, uint32_t lm_off, uint32_t blk, [[maybe_unused]] AddrT pa_t,
                                         [[maybe_unused]] AddrT pb_t, [[maybe_unused]] AddrT s_t, float (&acc)[RT][NT][2]) {
        if constexpr (M1) {
                // scales of this thread's rows, its parity's four sub-blocks; the odd sub-block's
                // weights reach the mma as 16*q, so its scale carries the 1/16
                float dsc[1][4], dmn[1][4];
#pragma unroll
                for (int r = 0; r < 1; r++) {
                    const uint4 hv = lds128<0>(boff + hdr_off);
                    const BlockHeader h{hv.x, hv.y, hv.z, hv.w};
                    const float d = half_bits_to_float(h.w0) * par_scale, dmin = half_bits_to_float(h.w0 >> 16);
                    uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
                    unpack_scales_packed(h, sc_lo, sc_hi, mn_lo, mn_hi);
                    // d*(2^23+sc) - d*2^23 in one fma: the product is exact inside the fma
                    const float nd = -d * 8388608.f, ndm = -dmin * 8388608.f;
                    const uint32_t scw[4] = {__byte_perm(sc_lo, 0x4B000000u, sel0), __byte_perm(sc_lo, 0x4B000000u, sel1),
                                             __byte_perm(sc_hi, 0x4B000000u, sel0), __byte_perm(sc_hi, 0x4B000000u, sel1)};
                    const uint32_t mnw[4] = {__byte_perm(mn_lo, 0x4B000000u, sel0), __byte_perm(mn_lo, 0x4B000000u, sel1),
                                             __byte_perm(mn_hi, 0x4B000000u, sel0), __byte_perm(mn_hi, 0x4B000000u, sel1)};
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        dsc[r][g] = fmaf(d, __uint_as_float(scw[g]), nd);
                        dmn[r][g] = fmaf(dmin, __uint_as_float(mnw[g]), ndm);
                    }
                }
                uint4 Sv[NT], Iv[NT];  // per group: sum(xi)*inv and inv of this parity's sub-block
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    Sv[nt] = load16((IND ? s_t : s0_addr) + (AddrT)blk * 64u, std::integral_constant<int, 0>{});
                    Iv[nt] = load16((IND ? s_t : s0_addr) + (AddrT)blk * 64u, std::integral_constant<int, 16>{});
                }
                // data lanes advance 1 KiB per block (4 groups x 256 B); zero lanes stay inside the
                // 1 KiB zero region, so the per-group offset g*256 is an immediate for both
                const AddrT pa = (IND ? pa_t : pa0) + blk * 4u * stride_a, pb = (IND ? pb_t : pb0) + blk * 4u * stride_b;
                const uint32_t lm_addr = boff + lm_off;
                uint32_t qh[4] = {0u, 0u, 0u, 0u};  // Q5_K: fifth bits of this thread's weights, all eight sub-blocks
                if constexpr (Q5) ldmatrix_x4<-32>(lm_addr, qh[0], qh[1], qh[2], qh[3]);
                auto do_group = [&](auto gc) {
                    constexpr int g = decltype(gc)::value;
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4<g * 32>(lm_addr, r0, r1, r2, r3);
                    [[maybe_unused]] constexpr uint32_t kLo = 0x0F0F0F0Fu, kHi = 0xF0F0F0F0u;
                    uint32_t e[4], o[4];
                    if constexpr (Q5) {
                        const uint32_t rr[4] = {r0, r1, r2, r3};
#pragma unroll
                        for (int i = 0; i < 4; i++) merge_fifth_bit<g>(rr[i], qh[i], e[i], o[i]);
                    } else {
                        e[0] = r0 & kLo; e[1] = r1 & kLo; e[2] = r2 & kLo; e[3] = r3 & kLo;  // q   (even sub-block)
                        o[0] = r0 & kHi; o[1] = r1 & kHi; o[2] = r2 & kHi; o[3] = r3 & kHi;  // 16q (odd sub-block)
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4 qa = load16(pa, std::integral_constant<int, g * 256>{});
                        const uint4 qb = load16(pb, std::integral_constant<int, g * 256>{});
                        int c01[4], c2[4];  // column pair = digits (d0, d1) resp. (d2, 0)
                        imma16832_first(c01, e[0], e[1], e[2], e[3], qa.x, qa.y);
                        imma16832_first(c2, e[0], e[1], e[2], e[3], qa.z, qa.w);
                        imma16832(c01, o[0], o[1], o[2], o[3], qb.x, qb.y);
                        imma16832(c2, o[0], o[1], o[2], o[3], qb.z, qb.w);
                        const uint32_t sbits = g == 0 ? Sv[nt].x : g == 1 ? Sv[nt].y : g == 2 ? Sv[nt].z : Sv[nt].w;
                        const float Sg = __uint_as_float(sbits);
                        const float Ig = __uint_as_float(g == 0 ? Iv[nt].x : g == 1 ? Iv[nt].y : g == 2 ? Iv[nt].z : Iv[nt].w);
                        // T = 2^14*sum(a d0) + (2^7*sum(a d1) + sum(a d2)) with a = q or 16q.  The
                        // bracket fits int32 (< 2^26); the whole of T need not (16q weights), so
                        // the top digit joins in float: its sum (< 2^19) times 2^14 is exact.
                        const int u_lo = c01[1] * 128 + c2[0], u_hi = c01[3] * 128 + c2[2];  // rows r, r+8
                        const bool hi = (bt & 2u) != 0;
                        const float v = fmaf((float)(hi ? c01[2] : c01[0]), 16384.f, (float)(hi ? u_hi : u_lo)) * Ig;
                        acc[0][nt][0] = fmaf(dsc[0][g], v, acc[0][nt][0]);
                        acc[0][nt][0] = fmaf(-dmn[0][g], Sg, acc[0][nt][0]);
                    }
                };
                do_group(std::integral_constant<int, 0>{});
                do_group(std::integral_constant<int, 1>{});
                do_group(std::integral_constant<int, 2>{});
                do_group(std::integral_constant<int, 3>{});
        }
    };

    for (uint32_t ti = 0; ti < my_tiles; ti++) {
        uint32_t tile = tile0 + ti * tstride;
        // IND: the unit's slot selects the staged row (data lanes only; zero lanes stay in the zero region),
        // its scales and the output row
        [[maybe_unused]] AddrT pa_t = pa0, pb_t = pb0, s_t = s0_addr;
        if constexpr (IND) {
            const uint32_t l = cur_l, vs = s_first + l;
            tile = cur_tl;
            cur_tl += tstride;
            while (cur_tl >= a.ntiles) cur_tl -= a.ntiles, cur_l++;
            pa_t += b_par == 0 ? l * K * 4u : 0u;
            pb_t += b_par == 1 ? l * K * 4u : 0u;
            s_t += l * nb * 64u;
            Y = vs >= a.m.n_slots ? a.m.Y2 + (uint64_t)(vs - a.m.n_slots) * N : a.m.Y + (uint64_t)vs * N;
        }
        // single-row calls: fetch this lane's residual value now, it is added when the tile is stored
        float res_pre = 0.f;
        if (FP && a.m.residual && wk == 0 && lane < 16u && tile * 16u + lane < N) res_pre = __ldg(a.m.residual + tile * 16u + lane);  // (FP is single-row: 16-row tiles)
        float acc[RT][NT][2];
#pragma unroll
        for (int t = 0; t < RT; t++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) acc[t][nt][0] = acc[t][nt][1] = 0.f;

        for (uint32_t c = 0; c < nchunks; c++) {
            const uint32_t bs = b0 + c * a.cb;
            const uint32_t nblk = c < nfull ? a.cb : a.rem;
            const uint32_t pitch = nblk * BB;
            const uint32_t lm_off = lm_row * pitch + lm_col, hdr_off = row_a * pitch;
            const uint32_t bar = bar0 + st * 8u;
            if (!failed) {
                uint32_t polls = 0;
                while (!mbar_try_wait(bar, ph)) {
                    if (++polls > kWaitPolls) {  // give up: flag it, keep the barriers matched
                        failed = 1;
                        if (lane == 0 && a.status) atomicExch(a.status, kDeviceTimeout);
                        break;
                    }
                }
            }
            uint32_t boff = ring + st * a.stage_bytes;
            for (uint32_t blk = bs; blk < bs + nblk; blk++, boff += BB) {
                if constexpr (M1) {
                m1_block(boff, hdr_off, lm_off, blk, pa_t, pb_t, s_t, acc);
                } else {
                // ---- several activation rows: every mma is one sub-block x four activation rows ----
                // headers of rows r and r+8 of each 16-row mma tile: d, dmin and the packed 6-bit scales and mins; the
                // float scale of a sub-block is formed when its group is processed (d*(2^23+sc) - d*2^23 in one fma: exact)
                float hd[RT][2], hm[RT][2], hnd[RT][2], hpm[RT][2];
                uint32_t sc_lo[RT][2], sc_hi[RT][2], mn_lo[RT][2], mn_hi[RT][2];
#pragma unroll
                for (int t = 0; t < RT; t++)
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const uint4 hv = lds128<0>(boff + hdr_off + (t * 16u + r * 8u) * pitch);
                        const BlockHeader h{hv.x, hv.y, hv.z, hv.w};
                        hd[t][r] = half_bits_to_float(h.w0);
                        hm[t][r] = -half_bits_to_float(h.w0 >> 16);  // the minimum enters with a minus sign
                        hnd[t][r] = -hd[t][r] * 8388608.f;
                        hpm[t][r] = -hm[t][r] * 8388608.f;
                        unpack_scales_packed(h, sc_lo[t][r], sc_hi[t][r], mn_lo[t][r], mn_hi[t][r]);
                    }
                const uint32_t lm_addr = boff + lm_off;
                uint32_t qh[RT][4];  // Q5_K: fifth bits of this thread's weights, all eight sub-blocks
#pragma unroll
                for (int t = 0; t < RT; t++) {
                    qh[t][0] = qh[t][1] = qh[t][2] = qh[t][3] = 0u;
                    if constexpr (Q5) ldmatrix_x4<-32>(lm_addr + t * 16u * pitch, qh[t][0], qh[t][1], qh[t][2], qh[t][3]);
                }
                const AddrT gx_blk = gx_addr + (AddrT)blk * 1024u;
                const AddrT gs_blk = gs_addr + (AddrT)blk * 256u;
                auto do_group = [&](auto gc) {
                    constexpr int g = decltype(gc)::value;
                    [[maybe_unused]] constexpr uint32_t kLo = 0x0F0F0F0Fu, kHi = 0xF0F0F0F0u;
                    uint32_t e[RT][4], o[RT][4];
                    // scales of sub-blocks 2g (even) and 2g+1 (odd) for rows r and r+8 of each mma tile
                    float dse[RT][2], dso[RT][2], dme[RT][2], dmo[RT][2];
#pragma unroll
                    for (int t = 0; t < RT; t++) {
                        uint32_t r0, r1, r2, r3;
                        ldmatrix_x4<g * 32>(lm_addr + t * 16u * pitch, r0, r1, r2, r3);
                        if constexpr (Q5) {
                            const uint32_t rr[4] = {r0, r1, r2, r3};
#pragma unroll
                            for (int i = 0; i < 4; i++) merge_fifth_bit<g>(rr[i], qh[t][i], e[t][i], o[t][i]);
                        } else {
                            e[t][0] = r0 & kLo; e[t][1] = r1 & kLo; e[t][2] = r2 & kLo; e[t][3] = r3 & kLo;  // q   (even sub-block)
                            o[t][0] = r0 & kHi; o[t][1] = r1 & kHi; o[t][2] = r2 & kHi; o[t][3] = r3 & kHi;  // 16q (odd sub-block)
                        }
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const uint32_t scw = g < 2 ? sc_lo[t][r] : sc_hi[t][r], mnw = g < 2 ? mn_lo[t][r] : mn_hi[t][r];
                            constexpr uint32_t se = 0x7440u + ((2 * g) & 3), so = 0x7440u + ((2 * g + 1) & 3);
                            dse[t][r] = fmaf(hd[t][r], __uint_as_float(__byte_perm(scw, 0x4B000000u, se)), hnd[t][r]);
                            dso[t][r] = fmaf(hd[t][r], __uint_as_float(__byte_perm(scw, 0x4B000000u, so)), hnd[t][r]);
                            dme[t][r] = fmaf(hm[t][r], __uint_as_float(__byte_perm(mnw, 0x4B000000u, se)), hpm[t][r]);
                            dmo[t][r] = fmaf(hm[t][r], __uint_as_float(__byte_perm(mnw, 0x4B000000u, so)), hpm[t][r]);
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        // the digits and the two floats of this thread's activation row: loaded once, used by every mma tile
                        const AddrT xa = gx_blk + (AddrT)(nt * 4u * NG) * 256u;
                        const uint4 qa = load16(xa, std::integral_constant<int, g * 256>{});        // even sub-block digits
                        const uint4 qb = load16(xa, std::integral_constant<int, g * 256 + 128>{});  // odd sub-block digits
                        const uint4 si = load16(gs_blk + (AddrT)(nt * nb) * 256u, std::integral_constant<int, g * 64>{});
                        const float Se = __uint_as_float(si.x), Ie = __uint_as_float(si.y);
                        const float So = __uint_as_float(si.z), Io = __uint_as_float(si.w);
#pragma unroll
                        for (int t = 0; t < RT; t++) {
                            int ce01[4], ce2[4], co01[4], co2[4];  // column pair = digits (d0, d1) resp. (d2, 0)
                            imma16832_first(ce01, e[t][0], e[t][1], e[t][2], e[t][3], qa.x, qa.y);
                            imma16832_first(ce2, e[t][0], e[t][1], e[t][2], e[t][3], qa.z, qa.w);
                            imma16832_first(co01, o[t][0], o[t][1], o[t][2], o[t][3], qb.x, qb.y);
                            imma16832_first(co2, o[t][0], o[t][1], o[t][2], o[t][3], qb.z, qb.w);
                            // T = 2^14*sum(a d0) + 2^7*sum(a d1) + sum(a d2), exact in int32: |T| < 2^31 for a = q; the odd
                            // sub-block of Q4_K arrives as a = 16q, every term is a multiple of 16 and T/16 is formed instead
#pragma unroll
                            for (int r = 0; r < 2; r++) {
                                const int te = ce01[2 * r] * 16384 + ce01[2 * r + 1] * 128 + ce2[2 * r];
                                const int to = Q5 ? co01[2 * r] * 16384 + co01[2 * r + 1] * 128 + co2[2 * r]
                                                  : co01[2 * r] * 1024 + co01[2 * r + 1] * 8 + (co2[2 * r] >> 4);
                                float s2 = acc[t][nt][r];
                                s2 = fmaf(dse[t][r], (float)te * Ie, s2);
                                s2 = fmaf(dme[t][r], Se, s2);
                                s2 = fmaf(dso[t][r], (float)to * Io, s2);
                                s2 = fmaf(dmo[t][r], So, s2);
                                acc[t][nt][r] = s2;
                            }
                        }
                    }
                };
                do_group(std::integral_constant<int, 0>{});
                do_group(std::integral_constant<int, 1>{});
                do_group(std::integral_constant<int, 2>{});
                do_group(std::integral_constant<int, 3>{});
                }
            }
            // the stage is free: refill it with the unit `stages` ahead
            __syncwarp();
            fence_proxy_async();
            if (u + a.stages < total_units) issue_next();
            u++;
            if (++st == a.stages) {
                st = 0;
                ph ^= 1u;
            }
        }

        // ---- tile epilogue: parities -> K slices -> bias -> Y -------------------
        float* pbuf = part + ((uint64_t)((ti & 1u) * nwarps + warp)) * (TOK * TR);
        if constexpr (M1) {
            // the two sub-block parities of a row sit in neighbouring lanes
            const float s = acc[0][0][0] + __shfl_xor_sync(0xFFFFFFFFu, acc[0][0][0], 1);
            if (c_par == 0) pbuf[row_a] = s;
        } else {
#pragma unroll
            for (int t = 0; t < RT; t++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    pbuf[(nt * 4u + bt) * TR + t * 16u + row_a] = acc[t][nt][0];
                    pbuf[(nt * 4u + bt) * TR + t * 16u + row_a + 8u] = acc[t][nt][1];
                }
        }
        if (a.wk > 1) {
            asm volatile("bar.sync %0, %1;" ::"r"(wt + 1u), "r"(a.wk * 32u) : "memory");
        } else {
            __syncwarp();
        }
        if (wk == 0) {
            const float* gbuf = part + ((uint64_t)((ti & 1u) * nwarps + warp)) * (TOK * TR);
            for (uint32_t idx = lane; idx < (uint32_t)TOK * TR; idx += 32u) {
                const uint32_t tok = idx / TR, row = tile * TR + (idx % TR);
                if (tok < M && row < N) {
                    float s = 0.f;
                    for (uint32_t k2 = 0; k2 < a.wk; k2++) s += gbuf[(uint64_t)k2 * (TOK * TR) + idx];
                    float yv = s + (a.m.bias ? a.m.bias[row] : 0.f);
                    if (FP) yv += res_pre;
                    if (BPQ4K_CHECK(tok < (IND || a.m.n_slots ? 1u : a.m.M) && row < N && idx < (uint32_t)TOK * TR, a.status))
                    Y[(uint64_t)tok * N + row + par_off] = yv;
                    // fused all-gather: the same value goes straight into every peer's gather buffer
                    if constexpr (PEER)
                        for (uint32_t p = 0; p < a.m.n_peers; p++) a.m.peer_Y[p][(uint64_t)tok * N + row + par_off] = yv;
                }
            }
        }
    }

    stamp(4);
    stamp(5);
#ifdef BPQ4K_STAMPS
    if (a.stamps && tid == 0 && blockIdx.y == 0 && blockIdx.x < kStampCtas) {
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        a.stamps[((uint64_t)a.stamp_slot * kStampCtas + blockIdx.x) * 8u + 7u] = smid | ((unsigned long long)gridDim.x << 32);
    }
#endif
}

// ---------------------------------------------------------------------------
// XG mode: quantise the activations once per call into global scratch, in the same layout
// the kernel above keeps in shared memory.
// Scratch layout: [1 KiB zeros][digits: tokens*K*4 B][SI: tokens*(K/32)*2 floats]
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_activations_kernel(const float* __restrict__ X, uint32_t M, uint32_t K,
                                                                   uint32_t tokens, uint8_t* __restrict__ scratch) {
    // the matmul kernel that follows may start its weight prefetch now; it waits for this grid to
    // complete before it reads the scratch
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint8_t* frag = scratch + kZeroBytes;
    float* SI = reinterpret_cast<float*>(frag + (uint64_t)tokens * K * 4u);
    const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x;
    if (gtid < kZeroBytes / 4u) reinterpret_cast<uint32_t*>(scratch)[gtid] = 0u;
    const uint32_t per_row = K / 8u, items = tokens * per_row;
    for (uint32_t base = blockIdx.x * blockDim.x; base < items; base += gridDim.x * blockDim.x) {
        const uint32_t it = base + threadIdx.x;
        const bool valid = it < items;
        const uint32_t tok = valid ? it / per_row : 0u;
        quantize_item(X, M, K, tok, valid ? it - tok * per_row : 0u, valid, frag, SI, tokens > 1u);
    }
}

// Launch one instantiation.  The grid is persistent: at most as many CTAs as can be
// resident at once (occupancy query, cached), never more than there are tile groups.
template <int NT, bool M1, bool XG, bool Q5 = false, bool XC = false, bool FP = false, bool IND = false, int RT = 1, bool PEER = false>
cudaError_t launch_one(const StreamArgs& sa, uint32_t groups, uint32_t slots_y, uint32_t threads, size_t smem,
                       int sm_count, uint32_t ctas_per_sm_override, bool pdl, cudaStream_t stream, uint32_t flat_grid = 0) {
    static KernelConfig kcfg;  // per instantiation; per-device slots and a mutex inside
    int occ = 1;
    if (cudaError_t e = kcfg.prepare(reinterpret_cast<const void*>(gemv_stream_kernel<NT, M1, XG, Q5, XC, FP, IND, RT, PEER>), threads, smem, &occ))
        return e;
    uint32_t per_sm = (uint32_t)occ;
    if (ctas_per_sm_override && ctas_per_sm_override < per_sm) per_sm = ctas_per_sm_override;
    // Every CTA walks ceil(groups/gx) tile groups.  Pick the smallest grid that needs no more
    // rounds than the full machine would, so that all CTAs carry (almost) the same load:
    // 448 groups on 148 SMs -> 4 rounds -> 112 CTAs of exactly 4, not 148 CTAs of 3 or 4.
    const uint64_t cap = (uint64_t)sm_count * per_sm;
    uint32_t gx = groups;
    if ((uint64_t)gx * slots_y > cap) {
        // CTAs per slot such that the whole 2-D grid fits the machine at once (never a partial second wave)
        uint32_t cap_x = (uint32_t)(cap / slots_y);
        if (cap_x == 0) cap_x = 1;
        const uint32_t rounds = (groups + cap_x - 1) / cap_x;
        gx = (groups + rounds - 1) / rounds;
    }
    if (gx == 0) gx = 1;
    if (flat_grid) gx = flat_grid, slots_y = 1;  // IND: the planner fixed the grid (one CTA per SM at most)
    StreamArgs sb = sa;
    if (!flat_grid && slots_y == 1 && !sa.m.n_slots) {
        // Direct form: every resident CTA slot gets a contiguous, balanced share of the tiles (one CTA more or
        // less keeps all SMs streaming; a grid that left SMs idle to equalise rounds ran at the per-SM rate).
        gx = (uint32_t)(groups < cap ? groups : cap);
        if (gx == 0) gx = 1;
        sb.contig = 1;
        sb.u_base = sa.ntiles / gx;
        sb.u_extra = sa.ntiles % gx;
    }
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    // Cluster staging: only the plain single-row form, only with a contiguous split, and only as many CTAs as the
    // device can keep resident as whole clusters (queried once per device, kernel and cluster size)
    uint32_t cs = (M1 && !XG && !XC && !IND && sb.contig && !(FP && sa.m.prologue == 1u)) ? sa.csize : 1u;  // (RMSNorm needs the whole row in every CTA)
    if (cs > 1u) {
        static std::mutex mu;
        static int max_clusters[16][5];  // [device][cluster size], 0 = not asked yet
        int dev = 0;
        cudaGetDevice(&dev);
        int mc = 0;
        if (dev >= 0 && dev < 16 && cs <= 4u) {
            std::lock_guard<std::mutex> lock(mu);
            mc = max_clusters[dev][cs];
            if (mc == 0) {
                cudaLaunchConfig_t q{};
                q.gridDim = dim3(cs * 64u);
                q.blockDim = dim3(threads);
                q.dynamicSmemBytes = smem;
                cudaLaunchAttribute qa[1];
                qa[0].id = cudaLaunchAttributeClusterDimension;
                qa[0].val.clusterDim.x = cs, qa[0].val.clusterDim.y = 1, qa[0].val.clusterDim.z = 1;
                q.attrs = qa;
                q.numAttrs = 1;
                if (cudaOccupancyMaxActiveClusters(&mc, gemv_stream_kernel<NT, M1, XG, Q5, XC, FP, IND, RT, PEER>, &q) != cudaSuccess || mc <= 0) {
                    cudaGetLastError();
                    mc = -1;
                }
                max_clusters[dev][cs] = mc;
            }
        }
        uint32_t gc = mc > 0 ? (uint32_t)mc * cs : 0u;
        if (gc > gx) gc = gx / cs * cs;
        if (gc >= cs && gc * 100u >= gx * 97u) {  // (a grid that lost more than 3 % of the SMs to whole clusters streams slower than it stages faster)
            gx = gc;
            sb.u_base = sa.ntiles / gx;
            sb.u_extra = sa.ntiles % gx;
            attr[na].id = cudaLaunchAttributeClusterDimension;
            attr[na].val.clusterDim.x = cs, attr[na].val.clusterDim.y = 1, attr[na].val.clusterDim.z = 1;
            na++;
        } else {
            cs = 1;
        }
    }
    sb.csize = cs;
    cfg.gridDim = dim3(gx, slots_y);
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_stream_kernel<NT, M1, XG, Q5, XC, FP, IND, RT, PEER>, sb);
    if (e != cudaSuccess && cs > 1u) {
        // a context that cannot place clusters (restricted SM sets): the same launch without them
        cudaGetLastError();
        sb.csize = 1;
        cfg.numAttrs = na - 1;  // the cluster attribute is the last one
        e = cudaLaunchKernelEx(&cfg, gemv_stream_kernel<NT, M1, XG, Q5, XC, FP, IND, RT, PEER>, sb);
    }
    return e;
}

static_assert(sizeof(CUtensorMap) == 128, "TmapCache::Entry::map must hold a CUtensorMap");

}  // namespace

bool gemv_stream_stamps_built() {
#ifdef BPQ4K_STAMPS
    return true;
#else
    return false;
#endif
}

size_t gemv_stream_scratch_bytes(uint32_t M, uint32_t K) {
    const uint32_t tokens = M <= 1 ? 1 : (M + 3) / 4 * 4;
    return kZeroBytes + (size_t)tokens * K * 4 + (size_t)tokens * (K / 32) * 8 + 256;
}

cudaError_t launch_gemv_stream(const MatmulArgs& m, const StreamTuning& tune, void* scratch, size_t scratch_bytes,
                               int* status_dev, int sm_count, TmapCache* tmaps, cudaStream_t stream, int* launches,
                               int qtype) {
    if (m.N == 0) return cudaSuccess;
    if (qtype != 12 && qtype != 13) return cudaErrorInvalidValue;
    const bool q5 = qtype == 13;
    const uint32_t block_bytes = q5 ? 176u : kBlockBytes, block_words = block_bytes / 4u;
    const bool indirect = m.n_slots != 0;
    const uint32_t M = indirect ? 1 : m.M;
    if (M == 0) return cudaSuccess;
    if (M > 16) return cudaErrorInvalidValue;  // callers split larger M
    const uint32_t nb = m.K / kQK;
    const bool m1 = M == 1;
    // Several activation rows and many weight rows: a warp takes 32 rows (two mma row tiles) through its ring at a
    // time, so the digits and scales of the activation rows are fetched once per two tiles (they are what loads
    // the shared-memory pipe, or L2 when they live in the global scratch).
    // Measured (M = 8): 8192 x 28672 69.6 against 93.5 us, 4096 x 14336 20.0 against 24.4 us; no gain where the digits sit
    // in shared memory (128256 x 4096: 98 against 100 us) and a loss at K = 8192, where twelve warps matter more.
    const bool peer = m.n_peers != 0 || m.slot_parity != nullptr;  // the fused all-gather's instantiations (16-row units only)
    const uint32_t rt = peer || tune.rows_per_unit == 16 ? 1u : tune.rows_per_unit == 32 ? (m1 || indirect ? 1u : 2u)
                        : (!m1 && !indirect && m.N >= 2048u && m.K >= 14336u && (uint64_t)M * m.K > 40960u) ? 2u : 1u;
    const uint32_t tile_rows = 16u * rt;
    const uint32_t ntiles = (m.N + tile_rows - 1) / tile_rows;
    const int NT = m1 ? 1 : (int)((M + 3) / 4);
    const uint32_t tokens = m1 ? 1 : NT * 4;

    // ---- plan ------------------------------------------------------------------
    constexpr uint32_t kSmemMax = 227 * 1024;
    // Defaults from tuning sweeps on B200 over the Llama-3 8B and 70B projection shapes:
    //   up to 640 tiles    all warps the kernel allows (16 with one activation row), K split as far
    //                      as possible while every tile group still gets its own resident CTA (one
    //                      round, everything in flight at once), 1-block stages, 2 deep
    //   more               8 warps, about 8 super-blocks per warp and tile, 5-block stages, 4 deep
    const uint64_t tiles_total = (uint64_t)ntiles * (indirect ? m.n_slots : 1);
    const bool small = tiles_total <= 640;
    // Several activation rows (sweeps over the same shapes, M = 2, 4, 8): the digits of all rows
    // should stay in shared memory, so the rings are narrower; with K > 4096 they do not fit
    // next to any ring and more warps hide the latency of reading them through L1/L2 instead.
    const bool wide_k = m.K > 4096;
    // (single row, rows of at most four super-blocks: a tile is over so quickly that 16 warps are needed to keep
    //  copies in flight -- 2048x768 expert matrices, 64 slots: 13.1 us against 14.8 us with 8 warps)
    uint32_t warps_m1 = small ? 16 : 8;
    // (not with more slots than SMs: those run as a unit list, whose CTAs stage several rows and need the room)
    if (!small && nb <= 4 && !(indirect && m.n_slots > (uint32_t)sm_count)) {  // only where 16 two-stage rings of whole rows fit next to the staged row
        const uint32_t cbw = nb < (q5 ? 3u : 5u) ? nb : (q5 ? 3u : 5u);
        if (16u * 2u * 16u * cbw * block_bytes + m.K * 4u + 8192u <= kSmemMax) warps_m1 = 16;
    }
    uint32_t warps = tune.warps ? tune.warps : m1 ? warps_m1 : NT == 1 ? (small || wide_k ? 16 : 8) : (!small && wide_k ? 12 : 8);
    if (!m1 && NT > 1 && warps > 12) warps = 12;  // the eight-row kernel is built for 384 threads (more registers each)
    if (rt == 2 && warps > 8) warps = 8;         // 32-row units: built for 256 threads
    uint32_t wk = tune.wk;
    if (!wk) {
        if (small) {
            wk = 1;
            // (up to 1.3 warps' worth of K slices per resident warp: 6144 x 4096 -- 384 tiles, 3072 slices on 2368 warps --
            //  runs 5.98 us split eight ways over 148 CTAs against 6.32 us split four ways over 96)
            while (wk * 2 <= warps && nb % (wk * 2) == 0 && tiles_total * (wk * 2) * 10u <= (uint64_t)sm_count * warps * 13u) wk *= 2;
        } else if (m1) {
            wk = nb >= 64 ? 8 : nb >= 32 ? 4 : nb >= 16 ? 2 : 1;
        } else {
            wk = !wide_k ? 1 : NT == 1 ? 8 : 4;
        }
    }
    if (wk > nb) wk = nb;
    if (wk > warps) wk = warps;
    while (wk > 1 && (warps % wk || nb % wk)) wk--;
    uint32_t wt = warps / wk;
    if (wk > 1 && wt > 15) wt = 15, warps = wt * wk;  // named barrier ids 1..15
    const uint32_t bpw = nb / wk;  // blocks per warp per tile
    // Stage = dense TMA box of 16 rows x cb blocks, then one box of rem blocks for the tail of
    // the warp's K range.  An odd cb keeps the 16-byte units of the eight rows an ldmatrix
    // touches in distinct bank groups (row pitch = cb*9 units).
    uint32_t cb = tune.cb ? tune.cb : m1 ? (small ? (bpw <= 2 ? bpw : 1) : (q5 ? 3 : 5)) : rt == 2 ? 2 : 3;  // Q5_K: 5 wide blocks leave no room for the ring
    if (cb > 256u / block_words) cb = 256u / block_words;  // box width <= 256 words
    if (cb > bpw) cb = bpw;
    uint32_t x_bytes = tokens * m.K * 4u, S_bytes = tokens * (m.K / 32u) * 8u;  // IND: times the local slots (set below)
    uint32_t stage_bytes = 0;
    auto layout = [&](bool xg, uint32_t stages, StreamArgs& sa) -> uint32_t {
        uint32_t off = kBarBytes;
        sa.off_zero = off; off += kZeroBytes;
        sa.off_S = off; off += xg ? 0 : align_up(S_bytes, 16);
        sa.off_x = align_up(off, 128); off = sa.off_x + (xg ? 0 : x_bytes);
        sa.off_part = align_up(off, 16); off = sa.off_part + 2u * warps * tokens * tile_rows * 4u;
        sa.off_ring = align_up(off, 128); off = sa.off_ring + warps * stages * stage_bytes;
        return off;
    };
    // Indirect form as one unit list (IND) when every CTA's share of it spans few enough slots for their
    // activation rows to sit side by side in shared memory; otherwise one grid row per slot.
    const uint32_t n_mats = indirect && m.W2 ? 2u : 1u;
    if (m.W2 && !indirect) return cudaErrorInvalidValue;
    uint32_t flat_grid = 0, nloc_max = 1, u_base = 0, u_extra = 0;
    if (indirect && !tune.force_scratch && tune.no_unit_list != 1) {
        const uint64_t U = (uint64_t)m.n_slots * n_mats * ntiles;
        if (U <= 0x7FFFFFFFull) {
            const uint64_t groups_flat = (U + wt - 1) / wt;
            const uint32_t G = (uint32_t)(groups_flat < (uint64_t)sm_count ? groups_flat : (uint64_t)sm_count);
            const uint32_t chunk = (uint32_t)((U + G - 1) / G);
            uint32_t nl = (chunk + ntiles - 2) / ntiles + 1;
            if (nl > m.n_slots * n_mats) nl = m.n_slots * n_mats;
            // One grid row per slot keeps every CTA on one slot (one staged row, less bookkeeping per tile) and is
            // 5-10 % faster while all slots' CTAs are resident at once (measured: 8 to 64 slots of 768x2048 and
            // 2048x768 experts).  With more slots than SMs it needs several waves, each paying the prologue again,
            // and the unit list wins (256 slots: 39.8 against 41.9 us).  Two stacks always share one unit list.
            const bool several_waves = m.n_slots > (uint32_t)sm_count;
            if (nl <= kMaxLocalSlots && (m.W2 || several_waves || tune.no_unit_list == 2)) {
                flat_grid = G, nloc_max = nl;
                u_base = (uint32_t)(U / G), u_extra = (uint32_t)(U % G);
            }
        }
    }
    if (m.W2 && !flat_grid) return cudaErrorInvalidValue;  // two stacks only as a unit list
    StreamArgs sa{};
    sa.m = m;
    sa.m.M = M;
    sa.nvslots = m.n_slots * n_mats;
    sa.u_base = u_base;
    sa.u_extra = u_extra;
    // activations in shared memory if they leave room for at least 2 stages per warp; with several
    // activation rows a narrower stage (down to 2 blocks) is tried before giving up on that
    bool xg = false;
    uint32_t stages = tune.stages ? tune.stages : (small ? 2 : 4);
    if (stages > kMaxStages) stages = kMaxStages;
    const bool fused = m.prologue != 0 || m.residual != nullptr;
    if (fused && !m1) return cudaErrorInvalidValue;                   // the fused forms are single-row
    if (indirect && m.residual) return cudaErrorInvalidValue;         // slots share no output row
    if (tune.force_scratch && !fused) xg = true;
    if (!xg) {
        const uint32_t cb_min = (m1 || tune.cb || cb < 2) ? cb : rt == 2 ? 1 : 2;
        auto fit = [&]() {
            for (uint32_t cb_try = cb; cb_try >= cb_min; cb_try--) {
                stage_bytes = tile_rows * cb_try * block_bytes;
                uint32_t s_try = stages;
                while (s_try >= 2 && layout(false, s_try, sa) > kSmemMax) s_try--;
                if (s_try >= 2) {
                    stages = s_try;
                    cb = cb_try;
                    return true;
                }
            }
            return false;
        };
        bool fits = false;
        if (flat_grid) {
            x_bytes *= nloc_max, S_bytes *= nloc_max;
            fits = fit();
            if (!fits) {  // the rows of several slots leave no room for the rings: one grid row per slot instead
                x_bytes /= nloc_max, S_bytes /= nloc_max;
                flat_grid = 0;
                if (m.W2) return cudaErrorInvalidValue;
            }
        }
        if (!fits) fits = fit();
        if (!fits) xg = true;
    }
    // several rows that fit in shared memory, 32K values or more: quantise them once per call (scratch) and
    // copy them in per CTA (measured: faster from there on; below, the extra launch costs more than it saves)
    const bool xc = !xg && !m1 && !indirect && (uint64_t)tokens * m.K >= 32768u && scratch &&
                    scratch_bytes >= gemv_stream_scratch_bytes(M, m.K);
    const uint32_t rem = bpw % cb;
    stage_bytes = tile_rows * cb * block_bytes;
    if (xg) {
        while (stages > 1 && layout(true, stages, sa) > kSmemMax) stages--;
        if (indirect || fused) return cudaErrorInvalidValue;  // these stage their activations in shared memory only
        if (!scratch || scratch_bytes < gemv_stream_scratch_bytes(M, m.K)) return cudaErrorInvalidValue;
    }
    const uint32_t smem = layout(xg, stages, sa);
    if (smem > kSmemMax) return cudaErrorInvalidValue;
    sa.wk = wk; sa.wt = wt; sa.cb = cb; sa.rem = rem; sa.bpw = bpw; sa.stages = stages; sa.stage_bytes = stage_bytes;
    sa.ntiles = ntiles; sa.tokens = tokens; sa.status = status_dev;
    // Long rows: the CTAs of a cluster share the staging of the activation row (4096 x 14336: 11.07 -> 10.33 us,
    // 8192 x 28672: 29.4 -> 27.9 us with pairs).  At K = 4096 a clustered launch starts ~0.5 us later than it stages faster.
    if (tune.stamps && tune.stamp_next && tune.stamp_launches) {
        sa.stamps = tune.stamps;
        sa.stamp_slot = (*tune.stamp_next)++ % tune.stamp_launches;
    }
    sa.csize = tune.cluster ? tune.cluster : (m1 && !indirect && m.K >= 14336u) ? 2u : 1u;
    {
        // whole ring before the wait while it is small (it lands long before the activations are needed); of a deep
        // ring only what keeps ~64 KB per SM in front of the activation loads
        const uint32_t per_stage = warps * stage_bytes;
        uint32_t pw = stages;
        if ((uint64_t)per_stage * stages > 96u * 1024u) pw = per_stage >= 64u * 1024u ? 1u : (64u * 1024u) / per_stage;
        if (tune.pre_wait) pw = tune.pre_wait >= 9 ? 0u : tune.pre_wait;
        sa.pre_wait = pw < stages ? pw : stages;
    }
    {
        const uint64_t rows_total = indirect ? m.w_total_rows : m.N;
        const uint32_t key_nb = (q5 ? (nb | 0x50000000u) : nb) | (rt << 24);  // keeps Q5_K maps apart from Q4_K maps of the same buffer, 32-row boxes from 16-row ones
        auto get_map = [&](uint32_t width_blocks, CUtensorMap* out, const uint8_t* Wp) -> cudaError_t {
            if (tmaps) {
                for (const auto& en : tmaps->entries)
                    if (en.W == Wp && en.rows == rows_total && en.row_bytes == m.w_row_bytes && en.nb == key_nb &&
                        en.cb == width_blocks) {
                        std::memcpy(out, en.map, sizeof(CUtensorMap));
                        return cudaSuccess;
                    }
            }
            EncodeTiledFn enc = encode_tiled_fn();
            if (!enc) return cudaErrorNotSupported;
            const cuuint64_t gdim[2] = {(cuuint64_t)nb * block_words, (cuuint64_t)rows_total};
            const cuuint64_t gstride[1] = {(cuuint64_t)m.w_row_bytes};
            const cuuint32_t box[2] = {width_blocks * block_words, tile_rows};
            const cuuint32_t estr[2] = {1u, 1u};
            const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(Wp), gdim, gstride, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
            if (tmaps) {
                auto& en = tmaps->entries[tmaps->next++ % TmapCache::kEntries];
                en.W = Wp; en.rows = rows_total; en.row_bytes = m.w_row_bytes; en.nb = key_nb; en.cb = width_blocks;
                std::memcpy(en.map, out, sizeof(CUtensorMap));
            }
            return cudaSuccess;
        };
        if (cudaError_t e = get_map(cb, &sa.tmap, m.W)) return e;
        if (rem) {
            if (cudaError_t e = get_map(rem, &sa.tmap_rem, m.W)) return e;
        } else {
            sa.tmap_rem = sa.tmap;
        }
        if (m.W2) {
            if (cudaError_t e = get_map(cb, &sa.tmap_b, m.W2)) return e;
            if (rem) {
                if (cudaError_t e = get_map(rem, &sa.tmap_b_rem, m.W2)) return e;
            } else {
                sa.tmap_b_rem = sa.tmap_b;
            }
        } else {
            sa.tmap_b = sa.tmap;
            sa.tmap_b_rem = sa.tmap_rem;
        }
    }

    const uint32_t groups = (ntiles + wt - 1) / wt;  // CTAs needed to give every tile a slot once
    const uint32_t slots_total = indirect ? m.n_slots : 1;

    if (xg || xc) {
        uint8_t* sc = static_cast<uint8_t*>(scratch);
        const uint32_t items = tokens * (m.K / 8u);
        uint32_t qgrid = (items + 255) / 256;
        if (qgrid < 4) qgrid = 4;  // the first 256 threads also clear the zero region
        quantize_activations_kernel<<<qgrid, 256, 0, stream>>>(m.X, M, m.K, tokens, sc);
        if (launches) ++*launches;
        sa.xfrag_g = sc;
        sa.S_g = reinterpret_cast<const float*>(sc + kZeroBytes + (size_t)tokens * m.K * 4u);
    }

    cudaError_t e = cudaSuccess;
    if (flat_grid) {
        if (xg || !m1) return cudaErrorInvalidValue;
        // single row staged per CTA: up to 16 warps stage it (helpers beyond the plan's warps leave afterwards)
        const uint32_t swarps_h = (m1 && !xg) ? (tune.staging_warps ? tune.staging_warps : 16u) : 0u;
        const uint32_t threads = (swarps_h > warps ? swarps_h : warps) * 32;
        const bool pdl = !tune.no_pdl;
        if (fused)
            e = q5 ? launch_one<1, true, false, true, false, true, true>(sa, groups, 1, threads, smem, sm_count, 1, pdl, stream, flat_grid)
                   : launch_one<1, true, false, false, false, true, true>(sa, groups, 1, threads, smem, sm_count, 1, pdl, stream, flat_grid);
        else
            e = q5 ? launch_one<1, true, false, true, false, false, true>(sa, groups, 1, threads, smem, sm_count, 1, pdl, stream, flat_grid)
                   : launch_one<1, true, false, false, false, false, true>(sa, groups, 1, threads, smem, sm_count, 1, pdl, stream, flat_grid);
        if (launches) ++*launches;
        return e;
    }
    MatmulArgs base = sa.m;
    for (uint32_t s0 = 0; s0 < slots_total; s0 += 65535u) {
        const uint32_t cnt = indirect ? min(65535u, m.n_slots - s0) : 1;
        if (indirect) {
            sa.m.offsets = base.offsets + s0;
            sa.m.x_rows = base.x_rows ? base.x_rows + s0 : nullptr;
            sa.m.X = base.x_rows ? base.X : base.X + (uint64_t)s0 * m.K;
            sa.m.Y = base.Y + (uint64_t)s0 * m.N;
        }
        // single row staged per CTA: up to 16 warps stage it (helpers beyond the plan's warps leave afterwards)
        const uint32_t swarps_h = (m1 && !xg) ? (tune.staging_warps ? tune.staging_warps : 16u) : 0u;
        const uint32_t threads = (swarps_h > warps ? swarps_h : warps) * 32;
#define BPQ4K_LAUNCH_RT(NT_, M1_, XG_, XC_, FP_, RT_, PEER_)                                                           \
    (q5 ? launch_one<NT_, M1_, XG_, true, XC_, FP_, false, RT_, PEER_>(sa, groups, cnt, threads, smem, sm_count, tune.ctas_per_sm, !tune.no_pdl, stream) \
        : launch_one<NT_, M1_, XG_, false, XC_, FP_, false, RT_, PEER_>(sa, groups, cnt, threads, smem, sm_count, tune.ctas_per_sm, !tune.no_pdl, stream))
#define BPQ4K_LAUNCH_NP(NT_, M1_, XG_, XC_, FP_) \
    ((M1_) || rt == 1 ? BPQ4K_LAUNCH_RT(NT_, M1_, XG_, XC_, FP_, 1, false) : BPQ4K_LAUNCH_RT(NT_, false, XG_, XC_, false, 2, false))
#define BPQ4K_LAUNCH(NT_, M1_, XG_, XC_, FP_) (peer ? BPQ4K_LAUNCH_RT(NT_, M1_, XG_, XC_, FP_, 1, true) : BPQ4K_LAUNCH_NP(NT_, M1_, XG_, XC_, FP_))
        if (peer && (indirect || fused || NT > 2)) return cudaErrorInvalidValue;  // the gather covers plain calls of up to eight rows
        if (m1 && fused) e = BPQ4K_LAUNCH_NP(1, true, false, false, true);
        else if (m1) e = xg ? BPQ4K_LAUNCH(1, true, true, false, false) : BPQ4K_LAUNCH(1, true, false, false, false);
        else if (xc) e = NT == 1 ? BPQ4K_LAUNCH(1, false, false, true, false) : NT == 2 ? BPQ4K_LAUNCH(2, false, false, true, false)
                       : NT == 3 ? BPQ4K_LAUNCH_NP(3, false, false, true, false) : BPQ4K_LAUNCH_NP(4, false, false, true, false);
        else if (xg) e = NT == 1 ? BPQ4K_LAUNCH(1, false, true, false, false) : NT == 2 ? BPQ4K_LAUNCH(2, false, true, false, false)
                       : NT == 3 ? BPQ4K_LAUNCH_NP(3, false, true, false, false) : BPQ4K_LAUNCH_NP(4, false, true, false, false);
        else e = NT == 1 ? BPQ4K_LAUNCH(1, false, false, false, false) : NT == 2 ? BPQ4K_LAUNCH(2, false, false, false, false)
               : NT == 3 ? BPQ4K_LAUNCH_NP(3, false, false, false, false) : BPQ4K_LAUNCH_NP(4, false, false, false, false);
#undef BPQ4K_LAUNCH
#undef BPQ4K_LAUNCH_NP
#undef BPQ4K_LAUNCH_RT
        if (launches) ++*launches;
        if (e != cudaSuccess) return e;
    }
    return e;
}

}  // namespace bpq4k
