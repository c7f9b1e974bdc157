// Bandwidth-bound Q6_K matmul for one activation row (decode: output head, attention and FFN
// tensors that "Q4_K_M" files keep in Q6_K).  Same machinery as the Q4_K streaming kernel: a
// persistent grid, per-warp shared-memory rings filled by 2-D tensor copies, the 6-bit codes
// assembled in registers, exact integer dot products on the tensor cores.
//
// Replaces the reference's q6k_matmul / q6k_matmul_wide shaders (runtime/kernels/quant_kq/
// q6k_matmul.wgsl, q6k_matmul_wide.wgsl; dispatch at runtime/model_runner.cpp:2032-2054, 4124-4135).
//
// Weight layout.  The file format's 210-byte super-block is not a multiple of 16 bytes, which
// bulk copies and ldmatrix need, so this kernel reads the PADDED layout (every block followed by
// 14 zero bytes, 224 bytes; bpq4k_kq_pack_host with BPQ4K_TYPE_Q6_K_PADDED writes it):
//   bytes   0-127  low nibbles: byte h*64+l holds weights h*128+l (low) and h*128+64+l (high), l < 64
//   bytes 128-191  bit pairs:   byte h*32+l holds the top two bits of weights h*128+{0,32,64,96}+l
//   bytes 192-207  16 signed scales, one per 16 weights        bytes 208-209  half d
// w = d*sc*(code - 32)  (runtime/gguf_loader.cpp:535-573).
//
// Arithmetic.  sum_k x_k w_k = sum over 16-weight groups of  d*sc*( sum code*x  -  32*sum x ).
// The activation row is quantised per 16-weight group to integers |xi| <= 2080000 written as three
// signed base-128 digits (as in the Q4_K kernel, but with one scale per 16 values because that is
// this format's scale granularity).  One mma.sync m16n8k32 (u8 x s8 -> s32) covers 16 rows x one
// 32-weight group; its 8 columns are [digit0, digit1, digit2, 0] of the group's first 16 weights
// (k >= 16 zeroed) and the same for the last 16 (k < 16 zeroed), so a single mma yields all six
// digit sums of both scale groups.  Thread t of a quad owns columns 2t, 2t+1: t = 0, 2 join the two
// high digits of one scale group, t = 1, 3 carry the low digit; every thread scales its part in
// float and the quad is summed at the end of the tile.
#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "kernels.h"
#include "q4k_common.cuh"
#include "stream_common.cuh"

namespace bpq4k {

namespace {

constexpr uint32_t kQ6Pad = 224, kQ6PadWords = 56;
constexpr uint32_t kMaxWarps6 = 16, kMaxStages6 = 8;
constexpr uint32_t kBarBytes6 = kMaxWarps6 * kMaxStages6 * 8;
constexpr uint32_t kWaitPolls6 = 1u << 22;
constexpr float kXiMax6 = 2080000.f;

struct Q6Args {
    CUtensorMap tmap, tmap_rem;
    MatmulArgs m;
    uint32_t wk, wt, cb, rem, bpw, stages, stage_bytes, ntiles;
    uint32_t off_S, off_x, off_part, off_ring;
    int* status;
    uint32_t tokens;  // activation-row slots of the several-row kernel (4 or 8)
};

// Quantise 8 consecutive activations v0, v1 (item c8 of the row; zeros for an idle lane).  The two items of a 16-value group sit in
// adjacent lanes.  Digits go to  frag + (k/32)*128 + digit*32 + k%32  (plane 3 of each 128 bytes is
// zero), the group's inv = max|x|/kXiMax6 and sum(xi)*inv to
//   SI[blk*32 + hh*8 + j] and SI[blk*32 + 16 + hh*8 + j],  group g16 = blk*16 + 2*j + hh.
__device__ __forceinline__ void q6_quantize_item(float4 v0, float4 v1, uint32_t c8, bool valid, uint8_t* frag, float* SI) {
    float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                       fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    float scale = 1.f, inv = 1.f;
    if (amax > 1e-30f && amax < 3e38f) {  // zero, tiny, inf or nan: leave unscaled
        scale = kXiMax6 / amax;
        inv = amax / kXiMax6;
    }
    const float xs[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t w0[2] = {0, 0}, w1[2] = {0, 0}, w2[2] = {0, 0};
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float vc = fminf(fmaxf(xs[i] * scale, -kXiMax6), kXiMax6);
        const int xi = __float2int_rn(vc);
        const int d2 = ((xi + 64) & 127) - 64;
        const int r1 = (xi - d2) >> 7;
        const int d1 = ((r1 + 64) & 127) - 64;
        const int d0 = (r1 - d1) >> 7;
        sum += xi;
        w0[i >> 2] |= (uint32_t)(d0 & 255) << (8 * (i & 3));
        w1[i >> 2] |= (uint32_t)(d1 & 255) << (8 * (i & 3));
        w2[i >> 2] |= (uint32_t)(d2 & 255) << (8 * (i & 3));
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    if (!valid) return;
    const uint32_t k0 = c8 * 8u;
    uint8_t* base = frag + (k0 >> 5) * 128u + (k0 & 31u);
    *reinterpret_cast<uint2*>(base) = make_uint2(w0[0], w0[1]);
    *reinterpret_cast<uint2*>(base + 32) = make_uint2(w1[0], w1[1]);
    *reinterpret_cast<uint2*>(base + 64) = make_uint2(w2[0], w2[1]);
    *reinterpret_cast<uint2*>(base + 96) = make_uint2(0u, 0u);
    if ((c8 & 1u) == 0) {
        const uint32_t g16 = k0 >> 4, blk = g16 >> 4, j16 = g16 & 15u;
        float* si = SI + blk * 32u + (j16 & 1u) * 8u + (j16 >> 1);
        si[0] = inv;
        si[16] = (float)sum * inv;
    }
}

__global__ void __launch_bounds__(512, 1) q6k_stream_kernel(const __grid_constant__ Q6Args a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t nwarps = blockDim.x >> 5;
    const uint32_t wk = warp % a.wk, wt = warp / a.wk;
    const uint32_t K = a.m.K, N = a.m.N;
    const uint32_t b0 = wk * a.bpw;
    const uint32_t nfull = a.bpw / a.cb;
    const uint32_t nchunks = nfull + (a.rem ? 1u : 0u);
    const float* X = a.m.X;
    float* Y = a.m.Y;
    // indirect (expert-stacked) form: blockIdx.y is the slot -- its expert's first row, activation row and output row
    uint32_t wrow0 = 0;
    if (a.m.n_slots) {
        const uint32_t s = blockIdx.y;
        wrow0 = a.m.offsets[s];
        if (a.m.offset_mul) wrow0 *= a.m.offset_mul;
        X += (uint64_t)(a.m.x_rows ? a.m.x_rows[s] : a.m.x_row_div ? s / a.m.x_row_div : s) * K;
        Y += (uint64_t)s * N;
    }
    // fused prologue on the activation row (see MatmulArgs::prologue): in the indirect form slot s takes row s of aux
    const float* AUX = a.m.aux ? a.m.aux + (a.m.n_slots ? (uint64_t)blockIdx.y * K : 0ull) : nullptr;

    const uint32_t tstride = gridDim.x * a.wt;
    const uint32_t tile0 = blockIdx.x * a.wt + wt;
    const uint32_t my_tiles = tile0 < a.ntiles ? (a.ntiles - tile0 + tstride - 1) / tstride : 0;
    const uint32_t total_units = my_tiles * nchunks;

    const uint32_t bar0 = smem_u32(smem) + warp * kMaxStages6 * 8u;
    const uint32_t ring = smem_u32(smem + a.off_ring) + warp * a.stages * a.stage_bytes;
    if (lane == 0) {
        for (uint32_t s = 0; s < a.stages; s++) mbar_init(bar0 + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    __syncwarp();

    // producer side: lane 0 issues one tensor copy (16 rows x cb or rem blocks) per unit
    uint32_t iss_tile = tile0, iss_c = 0, iss_st = 0;
    auto issue_next = [&]() {
        if (lane == 0) {
            const uint32_t bar = bar0 + iss_st * 8u;
            const bool full = iss_c < nfull;
            mbar_expect_tx(bar, 16u * kQ6Pad * (full ? a.cb : a.rem));
            tma_load_2d(ring + iss_st * a.stage_bytes, full ? &a.tmap : &a.tmap_rem, (b0 + iss_c * a.cb) * kQ6PadWords,
                        wrow0 + iss_tile * 16u, bar);
        }
        if (++iss_st == a.stages) iss_st = 0;
        if (++iss_c == nchunks) {
            iss_c = 0;
            iss_tile += tstride;
        }
    };
    {
        const uint32_t pre = min(a.stages, total_units);
        for (uint32_t i = 0; i < pre; i++) issue_next();
    }
    // Programmatic dependent launch: the weight prefetch above may overlap the tail of the preceding
    // kernel; X is read and Y written only after that kernel has finished.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    {
        // Fused prologue (the reference's q6k_matmul_norm.wgsl / *_down_gelu.wgsl forms and silu_mul_fused ahead of the
        // down projection, runtime/model_runner.cpp:3755-3766): the row is transformed while it is staged.
        const uint32_t prologue = AUX ? a.m.prologue : 0u;
        float rstd = 1.f;
        if (prologue == 1u) {
            float ss = 0.f;
            for (uint32_t i = tid; i < K / 4u; i += blockDim.x) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(X) + i);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
            float* red = reinterpret_cast<float*>(smem + a.off_part);
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.f;
            for (uint32_t w2 = 0; w2 < nwarps; w2++) tot += red[w2];
            rstd = 1.f / sqrtf(tot / (float)K + a.m.eps);
            __syncthreads();  // red is the partial-sum buffer of the main loop
        }
        // up to four 8-value items per thread and round, all loads issued before the first use
        constexpr int U = 4;
        const uint32_t per_row = K / 8u;
        for (uint32_t base = 0; base < per_row; base += blockDim.x * U) {
            const uint32_t nj = min((uint32_t)U, (per_row - base + blockDim.x - 1) / blockDim.x);  // uniform over the CTA
            float4 v[U][2];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const uint32_t it = base + j * blockDim.x + tid;
                v[j][0] = v[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if ((uint32_t)j < nj && it < per_row) {
                    const float4* xp = reinterpret_cast<const float4*>(X + (uint64_t)it * 8u);
                    v[j][0] = __ldg(xp);
                    v[j][1] = __ldg(xp + 1);
                    if (prologue) {
                        const float4* ap = reinterpret_cast<const float4*>(AUX + (uint64_t)it * 8u);
                        const float4 w0 = __ldg(ap), w1 = __ldg(ap + 1);
                        float* vf = reinterpret_cast<float*>(v[j]);
                        const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const float gte = vf[i];
                            if (prologue == 1u) {
                                vf[i] = gte * rstd * wf[i];
                            } else if (prologue == 2u) {
                                const float inner = 0.7978845608f * (gte + 0.044715f * gte * gte * gte);
                                vf[i] = 0.5f * gte * (1.f + tanhf(inner)) * wf[i];
                            } else {
                                vf[i] = __fdividef(gte, 1.f + __expf(-gte)) * wf[i];
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < U; j++) {
                const uint32_t it = base + j * blockDim.x + tid;
                if ((uint32_t)j < nj)
                    q6_quantize_item(v[j][0], v[j][1], it < per_row ? it : 0u, it < per_row, smem + a.off_x,
                                     reinterpret_cast<float*>(smem + a.off_S));
            }
        }
        __syncthreads();
    }

    // ---- per-lane constants ----
    const uint32_t r = lane >> 2, t = lane & 3u;
    const uint32_t hh = t >> 1, tpar = t & 1u;  // scale group inside a 32-weight group; digit part
    const uint32_t lm_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u, lm_col = (lane >> 4) * 16u;
    // B operand: column n = lane/4 -> digit plane n%4 (3 = zeros), half n/4; word t of that half
    const uint32_t bn = lane >> 2;
    const uint32_t x_lane = smem_u32(smem + a.off_x) + (bn & 3u) * 32u + (bn >> 2) * 16u + t * 4u;
    const uint32_t mask0 = (bn >> 2) ? 0u : 0xFFFFFFFFu, mask1 = ~mask0;
    const uint32_t s_lane = smem_u32(smem + a.off_S) + hh * 32u;
    const int mulc = tpar ? 1 : 128;            // (digit0, digit1) -> digit0*128 + digit1 ; (digit2, 0) -> digit2
    const float kf = tpar ? 1.f : 128.f;        // weight of that part in T = d0*2^14 + d1*2^7 + d2
    const float flag_s = tpar ? 0.f : 1.f;      // one thread per scale group adds the -32*sum(x) term
    const uint32_t sel_a = 0x8880u + hh * 0x1111u, sel_b = 0xAAA2u + hh * 0x1111u;  // sign-extending byte picks

    float* part = reinterpret_cast<float*>(smem + a.off_part);
    uint32_t st = 0, ph = 0, u = 0, failed = 0;

    for (uint32_t ti = 0; ti < my_tiles; ti++) {
        const uint32_t tile = tile0 + ti * tstride;
        float acc[2] = {0.f, 0.f}, acc_s[2] = {0.f, 0.f};
        for (uint32_t c = 0; c < nchunks; c++) {
            const uint32_t bs = b0 + c * a.cb;
            const uint32_t nblk = c < nfull ? a.cb : a.rem;
            const uint32_t pitch = nblk * kQ6Pad;
            const uint32_t bar = bar0 + st * 8u;
            if (!failed) {
                uint32_t polls = 0;
                while (!mbar_try_wait(bar, ph)) {
                    if (++polls > kWaitPolls6) {  // give up: flag it, keep the barriers matched
                        failed = 1;
                        if (lane == 0 && a.status) atomicExch(a.status, kDeviceTimeout);
                        break;
                    }
                }
            }
            uint32_t boff = ring + st * a.stage_bytes;
            for (uint32_t blk = bs; blk < bs + nblk; blk++, boff += kQ6Pad) {
                // d*scale of rows r and r+8 for this thread's eight scale groups (index j = h*4 + gg)
                float ds[2][8];
#pragma unroll
                for (int rr = 0; rr < 2; rr++) {
                    const uint32_t hdr = boff + (r + rr * 8u) * pitch + 192u;
                    const uint4 sv = lds128<0>(hdr);
                    const uint4 dv = lds128<16>(hdr);
                    const float d = half_bits_to_float(dv.x);
                    const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        // scale byte 2*j + hh of the block: word j/2, byte 2*(j%2) + hh
                        int sc;  // prmt with bit 3 of a selector nibble set copies the byte's sign (the intrinsic masks that bit)
                        asm("prmt.b32 %0, %1, 0, %2;" : "=r"(sc) : "r"(sw[j >> 1]), "r"((j & 1) ? sel_b : sel_a));
                        ds[rr][j] = d * (float)sc;
                    }
                }
                // this row's activation scales for the same eight groups: inv*kf and flagged sum
                float sx[8], so[8];
                {
                    const uint32_t sa = s_lane + blk * 128u;
                    const uint4 i0 = lds128<0>(sa), i1 = lds128<16>(sa), s0 = lds128<64>(sa), s1 = lds128<80>(sa);
                    const uint32_t iw[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
                    const uint32_t swd[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        sx[j] = __uint_as_float(iw[j]) * kf;
                        so[j] = __uint_as_float(swd[j]) * flag_s;
                    }
                }
                const uint32_t lm_addr = boff + lm_row * pitch + lm_col;
                const uint32_t xb = x_lane + blk * 1024u;
                auto do_half = [&](auto hc) {
                    constexpr int h = decltype(hc)::value;
                    uint32_t la[4], lb[4], lh[4];
                    ldmatrix_x4<h * 64>(lm_addr, la[0], la[1], la[2], la[3]);
                    ldmatrix_x4<h * 64 + 32>(lm_addr, lb[0], lb[1], lb[2], lb[3]);
                    ldmatrix_x4<128 + h * 32>(lm_addr, lh[0], lh[1], lh[2], lh[3]);
                    auto do_group = [&](auto gc) {
                        constexpr int gg = decltype(gc)::value;
                        constexpr int j = h * 4 + gg;
                        uint32_t q[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t lo = (gg & 1) ? lb[i] : la[i];
                            const uint32_t nib = (gg & 2) ? (lo >> 4) : lo;
                            const uint32_t hi = gg == 0 ? (lh[i] << 4) : gg == 1 ? (lh[i] << 2) : gg == 2 ? lh[i] : (lh[i] >> 2);
                            q[i] = (nib & 0x0F0F0F0Fu) | (hi & 0x30303030u);
                        }
                        uint32_t bw;
                        asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(bw) : "r"(xb), "n"(j * 128));
                        int cacc[4];
                        imma16832_first(cacc, q[0], q[1], q[2], q[3], bw & mask0, bw & mask1);
                        const float v0 = (float)(cacc[0] * mulc + cacc[1]);  // row r
                        const float v1 = (float)(cacc[2] * mulc + cacc[3]);  // row r+8
                        acc[0] = fmaf(v0, ds[0][j] * sx[j], acc[0]);
                        acc[1] = fmaf(v1, ds[1][j] * sx[j], acc[1]);
                        acc_s[0] = fmaf(ds[0][j], so[j], acc_s[0]);
                        acc_s[1] = fmaf(ds[1][j], so[j], acc_s[1]);
                    };
                    do_group(std::integral_constant<int, 0>{});
                    do_group(std::integral_constant<int, 1>{});
                    do_group(std::integral_constant<int, 2>{});
                    do_group(std::integral_constant<int, 3>{});
                };
                do_half(std::integral_constant<int, 0>{});
                do_half(std::integral_constant<int, 1>{});
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

        // ---- tile epilogue: quad -> K slices -> bias -> Y ----
        float s0 = fmaf(-32.f, acc_s[0], acc[0]), s1 = fmaf(-32.f, acc_s[1], acc[1]);
        s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 1);
        s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 1);
        s0 += __shfl_xor_sync(0xFFFFFFFFu, s0, 2);
        s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, 2);
        float* pbuf = part + ((uint64_t)((ti & 1u) * nwarps + warp)) * 16u;
        if (t == 0) {
            pbuf[r] = s0;
            pbuf[r + 8u] = s1;
        }
        if (a.wk > 1) {
            asm volatile("bar.sync %0, %1;" ::"r"(wt + 1u), "r"(a.wk * 32u) : "memory");
        } else {
            __syncwarp();
        }
        if (wk == 0 && lane < 16u) {
            const uint32_t row = tile * 16u + lane;
            if (row < N) {
                float s = 0.f;
                for (uint32_t k2 = 0; k2 < a.wk; k2++) s += pbuf[k2 * 16u + lane];
                float yv = s + (a.m.bias ? a.m.bias[row] : 0.f);
                if (a.m.residual) yv += a.m.residual[row];
                // double-buffered gather slots: the half this step writes (see MatmulArgs::slot_parity)
                const uint64_t par_off = a.m.slot_parity ? (uint64_t)(*reinterpret_cast<const volatile uint32_t*>(a.m.slot_parity) & 1u) * a.m.slot_parity_stride : 0ull;
                Y[row + par_off] = yv;
                for (uint32_t p = 0; p < a.m.n_peers; p++) a.m.peer_Y[p][row + par_off] = yv;
            }
        }
    }
}


// ---------------------------------------------------------------------------------------------
// Several activation rows (M = 2..8): the eight mma columns are four activation rows x the two
// 16-weight scale groups of a 32-weight group, one mma per digit.  Thread t of a quad then holds,
// for rows r and r+8 of the tile, both scale groups of activation row t.
//
// Layouts in shared memory (TOK = 4 or 8 row slots, rows past M are zero):
//   digits  frag + ((G*TOK + tok)*128) + w*16 + d*4 : the four k-bytes of word w (k = 4w..4w+3 of
//           32-weight group G) of digit d (d = 3: zero) -- one 16-byte load gives a thread the three
//           digit words of its B fragment, and the four rows of a tile are 128 bytes apart
//   scales  SI[((blk*8 + c)*TOK + tok)*4 + f%4],  c = f/4,  f = g16 (inv, 0..15) or 16 + g16 (sum*inv)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void q6_quantize_item_rows(float4 v0, float4 v1, uint32_t tok, uint32_t TOK, uint32_t c8, bool valid,
                                                      uint8_t* frag, float* SI) {
    float amax = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                       fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    float scale = 1.f, inv = 1.f;
    if (amax > 1e-30f && amax < 3e38f) {
        scale = kXiMax6 / amax;
        inv = amax / kXiMax6;
    }
    const float xs[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t w0[2] = {0, 0}, w1[2] = {0, 0}, w2[2] = {0, 0};
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float vc = fminf(fmaxf(xs[i] * scale, -kXiMax6), kXiMax6);
        const int xi = __float2int_rn(vc);
        const int d2 = ((xi + 64) & 127) - 64;
        const int r1 = (xi - d2) >> 7;
        const int d1 = ((r1 + 64) & 127) - 64;
        const int d0 = (r1 - d1) >> 7;
        sum += xi;
        w0[i >> 2] |= (uint32_t)(d0 & 255) << (8 * (i & 3));
        w1[i >> 2] |= (uint32_t)(d1 & 255) << (8 * (i & 3));
        w2[i >> 2] |= (uint32_t)(d2 & 255) << (8 * (i & 3));
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    if (!valid) return;
    const uint32_t k0 = c8 * 8u, G = k0 >> 5, w = (k0 & 31u) >> 2;
    uint4* dst = reinterpret_cast<uint4*>(frag + ((uint64_t)G * TOK + tok) * 128u + w * 16u);
    dst[0] = make_uint4(w0[0], w1[0], w2[0], 0u);
    dst[1] = make_uint4(w0[1], w1[1], w2[1], 0u);
    if ((c8 & 1u) == 0) {
        const uint32_t g16 = k0 >> 4, blk = g16 >> 4, f = g16 & 15u;
        SI[((blk * 8u + (f >> 2)) * TOK + tok) * 4u + (f & 3u)] = inv;
        SI[((blk * 8u + 4u + (f >> 2)) * TOK + tok) * 4u + (f & 3u)] = (float)sum * inv;
    }
}

template <int NT>
__global__ void __launch_bounds__(256, 1) q6k_stream_rows_kernel(const __grid_constant__ Q6Args a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TOK = NT * 4;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t nwarps = blockDim.x >> 5;
    const uint32_t wk = warp % a.wk, wt = warp / a.wk;
    const uint32_t K = a.m.K, N = a.m.N, M = a.m.M;
    const uint32_t b0 = wk * a.bpw;
    const uint32_t nfull = a.bpw / a.cb;
    const uint32_t nchunks = nfull + (a.rem ? 1u : 0u);
    const float* X = a.m.X;
    float* Y = a.m.Y;

    const uint32_t tstride = gridDim.x * a.wt;
    const uint32_t tile0 = blockIdx.x * a.wt + wt;
    const uint32_t my_tiles = tile0 < a.ntiles ? (a.ntiles - tile0 + tstride - 1) / tstride : 0;
    const uint32_t total_units = my_tiles * nchunks;

    const uint32_t bar0 = smem_u32(smem) + warp * kMaxStages6 * 8u;
    const uint32_t ring = smem_u32(smem + a.off_ring) + warp * a.stages * a.stage_bytes;
    if (lane == 0) {
        for (uint32_t s = 0; s < a.stages; s++) mbar_init(bar0 + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_proxy_async();
    __syncwarp();

    uint32_t iss_tile = tile0, iss_c = 0, iss_st = 0;
    auto issue_next = [&]() {
        if (lane == 0) {
            const uint32_t bar = bar0 + iss_st * 8u;
            const bool full = iss_c < nfull;
            mbar_expect_tx(bar, 16u * kQ6Pad * (full ? a.cb : a.rem));
            tma_load_2d(ring + iss_st * a.stage_bytes, full ? &a.tmap : &a.tmap_rem, (b0 + iss_c * a.cb) * kQ6PadWords,
                        iss_tile * 16u, bar);
        }
        if (++iss_st == a.stages) iss_st = 0;
        if (++iss_c == nchunks) {
            iss_c = 0;
            iss_tile += tstride;
        }
    };
    {
        const uint32_t pre = min(a.stages, total_units);
        for (uint32_t i = 0; i < pre; i++) issue_next();
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    {
        uint8_t* frag = smem + a.off_x;
        float* SI = reinterpret_cast<float*>(smem + a.off_S);
        const uint32_t nb = K / kQK, mrows = min(M, TOK);
        // rows past M: zero digits and scales (every slot of the layouts interleaves the rows)
        if (mrows < TOK) {
            for (uint32_t i = tid; i < TOK * K; i += blockDim.x) {  // word i of the digit area: row = (i / 32) % TOK
                if ((i >> 5) % TOK >= mrows) reinterpret_cast<uint32_t*>(frag)[i] = 0u;
            }
            for (uint32_t i = tid; i < nb * 8u * TOK * 4u; i += blockDim.x) {
                if ((i >> 2) % TOK >= mrows) SI[i] = 0.f;
            }
        }
        constexpr int U = 4;
        const uint32_t per_row = K / 8u, items = mrows * per_row;
        for (uint32_t base = 0; base < items; base += blockDim.x * U) {
            const uint32_t nj = min((uint32_t)U, (items - base + blockDim.x - 1) / blockDim.x);
            float4 v[U][2];
            uint32_t tok[U], c8[U];
#pragma unroll
            for (int j = 0; j < U; j++) {
                const uint32_t it = base + j * blockDim.x + tid;
                const bool ok = (uint32_t)j < nj && it < items;
                tok[j] = ok ? it / per_row : 0u;
                c8[j] = ok ? it - tok[j] * per_row : 0u;
                v[j][0] = v[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok) {
                    const float4* xp = reinterpret_cast<const float4*>(X + (uint64_t)tok[j] * K + (uint64_t)c8[j] * 8u);
                    v[j][0] = __ldg(xp);
                    v[j][1] = __ldg(xp + 1);
                }
            }
#pragma unroll
            for (int j = 0; j < U; j++) {
                const uint32_t it = base + j * blockDim.x + tid;
                if ((uint32_t)j < nj) q6_quantize_item_rows(v[j][0], v[j][1], tok[j], TOK, c8[j], it < items, frag, SI);
            }
        }
        __syncthreads();
    }

    const uint32_t r = lane >> 2, t = lane & 3u;
    const uint32_t lm_row = (lane & 7u) + ((lane >> 3) & 1u) * 8u, lm_col = (lane >> 4) * 16u;
    // B operand: column n = lane/4 -> activation row n/2 of the mma tile, scale group (half) n%2
    const uint32_t bn = lane >> 2, bhalf = bn & 1u;
    const uint32_t x_lane = smem_u32(smem + a.off_x) + (bn >> 1) * 128u + (bhalf * 4u + t) * 16u;  // + (G*TOK + nt*4)*128
    const uint32_t mask0 = bhalf ? 0u : 0xFFFFFFFFu, mask1 = ~mask0;
    const uint32_t s_lane = smem_u32(smem + a.off_S) + t * 16u;  // + ((blk*8 + c)*TOK + nt*4)*16

    float* part = reinterpret_cast<float*>(smem + a.off_part);
    uint32_t st = 0, ph = 0, u = 0, failed = 0;

    for (uint32_t ti = 0; ti < my_tiles; ti++) {
        const uint32_t tile = tile0 + ti * tstride;
        float acc[NT][2], acc_s[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc_s[nt][0] = acc_s[nt][1] = 0.f;
        for (uint32_t c = 0; c < nchunks; c++) {
            const uint32_t bs = b0 + c * a.cb;
            const uint32_t nblk = c < nfull ? a.cb : a.rem;
            const uint32_t pitch = nblk * kQ6Pad;
            const uint32_t bar = bar0 + st * 8u;
            if (!failed) {
                uint32_t polls = 0;
                while (!mbar_try_wait(bar, ph)) {
                    if (++polls > kWaitPolls6) {
                        failed = 1;
                        if (lane == 0 && a.status) atomicExch(a.status, kDeviceTimeout);
                        break;
                    }
                }
            }
            uint32_t boff = ring + st * a.stage_bytes;
            for (uint32_t blk = bs; blk < bs + nblk; blk++, boff += kQ6Pad) {
                const uint32_t lm_addr = boff + lm_row * pitch + lm_col;
                auto do_half = [&](auto hc) {
                    constexpr int h = decltype(hc)::value;
                    // d*scale of rows r, r+8 for the eight scale groups of this half (index 2*gg + column half)
                    float ds[2][8];
#pragma unroll
                    for (int rr = 0; rr < 2; rr++) {
                        const uint32_t hdr = boff + (r + rr * 8u) * pitch + 192u;
                        const uint4 sv = lds128<0>(hdr);
                        const uint4 dv = lds128<16>(hdr);
                        const float d = half_bits_to_float(dv.x);
                        const uint32_t swa = h ? sv.z : sv.x, swb = h ? sv.w : sv.y;
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            int sc;  // sign-extending pick of byte j%4
                            asm("prmt.b32 %0, %1, 0, %2;" : "=r"(sc) : "r"(j < 4 ? swa : swb), "r"(0x8880 + (j & 3) * 0x1111));
                            ds[rr][j] = d * (float)sc;
                        }
                    }
                    uint32_t la[4], lb[4], lh[4];
                    ldmatrix_x4<h * 64>(lm_addr, la[0], la[1], la[2], la[3]);
                    ldmatrix_x4<h * 64 + 32>(lm_addr, lb[0], lb[1], lb[2], lb[3]);
                    ldmatrix_x4<128 + h * 32>(lm_addr, lh[0], lh[1], lh[2], lh[3]);
                    uint32_t q[4][4];
#pragma unroll
                    for (int gg = 0; gg < 4; gg++)
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t lo = (gg & 1) ? lb[i] : la[i];
                            const uint32_t nib = (gg & 2) ? (lo >> 4) : lo;
                            const uint32_t hi = gg == 0 ? (lh[i] << 4) : gg == 1 ? (lh[i] << 2) : gg == 2 ? lh[i] : (lh[i] >> 2);
                            q[gg][i] = (nib & 0x0F0F0F0Fu) | (hi & 0x30303030u);
                        }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        // this thread's activation row (t of tile nt): inv and sum*inv of the half's eight scale groups
                        const uint32_t sa = s_lane + ((blk * 8u + 2u * h) * TOK + nt * 4u) * 16u;
                        const uint4 i0 = lds128<0>(sa), i1 = lds128<0>(sa + TOK * 16u);
                        const uint4 s0 = lds128<0>(sa + 4u * TOK * 16u), s1 = lds128<0>(sa + 5u * TOK * 16u);
                        const float inv[8] = {__uint_as_float(i0.x), __uint_as_float(i0.y), __uint_as_float(i0.z), __uint_as_float(i0.w),
                                              __uint_as_float(i1.x), __uint_as_float(i1.y), __uint_as_float(i1.z), __uint_as_float(i1.w)};
                        const float sm[8] = {__uint_as_float(s0.x), __uint_as_float(s0.y), __uint_as_float(s0.z), __uint_as_float(s0.w),
                                             __uint_as_float(s1.x), __uint_as_float(s1.y), __uint_as_float(s1.z), __uint_as_float(s1.w)};
                        const uint32_t xb = x_lane + (((blk * 8u + h * 4u) * TOK) + nt * 4u) * 128u;
#pragma unroll
                        for (int gg = 0; gg < 4; gg++) {
                            const uint4 dw = lds128<0>(xb + gg * TOK * 128u);  // digit words d0, d1, d2 of this column
                            int c0[4], c1[4], c2[4];
                            imma16832_first(c0, q[gg][0], q[gg][1], q[gg][2], q[gg][3], dw.x & mask0, dw.x & mask1);
                            imma16832_first(c1, q[gg][0], q[gg][1], q[gg][2], q[gg][3], dw.y & mask0, dw.y & mask1);
                            imma16832_first(c2, q[gg][0], q[gg][1], q[gg][2], q[gg][3], dw.z & mask0, dw.z & mask1);
#pragma unroll
                            for (int e = 0; e < 4; e++) {  // e: row r (0, 1) or r+8 (2, 3); column half e%2
                                const int rr = e >> 1, j = 2 * gg + (e & 1);
                                const float T = fmaf((float)c0[e], 16384.f, (float)(c1[e] * 128 + c2[e]));
                                acc[nt][rr] = fmaf(T, ds[rr][j] * inv[j], acc[nt][rr]);
                                acc_s[nt][rr] = fmaf(ds[rr][j], sm[j], acc_s[nt][rr]);
                            }
                        }
                    }
                };
                do_half(std::integral_constant<int, 0>{});
                do_half(std::integral_constant<int, 1>{});
            }
            __syncwarp();
            fence_proxy_async();
            if (u + a.stages < total_units) issue_next();
            u++;
            if (++st == a.stages) {
                st = 0;
                ph ^= 1u;
            }
        }

        // ---- tile epilogue: K slices -> bias -> Y ----
        float* pbuf = part + ((uint64_t)((ti & 1u) * nwarps + warp)) * (TOK * 16u);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            pbuf[(nt * 4u + t) * 16u + r] = fmaf(-32.f, acc_s[nt][0], acc[nt][0]);
            pbuf[(nt * 4u + t) * 16u + r + 8u] = fmaf(-32.f, acc_s[nt][1], acc[nt][1]);
        }
        if (a.wk > 1) {
            asm volatile("bar.sync %0, %1;" ::"r"(wt + 1u), "r"(a.wk * 32u) : "memory");
        } else {
            __syncwarp();
        }
        if (wk == 0) {
            for (uint32_t idx = lane; idx < TOK * 16u; idx += 32u) {
                const uint32_t tok = idx >> 4, row = tile * 16u + (idx & 15u);
                if (tok < M && row < N) {
                    float s = 0.f;
                    for (uint32_t k2 = 0; k2 < a.wk; k2++) s += pbuf[(uint64_t)k2 * (TOK * 16u) + idx];
                    Y[(uint64_t)tok * N + row] = s + (a.m.bias ? a.m.bias[row] : 0.f);
                }
            }
        }
    }
}

}  // namespace

// Up to 8 activation rows, Q6_K weights in the padded layout.  Returns cudaErrorInvalidValue when the
// shape does not fit the kernel (several rows of a long K need more shared memory than there is;
// the caller then goes row by row, or uses the plain kernel).
cudaError_t launch_q6k_stream(const MatmulArgs& m, const StreamTuning& tune, int* status_dev, int sm_count, TmapCache* tmaps,
                              cudaStream_t stream, int* launches) {
    if (m.N == 0) return cudaSuccess;
    if (m.M == 0 || m.M > 8) return cudaErrorInvalidValue;
    const bool indirect = m.n_slots != 0;                // slots of one row each, blockIdx.y = slot
    if (indirect && (m.M != 1 || m.n_peers || m.W2 || m.residual)) return cudaErrorInvalidValue;
    if ((m.prologue || m.residual) && m.M != 1) return cudaErrorInvalidValue;  // the fused forms are single-row
    const bool rows = m.M > 1;                           // the several-row kernel
    const uint32_t tokens = rows ? (m.M + 3) / 4 * 4 : 1;
    const uint32_t nb = m.K / kQK;
    const uint32_t ntiles = (m.N + 15) / 16;
    constexpr uint32_t kSmemMax = 227 * 1024;

    // plan: as the Q4_K kernel's single-row plan (small: everything in one round with K split over
    // the warps of a CTA; large: 8 warps, deeper rings)
    const uint64_t tiles_total = (uint64_t)ntiles * (indirect ? m.n_slots : 1);
    const bool small = tiles_total <= 640;
    const uint64_t rows_total = indirect ? m.w_total_rows : m.N;  // rows the tensor map may touch
    Q6Args qa{};
    uint32_t warps = 0, wk = 0, wt = 0, bpw = 0, cb = 0, rem = 0, stage_bytes = 0, stages = 0, smem = 0;
    auto plan = [&](uint32_t warps_want, uint32_t cb_want, uint32_t stages_want) -> bool {
        warps = warps_want > kMaxWarps6 ? kMaxWarps6 : warps_want;
        if (rows && warps > 8) warps = 8;  // the several-row kernel is built for 256 threads
        wk = tune.wk;
        if (!wk) {
            if (small) {
                wk = 1;
                while (wk * 2 <= warps && nb % (wk * 2) == 0 && tiles_total * (wk * 2) <= (uint64_t)sm_count * warps) wk *= 2;
            } else {
                wk = nb >= 64 ? 8 : nb >= 32 ? 4 : nb >= 16 ? 2 : 1;
            }
        }
        if (wk > nb) wk = nb;
        if (wk > warps) wk = warps;
        while (wk > 1 && (warps % wk || nb % wk)) wk--;
        wt = warps / wk;
        if (wk > 1 && wt > 15) wt = 15, warps = wt * wk;  // named barrier ids 1..15
        bpw = nb / wk;
        cb = cb_want ? cb_want : (small ? (bpw <= 2 ? bpw : 1) : 3);
        if (cb > 4) cb = 4;  // box width <= 256 words
        if (cb > bpw) cb = bpw;
        rem = bpw % cb;
        stage_bytes = 16 * cb * kQ6Pad;
        stages = stages_want > kMaxStages6 ? kMaxStages6 : stages_want;
        auto layout = [&](uint32_t st) -> uint32_t {
            uint32_t off = kBarBytes6;
            qa.off_S = off; off += tokens * nb * 128u;
            qa.off_x = align_up(off, 128); off = qa.off_x + tokens * m.K * 4u;
            qa.off_part = align_up(off, 16); off = qa.off_part + 2u * warps * tokens * 16u * 4u;
            qa.off_ring = align_up(off, 128); off = qa.off_ring + warps * st * stage_bytes;
            return off;
        };
        while (stages > 2 && layout(stages) > kSmemMax) stages--;
        smem = layout(stages);
        return smem <= kSmemMax;
    };
    // the tuned plan first; with a long K the digits leave less room: narrower stages, then fewer warps
    const uint32_t warps0 = tune.warps ? tune.warps : (small ? 16 : 8);
    const uint32_t stages0 = tune.stages ? tune.stages : (small ? 2 : 4);
    if (!plan(warps0, tune.cb, stages0) && !(rows && plan(warps0, 2, 2)) && !plan(warps0, 1, 2) && !plan(8, 1, 2) && !plan(4, 1, 2))
        return cudaErrorInvalidValue;
    qa.m = m;
    qa.tokens = tokens;
    qa.wk = wk; qa.wt = wt; qa.cb = cb; qa.rem = rem; qa.bpw = bpw; qa.stages = stages; qa.stage_bytes = stage_bytes;
    qa.ntiles = ntiles; qa.status = status_dev;

    auto get_map = [&](uint32_t width_blocks, CUtensorMap* out) -> cudaError_t {
        const uint32_t key_nb = nb | 0x60000000u;  // keeps these entries apart from the Q4_K maps of the cache
        if (tmaps) {
            for (const auto& en : tmaps->entries)
                if (en.W == m.W && en.rows == rows_total && en.row_bytes == m.w_row_bytes && en.nb == key_nb && en.cb == width_blocks) {
                    std::memcpy(out, en.map, sizeof(CUtensorMap));
                    return cudaSuccess;
                }
        }
        EncodeTiledFn enc = encode_tiled_fn();
        if (!enc) return cudaErrorNotSupported;
        const cuuint64_t gdim[2] = {(cuuint64_t)nb * kQ6PadWords, (cuuint64_t)rows_total};
        const cuuint64_t gstride[1] = {(cuuint64_t)m.w_row_bytes};
        const cuuint32_t box[2] = {width_blocks * kQ6PadWords, 16u};
        const cuuint32_t estr[2] = {1u, 1u};
        const CUresult res = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(m.W), gdim, gstride, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (res != CUDA_SUCCESS) return cudaErrorInvalidValue;
        if (tmaps) {
            auto& en = tmaps->entries[tmaps->next++ % TmapCache::kEntries];
            en.W = m.W; en.rows = rows_total; en.row_bytes = m.w_row_bytes; en.nb = key_nb; en.cb = width_blocks;
            std::memcpy(en.map, out, sizeof(CUtensorMap));
        }
        return cudaSuccess;
    };
    if (cudaError_t e = get_map(cb, &qa.tmap)) return e;
    if (rem) {
        if (cudaError_t e = get_map(rem, &qa.tmap_rem)) return e;
    } else {
        qa.tmap_rem = qa.tmap;
    }

    static KernelConfig kcfg[3];  // one per kernel variant; per-device slots inside
    const int variant = !rows ? 0 : tokens == 4 ? 1 : 2;
    {
        const void* fn = variant == 0 ? reinterpret_cast<const void*>(q6k_stream_kernel)
                       : variant == 1 ? reinterpret_cast<const void*>(q6k_stream_rows_kernel<1>)
                                      : reinterpret_cast<const void*>(q6k_stream_rows_kernel<2>);
        if (cudaError_t e = kcfg[variant].prepare(fn, warps * 32, smem, nullptr)) return e;
    }
    // persistent grid, one CTA per SM, balanced: the smallest grid that needs no more rounds than
    // the whole machine would
    const uint32_t groups = (ntiles + wt - 1) / wt;
    uint32_t gx = groups;
    const uint32_t slots_y = indirect ? m.n_slots : 1;
    if (slots_y > 65535u) return cudaErrorInvalidValue;
    {
        // all slots' CTAs resident at once (never a partial second wave), each slot's tiles in balanced rounds
        uint32_t cap_x = (uint32_t)sm_count / slots_y;
        if (cap_x == 0) cap_x = 1;
        if (gx > cap_x) {
            const uint32_t rounds = (groups + cap_x - 1) / cap_x;
            gx = (groups + rounds - 1) / rounds;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(gx, slots_y);
    cfg.blockDim = dim3(warps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tune.no_pdl ? 0 : 1;
    const cudaError_t e = variant == 0 ? cudaLaunchKernelEx(&cfg, q6k_stream_kernel, qa)
                        : variant == 1 ? cudaLaunchKernelEx(&cfg, q6k_stream_rows_kernel<1>, qa)
                                       : cudaLaunchKernelEx(&cfg, q6k_stream_rows_kernel<2>, qa);
    if (launches) ++*launches;
    return e;
}

}  // namespace bpq4k
