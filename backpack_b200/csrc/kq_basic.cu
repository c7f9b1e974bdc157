// Q5_K and Q6_K on the reference's packed layout (raw GGUF super-blocks, rows a whole number of
// words apart): the bit-exact dequantiser, the embedding-row gather, and a float-FMA matmul with
// one warp per output row.  Arithmetic follows the reference's CPU decode
// (runtime/gguf_loader.cpp:497-573) and its shaders (runtime/kernels/quant_kq/q5k_matmul.wgsl,
// q6k_matmul.wgsl, q6k_gather.wgsl, q6k_gather_batched.wgsl, q5k/q6k_matmul_batched4.wgsl).
//
// Q5_K super-block, 176 bytes: half d, half dmin, 12 packed scale/min bytes (as Q4_K), 32 bytes
//   of fifth bits (bit sb of byte i belongs to weight sb*32+i), 128 nibble bytes laid out as in
//   Q4_K.  w = (d*sc)*q - dmin*mn, q = nibble | bit<<4.
// Q6_K super-block, 210 bytes: 128 nibble bytes, 64 bytes of bit pairs, 16 signed byte scales
//   (one per 16 weights), half d at byte 208.  w = (d*sc)*(code - 32).  210 is not a multiple of
//   4, so blocks are only 2-byte aligned and these kernels read them with byte and 16-bit loads.
//   The padded layout (every block followed by 14 zero bytes: 224 bytes) is read the same way.
#include "kernels.h"
#include "q4k_common.cuh"

namespace bpq4k {

namespace {

constexpr uint32_t kQ5Bytes = 176, kQ6Bytes = 210;

// ---- Q5_K: lane l owns nibble word l (8 weights: four of sub-block 2g, four of 2g+1) -------------
struct Q5Lane {
    float s_even, s_odd, m_even, m_odd;
    uint32_t q_even[4], q_odd[4];
};

__device__ __forceinline__ Q5Lane q5k_lane(const uint8_t* __restrict__ p, uint32_t lane) {
    const uint4 hv = __ldg(reinterpret_cast<const uint4*>(p));
    const BlockHeader h{hv.x, hv.y, hv.z, hv.w};
    const uint32_t g = lane >> 3, j = lane & 7u;
    const uint32_t code = __ldg(reinterpret_cast<const uint32_t*>(p + 48) + lane);
    const uint32_t qh = __ldg(reinterpret_cast<const uint32_t*>(p + 16) + j);  // fifth bits of weights 4j..4j+3
    const float d = half_bits_to_float(h.w0), dmin = half_bits_to_float(h.w0 >> 16);
    uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
    unpack_scales_packed(h, sc_lo, sc_hi, mn_lo, mn_hi);
    Q5Lane r;
    r.s_even = __fmul_rn(d, (float)byte_of(sc_lo, sc_hi, 2 * g));
    r.s_odd = __fmul_rn(d, (float)byte_of(sc_lo, sc_hi, 2 * g + 1));
    r.m_even = __fmul_rn(dmin, (float)byte_of(mn_lo, mn_hi, 2 * g));
    r.m_odd = __fmul_rn(dmin, (float)byte_of(mn_lo, mn_hi, 2 * g + 1));
#pragma unroll
    for (int i = 0; i < 4; i++) {
        r.q_even[i] = ((code >> (8 * i)) & 15u) | (((qh >> (8 * i + 2 * g)) & 1u) << 4);
        r.q_odd[i] = ((code >> (8 * i + 4)) & 15u) | (((qh >> (8 * i + 2 * g + 1)) & 1u) << 4);
    }
    return r;
}

// ---- Q6_K: lane l owns weights l, l+32, l+64, l+96 of each 128-weight half ------------------------
struct Q6Lane {
    float ds[2][4];  // d*scale of the four weights of each half
    int q[2][4];
};

__device__ __forceinline__ Q6Lane q6k_lane(const uint8_t* __restrict__ p, uint32_t lane) {
    const float d = half_bits_to_float(__ldg(reinterpret_cast<const uint16_t*>(p + 208)));
    const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192);
    const uint32_t is = lane >> 4;
    Q6Lane r;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const uint32_t la = __ldg(p + half * 64 + lane), lb = __ldg(p + half * 64 + 32 + lane);
        const uint32_t hb = __ldg(p + 128 + half * 32 + lane);
        r.q[half][0] = (int)((la & 15u) | ((hb & 3u) << 4)) - 32;
        r.q[half][1] = (int)((lb & 15u) | (((hb >> 2) & 3u) << 4)) - 32;
        r.q[half][2] = (int)((la >> 4) | (((hb >> 4) & 3u) << 4)) - 32;
        r.q[half][3] = (int)((lb >> 4) | (((hb >> 6) & 3u) << 4)) - 32;
#pragma unroll
        for (int g = 0; g < 4; g++) r.ds[half][g] = __fmul_rn(d, (float)__ldg(sc + half * 8 + is + 2 * g));
    }
    return r;
}

// One warp per super-block; source row r is rows[r] when `rows` is given (embedding gather).
template <int QTYPE>
__global__ void __launch_bounds__(256) kq_dequant_kernel(const uint8_t* __restrict__ W, const uint32_t* __restrict__ rows,
                                                          uint32_t n_src_rows, uint32_t N, uint32_t nb, uint64_t w_row_bytes,
                                                          uint32_t q6_block_bytes, float* __restrict__ out) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const uint64_t total = (uint64_t)N * nb;
    const uint32_t K = nb * kQK;
    for (uint64_t blk = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < total; blk += warps) {
        const uint32_t row = (uint32_t)(blk / nb);
        const uint32_t b = (uint32_t)(blk - (uint64_t)row * nb);
        uint32_t src = rows ? rows[row] : row;
        float* o = out + (uint64_t)row * K + (uint64_t)b * kQK;
        if (src >= n_src_rows) {  // a token id outside the table: zeros, never an out-of-range read
#pragma unroll
            for (int i = 0; i < 8; i++) o[i * 32 + lane] = 0.f;
            continue;
        }
        if constexpr (QTYPE == 13) {
            const Q5Lane q = q5k_lane(W + (uint64_t)src * w_row_bytes + (uint64_t)b * kQ5Bytes, lane);
            float4 lo, hi;
            lo.x = __fsub_rn(__fmul_rn(q.s_even, (float)q.q_even[0]), q.m_even);
            lo.y = __fsub_rn(__fmul_rn(q.s_even, (float)q.q_even[1]), q.m_even);
            lo.z = __fsub_rn(__fmul_rn(q.s_even, (float)q.q_even[2]), q.m_even);
            lo.w = __fsub_rn(__fmul_rn(q.s_even, (float)q.q_even[3]), q.m_even);
            hi.x = __fsub_rn(__fmul_rn(q.s_odd, (float)q.q_odd[0]), q.m_odd);
            hi.y = __fsub_rn(__fmul_rn(q.s_odd, (float)q.q_odd[1]), q.m_odd);
            hi.z = __fsub_rn(__fmul_rn(q.s_odd, (float)q.q_odd[2]), q.m_odd);
            hi.w = __fsub_rn(__fmul_rn(q.s_odd, (float)q.q_odd[3]), q.m_odd);
            float* oo = o + (lane >> 3) * 64u + (lane & 7u) * 4u;
            __stcs(reinterpret_cast<float4*>(oo), lo);
            __stcs(reinterpret_cast<float4*>(oo + 32), hi);
        } else {
            const Q6Lane q = q6k_lane(W + (uint64_t)src * w_row_bytes + (uint64_t)b * q6_block_bytes, lane);
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int g = 0; g < 4; g++) __stcs(o + half * 128 + g * 32 + lane, __fmul_rn(q.ds[half][g], (float)q.q[half][g]));
        }
    }
}

// Float-FMA matmul: one warp per output row, MB activation rows per pass; w as the dequantiser
// computes it, acc += x*w, warp reduction by shuffles.  The always-available variant.
template <int QTYPE, int MB>
__global__ void __launch_bounds__(256) kq_gemv_fp32_kernel(MatmulArgs a, uint32_t q6_block_bytes) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t n = blockIdx.x * 8u + warp;
    if (n >= a.N) return;
    const uint32_t nb = a.K / kQK;
    const uint32_t m0 = blockIdx.y * MB;
    const uint32_t mcount = min((uint32_t)MB, a.M - m0);
    const uint8_t* wp = a.W + (uint64_t)n * a.w_row_bytes;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; m++) acc[m] = 0.f;
    for (uint32_t b = 0; b < nb; b++) {
        float w[8];
        uint32_t koff[8];
        if constexpr (QTYPE == 13) {
            const Q5Lane q = q5k_lane(wp + (uint64_t)b * kQ5Bytes, lane);
            const uint32_t base = (lane >> 3) * 64u + (lane & 7u) * 4u;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                w[i] = __fsub_rn(__fmul_rn(q.s_even, (float)q.q_even[i]), q.m_even);
                w[4 + i] = __fsub_rn(__fmul_rn(q.s_odd, (float)q.q_odd[i]), q.m_odd);
                koff[i] = base + i;
                koff[4 + i] = base + 32u + i;
            }
        } else {
            const Q6Lane q = q6k_lane(wp + (uint64_t)b * q6_block_bytes, lane);
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    w[half * 4 + g] = __fmul_rn(q.ds[half][g], (float)q.q[half][g]);
                    koff[half * 4 + g] = half * 128u + g * 32u + lane;
                }
        }
#pragma unroll
        for (int m = 0; m < MB; m++) {
            if ((uint32_t)m < mcount) {
                const float* xp = a.X + (uint64_t)(m0 + m) * a.K + (uint64_t)b * kQK;
                float s = acc[m];
#pragma unroll
                for (int i = 0; i < 8; i++) s = fmaf(__ldg(xp + koff[i]), w[i], s);
                acc[m] = s;
            }
        }
    }
    const float bias = a.bias ? a.bias[n] : 0.f;
#pragma unroll
    for (int m = 0; m < MB; m++) {
        float s = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (lane == 0 && (uint32_t)m < mcount) a.Y[(uint64_t)(m0 + m) * a.N + n] = s + bias;
    }
}

template <int QTYPE>
cudaError_t gemv_fp32_typed(const MatmulArgs& a, uint32_t q6bb, cudaStream_t stream, int* launches) {
    const uint32_t gx = (a.N + 7) / 8;
    MatmulArgs c = a;
    const uint32_t MB = a.M >= 8 ? 8 : a.M >= 4 ? 4 : a.M >= 2 ? 2 : 1;
    const uint32_t slab = 65535u * MB;  // gridDim.y limit
    for (uint32_t m0 = 0; m0 < a.M; m0 += slab) {
        c.M = min(slab, a.M - m0);
        c.X = a.X + (uint64_t)m0 * a.K;
        c.Y = a.Y + (uint64_t)m0 * a.N;
        const dim3 grid(gx, (c.M + MB - 1) / MB);
        switch (MB) {
            case 8: kq_gemv_fp32_kernel<QTYPE, 8><<<grid, 256, 0, stream>>>(c, q6bb); break;
            case 4: kq_gemv_fp32_kernel<QTYPE, 4><<<grid, 256, 0, stream>>>(c, q6bb); break;
            case 2: kq_gemv_fp32_kernel<QTYPE, 2><<<grid, 256, 0, stream>>>(c, q6bb); break;
            default: kq_gemv_fp32_kernel<QTYPE, 1><<<grid, 256, 0, stream>>>(c, q6bb); break;
        }
        if (launches) ++*launches;
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_kq_dequant_f32(int qtype, const uint8_t* W, const uint32_t* rows, uint32_t n_src_rows, uint32_t N,
                                  uint32_t K, uint64_t w_row_bytes, float* out, cudaStream_t stream) {
    const uint32_t nb = K / kQK;
    const uint64_t total = (uint64_t)N * nb;
    if (total == 0) return cudaSuccess;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    uint64_t ctas = (total + 7) / 8;
    const uint64_t cap = (uint64_t)sms * 8 * 4;
    if (ctas > cap) ctas = cap;
    if (qtype == 13) kq_dequant_kernel<13><<<(unsigned)ctas, 256, 0, stream>>>(W, rows, n_src_rows, N, nb, w_row_bytes, 0u, out);
    else if (qtype == 14) kq_dequant_kernel<14><<<(unsigned)ctas, 256, 0, stream>>>(W, rows, n_src_rows, N, nb, w_row_bytes, kQ6Bytes, out);
    else if (qtype == kQ6PaddedType) kq_dequant_kernel<14><<<(unsigned)ctas, 256, 0, stream>>>(W, rows, n_src_rows, N, nb, w_row_bytes, kQ6PaddedBytes, out);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_kq_gemv_fp32(int qtype, const MatmulArgs& a, cudaStream_t stream, int* launches) {
    if (a.N == 0 || a.M == 0) return cudaSuccess;
    if (qtype == 13) return gemv_fp32_typed<13>(a, 0u, stream, launches);
    if (qtype == 14) return gemv_fp32_typed<14>(a, kQ6Bytes, stream, launches);
    if (qtype == kQ6PaddedType) return gemv_fp32_typed<14>(a, kQ6PaddedBytes, stream, launches);
    return cudaErrorInvalidValue;
}

}  // namespace bpq4k
