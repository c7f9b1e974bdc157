// Straightforward Q4_K kernels: the bit-exact dequantiser and a float-FMA
// matmul with one warp per output row.  They are the arithmetic twin of the
// reference's shader (runtime/kernels/quant_kq/q4k_matmul.wgsl:37-94) and CPU
// decode (runtime/gguf_loader.cpp:455-496) and serve as the always-available
// variant; the bandwidth-tuned kernels live in q4k_gemv_stream.cu.
#include "kernels.h"
#include "q4k_common.cuh"

namespace bpq4k {

// ---------------------------------------------------------------------------
// Dequantise: one warp per super-block.  Lane l owns code word l (code bytes
// 4l..4l+3): group g = l/8 -> sub-blocks 2g (low nibbles) and 2g+1 (high).
// Each lane writes two float4, so eight lanes cover 128 contiguous bytes.
// HBM-bound on the 4 B/weight it writes (reads 0.5625 B/weight).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dequant_f32_kernel(const uint8_t* __restrict__ W, uint32_t N, uint32_t nb,
                                                           uint64_t w_row_bytes, float* __restrict__ out) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const uint64_t total = (uint64_t)N * nb;
    const uint32_t K = nb * kQK;
    for (uint64_t blk = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < total; blk += warps) {
        const uint32_t row = (uint32_t)(blk / nb);
        const uint32_t b = (uint32_t)(blk - (uint64_t)row * nb);
        const uint8_t* p = W + (uint64_t)row * w_row_bytes + (uint64_t)b * kBlockBytes;
        const uint4 hv = __ldg(reinterpret_cast<const uint4*>(p));
        const BlockHeader h{hv.x, hv.y, hv.z, hv.w};
        const uint32_t code = __ldg(reinterpret_cast<const uint32_t*>(p + 16) + lane);
        const float d = half_bits_to_float(h.w0);
        const float dmin = half_bits_to_float(h.w0 >> 16);
        uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
        unpack_scales_packed(h, sc_lo, sc_hi, mn_lo, mn_hi);
        const uint32_t g = lane >> 3;
        // (d*sc) and (dmin*mn) are rounded products; (d*sc)*q is rounded, then
        // the difference is rounded -- the same four float operations as
        // gguf_loader.cpp:480-492.  The _rn intrinsics are never contracted.
        const float s_even = __fmul_rn(d, (float)byte_of(sc_lo, sc_hi, 2 * g));
        const float s_odd = __fmul_rn(d, (float)byte_of(sc_lo, sc_hi, 2 * g + 1));
        const float m_even = __fmul_rn(dmin, (float)byte_of(mn_lo, mn_hi, 2 * g));
        const float m_odd = __fmul_rn(dmin, (float)byte_of(mn_lo, mn_hi, 2 * g + 1));
        float4 lo, hi;
        lo.x = __fsub_rn(__fmul_rn(s_even, (float)(code & 15u)), m_even);
        hi.x = __fsub_rn(__fmul_rn(s_odd, (float)((code >> 4) & 15u)), m_odd);
        lo.y = __fsub_rn(__fmul_rn(s_even, (float)((code >> 8) & 15u)), m_even);
        hi.y = __fsub_rn(__fmul_rn(s_odd, (float)((code >> 12) & 15u)), m_odd);
        lo.z = __fsub_rn(__fmul_rn(s_even, (float)((code >> 16) & 15u)), m_even);
        hi.z = __fsub_rn(__fmul_rn(s_odd, (float)((code >> 20) & 15u)), m_odd);
        lo.w = __fsub_rn(__fmul_rn(s_even, (float)((code >> 24) & 15u)), m_even);
        hi.w = __fsub_rn(__fmul_rn(s_odd, (float)(code >> 28)), m_odd);
        float* o = out + (uint64_t)row * K + (uint64_t)b * kQK + g * 64u + (lane & 7u) * 4u;
        __stcs(reinterpret_cast<float4*>(o), lo);
        __stcs(reinterpret_cast<float4*>(o + 32), hi);
    }
}

cudaError_t launch_dequant_f32(const uint8_t* W, uint32_t N, uint32_t K, uint64_t w_row_bytes, float* out,
                               cudaStream_t stream) {
    const uint32_t nb = K / kQK;
    const uint64_t total = (uint64_t)N * nb;
    if (total == 0) return cudaSuccess;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    uint64_t ctas = (total + 7) / 8;
    const uint64_t cap = (uint64_t)sms * 8 * 4;
    if (ctas > cap) ctas = cap;
    dequant_f32_kernel<<<(unsigned)ctas, 256, 0, stream>>>(W, N, nb, w_row_bytes, out);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Float-FMA matmul: one warp per output row, MB activation rows per pass.
// Lane l owns code word l of every block of its row (8 weights), reads the
// matching two float4 of each activation row, and the warp reduces with
// shuffles.  Arithmetic per weight is the shader's: w = (d*sc)*q - dmin*mn,
// acc += x*w (q4k_matmul.wgsl:66-76).  The direct form reads the weights
// ceil(M/MB) times, like the reference's batched8 shader re-reads them M/8
// times; it is the fallback and the cross-check, not the fast path.
// ---------------------------------------------------------------------------
template <int MB>
__global__ void __launch_bounds__(256) gemv_fp32_kernel(MatmulArgs a) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t n = blockIdx.x * 8u + warp;
    if (n >= a.N) return;
    const uint32_t nb = a.K / kQK;
    uint32_t m0 = blockIdx.y * MB;
    const float* X = a.X;
    float* Y = a.Y;
    uint64_t wrow = n;
    uint32_t mcount;
    if (a.n_slots) {  // indirect form: blockIdx.y is the slot, one activation row
        const uint32_t s = blockIdx.y;
        wrow += a.offsets[s];
        X += (uint64_t)(a.x_rows ? a.x_rows[s] : s) * a.K;
        Y += (uint64_t)s * a.N;
        m0 = 0;
        mcount = 1;
    } else {
        mcount = min((uint32_t)MB, a.M - m0);
    }
    const uint8_t* wp = a.W + wrow * a.w_row_bytes;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; m++) acc[m] = 0.f;
    const uint32_t g = lane >> 3;
    const uint32_t koff = g * 64u + (lane & 7u) * 4u;
    for (uint32_t b = 0; b < nb; b++) {
        const uint8_t* p = wp + (uint64_t)b * kBlockBytes;
        const uint4 hv = __ldg(reinterpret_cast<const uint4*>(p));
        const BlockHeader h{hv.x, hv.y, hv.z, hv.w};
        const uint32_t code = __ldg(reinterpret_cast<const uint32_t*>(p + 16) + lane);
        const float d = half_bits_to_float(h.w0);
        const float dmin = half_bits_to_float(h.w0 >> 16);
        uint32_t sc_lo, sc_hi, mn_lo, mn_hi;
        unpack_scales_packed(h, sc_lo, sc_hi, mn_lo, mn_hi);
        const float s_even = d * (float)byte_of(sc_lo, sc_hi, 2 * g);
        const float s_odd = d * (float)byte_of(sc_lo, sc_hi, 2 * g + 1);
        const float m_even = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g);
        const float m_odd = dmin * (float)byte_of(mn_lo, mn_hi, 2 * g + 1);
        float wl[4], wh[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            wl[j] = __fsub_rn(__fmul_rn(s_even, (float)((code >> (8 * j)) & 15u)), m_even);
            wh[j] = __fsub_rn(__fmul_rn(s_odd, (float)((code >> (8 * j + 4)) & 15u)), m_odd);
        }
#pragma unroll
        for (int m = 0; m < MB; m++) {
            if ((uint32_t)m < mcount) {
                const float* xp = X + (uint64_t)(m0 + m) * a.K + (uint64_t)b * kQK + koff;
                const float4 xl = __ldg(reinterpret_cast<const float4*>(xp));
                const float4 xh = __ldg(reinterpret_cast<const float4*>(xp + 32));
                float s = acc[m];
                s = fmaf(xl.x, wl[0], s); s = fmaf(xl.y, wl[1], s); s = fmaf(xl.z, wl[2], s); s = fmaf(xl.w, wl[3], s);
                s = fmaf(xh.x, wh[0], s); s = fmaf(xh.y, wh[1], s); s = fmaf(xh.z, wh[2], s); s = fmaf(xh.w, wh[3], s);
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
        if (lane == 0 && (uint32_t)m < mcount) Y[(uint64_t)(m0 + m) * a.N + n] = s + bias;
    }
}

cudaError_t launch_gemv_fp32(const MatmulArgs& a, cudaStream_t stream, int* launches) {
    if (a.N == 0) return cudaSuccess;
    const uint32_t gx = (a.N + 7) / 8;
    if (a.n_slots) {
        // gridDim.y is limited to 65535
        MatmulArgs c = a;
        for (uint32_t s0 = 0; s0 < a.n_slots; s0 += 65535u) {
            const uint32_t cnt = min(65535u, a.n_slots - s0);
            c.offsets = a.offsets + s0;
            c.x_rows = a.x_rows ? a.x_rows + s0 : nullptr;
            // with x_rows null the slot index selects the row: advance X too
            c.X = a.x_rows ? a.X : a.X + (uint64_t)s0 * a.K;
            c.Y = a.Y + (uint64_t)s0 * a.N;
            gemv_fp32_kernel<1><<<dim3(gx, cnt), 256, 0, stream>>>(c);
            if (launches) ++*launches;
        }
        return cudaGetLastError();
    }
    if (a.M == 0) return cudaSuccess;
    MatmulArgs c = a;
    // gridDim.y is limited to 65535: walk very tall activations in slabs.
    const uint32_t MB = a.M >= 8 ? 8 : a.M >= 4 ? 4 : a.M >= 2 ? 2 : 1;
    const uint32_t slab = 65535u * MB;
    for (uint32_t m0 = 0; m0 < a.M; m0 += slab) {
        c.M = min(slab, a.M - m0);
        c.X = a.X + (uint64_t)m0 * a.K;
        c.Y = a.Y + (uint64_t)m0 * a.N;
        const dim3 grid(gx, (c.M + MB - 1) / MB);
        switch (MB) {
            case 8: gemv_fp32_kernel<8><<<grid, 256, 0, stream>>>(c); break;
            case 4: gemv_fp32_kernel<4><<<grid, 256, 0, stream>>>(c); break;
            case 2: gemv_fp32_kernel<2><<<grid, 256, 0, stream>>>(c); break;
            default: gemv_fp32_kernel<1><<<grid, 256, 0, stream>>>(c); break;
        }
        if (launches) ++*launches;
    }
    return cudaGetLastError();
}

}  // namespace bpq4k
