// Shared device helpers for the Q4_K kernels: super-block field decode.
//
// Super-block layout (144 bytes, 256 weights), as the reference's shader and
// CPU decode consume it (runtime/kernels/quant_kq/q4k_matmul.wgsl:45-74,
// runtime/gguf_loader.cpp:460-493):
//   bytes 0-1   half d          bytes 2-3   half dmin
//   bytes 4-15  eight 6-bit scales and eight 6-bit mins, packed
//   bytes 16-143 code bytes; byte 16+g*32+i holds weight g*64+i in its low
//               nibble (sub-block 2g) and weight g*64+32+i in its high nibble
//               (sub-block 2g+1)
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace bpq4k {

constexpr uint32_t kQK = 256;
constexpr uint32_t kBlockBytes = 144;
constexpr uint32_t kBlockWords = 36;

// The first 16 bytes of a super-block as four words.
struct BlockHeader {
    uint32_t w0;  // d | dmin<<16
    uint32_t s0;  // packed bytes 4..7   (scales 0..3 low 6 bits, top 2 bits belong to scales 4..7)
    uint32_t s1;  // packed bytes 8..11  (mins 0..3, top 2 bits belong to mins 4..7)
    uint32_t s2;  // packed bytes 12..15 (low nibble: scales 4..7, high nibble: mins 4..7)
};

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    // __half2float is exact for every half, subnormals included.
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16 & 0xFFFFu)));
}

// All eight scales (and mins) of a block as two packed words of four bytes
// each: scales_lo holds sub-blocks 0..3, scales_hi sub-blocks 4..7.
__device__ __forceinline__ void unpack_scales_packed(const BlockHeader& h, uint32_t& sc_lo, uint32_t& sc_hi,
                                                     uint32_t& mn_lo, uint32_t& mn_hi) {
    sc_lo = h.s0 & 0x3F3F3F3Fu;
    mn_lo = h.s1 & 0x3F3F3F3Fu;
    sc_hi = (h.s2 & 0x0F0F0F0Fu) | ((h.s0 >> 2) & 0x30303030u);
    mn_hi = ((h.s2 >> 4) & 0x0F0F0F0Fu) | ((h.s1 >> 2) & 0x30303030u);
}

__device__ __forceinline__ uint32_t byte_of(uint32_t lo, uint32_t hi, uint32_t idx) {
    const uint32_t w = idx < 4 ? lo : hi;
    return (w >> ((idx & 3u) * 8u)) & 0xFFu;
}

}  // namespace bpq4k
