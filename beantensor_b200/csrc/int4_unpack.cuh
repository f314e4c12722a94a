// Nibble unpack shared by the int4 kernels: eight two's-complement nibbles of a 32-bit word become eight fp16 values
// w * s, each rounded once, in natural k order (byte j of the word holds k = 2j in its low and k = 2j + 1 in its high
// nibble). w is made exactly (a logic instruction puts the nibble, offset by 8, into the mantissa of 1024 or of
// 1024/16-scaled form; one HFMA2 removes the offsets), so the HMUL2 by the scale rounds the exact product w * s once:
// bit for bit f16_rne(float(w) * float(s)).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace btm {

__device__ __forceinline__ uint32_t i4_and_xor(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); // (a & b) ^ c
    return r;
}

// 8 two's-complement nibbles of a word -> 8 fp16 values v*s (one rounding each) in natural k order.
__device__ __forceinline__ uint4 dequant_word(uint32_t x, __half2 s2)
{
    const __half2 mul = __halves2half2(__ushort_as_half((unsigned short)0x3C00), __ushort_as_half((unsigned short)0x2C00)); // {1, 1/16}
    const __half2 add = __halves2half2(__ushort_as_half((unsigned short)0xE408), __ushort_as_half((unsigned short)0xD480)); // {-1032, -72}
    const uint32_t y = __byte_perm(x, x, 0x1010);
    const uint32_t z = __byte_perm(x, x, 0x3232);
    uint32_t p01 = i4_and_xor(y, 0x00F0000Fu, 0x64806408u);
    uint32_t p23 = i4_and_xor(y >> 8, 0x00F0000Fu, 0x64806408u);
    uint32_t p45 = i4_and_xor(z, 0x00F0000Fu, 0x64806408u);
    uint32_t p67 = i4_and_xor(z >> 8, 0x00F0000Fu, 0x64806408u);
    __half2 r0 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p01), mul, add), s2);
    __half2 r1 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p23), mul, add), s2);
    __half2 r2 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p45), mul, add), s2);
    __half2 r3 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p67), mul, add), s2);
    return make_uint4(*reinterpret_cast<uint32_t *>(&r0), *reinterpret_cast<uint32_t *>(&r1), *reinterpret_cast<uint32_t *>(&r2),
                      *reinterpret_cast<uint32_t *>(&r3));
}

} // namespace btm
