// Device-side decode of the 2-bit stored ternary values of the stream layout.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

// Two 2-bit stored values s = code + 1 (bits 2q..2q+1 and 16+2q..16+2q+1 of `word`, q = 0..7)
// -> packed bf16 pair of codes in {-1, 0, +1}, exactly.
//
// No shift is needed for the four positions of the low byte of each half: OR-ing the two bits
// into the mantissa of a bf16 constant whose unit-in-the-last-place makes them worth s gives
// base + s, and subtracting base + 1 leaves the code.
//   bits 0-1: 128 + s (0x4300), bits 2-3: 32 + s (0x4200), bits 4-5: 8 + s (0x4100);
//   bits 6-7 straddle the mantissa top bit and the exponent low bit of 2.0 (0x4000):
//   s = 0, 1, 2 -> 2.0, 3.0, 4.0 = 2 + s as well.
// Positions 4..7 are the same four after one shift by 8 (shared by the four registers).
// s = 3 never occurs in a validated stream.
__device__ __forceinline__ uint32_t mortar_decode_pair(uint32_t word, int q) {
    const uint32_t w = (q & 4) ? (word >> 8) : word;
    const int j = q & 3;
    const uint32_t mask = 0x00030003u << (2 * j);
    const uint32_t base = j == 0 ? 0x43004300u : j == 1 ? 0x42004200u : j == 2 ? 0x41004100u : 0x40004000u;
    const uint32_t bias = j == 0 ? 0x43014301u : j == 1 ? 0x42044204u : j == 2 ? 0x41104110u : 0x40404040u;
    // (w & mask) | base as ONE three-input logic op (left to the compiler it becomes two), then
    // the packed bf16 subtraction
    uint32_t v, r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(w), "r"(mask), "r"(base));
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(bias));
    return r;
}

// The same decode into a packed fp16 pair.  fp16 has 10 mantissa bits, so all four 2-bit positions
// of a byte lie inside the mantissa: the constants are 1024, 256, 64 and 16 (units in the last
// place 1, 1/4, 1/16, 1/64), the subtrahends those plus one.
__device__ __forceinline__ uint32_t mortar_decode_pair_h(uint32_t word, int q) {
    const uint32_t w = (q & 4) ? (word >> 8) : word;
    const int j = q & 3;
    const uint32_t mask = 0x00030003u << (2 * j);
    const uint32_t base = j == 0 ? 0x64006400u : j == 1 ? 0x5C005C00u : j == 2 ? 0x54005400u : 0x4C004C00u;
    const uint32_t bias = j == 0 ? 0x64016401u : j == 1 ? 0x5C045C04u : j == 2 ? 0x54105410u : 0x4C404C40u;
    uint32_t v, r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(w), "r"(mask), "r"(base));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(bias));
    return r;
}
