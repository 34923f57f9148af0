// Shared device helpers for the q4f16 kernels (sm_100a).
//
// Decode rule (what the reference's TIR computes, src/tir/op/op.cc:564,606,282 in the
// reference tree): q = (word >> 4*(k%8)) & 0xF, w = fp16(q - 7) * scale with ONE fp16
// round-to-nearest-even multiply.  The helpers below form (q - 7) exactly in fp16 with the
// "magic number" trick (OR the nibble into the mantissa of 1024.0, subtract) and then issue
// exactly one HMUL2 per pair, so every kernel that uses them reproduces the reference's
// dequantised weights bit for bit.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) {
  return *reinterpret_cast<__half2*>(&v);
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}

// Masks and the magic number live in constant memory on purpose.  Written as literals, ptxas
// encodes (w & mask) | magic as TWO instructions (an instruction has room for one 32-bit
// immediate); with the operands coming from the constant bank it is one LOP3, which halves the
// integer-pipe work of the unpack (measured: 8.2 -> 4.1 logic instructions per packed word, and
// the integer pipe was the busiest unit of the skinny matmul).
static __constant__ uint32_t kQ4Bits[3] = {0x000F000Fu, 0x00F000F0u, 0x64006400u};

// (a & b) | c in one LOP3.
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// The three constants, fetched once per kernel (q4_consts()) and kept in registers: a kernel
// whose loop contains a compiler memory barrier would otherwise re-read them every iteration.
struct Q4Consts {
  uint32_t lo, hi, magic;   // nibble 0 / nibble 1 of each 16-bit half; (1024, 1024)
};
__device__ __forceinline__ Q4Consts q4_consts() { return Q4Consts{kQ4Bits[0], kQ4Bits[1], kQ4Bits[2]}; }

// One packed word (8 nibbles, k0 lowest) -> four half2 of exact (q-7):
//   out[0] = (k0,k4)  out[1] = (k1,k5)  out[2] = (k2,k6)  out[3] = (k3,k7)
// 1 shift + 4 LOP3 + 4 half2 arithmetic ops.
__device__ __forceinline__ void q4_unpack_pairs(uint32_t w, __half2 (&out)[4], const Q4Consts& c) {
  const __half2 kSub = u32_as_h2(0x64076407u);         // (1031, 1031)
  const __half2 kSixteenth = u32_as_h2(0x2C002C00u);   // (1/16, 1/16)
  const __half2 kNeg71 = u32_as_h2(0xD470D470u);       // (-71, -71)
  uint32_t lo0 = lop3_and_or(w, c.lo, c.magic);        // 1024 + q0      , 1024 + q4
  uint32_t hi0 = lop3_and_or(w, c.hi, c.magic);        // 1024 + 16*q1   , 1024 + 16*q5
  uint32_t w8 = w >> 8;
  uint32_t lo1 = lop3_and_or(w8, c.lo, c.magic);       // q2, q6
  uint32_t hi1 = lop3_and_or(w8, c.hi, c.magic);       // q3, q7
  out[0] = __hsub2(u32_as_h2(lo0), kSub);                    // exact: q - 7
  out[1] = __hfma2(u32_as_h2(hi0), kSixteenth, kNeg71);      // exact: (64 + q) - 71
  out[2] = __hsub2(u32_as_h2(lo1), kSub);
  out[3] = __hfma2(u32_as_h2(hi1), kSixteenth, kNeg71);
}

// Same, followed by the single rounding multiply by the group's scale (both lanes = scale).
__device__ __forceinline__ void q4_dequant_pairs(uint32_t w, __half2 scale2, uint32_t (&out)[4], const Q4Consts& c) {
  __half2 v[4];
  q4_unpack_pairs(w, v, c);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = h2_as_u32(__hmul2(v[i], scale2));
}

// Dequantised word in natural order: out = (k0,k1) (k2,k3) (k4,k5) (k6,k7).
__device__ __forceinline__ uint4 q4_dequant_natural(uint32_t w, __half2 scale2, const Q4Consts& c) {
  uint32_t p[4];
  q4_dequant_pairs(w, scale2, p, c);
  uint4 o;
  o.x = __byte_perm(p[0], p[1], 0x5410);
  o.y = __byte_perm(p[2], p[3], 0x5410);
  o.z = __byte_perm(p[0], p[1], 0x7632);
  o.w = __byte_perm(p[2], p[3], 0x7632);
  return o;
}

// Weight layouts.  kLayoutReference: nibble j of a word is k % 8 = j (what the reference's encoder writes,
// python/tvm/relax/transform/legalize_ops.py in its tree does the decode the same way).  kLayoutPaired: the
// nibbles of a word sit in the order k0,k2,k4,k6,k1,k3,k5,k7, so that the four mask-and-or extractions of
// q4_unpack_pairs yield (k0,k1) (k2,k3) (k4,k5) (k6,k7): natural order without the four byte permutes.
// Same shape, same scales; a pure permutation inside every 32-bit word (b200_q4f16_repack / _unpack).
constexpr int kLayoutReference = 0, kLayoutPaired = 1;

// Reference word -> paired word and back (each is the other's inverse).
__host__ __device__ __forceinline__ uint32_t q4_word_to_paired(uint32_t w) {
  // nibble positions [0..7] of the result hold k0,k2,k4,k6,k1,k3,k5,k7
  return (w & 0xFu) | ((w >> 4) & 0xF0u) | ((w >> 8) & 0xF00u) | ((w >> 12) & 0xF000u) |
         ((w << 12) & 0xF0000u) | ((w << 8) & 0xF00000u) | ((w << 4) & 0xF000000u) | (w & 0xF0000000u);
}
__host__ __device__ __forceinline__ uint32_t q4_word_from_paired(uint32_t v) {
  return (v & 0xFu) | ((v >> 12) & 0xF0u) | ((v << 4) & 0xF00u) | ((v >> 8) & 0xF000u) |
         ((v << 8) & 0xF0000u) | ((v >> 4) & 0xF00000u) | ((v << 12) & 0xF000000u) | (v & 0xF0000000u);
}

// Dequantised word of the PAIRED layout in natural order: the four pairs are already (k0,k1) .. (k6,k7).
__device__ __forceinline__ uint4 q4_dequant_paired(uint32_t w, __half2 scale2, const Q4Consts& c) {
  uint32_t p[4];
  q4_dequant_pairs(w, scale2, p, c);
  return make_uint4(p[0], p[1], p[2], p[3]);
}
template <bool PAIRED>
__device__ __forceinline__ uint4 q4_dequant_ordered(uint32_t w, __half2 scale2, const Q4Consts& c) {
  return PAIRED ? q4_dequant_paired(w, scale2, c) : q4_dequant_natural(w, scale2, c);
}

}  // namespace b200
