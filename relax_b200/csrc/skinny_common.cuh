// Device helpers shared by the skinny (batch <= 16) q4f16 kernels: the warp-level MMA wrappers, the fp16x8
// elementwise pieces of the fused neighbours (residual add, RMSNorm scaling, SwiGLU), the layout of the
// staged activation block, the offset bookkeeping of the batch-1 fast form and the descriptor of the sum
// over tensor-parallel ranks.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "q4_common.cuh"

namespace b200 {
namespace skinny {

__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B + C with D and C in different registers (C: the negated offset sums of the fast form).
__device__ __forceinline__ void mma_16x8x16_c(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Eight fp16 at a time, fp32 inside, one round-to-nearest at the end (the same arithmetic as the
// stand-alone RMSNorm and SwiGLU kernels).
__device__ __forceinline__ uint4 add_f16x8(const uint4& a, const uint4& b) {
  uint4 o;
  const __half2* x = reinterpret_cast<const __half2*>(&a);
  const __half2* y = reinterpret_cast<const __half2*>(&b);
  __half2* r = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(x[j]), g = __half22float2(y[j]);
    r[j] = __floats2half2_rn(f.x + g.x, f.y + g.y);
  }
  return o;
}
__device__ __forceinline__ uint4 scale_f16x8(const uint4& a, float inv, const uint4& w) {
  uint4 o;
  const __half2* x = reinterpret_cast<const __half2*>(&a);
  const __half2* y = reinterpret_cast<const __half2*>(&w);
  __half2* r = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(x[j]), g = __half22float2(y[j]);
    r[j] = __floats2half2_rn(f.x * inv * g.x, f.y * inv * g.y);
  }
  return o;
}
__device__ __forceinline__ uint4 silu_mul_f16x8(const uint4& gate, const uint4& up) {
  uint4 o;
  const __half2* x = reinterpret_cast<const __half2*>(&gate);
  const __half2* y = reinterpret_cast<const __half2*>(&up);
  __half2* r = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 g = __half22float2(x[j]), u = __half22float2(y[j]);
    r[j] = __floats2half2_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
  }
  return o;
}

// Layout of the staged x block: one 16-byte slot per (8-k word jw, batch column).  Lane (g,t)
// reads column g of words 32c + 8t + i (i = 0..7), so the four lanes t of a row-group read
// words 8 apart in the same instruction and their slots must differ mod 8:
//   NC >= 8: NC slots per word, column XOR-ed with 2*((jw>>3)&3)  (= 2t);
//   NC <  8: NC slots per word plus NC slots of padding after every 8 words.
template <int NC>
struct XLayout {
  __device__ __forceinline__ static int slot(int jw, int col) {
    if (NC >= 8) return jw * NC + (col ^ (((jw >> 3) & 3) << 1));
    return NC * (jw + (jw >> 3)) + col;
  }
  // slots per 256-k chunk (32 words)
  static constexpr int kSlotsPerChunk = NC >= 8 ? 32 * NC : 36 * NC;
  // bytes for a block of `k` (multiple of 256)
  __host__ __device__ static constexpr size_t bytes(int k) { return (size_t)(k / 256) * kSlotsPerChunk * 16; }
};

// Offsets the raw nibble halves carry in the fast form: (w & 0x000F000F) | 0x64006400 = 1024 + q (even k of a
// word), (w & 0x00F000F0) | 0x54005400 = 64 + q (odd k); minus the zero point 7 that is 1031 and 71.
constexpr float kOffEven = 1031.f, kOffOdd = 71.f;
// sum over the eight k of one staged word of x_k * offset_k; v holds (x0,x1)(x2,x3)(x4,x5)(x6,x7).  In the paired
// weight layout the 1024-offset extractions hold k0,k1,k4,k5 and the 64-offset ones k2,k3,k6,k7.
__device__ __forceinline__ float offset_sum_f16x8(const uint4& v, bool paired) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), c = __half22float2(h[2]), d = __half22float2(h[3]);
  if (paired) return fmaf(kOffEven, (a.x + a.y) + (c.x + c.y), kOffOdd * ((b.x + b.y) + (d.x + d.y)));
  return fmaf(kOffEven, (a.x + c.x) + (b.x + d.x), kOffOdd * ((a.y + c.y) + (b.y + d.y)));
}
// One word of activations (x0..x7) in the order the unpack of a packed weight word produces its four pairs:
// (k0,k4)(k1,k5)(k2,k6)(k3,k7) for the reference's nibble order, natural order for the paired layout.
__device__ __forceinline__ uint4 staged_order(const uint4& v, bool paired) {
  if (paired) return v;
  uint4 q;
  q.x = __byte_perm(v.x, v.z, 0x5410);
  q.y = __byte_perm(v.x, v.z, 0x7632);
  q.z = __byte_perm(v.y, v.w, 0x5410);
  q.w = __byte_perm(v.y, v.w, 0x7632);
  return q;
}
// Where the fast form keeps minus the offset sum of group `grp` (counted from the start of the staged block):
// 32 floats per 256-k chunk, [lane pair t & 1][set: even / odd group][c0 c1 c0 c1], so that lane (g,t) fetches
// the accumulator input of a set -- rows g and g+8, columns 2t and 2t+1 = groups 4t+set and 4t+2+set -- with one
// 16-byte load.
__device__ __forceinline__ int corr_index(int grp) {
  const int j = grp & 7;
  return (grp >> 3) * 32 + ((j >> 2) * 2 + (j & 1)) * 4 + ((j >> 1) & 1);
}

constexpr int kMaxPeers = 8;

// Sum over tensor-parallel ranks fused into a row-parallel matmul.  y (this rank's partial result)
// lives in memory that every peer has mapped; the CTA that finishes last on this GPU publishes a
// flag to every rank; every CTA then waits for all ranks' flags and adds up its slice of the
// partial results in rank order (so every rank gets the same bits) into `out`.  Peer memory is
// read with plain volatile loads only.
struct PeerReduce {
  int world = 0;                            // <= 1: off
  int rank = 0;
  const __half* peer_y[kMaxPeers] = {};     // rank r's partial result as mapped on this GPU (peer_y[rank] == y)
  int* peer_flags[kMaxPeers] = {};          // rank r's flag array as mapped on this GPU
  int flag_base = 0;                        // this reduction's `world` slots inside a flag array
  const int* epoch = nullptr;               // device scalar: flags carry *epoch + 1 (grows from step to step)
  int* done_counter = nullptr;              // zero between launches
  __half* out = nullptr;                    // [M, N] fp16, local
  uint64_t wait_ns = 2000000000ull;         // how long to wait for the other GPUs' flags (option gemv.peer_wait_ms)
};


}  // namespace skinny
}  // namespace b200
