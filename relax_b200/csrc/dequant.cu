// Dequantise-only kernel: W fp16 [N,K] = decode(Wq u32 [N,K/8], S fp16 [N,K/32]).
//
// Replaces the reference's stand-alone `decode` PrimFunc (the kernel it runs when decode
// and matmul are not fused).  HBM-bound: 0.5625 B read + 2 B written per weight.  One
// thread per packed word: a warp reads 128 contiguous bytes and writes 512 contiguous
// bytes, so every sector moved is fully used.  Bit-exact by construction (q4_common.cuh).
#include "internal.h"
#include "q4_common.cuh"

namespace b200 {

constexpr int kDeqThreads = 256;
constexpr int kDeqUnroll = 4;

__global__ void __launch_bounds__(kDeqThreads)
q4f16_dequantize_kernel(const uint32_t* __restrict__ wq, const __half* __restrict__ scales,
                        uint4* __restrict__ w, int64_t n_words, int words_per_row) {
  // words_per_row = K/8; a group of 32 k is 4 consecutive words, and rows hold a whole number
  // of groups, so scale index = word index / 4.
  const Q4Consts qc = q4_consts();
  int64_t base = (int64_t)blockIdx.x * (kDeqThreads * kDeqUnroll) + threadIdx.x;
  uint32_t word[kDeqUnroll];
  __half sc[kDeqUnroll];
#pragma unroll
  for (int u = 0; u < kDeqUnroll; ++u) {
    int64_t i = base + (int64_t)u * kDeqThreads;
    bool ok = i < n_words;
    word[u] = ok ? __ldg(wq + i) : 0u;
    sc[u] = ok ? __ldg(scales + (i >> 2)) : __half(0.f);
  }
#pragma unroll
  for (int u = 0; u < kDeqUnroll; ++u) {
    int64_t i = base + (int64_t)u * kDeqThreads;
    if (i < n_words) w[i] = q4_dequant_natural(word[u], __half2(sc[u], sc[u]), qc);
  }
  (void)words_per_row;
}

int launch_dequantize(const uint32_t* wq, const __half* scales, __half* w, int64_t N, int64_t K,
                      cudaStream_t stream) {
  int64_t n_words = N * (K / 8);
  if (n_words == 0) return B200_OK;
  int64_t per_block = (int64_t)kDeqThreads * kDeqUnroll;
  int64_t blocks = (n_words + per_block - 1) / per_block;
  if (blocks > 0x7fffffffLL) return fail(B200_EINVAL, "dequantize: tensor too large (%lld words)", (long long)n_words);
  q4f16_dequantize_kernel<<<(unsigned)blocks, kDeqThreads, 0, stream>>>(wq, scales, reinterpret_cast<uint4*>(w),
                                                                        n_words, (int)(K / 8));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "dequantize launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

}  // namespace b200
