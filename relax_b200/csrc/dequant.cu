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

template <bool PAIRED>
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
    if (i < n_words) w[i] = q4_dequant_ordered<PAIRED>(word[u], __half2(sc[u], sc[u]), qc);
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
  if (current_layout() == kLayoutPaired)
    q4f16_dequantize_kernel<true><<<(unsigned)blocks, kDeqThreads, 0, stream>>>(wq, scales, reinterpret_cast<uint4*>(w),
                                                                              n_words, (int)(K / 8));
  else
    q4f16_dequantize_kernel<false><<<(unsigned)blocks, kDeqThreads, 0, stream>>>(wq, scales, reinterpret_cast<uint4*>(w),
                                                                               n_words, (int)(K / 8));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "dequantize launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

// Offline repack: one thread per 16 bytes (four words), grid-stride; in-place is allowed (each word depends on
// itself only).  HBM bound: 4 B read + 4 B written per word.
__global__ void __launch_bounds__(256)
q4f16_repack_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int64_t n_words, int to_paired) {
  const int64_t n4 = n_words >> 2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    for (int64_t i = t; i < n4; i += stride) {
      uint4 v = reinterpret_cast<const uint4*>(in)[i];
      if (to_paired) {
        v.x = q4_word_to_paired(v.x); v.y = q4_word_to_paired(v.y); v.z = q4_word_to_paired(v.z); v.w = q4_word_to_paired(v.w);
      } else {
        v.x = q4_word_from_paired(v.x); v.y = q4_word_from_paired(v.y); v.z = q4_word_from_paired(v.z); v.w = q4_word_from_paired(v.w);
      }
      reinterpret_cast<uint4*>(out)[i] = v;
    }
  }
  for (int64_t i = (vec ? (n4 << 2) : 0) + t; i < n_words; i += stride) {
    const uint32_t w = in[i];
    out[i] = to_paired ? q4_word_to_paired(w) : q4_word_from_paired(w);
  }
}

int launch_repack(const uint32_t* in, uint32_t* out, int64_t n_words, int layout, bool to_layout, cudaStream_t stream) {
  if (n_words == 0) return B200_OK;
  if (layout == kLayoutReference) {
    if (in != out) {
      cudaError_t e = cudaMemcpyAsync(out, in, (size_t)n_words * 4, cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) return fail(B200_ELAUNCH, "repack copy: %s", cudaGetErrorString(e));
    }
    return B200_OK;
  }
  int64_t blocks = (n_words / 4 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  q4f16_repack_kernel<<<(unsigned)blocks, 256, 0, stream>>>(in, out, n_words, to_layout ? 1 : 0);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "repack launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

}  // namespace b200
