// The last matmul of a decode step: logits[B, V] = h[B, H] . W[V, H]^T over fp16 weights (the output
// embedding is not quantised), fp32 accumulation, fp16 result, and optionally the greedy token of every row.
//
// The reference lowers this to its generic matmul (python/tvm/relax/transform/legalize_ops.py:203-264:
// fp32 accumulate, then astype) followed by an argmax; for 1..16 rows it is a pure weight stream (262 MB for a
// 32000 x 4096 table), so the kernel is built like the skinny q4 kernel without the dequantisation: HBM bound.
//
//   CTA = 8 warps, two CTAs per SM (16 warps, one CTA, for 9..16 rows), a CTA takes 16-row tiles of W round
//   robin.  Warp w takes the 32-k chunks w, w + warps, ... of the tile: lane (g, t) loads 16 bytes of row g and of row g + 8 at k = chunk + 8 t (a warp
//   instruction covers 64 contiguous bytes of each of 8 rows) and feeds them to two mma.sync.m16n8k16 whose k
//   index is permuted accordingly; the activation rows sit in shared memory (row pitch padded by 64 bytes: the
//   eight lanes of a quarter warp hit distinct banks), lane (g, t) reads 16 bytes of batch row g at the same k.
//   Four chunks (eight 16-byte loads per lane) are in flight per warp.  Tile end: the warps' partial sums are
//   added in warp order through shared memory, rounded to fp16 and stored; every thread keeps the best
//   (value, index) it has produced.  Kernel end: the CTA's best per batch row goes to a scratch array, the CTA
//   that finishes last picks the winners (ties: lowest index) and writes the tokens.
#include "internal.h"
#include "skinny_common.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace {

using namespace ptx;
using skinny::mma_16x8x16;

// warps per CTA: 8 with two CTAs per SM for up to 8 batch rows; 16 in the one CTA per SM that two column blocks'
// activations leave room for (the loads in flight per SM are what the rate depends on)
__host__ __device__ constexpr int warps_of(int ncb) { return ncb == 1 ? 8 : 16; }
constexpr int kTileRows = 16;
constexpr int kUnroll = 4;            // 32-k chunks in flight per warp
constexpr int kPadBytes = 64;

struct Best {
  float v;
  int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
  // larger value wins; equal values: the lower index (what a sequential argmax returns)
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// NCB: column blocks of 8 batch rows (1 or 2).
template <int NCB>
__global__ void __launch_bounds__(warps_of(NCB) * 32, NCB == 1 ? 2 : 1)
f16_lm_head_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ logits,
                   int* __restrict__ tokens, float* __restrict__ scratch, int B, int V, int H, int token_offset) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int pitch = H * 2 + kPadBytes;                       // bytes per staged activation row
  unsigned char* xs = smem;                                  // [8 * NCB][pitch]
  float* red = reinterpret_cast<float*>(smem + (size_t)8 * NCB * pitch);   // [kWarps][16 rows][8 * NCB]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  constexpr int NC = 8 * NCB;
  constexpr int kWarps = warps_of(NCB);
  constexpr int kThreads = kWarps * 32;

  pdl_launch_dependents();
  pdl_wait();                                                // x is the previous kernel's output
  for (int i = tid; i < NC * (H / 8); i += kThreads) {
    const int m = i / (H / 8), j = i - m * (H / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < B) v = *reinterpret_cast<const uint4*>(x + (int64_t)m * H + j * 8);
    *reinterpret_cast<uint4*>(xs + (size_t)m * pitch + j * 16) = v;
  }
  __syncthreads();

  const int nchunks = H / 32;
  const int ntiles = (V + kTileRows - 1) / kTileRows;
  // final-sum role: thread (column c, row r) of the tile
  const int fr = tid & 15, fc = tid >> 4;
  Best best = {-INFINITY, 0x7fffffff};
  for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int row0 = tile * kTileRows;
    const int ra = min(row0 + g, V - 1), rb = min(row0 + g + 8, V - 1);      // clamped: rows past the end are not stored
    const __half* wa = w + (int64_t)ra * H + t * 8;
    const __half* wb = w + (int64_t)rb * H + t * 8;
    float acc[NCB][4];
#pragma unroll
    for (int cb = 0; cb < NCB; ++cb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[cb][i] = 0.f;
    for (int c0 = warp; c0 < nchunks; c0 += kWarps * kUnroll) {
      uint4 va[kUnroll], vb[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int c = c0 + u * kWarps;
        if (c < nchunks) {
          va[u] = *reinterpret_cast<const uint4*>(wa + c * 32);
          vb[u] = *reinterpret_cast<const uint4*>(wb + c * 32);
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int c = c0 + u * kWarps;
        if (c < nchunks) {
#pragma unroll
          for (int cb = 0; cb < NCB; ++cb) {
            const uint4 xq = *reinterpret_cast<const uint4*>(xs + (size_t)(cb * 8 + g) * pitch + (c * 32 + t * 8) * 2);
            mma_16x8x16(acc[cb], va[u].x, vb[u].x, va[u].y, vb[u].y, xq.x, xq.y);
            mma_16x8x16(acc[cb], va[u].z, vb[u].z, va[u].w, vb[u].w, xq.z, xq.w);
          }
        }
      }
    }
    // partial sums of this warp: rows g, g + 8; columns cb * 8 + 2 t, + 1
#pragma unroll
    for (int cb = 0; cb < NCB; ++cb) {
      float* r0 = red + ((size_t)warp * 16 + g) * NC + cb * 8 + 2 * t;
      float* r1 = red + ((size_t)warp * 16 + g + 8) * NC + cb * 8 + 2 * t;
      r0[0] = acc[cb][0]; r0[1] = acc[cb][1];
      r1[0] = acc[cb][2]; r1[1] = acc[cb][3];
    }
    __syncthreads();
    if (fc < NC) {
      float s = 0.f;
#pragma unroll
      for (int q = 0; q < kWarps; ++q) s += red[((size_t)q * 16 + fr) * NC + fc];
      const int row = row0 + fr;
      if (fc < B && row < V) {
        const __half hv = __float2half_rn(s);
        if (logits) logits[(int64_t)fc * V + row] = hv;
        best = better(best, Best{__half2float(hv), row});
      }
    }
    __syncthreads();                                         // red is reused by the next tile
  }
  if (tokens == nullptr) return;

  // ---- greedy token per batch row: CTA's best -> scratch, the last CTA picks the winners ----------------
  // scratch: [gridDim.x][16] (value, index) pairs as 2 floats, then one int counter (zero between launches)
  if (fc < NC) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {                        // the 16 row slots of a column are 16 consecutive lanes
      Best other;
      other.v = __shfl_xor_sync(0xffffffffu, best.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, best.i, o);
      best = better(best, other);
    }
    if (fr == 0 && fc < B) {
      float* slot = scratch + ((size_t)blockIdx.x * 16 + fc) * 2;
      slot[0] = best.v;
      slot[1] = __int_as_float(best.i);
    }
  }
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  int* counter = reinterpret_cast<int*>(scratch + (size_t)gridDim.x * 16 * 2);
  if (tid == 0) s_last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // 16 threads per batch row walk the CTAs' entries
  {
    const int c = tid >> 4, sl = tid & 15;
    Best b = {-INFINITY, 0x7fffffff};
    if (c < B) {
      for (int q = sl; q < (int)gridDim.x; q += 16) {
        const volatile float* slot = scratch + ((size_t)q * 16 + c) * 2;
        b = better(b, Best{slot[0], __float_as_int(slot[1])});
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      Best other;
      other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = better(b, other);
    }
    // (a row whose logits are all NaN has no winner: it gets the table's first token)
    if (c < B && sl == 0) tokens[c] = (b.i == 0x7fffffff ? 0 : b.i) + token_offset;
  }
  if (tid == 0) *counter = 0;                                // ready for the next launch in the stream
}

}  // namespace

int64_t lm_head_scratch_bytes() { return ((int64_t)sm_count() * 2 * 16 * 2 + 4) * (int64_t)sizeof(float); }

int launch_lm_head(const __half* x, const __half* w, __half* logits, int* tokens, float* scratch, int64_t B, int64_t V,
                   int64_t H, int64_t token_offset, cudaStream_t stream) {
  const int ncb = B <= 8 ? 1 : 2;
  const size_t smem = (size_t)8 * ncb * (H * 2 + kPadBytes) + (size_t)warps_of(ncb) * 16 * 8 * ncb * sizeof(float);
  if (smem > 227 * 1024) return B200_ENOTREADY;
  const int ntiles = (int)((V + kTileRows - 1) / kTileRows);
  int grid = sm_count() * (ncb == 1 ? 2 : 1);
  if (grid > ntiles) grid = ntiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)warps_of(ncb) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 1 : 0;
  cudaError_t e;
  if (ncb == 1) {
    e = cudaFuncSetAttribute(f16_lm_head_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaLaunchKernelEx(&cfg, f16_lm_head_kernel<1>, x, w, logits, tokens, scratch, (int)B, (int)V, (int)H, (int)token_offset);
  } else {
    e = cudaFuncSetAttribute(f16_lm_head_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = cudaLaunchKernelEx(&cfg, f16_lm_head_kernel<2>, x, w, logits, tokens, scratch, (int)B, (int)V, (int)H, (int)token_offset);
  }
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "lm_head launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

}  // namespace b200
