// Skinny q4f16 matmul for decode: y[M,N] = x[M,K] . decode(Wq,S)^T with 1 <= M <= 16.
//
// Replaces the fused decode+matmul+astype PrimFunc of the reference for small M (the
// reference would run it as MetaSchedule-tuned CUDA C, src/relax/transform/meta_schedule.cc;
// there is no hand-written kernel to mirror).  The kernel is HBM-bound: per launch it must
// move N*K/2 bytes of packed weights and N*K/16 bytes of scales once; x and y are noise.
//
// Work split.  A CTA owns 16*RT consecutive rows of W and the whole K range; its warps take
// 256-wide slices of K round-robin and the partial sums meet in shared memory at the end.
// Inside a warp the products run on the tensor cores as mma.sync m16n8k16 (A = 16 weight
// rows, B = up to 8 batch columns), because at 1.6 ALU instructions per weight for the
// dequantisation there is no issue bandwidth left for one FFMA + one CVT per weight.
//
// Thread <-> data mapping (lane = 4*g + t).  In a slice, thread t of row-group g loads the
// 16-byte words of groups 8c+2t and 8c+2t+1 of rows g and g+8: one uint4 is exactly one
// scale group (32 nibbles), four neighbouring lanes read 128 contiguous bytes of a row.
// A packed word unpacks to the pairs (k0,k4)(k1,k5)(k2,k6)(k3,k7); instead of shuffling the
// weights back into order, x is staged in shared memory in that same permuted order once
// per CTA, so an A fragment and its B fragment always agree on which k sits where.  Each
// dequantised weight is the reference's fp16 value (one HMUL2 after an exact q-7); only
// the fp32 summation order differs from the reference's sequential loop.
#include "internal.h"
#include "q4_common.cuh"
#include "skinny_common.cuh"

namespace b200 {

namespace {

constexpr int kChunkGroups = 8;    // groups of 32 k per warp-slice
constexpr int kChunkK = 256;       // k per warp-slice

__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Shared-memory slot of batch column `col` inside the 8-k word `jw` of the staged x block.
// With 8 or 16 stored columns the four lanes t of a row-group read words 1 KB apart, which
// would land on the same banks; XOR-ing 2*t into the column spreads them over all 8 slots.
template <int NC>
__device__ __forceinline__ int x_slot(int jw, int col) {
  return NC >= 8 ? jw * NC + (col ^ (((jw >> 3) & 3) << 1)) : jw * NC + col;
}

// One slice's worth of packed weights and scales held in registers.
template <int RT>
struct Slice {
  uint4 w[RT][2][2];     // [row tile][row g / g+8][group u]
  __half2 s[RT][2][2];   // scale of that group, broadcast to both lanes
};

template <int NC, int RT>
__global__ void __launch_bounds__(512)
q4f16_gemv_stream_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ wq,
                         const __half* __restrict__ scales, __half* __restrict__ y, int M, int N, int K,
                         int kblk, int paired) {
  constexpr int MT = (NC + 7) / 8;           // n8 column tiles
  constexpr int TILE_N = 16 * RT;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* xs = reinterpret_cast<uint4*>(smem_raw);  // [kblk/8 words][NC] permuted x

  const Q4Consts qc = q4_consts();
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int G = K >> 5;                       // scale groups per row
  const int words_per_row = K >> 3;
  const int row0 = blockIdx.x * TILE_N;

  // Rows this thread streams (clamped so out-of-range rows re-read the last row; their
  // results are dropped at the store).
  const uint32_t* wrow[RT][2];
  const __half* srow[RT][2];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int r = row0 + rt * 16 + g + 8 * h;
      r = r < N ? r : N - 1;
      wrow[rt][h] = wq + (int64_t)r * words_per_row;
      srow[rt][h] = scales + (int64_t)r * G;
    }

  auto load_slice = [&](int c, Slice<RT>& sl) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      int gi = c * kChunkGroups + 2 * t + u;
      bool ok = gi < G;
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (ok) {
            sl.w[rt][h][u] = ldg_stream(reinterpret_cast<const uint4*>(wrow[rt][h] + gi * 4));
            __half sc = __ldg(srow[rt][h] + gi);
            sl.s[rt][h][u] = __half2(sc, sc);
          } else {
            sl.w[rt][h][u] = make_uint4(0, 0, 0, 0);
            sl.s[rt][h][u] = __half2(__half(0.f), __half(0.f));   // w = -7 * 0: contributes nothing
          }
        }
    }
  };

  float acc[RT][MT][4];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[rt][mt][i] = 0.f;

  const int nchunks = (G + kChunkGroups - 1) / kChunkGroups;
  const int chunks_per_blk = kblk / kChunkK;

  // Weights do not depend on the previous kernel in the stream: start the first slice's loads
  // before waiting on it (programmatic dependent launch); x does, so it is read afterwards.
  Slice<RT> cur, nxt;
  {
    int c_first = warp;
    if (c_first < nchunks && c_first < chunks_per_blk) load_slice(c_first, cur);
  }
  pdl_wait();

  for (int cb = 0; cb < nchunks; cb += chunks_per_blk) {
    // ---- stage x[:, cb*256 .. +kblk) into shared memory, permuted per 8 k ----------------
    if (cb > 0) __syncthreads();
    {
      const int words = kblk >> 3;
      const int k0 = cb * kChunkK;
      for (int i = tid; i < words * NC; i += blockDim.x) {
        int j = i / NC, m = i - j * NC;
        int k = k0 + j * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < M && k < K) v = *reinterpret_cast<const uint4*>(x + (int64_t)m * K + k);
        // (k0,k4)(k1,k5)(k2,k6)(k3,k7) for the reference's nibble order, natural order for the paired layout
        xs[x_slot<NC>(j, m)] = skinny::staged_order(v, paired != 0);
      }
    }
    __syncthreads();

    const int c_end = min(nchunks, cb + chunks_per_blk);
    int c = cb + warp;
    if (cb > 0 && c < c_end) load_slice(c, cur);
    for (; c < c_end; c += nwarps) {
      const int cn = c + nwarps;
      const bool more = cn < c_end;
      if (more) load_slice(cn, nxt);
      else if (cb + chunks_per_blk >= nchunks) pdl_launch_dependents();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int gi = c * kChunkGroups + 2 * t + u;
        const int jbase = (gi - cb * kChunkGroups) * 4;   // word index inside the staged block
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
          uint4 b[MT];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            int col = g + 8 * mt;
            b[mt] = (col < NC) ? xs[x_slot<NC>(jbase + wd, col)] : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int rt = 0; rt < RT; ++rt) {
            uint32_t a_lo[4], a_hi[4];
            const uint4& w0 = cur.w[rt][0][u];
            const uint4& w1 = cur.w[rt][1][u];
            uint32_t word0 = wd == 0 ? w0.x : wd == 1 ? w0.y : wd == 2 ? w0.z : w0.w;
            uint32_t word1 = wd == 0 ? w1.x : wd == 1 ? w1.y : wd == 2 ? w1.z : w1.w;
            q4_dequant_pairs(word0, cur.s[rt][0][u], a_lo, qc);
            q4_dequant_pairs(word1, cur.s[rt][1][u], a_hi, qc);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_16x8x16(acc[rt][mt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[mt].x, b[mt].y);
              mma_16x8x16(acc[rt][mt], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[mt].z, b[mt].w);
            }
          }
        }
      }
      if (more) cur = nxt;
    }
  }

  // ---- cross-warp reduction and store -------------------------------------------------------
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem_raw);   // [nwarps][RT*MT*128]
  constexpr int PER_WARP = RT * MT * 128;
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp * PER_WARP + ((rt * MT + mt) * 4 + i) * 32 + lane] = acc[rt][mt][i];
  __syncthreads();
  for (int e = tid; e < PER_WARP; e += blockDim.x) {
    float sum = 0.f;
    for (int w = 0; w < nwarps; ++w) sum += red[w * PER_WARP + e];
    int ln = e & 31;
    int q = e >> 5;
    int i = q & 3;
    int mt = (q >> 2) % MT;
    int rt = (q >> 2) / MT;
    int row = row0 + rt * 16 + (ln >> 2) + 8 * (i >> 1);
    int col = mt * 8 + 2 * (ln & 3) + (i & 1);
    if (row < N && col < M) y[(int64_t)col * N + row] = __float2half_rn(sum);
  }
}

template <int NC, int RT>
int launch_stream(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int M, int N, int K,
                  cudaStream_t stream) {
  constexpr int MT = (NC + 7) / 8;
  constexpr int TILE_N = 16 * RT;
  int warps = (int)options().gemv_warps;
  if (warps <= 0) warps = 8;
  if (warps > 16) warps = 16;
  // x block: as much of K as fits a 64 KB budget, in multiples of one warp-slice.
  const int kpad = ((K + kChunkK - 1) / kChunkK) * kChunkK;
  int kblk = (64 * 1024 / (NC * 2) / kChunkK) * kChunkK;
  if (kblk > kpad) kblk = kpad;
  size_t smem = (size_t)NC * kblk * 2;
  size_t red = (size_t)warps * RT * MT * 128 * sizeof(float);
  if (red > smem) smem = red;
  auto kern = q4f16_gemv_stream_kernel<NC, RT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemv: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((N + TILE_N - 1) / TILE_N));
  cfg.blockDim = dim3((unsigned)(warps * 32));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, x, wq, scales, y, M, N, K, kblk, (int)(current_layout() == kLayoutPaired));
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemv launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

}  // namespace

int launch_gemv_stream(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M,
                       int64_t N, int64_t K, cudaStream_t stream) {
  int m = (int)M, n = (int)N, k = (int)K;
  if (m == 1) return launch_stream<1, 1>(x, wq, scales, y, m, n, k, stream);
  if (m == 2) return launch_stream<2, 1>(x, wq, scales, y, m, n, k, stream);
  if (m <= 4) return launch_stream<4, 1>(x, wq, scales, y, m, n, k, stream);
  if (m <= 8) return launch_stream<8, 1>(x, wq, scales, y, m, n, k, stream);
  return launch_stream<16, 1>(x, wq, scales, y, m, n, k, stream);
}

int launch_gemv_pipe(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                     int64_t K, cudaStream_t stream);

int launch_gemv(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                int64_t K, cudaStream_t stream) {
  if (N == 0 || M == 0) return B200_OK;
  const int64_t variant = options().gemv_variant;
  if (variant != 1) {
    int rc = launch_gemv_pipe(x, wq, scales, y, M, N, K, stream);
    if (rc != B200_ENOTREADY) return rc;   // ENOTREADY = shape outside the pipelined kernel's domain
  }
  return launch_gemv_stream(x, wq, scales, y, M, N, K, stream);
}

}  // namespace b200
