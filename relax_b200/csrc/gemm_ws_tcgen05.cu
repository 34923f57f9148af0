// Weight-stationary q4f16 matmul on the 5th-generation tensor cores for mid-sized batches
// (16 < M <= 128, and M = 9..16 where it beats the skinny kernel): y[M,N] = x[M,K] . decode(Wq,S)^T.
//
// Decode at batch 16..128 is still bound by streaming the weights once, so the roles of the prefill
// kernel are swapped: the MMA's M dimension is 128 WEIGHT rows (A operand = dequantised weights), its
// N dimension is the batch (B operand = x, 16..128 columns).  A CTA owns 128 weight rows and a slice
// of K; the `ksplit` CTAs of a thread-block cluster that share a row tile add their fp32 partial
// tiles through distributed shared memory in rank order (deterministic), so small N still fills
// the GPU (N = 4096: 32 row tiles x 4 K slices = 128 CTAs) without atomics or a scratch buffer.
//
//   warp 0      TMA producer: x block {64 k, NB batch rows} (128-byte swizzle), packed weights
//               {16 words = 128 k, 128 rows} (64-byte swizzle), scales {8 groups = 256 k, 128 rows}
//   warps 8-15  dequantisers: thread (row, half) turns 4 packed words of one scale group into 32 fp16
//               (exact q-7, one HMUL2 by the scale: the reference's rounding) and stores them as its
//               part of row `row` of the K-major SWIZZLE_128B operand tile
//   warp 1      one thread issues tcgen05.mma kind::f16 (M=128, N=NB, K=16) four times per K block;
//               fp32 accumulator [128 rows x NB] in TMEM
//   warps 4-7   epilogue: tcgen05.ld -> this CTA's partial tile in shared memory; after the cluster
//               barrier CTA r adds up batch columns r, r+ksplit, ... over all ranks and stores fp16
//
// Every mbarrier wait is bounded; a wait that runs out raises a block-wide abort flag and a device
// error word, all loops then run through without waiting (cluster barriers are still reached by
// every thread), TMEM is freed and the kernel ends.
#include <cooperative_groups.h>

#include "internal.h"
#include "q4_common.cuh"
#include "sm100_ptx.cuh"
#include "tmap.h"

namespace b200 {

__device__ int g_gemm_ws_error = 0;

namespace {

namespace cg = cooperative_groups;
using namespace ptx;

constexpr int BR = 128;            // weight rows per tile (UMMA M)
constexpr int BK = 64;             // k per MMA stage (one 128-byte swizzled row of fp16)
constexpr int kMaxNB = 128;        // batch columns (UMMA N), multiple of 16
constexpr int SX = 4;              // x stages
constexpr int SW = 3;              // dequantised-weight stages
constexpr int SR = 3;              // packed-weight stages (128 k each = two K blocks)
constexpr int SS = 2;              // scale stages (256 k each = four K blocks)
constexpr int kWBytes = BR * BK * 2;          // 16384
constexpr int kXBytesMax = kMaxNB * BK * 2;   // 16384
constexpr int kRawBytes = BR * 64;            // 8192: 128 rows x 16 words
constexpr int kScBytes = BR * 16;             // 2048: 128 rows x 8 scales
constexpr int kNumThreads = 512;
constexpr int kDequantWarps = 8;
constexpr uint64_t kWaitNs = 4000000000ull;   // 4 s

struct Smem {
  // all operand buffers are multiples of 1024 bytes, the struct is placed 1024-aligned
  unsigned char w[SW][kWBytes];
  unsigned char x[SX][kXBytesMax];
  unsigned char raw[SR][kRawBytes];
  unsigned char sc[SS][kScBytes];
  float part[kMaxNB * BR];                      // this CTA's partial tile, [batch column][weight row]
  uint64_t x_full[SX], x_empty[SX];
  uint64_t w_full[SW], w_empty[SW];
  uint64_t raw_full[SR], raw_empty[SR];
  uint64_t sc_full[SS], sc_empty[SS];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

struct WsParams {
  CUtensorMap tm_x;    // fp16   {K, M},     box {64, NB},   SWIZZLE_128B
  CUtensorMap tm_w;    // uint32 {K/8, N},   box {16, 128},  SWIZZLE_64B
  CUtensorMap tm_s;    // fp16   {K/32, N},  box {8, 128}
  __half* y;
  int M, N, K;
  int NB;              // batch columns of the MMA: M rounded up to 16
  int ksplit;          // CTAs per cluster = K slices
  int kb_total;        // K / 64
  uint32_t tmem_cols;  // power of two >= max(32, NB)
};

__device__ __forceinline__ void wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (*abort_flag) return;
  if (!mbar_wait_ns(bar, parity, kWaitNs)) {
    *abort_flag = 1;
    atomicExch(&g_gemm_ws_error, code);
  }
}

__global__ void __launch_bounds__(kNumThreads, 1)
q4f16_gemm_ws_tcgen05_kernel(const __grid_constant__ WsParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u));
  volatile int* abort_flag = &sm.abort_flag;
  cg::cluster_group cluster = cg::this_cluster();

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int krank = (int)cluster.block_rank();          // K slice of this CTA (gridDim.x == ksplit)
  const int row0 = blockIdx.y * BR;
  // K blocks of 64, handed out in units of 4 (= one scale stage of 256 k), the first slices one unit longer
  const int units = p.kb_total >> 2;
  const int ubase = units / p.ksplit, uextra = units % p.ksplit;
  const int u0 = krank * ubase + min(krank, uextra);
  const int kb0 = u0 * 4;
  const int num_kb = (ubase + (krank < uextra ? 1 : 0)) * 4;
  const int xbytes = p.NB * BK * 2;

  if (tid == 0) {
    sm.abort_flag = 0;
    for (int i = 0; i < SX; ++i) { mbar_init(&sm.x_full[i], 1); mbar_init(&sm.x_empty[i], 1); }
    for (int i = 0; i < SW; ++i) { mbar_init(&sm.w_full[i], kDequantWarps); mbar_init(&sm.w_empty[i], 1); }
    for (int i = 0; i < SR; ++i) { mbar_init(&sm.raw_full[i], 1); mbar_init(&sm.raw_empty[i], kDequantWarps); }
    for (int i = 0; i < SS; ++i) { mbar_init(&sm.sc_full[i], 1); mbar_init(&sm.sc_empty[i], kDequantWarps); }
    mbar_init(&sm.acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&p.tm_x);
      prefetch_tmap(&p.tm_w);
      prefetch_tmap(&p.tm_s);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int gk = kb0 + kb;                       // global K block
        if ((kb & 3) == 0) {
          const int it = kb >> 2, s = it % SS;
          if (it >= SS) wait_or_abort(&sm.sc_empty[s], ((it / SS) - 1) & 1, abort_flag, 2);
          mbar_arrive_expect_tx(&sm.sc_full[s], kScBytes);
          tma_load_2d(sm.sc[s], &p.tm_s, (gk >> 2) * 8, row0, &sm.sc_full[s]);
        }
        if ((kb & 1) == 0) {
          const int it = kb >> 1, s = it % SR;
          if (it >= SR) wait_or_abort(&sm.raw_empty[s], ((it / SR) - 1) & 1, abort_flag, 3);
          mbar_arrive_expect_tx(&sm.raw_full[s], kRawBytes);
          tma_load_2d(sm.raw[s], &p.tm_w, (gk >> 1) * 16, row0, &sm.raw_full[s]);
        }
        {
          const int s = kb % SX;
          if (kb >= SX) wait_or_abort(&sm.x_empty[s], ((kb / SX) - 1) & 1, abort_flag, 1);
          mbar_arrive_expect_tx(&sm.x_full[s], xbytes);
          tma_load_2d(sm.x[s], &p.tm_x, gk * BK, 0, &sm.x_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16_f32(BR, p.NB);
      for (int kb = 0; kb < num_kb; ++kb) {
        const int sx = kb % SX, sw = kb % SW;
        wait_or_abort(&sm.x_full[sx], (kb / SX) & 1, abort_flag, 5);
        wait_or_abort(&sm.w_full[sw], (kb / SW) & 1, abort_flag, 6);
        tc_fence_after_sync();
        const uint64_t da = umma_desc_k128(smem_u32(sm.w[sw]));
        const uint64_t db = umma_desc_k128(smem_u32(sm.x[sx]));
#pragma unroll
        for (int k16 = 0; k16 < BK / 16; ++k16)
          umma_f16_ss(tmem_base, da + (uint64_t)(2 * k16), db + (uint64_t)(2 * k16), idesc, (kb | k16) != 0);
        umma_commit(&sm.x_empty[sx]);
        umma_commit(&sm.w_empty[sw]);
      }
      umma_commit(&sm.acc_full);
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ epilogue, part 1: TMEM -> this CTA's partial tile
    const int ew = warp - 4;                       // TMEM lane quadrant this warp may read
    wait_or_abort(&sm.acc_full, 0, abort_flag, 7);
    tc_fence_after_sync();
    const int r = ew * 32 + lane;                  // weight row inside the tile = TMEM lane
    const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16);
    for (int c0 = 0; c0 < p.NB; c0 += 32) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(taddr + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 32; ++q)
        if (c0 + q < p.NB) sm.part[(c0 + q) * BR + r] = num_kb > 0 ? __uint_as_float(v[q]) : 0.f;
    }
    tc_fence_before_sync();
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ dequantisers
    const int t = tid - 256;
    const int r = t & 127;                          // weight row inside the tile
    const int half = t >> 7;                        // which 32-k half (= scale group) of each K block
    const int r8 = r & 7;
    const Q4Consts qc = q4_consts();
    uint4 pk[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};   // this thread's words of the two K blocks of a raw stage
    uint32_t sc2[2] = {0, 0};                       // this thread's 4 scales of a scale stage (one per K block)
    for (int kb = 0; kb < num_kb; ++kb) {
      if ((kb & 3) == 0) {
        const int it = kb >> 2, s = it % SS;
        wait_or_abort(&sm.sc_full[s], (it / SS) & 1, abort_flag, 8);
        // row r holds 8 scales (groups of this 256-k span); K block j of the span uses groups 2j, 2j+1
        const __half* srow = reinterpret_cast<const __half*>(sm.sc[s] + r * 16);
        const uint32_t a0 = __half_as_ushort(srow[0 + half]), a1 = __half_as_ushort(srow[2 + half]);
        const uint32_t a2 = __half_as_ushort(srow[4 + half]), a3 = __half_as_ushort(srow[6 + half]);
        sc2[0] = a0 | (a1 << 16);
        sc2[1] = a2 | (a3 << 16);
        pin_loaded(sc2[0]);
        pin_loaded(sc2[1]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.sc_empty[s]);
      }
      if ((kb & 1) == 0) {
        const int it = kb >> 1, s = it % SR;
        wait_or_abort(&sm.raw_full[s], (it / SR) & 1, abort_flag, 9);
        // row r holds 64 bytes = 4 chunks of 16 (chunk c = words 4c..4c+3); 64-byte swizzle: chunk ^= (r >> 1) & 3
        const unsigned char* rr = sm.raw[s] + r * 64;
        const int sx = (r >> 1) & 3;
        pk[0] = *reinterpret_cast<const uint4*>(rr + (((0 + half) ^ sx) << 4));    // K block 0: chunks 0,1
        pk[1] = *reinterpret_cast<const uint4*>(rr + (((2 + half) ^ sx) << 4));    // K block 1: chunks 2,3
        pin_loaded(pk[0]);
        pin_loaded(pk[1]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.raw_empty[s]);
      }
      const int sw = kb % SW;
      if (kb >= SW) wait_or_abort(&sm.w_empty[sw], ((kb / SW) - 1) & 1, abort_flag, 10);
      const uint32_t scw = sc2[(kb >> 1) & 1];
      const __half sch = __ushort_as_half((unsigned short)((kb & 1) ? (scw >> 16) : (scw & 0xffffu)));
      const __half2 s2 = __half2(sch, sch);
      const uint4 words = pk[kb & 1];
      unsigned char* wrow = sm.w[sw] + r * 128;       // 8-row atoms of 1024 B, rows 128 B apart
      const uint32_t wd[4] = {words.x, words.y, words.z, words.w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 o = q4_dequant_natural(wd[c], s2, qc);
        *reinterpret_cast<uint4*>(wrow + (((4 * half + c) ^ r8) << 4)) = o;
      }
      fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core's async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.w_full[sw]);
    }
  }

  // ---------------------------------------------------------------------- sum over the K slices
  cluster.sync();                                    // every CTA's partial tile is complete and visible
  if (warp >= 4 && warp < 8) {
    const int r = (warp - 4) * 32 + lane;
    const int row = row0 + r;
    for (int c = krank; c < p.M; c += p.ksplit) {      // this CTA's batch columns
      float sum = 0.f;
      for (int q = 0; q < p.ksplit; ++q) {
        const float* remote = cluster.map_shared_rank(sm.part, q);
        sum += remote[c * BR + r];
      }
      if (row < p.N) p.y[(int64_t)c * p.N + row] = __float2half_rn(sum);
    }
  }
  cluster.sync();                                    // nobody leaves while a peer still reads its tile

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

}  // namespace

// Returns B200_ENOTREADY when the shape is outside what this kernel takes.
int launch_gemm_ws(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                   int64_t K, cudaStream_t stream) {
  if (M < 1 || M > kMaxNB || K % 256 != 0 || K < 256 || (reinterpret_cast<uintptr_t>(scales) & 15u)) return B200_ENOTREADY;
  WsParams p;
  int rc;
  p.NB = (int)((M + 15) / 16) * 16;
  {
    const uint64_t d[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t s[1] = {(uint64_t)K * 2};
    const uint32_t b[2] = {BK, (uint32_t)p.NB};
    if ((rc = make_tmap(&p.tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }
  {
    const uint64_t d[2] = {(uint64_t)(K / 8), (uint64_t)N};
    const uint64_t s[1] = {(uint64_t)(K / 2)};
    const uint32_t b[2] = {16, BR};
    if ((rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, wq, d, s, b, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
  }
  {
    const uint64_t d[2] = {(uint64_t)(K / 32), (uint64_t)N};
    const uint64_t s[1] = {(uint64_t)(K / 32) * 2};
    const uint32_t b[2] = {8, BR};
    if ((rc = make_tmap(&p.tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, scales, d, s, b, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
  }
  p.y = y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.kb_total = (int)(K / BK);
  p.tmem_cols = p.NB <= 32 ? 32 : (p.NB <= 64 ? 64 : 128);
  const int row_tiles = (int)((N + BR - 1) / BR);
  // K slices: enough CTAs to cover the SMs, at most 8 per cluster, at least one 256-k unit per slice
  const int sms = sm_count();
  int ksplit = 1;
  const int units = p.kb_total / 4;
  while (ksplit < 8 && row_tiles * ksplit * 2 <= sms + sms / 4 && ksplit * 2 <= units) ksplit *= 2;
  if (options().gemm_ws_ksplit > 0) ksplit = (int)options().gemm_ws_ksplit;
  if (ksplit > units) ksplit = units;
  p.ksplit = ksplit;

  const size_t smem = sizeof(Smem) + 1024;
  auto kern = q4f16_gemm_ws_tcgen05_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemm_ws: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ksplit, (unsigned)row_tiles);
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemm_ws launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

int gemm_ws_error_read_and_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_ws_error, sizeof(int)) != cudaSuccess) return 0xff;
  if (v) cudaMemcpyToSymbol(g_gemm_ws_error, &zero, sizeof(int));
  return v & 0xff;
}

}  // namespace b200
