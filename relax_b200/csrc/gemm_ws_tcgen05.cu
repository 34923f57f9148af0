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
constexpr int kMaxStages = 8;
constexpr int kWBytes = BR * BK * 2;          // 16384: one dequantised K block
constexpr int kRawBytes = BR * 64 * 2;        // 16384: 128 rows x 32 words = 256 k = four K blocks
constexpr int kScBytes = BR * 16;             // 2048:  128 rows x 8 scales  = 256 k
constexpr int kNumThreads = 512;
constexpr int kDequantWarps = 8;
constexpr uint64_t kWaitNs = 4000000000ull;   // 4 s

// A single thread sustains only ~2 tiled TMA loads per microsecond whatever their size, so every
// load carries several K blocks (3-D boxes: the K block is the outer coordinate) and the three
// kinds of load are issued by three different warps.
struct WsParams {
  CUtensorMap tm_x;    // fp16   {64, M, K/64},    box {64, NB, XK},   SWIZZLE_128B: [K block][batch row][128 B]
  CUtensorMap tm_w;    // uint32 {16, N, K/128},   box {16, 128, 2},   SWIZZLE_64B:  [128-k half][row][64 B]
  CUtensorMap tm_s;    // fp16   {K/32, N},        box {8, 128}
  __half* y;
  int M, N, K;
  int NB;              // batch columns of the MMA: M rounded up to 16
  int XK;              // K blocks per x load (2 or 4)
  int WK;              // K blocks per dequantised-weight stage (4 or 2): one hand-shake with the MMA thread per stage
  int SX, SW, SR;      // ring depths: x loads, dequantised stages, packed 256-k spans (weights + scales)
  int ksplit;          // CTAs per cluster = K slices
  int kb_total;        // K / 64
  uint32_t tmem_cols;  // power of two >= max(32, NB)
};

struct Bars {
  uint64_t x_full[kMaxStages], x_empty[kMaxStages];
  uint64_t w_full[kMaxStages], w_empty[kMaxStages];
  uint64_t r_full[kMaxStages], r_empty[kMaxStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return;   // completed barrier: no read of the flag on the fast path
  if (*abort_flag) return;
  if (!mbar_wait_ns(bar, parity, kWaitNs)) {
    *abort_flag = 1;
    atomicExch(&g_gemm_ws_error, code);
  }
}

// Same for the roles that are off the critical path (TMA producers, epilogue warps): they sleep
// between polls, so their polling does not take issue slots from the dequantisers.
__device__ __forceinline__ void wait_or_abort_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (*abort_flag) return;
  if (!mbar_wait_ns_relaxed(bar, parity, kWaitNs)) {
    *abort_flag = 1;
    atomicExch(&g_gemm_ws_error, code);
  }
}

// Position in a ring of `n` stages without divisions (the ring depths are run-time values and a
// single issuing thread cannot afford integer divisions per K block): stage index + wrap parity.
struct Ring {
  int s = 0;
  uint32_t phase = 0;      // number of completed wraps, mod 2
  bool wrapped = false;    // at least one wrap so far
  __device__ __forceinline__ void next(int n) {
    if (++s == n) { s = 0; phase ^= 1; wrapped = true; }
  }
};

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int32_t c0, int32_t c1, int32_t c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Shared memory (1024-aligned base): x ring [SX][XK][NB][128 B] | w ring [SW][WK][16 KB] | raw ring [SR][16 KB]
// | scale ring [SR][2 KB] | barriers.  After the main loop the x ring is reused for this CTA's
// partial tile [batch column][weight row] fp32 (NB * 512 B <= SX * XK * NB * 128 B since XK >= 2, SX >= 2).
__global__ void __launch_bounds__(kNumThreads, 1)
q4f16_gemm_ws_tcgen05_kernel(const __grid_constant__ WsParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* base = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  const int xstage = p.XK * p.NB * 128;
  unsigned char* x_ring = base;
  unsigned char* w_ring = x_ring + (size_t)p.SX * xstage;
  const int wstage = p.WK * kWBytes;
  unsigned char* raw_ring = w_ring + (size_t)p.SW * wstage;
  unsigned char* sc_ring = raw_ring + (size_t)p.SR * kRawBytes;
  Bars& bar = *reinterpret_cast<Bars*>(sc_ring + (size_t)p.SR * kScBytes);
  float* part = reinterpret_cast<float*>(x_ring);
  volatile int* abort_flag = &bar.abort_flag;
  cg::cluster_group cluster = cg::this_cluster();

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int krank = (int)cluster.block_rank();          // K slice of this CTA (gridDim.x == ksplit)
  const int row0 = blockIdx.y * BR;
  // K blocks of 64, handed out in units of 4 (= one 256-k span), the first slices one unit longer
  const int units = p.kb_total >> 2;
  const int ubase = units / p.ksplit, uextra = units % p.ksplit;
  const int u0 = krank * ubase + min(krank, uextra);
  const int kb0 = u0 * 4;
  const int num_kb = (ubase + (krank < uextra ? 1 : 0)) * 4;

  if (tid == 0) {
    bar.abort_flag = 0;
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bar.x_full[i], 1); mbar_init(&bar.x_empty[i], 1);
      mbar_init(&bar.w_full[i], kDequantWarps); mbar_init(&bar.w_empty[i], 1);
      mbar_init(&bar.r_full[i], 2); mbar_init(&bar.r_empty[i], kDequantWarps);
    }
    mbar_init(&bar.acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar.tmem_base, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bar.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer: x (XK K blocks per load)
    if (lane == 0) {
      prefetch_tmap(&p.tm_x);
      Ring rx;
      for (int kb = 0; kb < num_kb; kb += p.XK, rx.next(p.SX)) {
        if (rx.wrapped) wait_or_abort_relaxed(&bar.x_empty[rx.s], rx.phase ^ 1, abort_flag, 1);
        mbar_arrive_expect_tx(&bar.x_full[rx.s], xstage);
        tma_load_3d(x_ring + (size_t)rx.s * xstage, &p.tm_x, 0, 0, kb0 + kb, &bar.x_full[rx.s]);
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ TMA producers: packed weights (warp 2), scales (warp 3), 256 k per load
    if (lane == 0) {
      prefetch_tmap(warp == 2 ? &p.tm_w : &p.tm_s);
      Ring rr;
      for (int kb = 0; kb < num_kb; kb += 4, rr.next(p.SR)) {
        const int s = rr.s;
        const int gk = kb0 + kb;
        if (rr.wrapped) wait_or_abort_relaxed(&bar.r_empty[s], rr.phase ^ 1, abort_flag, 3);
        if (warp == 2) {
          mbar_arrive_expect_tx(&bar.r_full[s], kRawBytes);
          tma_load_3d(raw_ring + (size_t)s * kRawBytes, &p.tm_w, 0, row0, gk >> 1, &bar.r_full[s]);
        } else {
          mbar_arrive_expect_tx(&bar.r_full[s], kScBytes);
          tma_load_2d(sc_ring + (size_t)s * kScBytes, &p.tm_s, (gk >> 2) * 8, row0, &bar.r_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16_f32(BR, p.NB);
      // The issuing thread is the pace-maker when the batch is narrow (an MMA of N = 16 is short):
      // one wait and one commit per stage of WK K blocks, descriptors advanced by constants.
      Ring rx, rw;
      int xslab = 0;
      uint32_t first = 0;                               // 0 until the first MMA has been issued
      for (int kb = 0; kb < num_kb; kb += p.WK, rw.next(p.SW)) {
        wait_or_abort(&bar.w_full[rw.s], rw.phase, abort_flag, 6);
        uint64_t da = umma_desc_k128(smem_u32(w_ring + (size_t)rw.s * wstage));
        for (int j = 0; j < p.WK; ++j, da += (uint64_t)(kWBytes >> 4)) {
          if (xslab == 0) wait_or_abort(&bar.x_full[rx.s], rx.phase, abort_flag, 5);
          tc_fence_after_sync();
          const uint64_t db = umma_desc_k128(smem_u32(x_ring + (size_t)rx.s * xstage + (size_t)xslab * p.NB * 128));
          umma_f16_ss(tmem_base, da, db, idesc, first);
          first = 1;
          umma_f16_ss(tmem_base, da + 2, db + 2, idesc, 1);
          umma_f16_ss(tmem_base, da + 4, db + 4, idesc, 1);
          umma_f16_ss(tmem_base, da + 6, db + 6, idesc, 1);
          if (++xslab == p.XK) {
            umma_commit(&bar.x_empty[rx.s]);
            xslab = 0;
            rx.next(p.SX);
          }
        }
        umma_commit(&bar.w_empty[rw.s]);
      }
      umma_commit(&bar.acc_full);
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ dequantisers
    const int t = tid - 256;
    const int r = t & 127;                          // weight row inside the tile
    const int half = t >> 7;                        // which 32-k half (= scale group) of each K block
    const int r8 = r & 7;
    const int sx64 = (r >> 1) & 3;                  // 64-byte swizzle phase of row r
    const Q4Consts qc = q4_consts();
    Ring rr, rw;
    for (int it = 0; it * 4 < num_kb; ++it, rr.next(p.SR)) {
      const int s = rr.s;
      wait_or_abort(&bar.r_full[s], rr.phase, abort_flag, 8);
      // this thread's share of the 256-k span: one 16-byte chunk (4 words = one scale group) and
      // one scale per K block.  Span layout: [128-k half h2][row][64 B]; K block j = half j>>1,
      // chunks 2*(j&1), 2*(j&1)+1 of the row; scales: row r holds groups 0..7, K block j uses 2j, 2j+1.
      uint4 pk[4];
      uint32_t scb[4];
      const unsigned char* rbase = raw_ring + (size_t)s * kRawBytes + r * 64;
      const __half* srow = reinterpret_cast<const __half*>(sc_ring + (size_t)s * kScBytes + r * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pk[j] = *reinterpret_cast<const uint4*>(rbase + (j >> 1) * (BR * 64) + (((2 * (j & 1) + half) ^ sx64) << 4));
        scb[j] = __half_as_ushort(srow[2 * j + half]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pin_loaded(pk[j]);
        pin_loaded(scb[j]);
      }
      fence_proxy_async_smem();              // generic reads ordered before the TMA refill (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.r_empty[s]);
      // one dequantised stage = WK K blocks: one wait, one proxy fence and one arrival per stage
      for (int j0 = 0; j0 < 4; j0 += p.WK, rw.next(p.SW)) {
        if (rw.wrapped) wait_or_abort(&bar.w_empty[rw.s], rw.phase ^ 1, abort_flag, 10);
        unsigned char* wst = w_ring + (size_t)rw.s * wstage + r * 128;     // 8-row atoms of 1024 B, rows 128 B apart
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < j0 || j >= j0 + p.WK) continue;
          const __half sch = __ushort_as_half((unsigned short)scb[j]);
          const __half2 s2 = __half2(sch, sch);
          unsigned char* wrow = wst + (j - j0) * kWBytes;
          const uint32_t wd[4] = {pk[j].x, pk[j].y, pk[j].z, pk[j].w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 o = q4_dequant_natural(wd[c], s2, qc);
            *reinterpret_cast<uint4*>(wrow + (((4 * half + c) ^ r8) << 4)) = o;
          }
        }
        fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar.w_full[rw.s]);
      }
    }
  }

  // ---------------------------------------------------------------------- TMEM -> this CTA's partial tile
  if (warp >= 4 && warp < 8) {
    const int ew = warp - 4;                       // TMEM lane quadrant this warp may read
    // acc_full is committed after every MMA (and with it every read of the x ring) has completed,
    // so the x ring may now be overwritten with the partial tile
    wait_or_abort_relaxed(&bar.acc_full, 0, abort_flag, 7);
    tc_fence_after_sync();
    const int r = ew * 32 + lane;                  // weight row inside the tile = TMEM lane
    const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16);
    for (int c0 = 0; c0 < p.NB; c0 += 32) {
      uint32_t v[32];
      tmem_ld_32x32b_x32(taddr + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 32; ++q)
        if (c0 + q < p.NB) part[(c0 + q) * BR + r] = num_kb > 0 ? __uint_as_float(v[q]) : 0.f;
    }
    tc_fence_before_sync();
  }

  // ---------------------------------------------------------------------- sum over the K slices
  cluster.sync();                                    // every CTA's partial tile is complete and visible
  if (warp >= 4 && warp < 8) {
    const int r = (warp - 4) * 32 + lane;
    const int row = row0 + r;
    for (int c = krank; c < p.M; c += p.ksplit) {      // this CTA's batch columns
      float sum = 0.f;
      for (int q = 0; q < p.ksplit; ++q) {
        const float* remote = cluster.map_shared_rank(part, q);
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
  p.XK = p.NB <= 64 ? 4 : 2;
  {
    const uint64_t d[3] = {BK, (uint64_t)M, (uint64_t)(K / BK)};
    const uint64_t s[2] = {(uint64_t)K * 2, BK * 2};
    const uint32_t b[3] = {BK, (uint32_t)p.NB, (uint32_t)p.XK};
    if ((rc = make_tmap(&p.tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, x, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }
  {
    const uint64_t d[3] = {16, (uint64_t)N, (uint64_t)(K / 128)};
    const uint64_t s[2] = {(uint64_t)(K / 2), 64};
    const uint32_t b[3] = {16, BR, 2};
    if ((rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, wq, d, s, b, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
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

  // ring depths: the dequantised ring gets what the x ring and the packed ring leave
  p.WK = p.NB <= 16 ? 4 : 2;
  p.SX = p.NB <= 64 ? 3 : 2;
  p.SR = p.NB <= 64 ? 3 : 2;
  const size_t xstage = (size_t)p.XK * p.NB * 128;
  const size_t wstage = (size_t)p.WK * kWBytes;
  const size_t fixed = 1024 + p.SX * xstage + p.SR * (size_t)(kRawBytes + kScBytes) + sizeof(Bars) + 256;
  int sw = (int)((227 * 1024 - fixed) / wstage);
  if (sw > 4) sw = 4;
  if (sw < 2) return B200_ENOTREADY;
  p.SW = sw;
  const size_t smem = fixed + (size_t)p.SW * wstage;
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
