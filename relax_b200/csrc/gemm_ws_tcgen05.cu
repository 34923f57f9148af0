// Weight-stationary q4f16 matmul on the 5th-generation tensor cores for mid-sized batches
// (M <= 128; the dispatcher gives it 17..128 rows, and 9..16 where it beats the skinny kernel):
// y[M,N] = x[M,K] . decode(Wq,S)^T.
//
// Decode at batch 16..128 is still bound by streaming the weights once, so the roles of the prefill
// kernel are swapped: the MMA's M dimension is 128 WEIGHT rows (A operand = dequantised weights), its
// N dimension is the batch (B operand = x, 16..128 columns).  A CTA owns 128 weight rows and a slice
// of K; the `ksplit` CTAs of a thread-block cluster that share a row tile add their fp32 partial
// tiles through distributed shared memory in rank order (deterministic), so small N still fills
// the GPU (N = 4096: 32 row tiles x 4 K slices = 128 CTAs) without atomics or a scratch buffer.
//
//   warps 0,2,3 TMA producers: x (WK K blocks of {64 k, NB batch rows} per load, 128-byte swizzle), packed
//               weights (256 k per load: whole 128-byte lines of 128 rows, 128-byte swizzle), scales
//               {8 groups = 256 k, 128 rows}; the first ring-full of weights is requested during set-up
//   warps 8-23  dequantisers, two groups of 8 warps that take alternate 256-k spans (a group's load ->
//               convert -> store -> fence -> arrive chain is latency bound; two chains in flight double
//               the rate): thread (row, half) turns 4 packed words of one scale group into 32 fp16
//               (exact q-7, one HMUL2 by the scale: the reference's rounding) and stores them as its
//               part of row `row` of the K-major SWIZZLE_128B operand tile
//   warp 1      one thread issues tcgen05.mma kind::f16 (M=128, N=NB, K=16) four times per K block;
//               fp32 accumulator [128 rows x NB] in TMEM.  An MMA of N <= 128 takes 60-64 clocks, so this
//               thread has about 250 clocks per K block: its loop is kept to a few dozen instructions
//               (one wait each on the weight and the x stage per WK K blocks, descriptors advanced by
//               32-bit adds, ring cursors without divisions); a lone thread runs some 10-15 clocks per
//               instruction, and a longer loop is what the whole kernel then waits for
//   warps 4-7   epilogue: tcgen05.ld -> this CTA's partial tile in shared memory; after the cluster
//               barrier CTA r adds up batch columns r, r+ksplit, ... over all ranks (every thread of
//               the CTA takes part, all of a column's remote loads in flight together) and stores fp16
//
// Launched with programmatic dependent launch: set-up and the weight loads run ahead of the previous
// kernel's end; the loads of x and the stores of y wait for it.
//
// Every mbarrier wait is bounded; a wait that runs out raises a block-wide abort flag and a device
// error word, all loops then run through without waiting (cluster barriers are still reached by
// every thread), TMEM is freed and the kernel ends.
#include <cooperative_groups.h>

#include <type_traits>

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
constexpr int kRawBytes = BR * 128;           // 16384: 128 rows x 32 words = 256 k = four K blocks, one 128-byte line per row
constexpr int kScBytes = BR * 16;             // 2048:  128 rows x 8 scales  = 256 k
constexpr int kDequantWarps = 8;           // per group
constexpr int kDequantGroups = 2;          // alternate 256-k spans
constexpr int kNumThreads = 256 + kDequantGroups * kDequantWarps * 32;   // 768
constexpr uint64_t kWaitNs = 4000000000ull;   // 4 s

// A single thread sustains only ~2 tiled TMA loads per microsecond whatever their size, so every
// load carries several K blocks (3-D boxes: the K block is the outer coordinate) and the three
// kinds of load are issued by three different warps.
struct WsParams {
  CUtensorMap tm_x;    // fp16   {64, M, K/64},    box {64, NB, WK},   SWIZZLE_128B: [K block][batch row][128 B]
  CUtensorMap tm_w;    // uint32 {K/8, N},         box {32, 128},      SWIZZLE_128B: [row][128 B] (whole lines: 64-byte pieces
                       //                                                    halve the rate the weights arrive at)
  CUtensorMap tm_s;    // fp16   {K/32, N},        box {8, 128}
  __half* y;
  int M, N, K;
  int NB;              // batch columns of the MMA: M rounded up to 16
  int WK;              // K blocks per stage of the x ring and of the dequantised-weight ring (4 or 2): the kernel's template value
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

// Shared memory (1024-aligned base): x ring [SX][WK][NB][128 B] | w ring [SW][WK][16 KB] | raw ring [SR][16 KB]
// | scale ring [SR][2 KB] | barriers.  After the main loop the x ring is reused for this CTA's
// partial tile [batch column][weight row] fp32 (NB * 512 B <= SX * WK * NB * 128 B since SX * WK >= 4).
// WK: K blocks per stage of the x ring and of the dequantised ring (2 or 4).  PAIRED: nibble order of the packed
// words (q4_common.cuh).
template <int WK, bool PAIRED>
__global__ void __launch_bounds__(kNumThreads, 1)
q4f16_gemm_ws_tcgen05_kernel(const __grid_constant__ WsParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* base = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  const int xstage = WK * p.NB * 128;
  unsigned char* x_ring = base;
  unsigned char* w_ring = x_ring + (size_t)p.SX * xstage;
  constexpr int wstage = WK * kWBytes;
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

  const int nspans = num_kb >> 2;
  if (tid == 0) {
    bar.abort_flag = 0;
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(&bar.x_full[i], 1); mbar_init(&bar.x_empty[i], 1);
      mbar_init(&bar.w_full[i], kDequantWarps); mbar_init(&bar.w_empty[i], 1);
    }
    mbar_init(&bar.acc_full, 1);
    mbar_fence_init();
  }
  if (tid == 64) {
    // The weights depend on nothing: the thread that will stream them sets up the packed ring's barriers itself
    // and fills the ring at once, ahead of the rest of the set-up (barriers, TMEM allocation, the block-wide sync).
    for (int i = 0; i < kMaxStages; ++i) { mbar_init(&bar.r_full[i], 2); mbar_init(&bar.r_empty[i], kDequantWarps); }
    mbar_fence_init();
    for (int i = 0; i < p.SR && i < nspans; ++i) {
      const int gk = kb0 + 4 * i;
      mbar_arrive_expect_tx(&bar.r_full[i], kRawBytes);
      tma_load_2d(raw_ring + (size_t)i * kRawBytes, &p.tm_w, (gk >> 2) * 32, row0, &bar.r_full[i]);
      mbar_arrive_expect_tx(&bar.r_full[i], kScBytes);
      tma_load_2d(sc_ring + (size_t)i * kScBytes, &p.tm_s, (gk >> 2) * 8, row0, &bar.r_full[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc(&bar.tmem_base, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bar.tmem_base;
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer: x (WK K blocks per load)
    if (lane == 0) {
      prefetch_tmap(&p.tm_x);
      pdl_wait();                                     // x may be the previous kernel's output
      Ring rx;
      for (int kb = 0; kb < num_kb; kb += WK, rx.next(p.SX)) {
        // (not the sleeping wait: a nanosleep lasts far longer than the time a stage takes, and a ring of two or
        // three stages then runs at the pace of the sleeps)
        if (rx.wrapped) wait_or_abort(&bar.x_empty[rx.s], rx.phase ^ 1, abort_flag, 1);
        mbar_arrive_expect_tx(&bar.x_full[rx.s], xstage);
        tma_load_3d(x_ring + (size_t)rx.s * xstage, &p.tm_x, 0, 0, kb0 + kb, &bar.x_full[rx.s]);
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ TMA producers: packed weights (warp 2), scales (warp 3), 256 k per load
    if (lane == 0) {
      // the first SR spans were requested during set-up: the cursor starts one trip round the ring later
      Ring rr;
      rr.phase = 1;
      rr.wrapped = true;
      for (int kb = 4 * p.SR; kb < num_kb; kb += 4, rr.next(p.SR)) {
        const int s = rr.s;
        const int gk = kb0 + kb;
        if (rr.wrapped) wait_or_abort(&bar.r_empty[s], rr.phase ^ 1, abort_flag, 3);
        if (warp == 2) {
          mbar_arrive_expect_tx(&bar.r_full[s], kRawBytes);
          tma_load_2d(raw_ring + (size_t)s * kRawBytes, &p.tm_w, (gk >> 2) * 32, row0, &bar.r_full[s]);
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
      // descriptor = constant fields | (shared-memory address >> 4) in bits 0-13: stepping through the rings
      // adds to the low word only (every address is below 256 KB, so nothing carries out of the field)
      const uint64_t dconst = umma_desc_k128(0);
      const uint32_t a0 = (smem_u32(w_ring) & 0x3FFFFu) >> 4, b0 = (smem_u32(x_ring) & 0x3FFFFu) >> 4;
      const uint32_t a_step = (uint32_t)wstage >> 4, b_step = (uint32_t)xstage >> 4, b_kb = (uint32_t)(p.NB * 128) >> 4;
      const uint32_t SW = (uint32_t)p.SW, SX = (uint32_t)p.SX;
      uint32_t ws = 0, wphase = 0, xs = 0, xphase = 0;
      // The issue of a tcgen05.mma holds this thread until the tensor core takes it (the time of the loop and
      // the time of the MMAs add up, measured), and a lone thread spends 10-15 clocks per instruction, more on a
      // taken branch: the loop is straight-line code, one branch for both waits, cursors advanced by selects.
      auto stage = [&](uint32_t acc_first) {
        uint64_t* wf = &bar.w_full[ws];
        uint64_t* xf = &bar.x_full[xs];
        const bool ready = mbar_try_wait(wf, wphase) & mbar_try_wait(xf, xphase);
        if (!ready) {
          wait_or_abort(wf, wphase, abort_flag, 6);
          wait_or_abort(xf, xphase, abort_flag, 5);
        }
        tc_fence_after_sync();
        const uint64_t da = dconst | (uint64_t)(a0 + ws * a_step);
        const uint64_t db = dconst | (uint64_t)(b0 + xs * b_step);
#pragma unroll
        for (int j = 0; j < WK; ++j) {
#pragma unroll
          for (int k16 = 0; k16 < 4; ++k16) {
            // +16 k inside the swizzled 128-byte row = +32 bytes = +2 in the descriptor's 16-byte units
            umma_f16_ss(tmem_base, da + (uint64_t)(j * (kWBytes >> 4) + 2 * k16), db + (uint64_t)(j * b_kb + 2 * k16), idesc,
                        (j | k16) == 0 ? acc_first : 1u);
          }
        }
        umma_commit(&bar.x_empty[xs]);
        umma_commit(&bar.w_empty[ws]);
        ws = ws + 1 == SW ? 0 : ws + 1;
        wphase ^= (uint32_t)(ws == 0);
        xs = xs + 1 == SX ? 0 : xs + 1;
        xphase ^= (uint32_t)(xs == 0);
      };
      if (num_kb > 0) stage(0);
      for (int kb = WK; kb < num_kb; kb += WK) stage(1);
      umma_commit(&bar.acc_full);
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ dequantisers
    const int t = (tid - 256) & 255;
    const int grp = (tid - 256) >> 8;               // this group converts the spans whose index is grp mod 2
    const int r = t & 127;                          // weight row inside the tile
    const int half = t >> 7;                        // which 32-k half (= scale group) of each K block
    const int r8 = r & 7;
    const Q4Consts qc = q4_consts();
    Ring rr, rw;
    for (int it = 0; it * 4 < num_kb; ++it, rr.next(p.SR)) {
      if ((it & 1) != grp) {                        // the other group's span: keep the ring cursors in step
#pragma unroll
        for (int j0 = 0; j0 < 4; j0 += WK) rw.next(p.SW);
        continue;
      }
      const int s = rr.s;
      wait_or_abort(&bar.r_full[s], rr.phase, abort_flag, 8);
      // this thread's share of the 256-k span: one 16-byte chunk (4 words = one scale group) and
      // one scale per K block.  Span layout: [128-k half h2][row][64 B]; K block j = half j>>1,
      // chunks 2*(j&1), 2*(j&1)+1 of the row; scales: row r holds groups 0..7, K block j uses 2j, 2j+1.
      uint4 pk[4];
      uint32_t scb[4];
      const unsigned char* rbase = raw_ring + (size_t)s * kRawBytes + r * 128;
      const __half* srow = reinterpret_cast<const __half*>(sc_ring + (size_t)s * kScBytes + r * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        pk[j] = *reinterpret_cast<const uint4*>(rbase + (((2 * j + half) ^ r8) << 4));   // 128-byte swizzle: chunk ^ (row % 8)
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
#pragma unroll
      for (int j0 = 0; j0 < 4; j0 += WK, rw.next(p.SW)) {
        if (rw.wrapped) wait_or_abort(&bar.w_empty[rw.s], rw.phase ^ 1, abort_flag, 10);
        unsigned char* wst = w_ring + (size_t)rw.s * wstage + r * 128;     // 8-row atoms of 1024 B, rows 128 B apart
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < j0 || j >= j0 + WK) continue;
          const __half sch = __ushort_as_half((unsigned short)scb[j]);
          const __half2 s2 = __half2(sch, sch);
          unsigned char* wrow = wst + (j - j0) * kWBytes;
          const uint32_t wd[4] = {pk[j].x, pk[j].y, pk[j].z, pk[j].w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 o = q4_dequant_ordered<PAIRED>(wd[c], s2, qc);
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
  pdl_wait();                                        // y may still be read by the previous kernel
  {
    // This CTA's batch columns are krank, krank + ksplit, ...  A work item is (column, four consecutive weight
    // rows): one 16-byte load per rank, all of a thread's loads in flight together; a warp covers a column's 128
    // rows.  The ranks are added in rank order whatever the unrolling: deterministic.
    const int ncols = p.M > krank ? (p.M - krank + p.ksplit - 1) / p.ksplit : 0;
    const bool vec_store = (p.N & 3) == 0;
    auto item = [&](auto ks_tag, int c, int rg) {
      constexpr int KS = decltype(ks_tag)::value;
      float4 v[KS];
#pragma unroll
      for (int q = 0; q < KS; ++q) v[q] = *reinterpret_cast<const float4*>(cluster.map_shared_rank(part, q) + c * BR + rg * 4);
      float4 sum = v[0];
#pragma unroll
      for (int q = 1; q < KS; ++q) { sum.x += v[q].x; sum.y += v[q].y; sum.z += v[q].z; sum.w += v[q].w; }
      const int row = row0 + rg * 4;
      __half* dst = p.y + (int64_t)c * p.N + row;
      if (vec_store && row + 4 <= p.N) {
        uint2 o;
        o.x = h2_as_u32(__floats2half2_rn(sum.x, sum.y));
        o.y = h2_as_u32(__floats2half2_rn(sum.z, sum.w));
        *reinterpret_cast<uint2*>(dst) = o;
      } else {
        if (row + 0 < p.N) dst[0] = __float2half_rn(sum.x);
        if (row + 1 < p.N) dst[1] = __float2half_rn(sum.y);
        if (row + 2 < p.N) dst[2] = __float2half_rn(sum.z);
        if (row + 3 < p.N) dst[3] = __float2half_rn(sum.w);
      }
    };
    for (int it = tid; it < ncols * 32; it += kNumThreads) {
      const int c = krank + (it >> 5) * p.ksplit, rg = it & 31;
      switch (p.ksplit) {
        case 1: item(std::integral_constant<int, 1>{}, c, rg); break;
        case 2: item(std::integral_constant<int, 2>{}, c, rg); break;
        case 4: item(std::integral_constant<int, 4>{}, c, rg); break;
        case 8: item(std::integral_constant<int, 8>{}, c, rg); break;
        default: {                                   // a K with fewer 256-k units than the next power of two
          float sum[4] = {0.f, 0.f, 0.f, 0.f};
          for (int q = 0; q < p.ksplit; ++q) {
            const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(part, q) + c * BR + rg * 4);
            sum[0] += v.x; sum[1] += v.y; sum[2] += v.z; sum[3] += v.w;
          }
          for (int i = 0; i < 4; ++i)
            if (row0 + rg * 4 + i < p.N) p.y[(int64_t)c * p.N + row0 + rg * 4 + i] = __float2half_rn(sum[i]);
        }
      }
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
  // K blocks per stage: a whole 256-k span for a narrow batch (x stages are small), half a span otherwise
  p.WK = p.NB <= 32 ? 4 : 2;
  if (options().gemm_ws_xk == 2 || options().gemm_ws_xk == 4) p.WK = (int)options().gemm_ws_xk;
  {
    const uint64_t d[3] = {BK, (uint64_t)M, (uint64_t)(K / BK)};
    const uint64_t s[2] = {(uint64_t)K * 2, BK * 2};
    const uint32_t b[3] = {BK, (uint32_t)p.NB, (uint32_t)p.WK};
    if ((rc = make_tmap(&p.tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, x, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }
  {
    const uint64_t d[2] = {(uint64_t)(K / 8), (uint64_t)N};
    const uint64_t s[1] = {(uint64_t)(K / 2)};
    const uint32_t b[2] = {32, BR};
    if ((rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, wq, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
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

  // Ring depths.  Dequantised ring: its minimum.  At least one stage more than a span holds (P = 4 / WK
  // stages): the two dequantiser groups share the ring's slots; a group that starts stage n has last waited for
  // the consumption of stage n - P - 1 - SW, and its parity wait on w_empty for stage n - SW is only
  // unambiguous if stage n - 2 SW is known to be consumed: n - P - 1 - SW >= n - 2 SW, i.e. SW >= P + 1 (a
  // shallower ring lets a group run two phases ahead of a barrier, pass the wait at once and overwrite a stage
  // that is still being read).  x ring: enough for the partial tile that reuses it (SX * WK >= 4) and for the L2
  // latency.  Packed ring: the rest (even, see below); its depth is the number of 18 KB requests an SM keeps in
  // flight to HBM.
  const int sw_min = 4 / p.WK + 1;
  p.SW = options().gemm_ws_w_stages > sw_min ? (int)options().gemm_ws_w_stages : sw_min;
  p.SX = p.NB <= 64 ? 3 : 2;
  if (options().gemm_ws_x_stages > 0) p.SX = (int)options().gemm_ws_x_stages;
  if (p.SX * p.WK < 4) p.SX = 4 / p.WK;
  const size_t xstage = (size_t)p.WK * p.NB * 128;
  const size_t wstage = (size_t)p.WK * kWBytes;
  const size_t others = 1024 + p.SX * xstage + p.SW * wstage + sizeof(Bars) + 256;
  const size_t cap = 227 * 1024;
  if (p.SX > kMaxStages || p.SW > kMaxStages || others + 2 * (size_t)(kRawBytes + kScBytes) > cap) return B200_ENOTREADY;
  int sr = (int)((cap - others) / (kRawBytes + kScBytes));
  if (sr > kMaxStages) sr = kMaxStages;
  if (options().gemm_ws_r_stages >= 2 && options().gemm_ws_r_stages < sr) sr = (int)options().gemm_ws_r_stages;
  // An even depth: the two dequantiser groups take alternate spans, so every slot of the ring then belongs to one
  // group, which waits for a slot's next load only after it has consumed the previous one itself (with an odd
  // depth the groups would share slots, and a load that completes out of order could let a group's parity wait
  // pass one phase early).
  sr &= ~1;
  if (sr < 2) return B200_ENOTREADY;
  p.SR = sr;
  const size_t fixed = 1024 + p.SX * xstage + p.SR * (size_t)(kRawBytes + kScBytes) + sizeof(Bars) + 256;
  const size_t smem = fixed + (size_t)p.SW * wstage;
  const bool paired = current_layout() == kLayoutPaired;
  auto kern = p.WK == 4 ? (paired ? q4f16_gemm_ws_tcgen05_kernel<4, true> : q4f16_gemm_ws_tcgen05_kernel<4, false>)
                        : (paired ? q4f16_gemm_ws_tcgen05_kernel<2, true> : q4f16_gemm_ws_tcgen05_kernel<2, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemm_ws: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ksplit, (unsigned)row_tiles);
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ksplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 2 : 1;
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
