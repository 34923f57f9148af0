// Prefill q4f16 matmul on the 5th-generation tensor cores: y[M,N] = x[M,K] . decode(Wq,S)^T.
//
// Replaces the fused decode+matmul+astype PrimFunc of the reference for large M (reference:
// python/tvm/relax/transform/legalize_ops.py:203-264 for the matmul semantics; its own GPU
// route would be a MetaSchedule-tuned mma.sync kernel, src/relax/transform/meta_schedule.cc).
// Tensor-core bound: 2*M*N*K flop against N*K/2 bytes of weights.
//
// One persistent CTA per SM, output tile 256 tokens x 256 weight rows, K in blocks of 64.  The
// tile is two 128-token halves that share every dequantised weight block: the int4 -> fp16
// conversion runs on the CUDA cores at roughly the rate one 128x256 MMA stream consumes it, so
// each converted block has to feed two of them for the tensor pipe to be the limit.
//
//   warp 0      TMA producer for x: box {64 k, 256 rows} fp16, 128-byte swizzle -> ring A
//               (rows 0-127 and 128-255 of the box are the two halves' A operands)
//   warp 2      TMA producer for the packed weights (box {16 words = 128 k, 256 rows}, 64-byte
//               swizzle) -> ring RAW.  The scales (16 bytes per row and 256 k) are read straight from
//               global memory by the dequantisers, one span ahead: that leaves room for a third
//               stage of the dequantised operand.
//   warps 8-23  dequantisers (two groups of 8 warps on alternate K blocks): thread r owns weight row r of the tile.  Per K block it turns 8
//               packed words into 64 fp16 (exact q-7, one HMUL2 by the scale: the reference's
//               rounding) and stores them as the 128-byte row r of the UMMA operand tile, chunk
//               c at position c ^ (r % 8): the canonical K-major SWIZZLE_128B layout a TMA load
//               would have produced -> ring B (generic-proxy stores, fence.proxy.async, mbarrier)
//   warp 1      MMA issuer: one thread issues tcgen05.mma.cta_group::1.kind::f16 (M=128, N=256,
//               K=16) four times per K block and half, A and B from shared-memory descriptors,
//               fp32 accumulators in TMEM (all 512 columns: 256 per half); tcgen05.commit hands
//               the A and B stages back and, after the last K block, publishes each half.
//   warps 4-7, 24-27  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, fp32 -> fp16 (RN),
//               16-byte global stores into row-major y; a warp reads the TMEM lane quadrant
//               (warp & 3), warps 4-7 take columns 0..127 of a half and warps 24-27 columns 128..255.
//               The halves are drained in order and handed back one by one, so the next tile's
//               MMAs on half 0 start while half 1 is still drained.
//
// Out-of-range rows (M, N tails) and columns (K tail) are zero-filled by the TMA unit: a zero
// scale makes the weight +-0, a zero x makes the product 0, the epilogue skips them.
// Every mbarrier wait is bounded; a wait that runs out raises a block-wide abort flag and a
// device error word, all loops then run through without waiting, TMEM is freed and the kernel ends.
#include "internal.h"
#include "q4_common.cuh"
#include "sm100_ptx.cuh"
#include "tmap.h"

namespace b200 {

__device__ int g_gemm_error = 0;

namespace {

using namespace ptx;

constexpr int BM = 128;            // tokens per half tile (UMMA M)
constexpr int BMT = 2 * BM;        // tokens per tile: two halves share each dequantised weight block
constexpr int BN = 256;            // weight rows per tile (UMMA N)
constexpr int BK = 64;             // k per MMA stage (one 128-byte swizzled row of fp16)
constexpr int SA = 3;              // x stages
constexpr int SB = 3;              // dequantised-weight stages (the conversion of a K block runs ahead of the MMA of the one before)
constexpr int SR = 2;              // packed-weight stages (128 k each = two K blocks)
constexpr int kABytes = BMT * BK * 2;         // 32768: half h at +h*16384
constexpr int kBBytes = BN * BK * 2;          // 32768
constexpr int kRawBytes = BN * 64;            // 16384: 256 rows x 16 words
constexpr int kScBytes = BN * 16;             // 4096:  256 rows x 8 scales
constexpr int kDequantWarps = 8;          // per group; two groups take alternate K blocks
constexpr int kDequantGroups = 2;
constexpr int kNumThreads = 256 + kDequantGroups * kDequantWarps * 32 + 128;   // 896: warps 24-27 are a second set of epilogue warps
constexpr uint32_t kTmemCols = 512;
constexpr uint64_t kWaitNs = 4000000000ull;   // 4 s

struct Smem {
  // all operand buffers are multiples of 1024 bytes, the struct is placed 1024-aligned
  unsigned char a[SA][kABytes];
  unsigned char b[SB][kBBytes];
  unsigned char raw[SR][kRawBytes];
  // The x ring and the dequantised ring advance one stage per K block in lock step (same depth), so stage s of
  // both shares one pair of barriers: `full` collects the x load's bytes and the dequantiser warps' arrivals,
  // `empty` is one tcgen05.commit that both the x producer and the dequantisers wait for.  One wait and one commit
  // per K block for the MMA-issuing thread, whose own instructions add to the MMAs' time.
  uint64_t full[SB], empty[SB];
  uint64_t raw_full[SR], raw_empty[SR];
  uint64_t acc_full[2], acc_empty[2];   // one pair per half
  uint32_t tmem_base;
  int abort_flag;
};

struct GemmParams {
  CUtensorMap tm_x;    // fp16   {K, M},     box {64, 256}, SWIZZLE_128B
  CUtensorMap tm_w;    // uint32 {K/8, N},   box {16, 256}, SWIZZLE_64B
  const __half* scales;
  __half* y;
  int M, N, K;
  int tiles_m, tiles_n;
  int scales_vec;      // scale rows are 16-byte aligned and whole 256-k spans: one 16-byte load per span
};

// Work units of one CTA, in order.  Whole waves of 256-token tiles first; if the last, partial
// wave has at most half as many tiles as there are CTAs, its tiles are cut into their two
// 128-token halves and spread over twice as many CTAs (a half on its own converts the weights
// for 128 tokens only, so it runs at the conversion rate, but the wave is half as long).
struct Work {
  int tn;        // weight-row tile
  int tok0;      // first token
  int nhalf;     // 128-token halves to compute (1 or 2)
};
__device__ __forceinline__ bool get_work(const GemmParams& p, int i, Work& w) {
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = (int)gridDim.x, b = (int)blockIdx.x;
  const int full_waves = tiles / grid;
  const int rem = tiles - full_waves * grid;
  int tile, half = -1;
  if (i < full_waves) {
    tile = b + i * grid;
  } else if (i == full_waves && rem > 0) {
    if (2 * rem <= grid) {
      if (b >= 2 * rem) return false;
      tile = full_waves * grid + (b >> 1);
      half = b & 1;
    } else {
      if (b >= rem) return false;
      tile = full_waves * grid + b;
    }
  } else {
    return false;
  }
  const int tm = tile % p.tiles_m;
  w.tn = tile / p.tiles_m;
  w.tok0 = tm * BMT + (half > 0 ? BM : 0);
  w.nhalf = (half < 0 && w.tok0 + BM < p.M) ? 2 : 1;
  // a second half that holds no token is still a unit (its CTA idles through it): every role
  // sees the same list
  return true;
}

// 8 scales (one 256-k span) of weight row `grow`; zero for rows >= N and groups past the end (a
// zero scale makes the weight +-0).
__device__ __forceinline__ uint4 load_scales(const GemmParams& p, int grow, int span) {
  const int G = p.K >> 5;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (grow >= p.N || span * 8 >= G) return v;
  const __half* srow = p.scales + (int64_t)grow * G + span * 8;
  if (p.scales_vec) return __ldg(reinterpret_cast<const uint4*>(srow));
  uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t bits = span * 8 + j < G ? (uint32_t)__half_as_ushort(__ldg(srow + j)) : 0u;
    w[j >> 1] |= bits << (16 * (j & 1));
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Bounded wait that also honours (and raises) the block-wide abort flag.  The MMA thread runs
// through here twice per K block: a barrier that has already completed costs one try_wait, not a
// shared-memory read of the flag first (measured +4 % on the whole kernel).
__device__ __forceinline__ void wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return;
  if (*abort_flag) return;
  if (!mbar_wait_ns(bar, parity, kWaitNs)) {
    *abort_flag = 1;
    atomicExch(&g_gemm_error, code);
  }
}

// Same for the roles that are off the critical path (TMA producers, epilogue warps): they sleep
// between polls, so their polling does not take issue slots from the dequantisers.
__device__ __forceinline__ void wait_or_abort_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (*abort_flag) return;
  if (!mbar_wait_ns_relaxed(bar, parity, kWaitNs)) {
    *abort_flag = 1;
    atomicExch(&g_gemm_error, code);
  }
}

template <bool PAIRED>   // nibble order of the packed words (q4_common.cuh): the paired order needs no byte permutes
__global__ void __launch_bounds__(kNumThreads, 1)
q4f16_gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u));
  volatile int* abort_flag = &sm.abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int num_kb = (p.K + BK - 1) / BK;

  if (tid == 0) {
    sm.abort_flag = 0;
    static_assert(SA == SB, "the x ring and the dequantised ring share their barriers");
    for (int i = 0; i < SB; ++i) { mbar_init(&sm.full[i], 1 + kDequantWarps); mbar_init(&sm.empty[i], 1); }
    for (int i = 0; i < SR; ++i) { mbar_init(&sm.raw_full[i], 1); mbar_init(&sm.raw_empty[i], kDequantGroups * kDequantWarps); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 8); }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sm.tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer: x
    if (lane == 0) {
      prefetch_tmap(&p.tm_x);
      uint32_t it = 0;
      Work w;
      for (int i = 0; get_work(p, i, w); ++i) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % SA;
          const uint32_t round = it / SA;
          if (round > 0) wait_or_abort_relaxed(&sm.empty[s], (round - 1) & 1, abort_flag, 1);
          mbar_arrive_expect_tx(&sm.full[s], kABytes);
          tma_load_2d(sm.a[s], &p.tm_x, kb * BK, w.tok0, &sm.full[s]);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ TMA producer: packed W, scales
    if (lane == 0) {
      prefetch_tmap(&p.tm_w);
      uint32_t it_raw = 0;
      Work w;
      for (int i = 0; get_work(p, i, w); ++i) {
        const int tn = w.tn;
        for (int kb = 0; kb < num_kb; ++kb) {
          if ((kb & 1) == 0) {
            const int s = it_raw % SR;
            const uint32_t round = it_raw / SR;
            if (round > 0) wait_or_abort_relaxed(&sm.raw_empty[s], (round - 1) & 1, abort_flag, 3);
            mbar_arrive_expect_tx(&sm.raw_full[s], kRawBytes);
            tma_load_2d(sm.raw[s], &p.tm_w, (kb >> 1) * 16, tn * BN, &sm.raw_full[s]);
            ++it_raw;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    {
      // The whole warp walks the loop (waits, cursors, descriptor arithmetic are warp-uniform, so the compiler can
      // keep them on the uniform datapath); only the tcgen05 instructions themselves are issued by one lane.
      const bool leader = lane == 0;
      constexpr uint32_t idesc = umma_idesc_f16_f32(BM, BN);
      // The issue of a tcgen05.mma holds this thread until the tensor core takes the instruction, so the time of
      // this loop's own instructions ADDS to the MMAs' time (measured with a micro-benchmark, and a lone thread
      // spends 10-15 clocks per instruction, more on a taken branch).  Hence: straight-line code per K block, one
      // wait and one commit (the two rings share their barriers), ring cursors advanced by selects, descriptors by 32-bit adds to the address field
      // (bits 0-13, in 16-byte units; every operand sits below 256 KB, so nothing carries out of the field), the
      // first K block of a tile (which waits for the drained accumulators) peeled out of the loop.
      const uint64_t dconst = umma_desc_k128(0);
      const uint32_t a_base = (smem_u32(sm.a[0]) & 0x3FFFFu) >> 4, b_base = (smem_u32(sm.b[0]) & 0x3FFFFu) >> 4;
      constexpr uint32_t a_step = kABytes >> 4, b_step = kBBytes >> 4, half_off = (BM * BK * 2) >> 4;
      uint32_t sb = 0, pb = 0;                              // stage and phase of the two rings (they advance together)
      uint32_t it_tile = 0;
      auto operands_ready = [&]() {
        wait_or_abort(&sm.full[sb], pb, abort_flag, 5);
        tc_fence_after_sync();
      };
      auto release_and_advance = [&]() {
        if (leader) umma_commit(&sm.empty[sb]);
        sb = sb + 1 == SB ? 0 : sb + 1;
        pb ^= (uint32_t)(sb == 0);
      };
      Work w;
      for (int i = 0; get_work(p, i, w); ++i, ++it_tile) {
        const int nhalf = w.nhalf;                            // second half all padding or not ours: skip it
        // ---- first K block: each half's accumulator must have been drained by the epilogue of the tile before
        {
          operands_ready();
          const uint64_t db = dconst | (uint64_t)(b_base + sb * b_step);
          for (int h = 0; h < nhalf; ++h) {
            if (it_tile > 0) {
              wait_or_abort(&sm.acc_empty[h], (it_tile - 1) & 1, abort_flag, 4);
              tc_fence_after_sync();
            }
            const uint64_t da = dconst | (uint64_t)(a_base + sb * a_step + h * half_off);
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16) {
              // advancing 16 fp16 along K inside the swizzled 128-byte row = +32 bytes = +2 in the
              // descriptor's 16-byte address units
              if (leader) umma_f16_ss(tmem_base + (uint32_t)h * BN, da + (uint64_t)(2 * k16), db + (uint64_t)(2 * k16), idesc, k16 != 0);
            }
          }
          if (num_kb == 1) {
            if (leader) umma_commit(&sm.acc_full[0]);
            if (nhalf == 2 && leader) umma_commit(&sm.acc_full[1]);
          }
          release_and_advance();
        }
        // ---- the other K blocks
        if (nhalf == 2) {
          // Both halves' accumulators are ours: the two independent accumulation chains are issued alternately
          // (measured 2-5 % faster than one half after the other).
          for (int kb = 1; kb < num_kb; ++kb) {
            operands_ready();
            const uint64_t da0 = dconst | (uint64_t)(a_base + sb * a_step);
            const uint64_t da1 = da0 + (uint64_t)half_off;
            const uint64_t db = dconst | (uint64_t)(b_base + sb * b_step);
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16) {
              if (leader) umma_f16_ss(tmem_base, da0 + (uint64_t)(2 * k16), db + (uint64_t)(2 * k16), idesc, 1);
              if (leader) umma_f16_ss(tmem_base + (uint32_t)BN, da1 + (uint64_t)(2 * k16), db + (uint64_t)(2 * k16), idesc, 1);
            }
            if (kb == num_kb - 1) {
              if (leader) umma_commit(&sm.acc_full[0]);
              if (leader) umma_commit(&sm.acc_full[1]);
            }
            release_and_advance();
          }
        } else {
          for (int kb = 1; kb < num_kb; ++kb) {
            operands_ready();
            const uint64_t da = dconst | (uint64_t)(a_base + sb * a_step);
            const uint64_t db = dconst | (uint64_t)(b_base + sb * b_step);
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16)
              if (leader) umma_f16_ss(tmem_base, da + (uint64_t)(2 * k16), db + (uint64_t)(2 * k16), idesc, 1);
            if (kb == num_kb - 1 && leader) umma_commit(&sm.acc_full[0]);
            release_and_advance();
          }
        }
        // a skipped half still takes part in the hand-shake so that the parities stay in step
        if (nhalf == 1 && leader) umma_commit(&sm.acc_full[1]);
      }
    }
  } else if ((warp >= 4 && warp < 8) || warp >= 24) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp & 3;                       // TMEM lane quadrant this warp may read
    const int chalf = warp >= 24 ? 1 : 0;          // which 128 columns of each half this warp drains
    uint32_t it_tile = 0;
    const bool vec_ok = (p.N % 8) == 0;
    Work w;
    for (int i = 0; get_work(p, i, w); ++i, ++it_tile) {
      const int tn = w.tn;
      for (int h = 0; h < 2; ++h) {
        wait_or_abort_relaxed(&sm.acc_full[h], it_tile & 1, abort_flag, 7);
        tc_fence_after_sync();
        const int row = w.tok0 + h * BM + ew * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(ew * 32) << 16) + (uint32_t)h * BN;
        if (h < w.nhalf && w.tok0 + h * BM < p.M) {  // (warp-uniform) half computed and holds real tokens
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + chalf * 128, v);
          tmem_ld_wait();
#pragma unroll 1
          for (int c = chalf * 4; c < chalf * 4 + 4; ++c) {
            // pack this chunk, start the next chunk's TMEM load, then store: the load's latency
            // overlaps the stores
            uint4 o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              o[q].x = h2_as_u32(__floats2half2_rn(__uint_as_float(v[8 * q + 0]), __uint_as_float(v[8 * q + 1])));
              o[q].y = h2_as_u32(__floats2half2_rn(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3])));
              o[q].z = h2_as_u32(__floats2half2_rn(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5])));
              o[q].w = h2_as_u32(__floats2half2_rn(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7])));
            }
            if (c + 1 < chalf * 4 + 4) tmem_ld_32x32b_x32(taddr + (c + 1) * 32, v);
            const int col0 = tn * BN + c * 32;
            if (row < p.M && col0 < p.N) {
              __half* dst = p.y + (int64_t)row * p.N + col0;
              if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + 8 * q) = o[q];
              } else {
                const __half* oh = reinterpret_cast<const __half*>(o);
#pragma unroll
                for (int q = 0; q < 32; ++q)
                  if (col0 + q < p.N) dst[q] = oh[q];
              }
            }
            tmem_ld_wait();
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.acc_empty[h]);
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ dequantisers
    // Two groups of 8 warps; group g converts the K blocks whose running index is g mod 2 (= ring
    // stage g of the dequantised operand), so two K blocks are in conversion at any time and the
    // wait -> convert -> fence -> arrive latency of one overlaps the other's.  Both groups take part
    // in the hand-shake of every packed / scale stage.
    const int grp = (tid - 256) >> 8;
    const int r = (tid - 256) & 255;                // weight row inside the tile, 0..255
    const int r8 = r & 7;
    const Q4Consts qc = q4_consts();
    uint32_t it_raw = 0, it_b = 0;
    Work w;
    for (int i = 0; get_work(p, i, w); ++i) {
      const int tn = w.tn;
      const int grow = tn * BN + r;                 // global weight row (may be >= N: zero-filled)
      uint4 sc4 = make_uint4(0, 0, 0, 0);           // 8 scales of the current 256-k span
      uint4 sc_next = load_scales(p, grow, 0);      // ... and of the next one
      uint4 pa = make_uint4(0, 0, 0, 0), pb = pa;   // this group's 8 packed words of the current pair of K blocks
      for (int kb = 0; kb < num_kb; ++kb, ++it_b) {
        if ((kb & 3) == 0) {
          // the 8 scales of this row's next 256-k span come straight from global memory (L2): one
          // 16-byte load per span and thread, fetched one span ahead of its use
          sc4 = sc_next;
          sc_next = load_scales(p, grow, (kb >> 2) + 1);
        }
        if ((kb & 1) == 0) {
          const int s = it_raw % SR;
          wait_or_abort(&sm.raw_full[s], (it_raw / SR) & 1, abort_flag, 9);
          // row r holds 64 bytes = 4 chunks of 16; 64-byte swizzle: chunk ^= (r >> 1) & 3
          const unsigned char* rr = sm.raw[s] + r * 64;
          const int x = (r >> 1) & 3;
          // this group's K block of the pair (kb, kb+1) is the one whose running index has its parity
          const int mine = ((it_b & 1) == (uint32_t)grp) ? 0 : 2;      // chunks 0,1 (kb) or 2,3 (kb+1)
          pa = *reinterpret_cast<const uint4*>(rr + ((mine ^ x) << 4));
          pb = *reinterpret_cast<const uint4*>(rr + (((mine + 1) ^ x) << 4));
          pin_loaded(pa);                                  // loads returned before the stage is released
          pin_loaded(pb);
          fence_proxy_async_smem();              // generic reads ordered before the TMA refill (async proxy)
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.raw_empty[s]);
          ++it_raw;
        }
        if ((it_b & 1) != (uint32_t)grp) continue;   // the other group's K block
        // ---- this K block: words 8*(kb&1) .. +7 of pk, scale groups 2*(kb&3), 2*(kb&3)+1
        const int sb = it_b % SB;
        const uint32_t b_round = it_b / SB;
        if (b_round > 0) wait_or_abort(&sm.empty[sb], (b_round - 1) & 1, abort_flag, 10);
        const uint32_t scw = (kb & 2) ? ((kb & 1) ? sc4.w : sc4.z) : ((kb & 1) ? sc4.y : sc4.x);
        const __half2 scp = u32_as_h2(scw);
        const __half2 s_lo = __half2(__low2half(scp), __low2half(scp));
        const __half2 s_hi = __half2(__high2half(scp), __high2half(scp));
        const uint4 p0 = pa, p1 = pb;
        unsigned char* brow = sm.b[sb] + r * 128;     // 8-row atoms of 1024 B, rows 128 B apart
        const uint32_t words[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 o = q4_dequant_ordered<PAIRED>(words[c], c < 4 ? s_lo : s_hi, qc);
          *reinterpret_cast<uint4*>(brow + ((c ^ r8) << 4)) = o;
        }
        fence_proxy_async_smem();          // generic-proxy stores -> visible to the tensor core's async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.full[sb]);
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  if (*abort_flag) {
    // loads may still be in flight into this CTA's shared memory: let them land before it is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

int launch_gemm(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                int64_t K, cudaStream_t stream) {
  if (M == 0 || N == 0) return B200_OK;
  GemmParams p;
  int rc;
  {
    const uint64_t d[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t s[1] = {(uint64_t)K * 2};
    const uint32_t b[2] = {BK, BMT};
    if ((rc = make_tmap(&p.tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }
  {
    const uint64_t d[2] = {(uint64_t)(K / 8), (uint64_t)N};
    const uint64_t s[1] = {(uint64_t)(K / 2)};
    const uint32_t b[2] = {16, BN};
    if ((rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, wq, d, s, b, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
  }
  p.scales_vec = (K % 256 == 0) && ((reinterpret_cast<uintptr_t>(scales) & 15u) == 0);
  p.scales = scales;
  p.y = y;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.tiles_m = (int)((M + BMT - 1) / BMT);
  p.tiles_n = (int)((N + BN - 1) / BN);
  const int tiles = p.tiles_m * p.tiles_n;
  int grid = sm_count();
  if (options().gemm_max_ctas > 0 && grid > options().gemm_max_ctas) grid = (int)options().gemm_max_ctas;
  // fewer tiles than CTAs: the tiles run as 128-token halves on twice as many CTAs (see get_work)
  if (grid > 2 * tiles) grid = 2 * tiles;
  else if (grid > tiles && grid < 2 * tiles) grid = tiles;
  const size_t smem = sizeof(Smem) + 1024;
  auto kern = current_layout() == kLayoutPaired ? q4f16_gemm_tcgen05_kernel<true> : q4f16_gemm_tcgen05_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemm: cudaFuncSetAttribute(%zu): %s", smem, cudaGetErrorString(e));
  kern<<<grid, kNumThreads, smem, stream>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemm launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

int gemm_error_read_and_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)) != cudaSuccess) return 0xff;
  if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
  return v & 0xff;
}

int device_error_flags_read_and_clear() {
  return gemv_pipe_error_read_and_clear() | (gemm_error_read_and_clear() << 8) | (gemm_ws_error_read_and_clear() << 16) |
         ((layer_error_read_and_clear() & 0x7f) << 24);
}

}  // namespace b200
