// Skinny q4f16 matmul, pipelined form: CTAs fed by TMA.
//
// The register-streaming kernel in gemv.cu can keep only a couple of KB per warp in flight,
// far short of the ~40 KB per SM that HBM3e needs to stay busy.  Here two producer threads per
// CTA each issue one tiled TMA load per stage (packed weights; scales) into a ring of
// shared-memory stages and CW consumer warps drain it:
//
//   stage      = 16 rows of W x CH chunks of 256 k.  The weights are seen through a 3-D tensor
//                map (32 words = 256 k | row | 256-k chunk) so that one box {32,16,CH} lands as
//                [chunk][row][128 B] with the 128-byte swizzle: the eight rows a warp reads in
//                one instruction then sit in eight different bank groups.  The scales use the
//                same trick with 16-byte units ([chunk][row][8 scales]).  Rows past N and chunks
//                past K are zero-filled by the TMA unit (zero scale => zero weight).
//   consumer w = takes chunks w, w + CW, ... of a stage.  Lane (g,t) owns, for rows g and g+8,
//                the scale groups 2t and 2t+1 of the chunk (two 16-byte words per row and one
//                32-bit pair of scales per row); it copies them to registers, hands the stage
//                back, dequantises (exact q-7, one HMUL2 by the scale, as the reference rounds)
//                and feeds mma.sync m16n8k16 with x fragments read from a copy of x kept in
//                shared memory in the matching permuted order.
//   row tile   = 16 rows over the whole K range; each warp leaves its partial sums in shared
//                memory and bumps a counter; the warp that arrives last adds them up (in warp
//                order, so the result does not depend on who is last) and stores fp16.  Nobody
//                waits at a tile boundary, so the warps drift apart and the shared-memory loads
//                of one overlap the arithmetic of another.
//   CTA        = row tiles blockIdx.x, blockIdx.x + gridDim.x, ...
//
// When x does not fit beside the ring (large M*K) the K range is cut into blocks: x is restaged
// per block and per-tile partial sums are carried in a small shared-memory array.
//
// Programmatic dependent launch: the weights never depend on the previous kernel in the stream,
// so the producer starts copying before griddepcontrol.wait; only the consumers (which read x
// and write y) wait.  Several CTAs fit on one SM, so the CTAs of the next launch move in as
// those of the previous one leave and their first copies are in flight while it drains.
//
// Two arithmetic forms share the pipeline (template flag FAST):
//
//   exact  every weight is rounded to fp16 as the reference does, w = RN16((q-7) * s), before the
//          fp32 accumulation: 1 shift + 4 LOP3 + 4 half2 ops + 4 HMUL2 per packed word.  Results
//          differ from the reference only by the fp32 summation order.  Any batch 1..16.
//   fast   (batch 1) the scale is applied to fp32 GROUP SUMS instead: y = sum_g s_g * sum_{k in g} x_k (q_k - 7).
//          * The nibbles go to the tensor core as they come out of the LOP3, still carrying their
//            magic-number offset (1024 + q for even k, 64 + q for odd k: both exact in fp16); the
//            offset's share, C_g = sum_k x_k * (1031 | 71), is formed once per activation block
//            while x is staged and enters the MMA as its (negated) accumulator input.
//          * A lane keeps owning two whole groups (two 16-byte loads per row), and the eight
//            columns of the MMA keep the groups apart: column c receives x only in the k slots
//            that lane t = c supplies (B is zero everywhere else), so D[:, c] is the group sum of
//            the group lane c holds.  Eight MMAs run into the same accumulator, then two FFMA per
//            row apply the scales.
//          1 shift + 4 LOP3 per packed word and 8 FFMA + 8 conversions per 16 words: about a third
//          of the exact form's issue slots, which was its limit.
//          The unrounded weight differs from the reference's by at most half an fp16 ulp, so
//          |y - y_ref| <= 2^-11 * sum|x*w| (typically 3e-4 of the output's spread); an activation
//          with a single 1.0 still reproduces the reference's weight bit for bit.
//
// Requires K % 256 == 0 and 16-byte aligned scales (tensor-map stride rules); other shapes use
// the register-streaming kernel.
#include "internal.h"
#include "q4_common.cuh"
#include "skinny_common.cuh"
#include "sm100_ptx.cuh"
#include "tmap.h"

namespace b200 {

__device__ int g_gemv_pipe_error = 0;   // set when a bounded wait gives up

namespace {

using namespace ptx;
using namespace skinny;

constexpr int kRows = 16;                // rows per stage / row tile
constexpr int kMaxStages = 8;
constexpr uint64_t kConsumerWaitNs = 2000000000ull;     // 2 s: a stage copy takes microseconds
constexpr uint64_t kProducerWaitNs = 30000000000ull;    // 30 s: may span the previous kernel's whole run

enum { kPrologueNone = 0, kPrologueRmsNorm = 1, kPrologueSwiGLU = 2 };

// Rotary embedding + KV append in the epilogue of the qkv matmul (batch 1, fast form).  The weight rows are then
// fetched through a 5-D tensor map whose 16-row tile is dims d0..d0+7 of one 128-wide head AND their rotate-half
// partners d0+64..d0+71, so a tile holds both members of every pair it produces (rows r and r + 8).
struct RopeOut {
  const float* cos_t = nullptr;   // fp32 [max_pos, 64]
  const float* sin_t = nullptr;
  const int* pos = nullptr;       // device scalar: position of the new token
  __half* q_out = nullptr;        // [nh * 128] rotated query
  __half* k_cache = nullptr;      // [max_ctx, nh, 128]: rotated key goes to slot *pos
  __half* v_cache = nullptr;      // value likewise (not rotated)
  int nh = 0;                     // heads of this rank: rows are q heads | k heads | v heads
  int on = 0;
};

struct PipeParams {
  CUtensorMap tm_w;   // uint32 {32, N, K/256}, box {32, 16, CH}, 128B swizzle
  CUtensorMap tm_s;   // fp16   {8, N, K/256},  box {8, 16, CH}
  const __half* x;
  __half* y;
  int M, N, K;
  int kblk;        // k per x block (multiple of the stage's k, or >= K)
  int nstages;
  int ntiles;      // ceil(N / 16)
  int tiles_per_cta;
  // what the staging of x applies on the way in (the neighbours of the matmul in a decoder layer)
  const __half* delta;       // RmsNorm: added to x first (or null)
  const __half* norm_w;      // RmsNorm: weight [K]
  __half* x_out;             // RmsNorm: fp16(x + delta) is written here by CTA 0 (or null)
  float eps;
  int paired;                // nibble order of the packed words: 0 reference, 1 paired (q4_common.cuh)
  RopeOut rope;
  PeerReduce red;
};

// The arithmetic of the fast form over the first NU of a warp's U chunks of one stage (see the comment at its call
// site in the kernel).  NU < U: the other chunks lie past K (zero-filled) and are skipped, so a short K costs what it
// holds and not a whole stage.
template <int NU, int U, int MT, int kXUnit, int kCUnit>
__device__ __forceinline__ void fast_stage_fn(float (&acc)[2][MT][4], const uint4 (&w)[U][2][2], const uint2 (&sc)[U][2],
                                            const uint4* xb, int x_mul, const float4* cu, const Q4Consts& qc,
                                            uint32_t magic_hi) {
  float d[U][2][4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t a[U][2][8];      // raw (offset) nibble pairs: [0..3] first MMA (rows g, g+8: even k, odd k), [4..7] second
    uint4 b[U][2];
#pragma unroll
    for (int u = 0; u < NU; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t w0 = wd == 0 ? w[u][0][h].x : wd == 1 ? w[u][0][h].y : wd == 2 ? w[u][0][h].z : w[u][0][h].w;
        const uint32_t w1 = wd == 0 ? w[u][1][h].x : wd == 1 ? w[u][1][h].y : wd == 2 ? w[u][1][h].z : w[u][1][h].w;
        b[u][h] = xb[x_mul * (u * kXUnit + 4 * h + wd)];      // (lanes that own no column all read one zero slot)
        a[u][h][0] = lop3_and_or(w0, qc.lo, qc.magic);
        a[u][h][1] = lop3_and_or(w1, qc.lo, qc.magic);
        a[u][h][2] = lop3_and_or(w0, qc.hi, magic_hi);
        a[u][h][3] = lop3_and_or(w1, qc.hi, magic_hi);
        const uint32_t w0s = w0 >> 8, w1s = w1 >> 8;
        a[u][h][4] = lop3_and_or(w0s, qc.lo, qc.magic);
        a[u][h][5] = lop3_and_or(w1s, qc.lo, qc.magic);
        a[u][h][6] = lop3_and_or(w0s, qc.hi, magic_hi);
        a[u][h][7] = lop3_and_or(w1s, qc.hi, magic_hi);
      }
#pragma unroll
    for (int u = 0; u < NU; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (wd == 0) {
          const float4 c = cu[u * kCUnit + h];
          mma_16x8x16_c(d[u][h], a[u][h][0], a[u][h][1], a[u][h][2], a[u][h][3], b[u][h].x, b[u][h].y, c.x, c.y, c.z, c.w);
        } else {
          mma_16x8x16(d[u][h], a[u][h][0], a[u][h][1], a[u][h][2], a[u][h][3], b[u][h].x, b[u][h].y);
        }
      }
#pragma unroll
    for (int u = 0; u < NU; ++u)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        mma_16x8x16(d[u][h], a[u][h][4], a[u][h][5], a[u][h][6], a[u][h][7], b[u][h].z, b[u][h].w);
  }
#pragma unroll
  for (int u = 0; u < NU; ++u) {
    // scales of groups 4t'+0..3: (s0, s1) (s2, s3); even groups belong to set 0, odd ones to set 1
    const float2 g01 = __half22float2(u32_as_h2(sc[u][0].x)), g23 = __half22float2(u32_as_h2(sc[u][0].y));
    const float2 h01 = __half22float2(u32_as_h2(sc[u][1].x)), h23 = __half22float2(u32_as_h2(sc[u][1].y));
    acc[0][0][0] = fmaf(g01.x, d[u][0][0], acc[0][0][0]);
    acc[0][0][0] = fmaf(g23.x, d[u][0][1], acc[0][0][0]);
    acc[1][0][0] = fmaf(g01.y, d[u][1][0], acc[1][0][0]);
    acc[1][0][0] = fmaf(g23.y, d[u][1][1], acc[1][0][0]);
    acc[0][0][2] = fmaf(h01.x, d[u][0][2], acc[0][0][2]);
    acc[0][0][2] = fmaf(h23.x, d[u][0][3], acc[0][0][2]);
    acc[1][0][2] = fmaf(h01.y, d[u][1][2], acc[1][0][2]);
    acc[1][0][2] = fmaf(h23.y, d[u][1][3], acc[1][0][2]);
  }
}

// Shared memory carve-up (after rounding the base up to 1024 bytes):
//   ring:  nstages * kStageBytes
//   bars:  full[kMaxStages] empty[kMaxStages] red_full[kMaxStages+1] red_empty[kMaxStages+1]
//   xs:    XLayout::bytes(kblk)     permuted x block
//   corr:  (fast form) 32 floats per 256-k chunk: minus the offset sum of each group, see corr_index()
//   red:   (nstages+1) * CW * kOut * 4   per-warp partial sums of a tile, one buffer per tile in flight
//   accs:  tiles_per_cta * kOut * 4 (only when K is cut into several blocks)
//
// Warps: CW consumers, then one TMA warp (two issuing lanes), then one epilogue warp.
template <int NC, int CW, int CH, int PRO, bool FAST>
__global__ void __launch_bounds__((CW + 2) * 32, FAST ? 2 : 1)
q4f16_gemv_pipe_kernel(const __grid_constant__ PipeParams p) {
  constexpr int MT = (NC + 7) / 8;
  static_assert(!FAST || NC == 1, "the fast form is the batch-1 kernel");
  // outputs per row tile as one consumer warp leaves them: the exact form stores whole MMA fragments,
  // the fast form one value per row (padded to two)
  constexpr int NCP = 2;
  constexpr int kOut = FAST ? kRows * NCP : MT * 128;
  constexpr int KC = 256 * CH;             // k per stage
  constexpr int kWBytes = CH * kRows * 128;           // [chunk][row][128 B], 128B-swizzled
  constexpr int kSBytes = CH * kRows * 16;            // [chunk][row][8 scales = 16 B]
  constexpr int kStageBytes = kWBytes + kSBytes;      // a multiple of 1024, as the swizzle needs
  constexpr int U = CH / CW;                          // chunks per warp per stage
  using XL = XLayout<NC>;
  static_assert(CH % CW == 0 && U >= 1, "each consumer warp takes whole chunks");
  static_assert(kStageBytes % 1024 == 0, "stage alignment");
  extern __shared__ unsigned char smem_unaligned[];
  // Round the base up to 1024 bytes by OFFSETTING the shared array (not by casting through an
  // integer): the compiler then still knows these are shared-memory addresses and emits LDS/STS.
  unsigned char* ring = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)p.nstages * kStageBytes);
  uint64_t* empty = full + kMaxStages;
  uint64_t* red_full = empty + kMaxStages;
  uint64_t* red_empty = red_full + kMaxStages + 1;
  uint4* xs = reinterpret_cast<uint4*>(red_empty + kMaxStages + 1);
  float* negcorr = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + XL::bytes(p.kblk));
  float* red = negcorr + (FAST ? (p.kblk >> 8) * 32 : 0);
  const int nred = p.nstages + 1;
  float* accs = red + nred * CW * kOut;

  __shared__ int s_abort;                    // set once a bounded wait gives up: later waits are skipped
  __shared__ uint4 s_zero;                   // fast form: what the lanes without an activation column feed the MMA

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int nkb = (p.K + p.kblk - 1) / p.kblk;

  if (tid == 0) {
    s_abort = 0;
    s_zero = make_uint4(0, 0, 0, 0);
    for (int s = 0; s < p.nstages; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], CW);
    }
    for (int s = 0; s < nred; ++s) {
      mbar_init(&red_full[s], CW);
      mbar_init(&red_empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == CW) {
    // ------------------------------------------------------------------ producer warp
    // lane 0 loads the packed weights, lane 1 the scales: one tiled load per stage each (the two
    // lanes run as independent threads; one thread issuing both would halve the issue rate).
    const bool is_w = lane == 0;
    if (lane < 2) {
      prefetch_tmap(is_w ? &p.tm_w : &p.tm_s);
      const uint64_t policy = policy_evict_first();
      int s = 0;
      uint32_t round = 0;              // how many times the ring has wrapped
      for (int kb = 0; kb < nkb; ++kb) {
        const int k_lo = kb * p.kblk;
        const int k_hi = min(p.K, k_lo + p.kblk);
        for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
          const int row0 = tile * kRows;
          for (int k0 = k_lo; k0 < k_hi; k0 += KC, s = (s + 1 == p.nstages ? 0 : s + 1), round += (s == 0)) {
            if (round > 0) {
              // Legitimately as long as the previous kernel in the stream runs (the consumers
              // that free the stages sit in griddepcontrol.wait until then): bound it by time.
              if (*(volatile int*)&s_abort || !mbar_wait_ns_relaxed(&empty[s], (round - 1) & 1, kProducerWaitNs)) {
                atomicExch(&g_gemv_pipe_error, 1);
                *(volatile int*)&s_abort = 1;
                return;   // copies already issued land in stages the consumers still own
              }
            }
            unsigned char* st = ring + (size_t)s * kStageBytes;
            // out-of-range parts of a box are zero-filled and still counted in the byte total
            if (p.rope.on) {
              // tile = (128-row unit, 8 dims): rows {dim, half} = coordinates (.., (tile % 8) * 8, 0, tile / 8, ..)
              mbar_arrive_expect_tx(&full[s], is_w ? kWBytes : kSBytes);
              tma_load_5d_hint(is_w ? st : st + kWBytes, is_w ? &p.tm_w : &p.tm_s, 0, (tile & 7) * 8, 0, tile >> 3, k0 >> 8,
                               &full[s], policy);
            } else if (is_w) {
              mbar_arrive_expect_tx(&full[s], kWBytes);
              tma_load_3d_hint(st, &p.tm_w, 0, row0, k0 >> 8, &full[s], policy);
            } else {
              mbar_arrive_expect_tx(&full[s], kSBytes);
              tma_load_3d_hint(st + kWBytes, &p.tm_s, 0, row0, k0 >> 8, &full[s], policy);
            }
          }
        }
      }
    }
    return;
  }

  if (warp == CW + 1) {
    // ------------------------------------------------------------------ epilogue warp
    // Adds up the CW partial sums of each finished tile in warp order (the result does not depend
    // on which consumer finished last), carries them across K blocks, stores fp16.
    pdl_wait();                                  // y may still be read by the previous kernel
    int rb = 0;
    uint32_t rround = 0;
    const int rope_pos = (FAST && p.rope.on) ? *p.rope.pos : 0;
    for (int kb = 0; kb < nkb; ++kb) {
      int slot = 0;
      for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++slot) {
        // rotary mode: lane 2r holds row r of the tile = dim (tile % 8) * 8 + r % 8 of half r / 8 of unit tile / 8;
        // its cosine and sine are fetched before the wait for the partial sums
        float rope_c = 1.f, rope_s = 0.f;
        if (FAST && p.rope.on && (tile >> 3) < 2 * p.rope.nh) {
          const int i = (tile & 7) * 8 + ((lane >> 1) & 7);
          rope_c = p.rope.cos_t[(int64_t)rope_pos * 64 + i];
          rope_s = p.rope.sin_t[(int64_t)rope_pos * 64 + i];
        }
        if (!mbar_try_wait(&red_full[rb], rround & 1)) {
          if (!*(volatile int*)&s_abort && !mbar_wait_ns_relaxed(&red_full[rb], rround & 1, kProducerWaitNs)) {
            atomicExch(&g_gemv_pipe_error, 4);
            *(volatile int*)&s_abort = 1;
          }
        }
        const float* rbuf = red + rb * (CW * kOut);
#pragma unroll
        for (int q = 0; q < (kOut + 31) / 32; ++q) {
          const int e = q * 32 + lane;
          if (kOut % 32 != 0 && e >= kOut) break;
          float sum = 0.f;
#pragma unroll
          for (int w2 = 0; w2 < CW; ++w2) sum += rbuf[w2 * kOut + e];
          if (nkb > 1) {
            float* a = accs + slot * kOut + e;
            if (kb > 0) sum += *a;
            if (kb < nkb - 1) *a = sum;
          }
          if (FAST && p.rope.on) {
            // (one K block, one batch column: checked by the launcher)  q | k rows: rotate with the partner (row r ^ 8
            // = lane ^ 16) on the fp16-rounded matmul results, as the separate kernel does; v rows: copy.
            const float vr = __half2float(__float2half_rn(sum));
            const float pv = __shfl_xor_sync(0xffffffffu, vr, 16);
            if ((lane & 1) == 0) {
              const int r = lane >> 1, u = tile >> 3, nh = p.rope.nh;
              const int d = (tile & 7) * 8 + (r & 7) + (r < 8 ? 0 : 64);
              const float rot = r < 8 ? vr * rope_c - pv * rope_s : vr * rope_c + pv * rope_s;
              if (u < nh) p.rope.q_out[u * 128 + d] = __float2half_rn(rot);
              else if (u < 2 * nh) p.rope.k_cache[((int64_t)rope_pos * nh + (u - nh)) * 128 + d] = __float2half_rn(rot);
              else p.rope.v_cache[((int64_t)rope_pos * nh + (u - 2 * nh)) * 128 + d] = __float2half_rn(vr);
            }
          } else if (kb == nkb - 1) {
            int row, col;
            if (FAST) {
              row = tile * kRows + e / NCP;      // [row][column] as the consumers stored it
              col = e % NCP;
            } else {
              const int i = q & 3, mt = q >> 2;  // MMA fragment order
              row = tile * kRows + (lane >> 2) + 8 * (i >> 1);
              col = mt * 8 + 2 * (lane & 3) + (i & 1);
            }
            if (row < p.N && col < p.M) p.y[(int64_t)col * p.N + row] = __float2half_rn(sum);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_empty[rb]);
        rb = rb + 1 == nred ? 0 : rb + 1;
        rround += (rb == 0);
      }
    }
    if (p.red.world > 1) {
      // ---- this GPU's partial result is complete once every CTA has come through here ----------
      __threadfence();                            // this CTA's stores to y are in L2, where the peers read them
      __syncwarp();
      const int e = *p.red.epoch + 1;
      int last = 0;
      if (lane == 0) last = atomicAdd(p.red.done_counter, 1) == (int)gridDim.x - 1;
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        if (lane == 0) *p.red.done_counter = 0;
        __threadfence_system();
        // tell every rank (this one included) that rank `rank`'s partial result is complete
        if (lane < p.red.world) st_release_sys(p.red.peer_flags[lane] + p.red.flag_base + p.red.rank, e);
      }
      // every CTA waits for every rank's flag (all CTAs of the grid are resident, none of them is
      // waiting for an SM), then adds up its own slice of the result
      if (lane < p.red.world) {
        const int* f = p.red.peer_flags[p.red.rank] + p.red.flag_base + lane;
        const uint64_t t0 = globaltimer_ns();
        while (ld_acquire_sys(f) < e) {
          if (globaltimer_ns() - t0 > p.red.wait_ns) {   // a rank never published: give up, flag the error
            atomicExch(&g_gemv_pipe_error, 16);
            break;
          }
        }
      }
      __syncwarp();
    }
    goto tail;
  }

  // -------------------------------------------------------------------- consumer warps
  {
  const int g = lane >> 2;
  const int t = lane & 3;
  constexpr int kConsumers = CW * 32;

  // Per-thread offsets inside a stage (chunk `warp`; further chunks of this warp are CW chunks on).
  //   weights: row g at (chunk*16 + g)*128, 16-byte unit j at ((j ^ g) << 4); row g+8 is 1024 on
  //   (same swizzle phase).
  //   A lane owns 16-byte units 2t and 2t+1 (scale groups 2t, 2t+1 of the chunk), which differ in address
  //   bit 4 only.
  const uint32_t w_off = (uint32_t)((warp * kRows + g) * 128 + (((2 * t) ^ g) << 4));
  //   scales: exact form one 32-bit pair (groups 2t, 2t+1) per row; fast form the four groups 4t'..4t'+3 of the
  //   two output columns the lane holds (t' = t & 1; lanes t >= 2 hold columns that stay empty)
  const uint32_t s_off = FAST ? (uint32_t)(kWBytes + (warp * kRows + g) * 16 + (t & 1) * 8)
                              : (uint32_t)(kWBytes + (warp * kRows + g) * 16 + t * 4);
  // x: words 32*chunk + 8t + i of the staged block, column g (the k-block offset is added per stage).
  // Lanes whose batch column does not exist (g >= NC) read column 0: what they feed into the MMA only
  // reaches output columns >= NC, which are never stored.  (Fast form: see x_own below.)
  const int xcol = NC >= 8 ? g : (g < NC ? g : 0);
  const uint4* x_thr = xs + (NC >= 8 ? (warp * 32 + 8 * t) * NC + (g ^ (2 * t)) : NC * (warp * 36 + 9 * t) + xcol);
  constexpr int kXStage = CH * XL::kSlotsPerChunk;   // slots per stage
  constexpr int kXUnit = CW * XL::kSlotsPerChunk;    // slots between this warp's chunks
  // fast form: column c of the MMA is the group that lane t = c holds, so the activation goes into the B
  // fragment of the lanes with g == t only (B[k slots of lane t][column g]); every other lane feeds zeros
  const bool x_own = g == t;
  const int x_mul = x_own ? 1 : 0;
  // offset sums of the chunk: [t & 1][set] four floats each
  const float4* c_thr = reinterpret_cast<const float4*>(negcorr) + warp * 8 + (t & 1) * 2;
  constexpr int kCStage = CH * 8;                    // float4 per stage
  constexpr int kCUnit = CW * 8;

  const Q4Consts qc = q4_consts();
  const uint32_t magic_hi = 0x54005400u;         // (64, 64): a nibble in mantissa bits 4..7 counts 1 per step

  // exact form: two accumulation chains over the whole tile, consecutive MMAs alternate between them so the
  // tensor pipe never waits on its own result.  fast form: acc[0] is the scaled total, the per-group sums
  // live in registers of their own.
  float acc[2][MT][4];

  // One chunk (rows g and g+8, groups 2t and 2t+1) into the accumulators.  The weights are
  // rounded to fp16 exactly as the reference does: (q-7) * scale, one HMUL2 per pair.
  auto chunk = [&](const uint4 (&w)[2][2], const uint32_t (&sc)[2], const uint4* xu) {
    const __half2 sp0 = u32_as_h2(sc[0]), sp1 = u32_as_h2(sc[1]);   // (scale of group 2t, of group 2t+1)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const __half2 s0 = h ? __high2half2(sp0) : __low2half2(sp0);
      const __half2 s1 = h ? __high2half2(sp1) : __low2half2(sp1);
      const uint32_t wr0[4] = {w[0][h].x, w[0][h].y, w[0][h].z, w[0][h].w};
      const uint32_t wr1[4] = {w[1][h].x, w[1][h].y, w[1][h].z, w[1][h].w};
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        uint4 b[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) b[mt] = xu[(4 * h + wd) * NC + 8 * mt];
        uint32_t a_lo[4], a_hi[4];
        q4_dequant_pairs(wr0[wd], s0, a_lo, qc);
        q4_dequant_pairs(wr1[wd], s1, a_hi, qc);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma_16x8x16(acc[0][mt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[mt].x, b[mt].y);
          mma_16x8x16(acc[1][mt], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[mt].z, b[mt].w);
        }
      }
    }
  };

  // Fast form, the U chunks of one stage together.  Set h = 0 / 1 is the lane's 16-byte unit 2t / 2t+1 (an even /
  // odd group); its four words for rows g and g+8 give eight MMAs into one accumulator d[u][h] that starts at
  // minus the offset sums.  Afterwards d[u][h][0], [1] are row g's sums over groups 4t+h and 4t+2+h, [2], [3] row
  // g+8's.  The MMAs are issued round-robin over the 2U accumulators (an MMA that follows the one it depends on
  // waits out the tensor pipe's whole latency; with the accumulators interleaved nothing waits).
  auto fast_stage = [&](int nu, const uint4 (&w)[U][2][2], const uint2 (&sc)[U][2], const uint4* xu, const float4* cu) {
    static_assert(!FAST || U == 2, "the dispatch below lists the chunk counts of U = 2");
    const uint4* xb = x_own ? xu : &s_zero;
    if (nu >= 2) fast_stage_fn<(U < 2 ? U : 2), U, MT, kXUnit, kCUnit>(acc, w, sc, xb, x_mul, cu, qc, magic_hi);
    else if (nu == 1) fast_stage_fn<1, U, MT, kXUnit, kCUnit>(acc, w, sc, xb, x_mul, cu, qc, magic_hi);
  };
  // Fast form: this warp's share of stage `s` into registers; the stage goes back to the producer at once.
  auto fast_load = [&](int s, uint32_t round, uint4 (&w)[U][2][2], uint2 (&sc)[U][2]) {
    // On a timeout the kernel keeps going without waiting (results are garbage, the error flag says so) so
    // that every warp still reaches the named barriers and the CTA ends.
    if (!mbar_try_wait(&full[s], round & 1)) {
      if (!*(volatile int*)&s_abort && !mbar_wait_ns(&full[s], round & 1, kConsumerWaitNs)) {
        atomicExch(&g_gemv_pipe_error, 2);
        *(volatile int*)&s_abort = 1;
      }
    }
    const unsigned char* st = ring + (size_t)s * kStageBytes;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const unsigned char* su = st + u * (CW * kRows * 128);
      w[u][0][0] = *reinterpret_cast<const uint4*>(su + w_off);
      w[u][0][1] = *reinterpret_cast<const uint4*>(su + (w_off ^ 16u));
      w[u][1][0] = *reinterpret_cast<const uint4*>(su + w_off + 1024);
      w[u][1][1] = *reinterpret_cast<const uint4*>(su + (w_off ^ 16u) + 1024);
      const unsigned char* ss = st + u * (CW * kRows * 16);
      sc[u][0] = *reinterpret_cast<const uint2*>(ss + s_off);
      sc[u][1] = *reinterpret_cast<const uint2*>(ss + s_off + 128);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      pin_loaded(w[u][0][0]);
      pin_loaded(w[u][0][1]);
      pin_loaded(w[u][1][0]);
      pin_loaded(w[u][1][1]);
      pin_loaded(sc[u][0].x);
      pin_loaded(sc[u][0].y);
      pin_loaded(sc[u][1].x);
      pin_loaded(sc[u][1].y);
    }
    fence_proxy_async_smem();   // generic reads ordered before the TMA refill (async proxy)
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);            // all of this warp's share is in registers
  };

  // Stores one staged word (eight activations of one batch column) in the permuted order the unpack
  // produces; the fast form also returns its offset sum.
  auto stage_word = [&](int j, int m, const uint4& v) -> float {
    xs[XL::slot(j, m)] = staged_order(v, p.paired != 0);
    return FAST ? offset_sum_f16x8(v, p.paired != 0) : 0.f;
  };
  // Fast form (one batch column): minus the offset sum of scale group `grp`, twice (rows g and g+8 of the
  // accumulator fragment).
  auto store_group_sum = [&](int grp, float psum) {
    const int ci = corr_index(grp);
    negcorr[ci] = -psum;
    negcorr[ci + 2] = -psum;
  };

  int s = 0;                                     // ring slot of the current stage
  uint32_t round = 0;                            // how many times the ring has wrapped
  int rb = 0;                                    // reduction buffer of the current tile
  uint32_t rround = 0;
  // Fast form: the weights never depend on the previous kernel, and with its CTAs resident beside the previous
  // launch's they are in shared memory long before that kernel ends; so this warp's share of the FIRST stage is
  // already in registers when the wait for the activations returns.
  uint4 fw[U][2][2];
  uint2 fsc[U][2];
  if (FAST) fast_load(0, 0, fw, fsc);
  pdl_wait();                                    // x may be the previous kernel's output
  // ---- RMSNorm prologue: r = fp16(x + delta), inv[m] = rsqrt(mean(r^2) + eps) for every row ------
  // Every CTA computes the statistics itself (K values per row: nothing next to its share of W);
  // CTA 0 also writes r out as the updated residual stream.
  __shared__ float s_part[16][CW];
  __shared__ float s_inv[16];
  // One activation row of at most 2 * 8 * kConsumers values: a thread's two 8-value words are the
  // same in the statistics pass and in the staging pass, so x, delta and the norm weight are loaded
  // once, all six loads in flight together, and kept in registers across the two barriers.
  const bool rms_one_pass = PRO == kPrologueRmsNorm && NC == 1 && nkb == 1 && p.K <= kConsumers * 16;
  uint4 rms_keep[2], rms_w[2];
  if (PRO == kPrologueRmsNorm && rms_one_pass) {
    uint4 d[2];
    bool live[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int k = (tid + r * kConsumers) * 8;
      live[r] = k < p.K;
      rms_keep[r] = d[r] = rms_w[r] = make_uint4(0, 0, 0, 0);
      if (live[r]) {
        rms_keep[r] = *reinterpret_cast<const uint4*>(p.x + k);
        if (p.delta) d[r] = *reinterpret_cast<const uint4*>(p.delta + k);
        rms_w[r] = *reinterpret_cast<const uint4*>(p.norm_w + k);
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (!live[r]) continue;
      const int k = (tid + r * kConsumers) * 8;
      if (p.delta) rms_keep[r] = add_f16x8(rms_keep[r], d[r]);
      if (p.x_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(p.x_out + k) = rms_keep[r];
      const __half2* h = reinterpret_cast<const __half2*>(&rms_keep[r]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_part[0][warp] = ss;
  } else if (PRO == kPrologueRmsNorm) {
    // four rows at a time so that eight independent loads are in flight per thread
    constexpr int R = NC >= 8 ? 4 : 1;
    for (int m0 = 0; m0 < p.M; m0 += R) {
      float ss[R];
#pragma unroll
      for (int r = 0; r < R; ++r) ss[r] = 0.f;
      for (int k = tid * 8; k < p.K; k += kConsumers * 8) {
        uint4 v[R], d[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int m = min(m0 + r, p.M - 1);
          v[r] = *reinterpret_cast<const uint4*>(p.x + (int64_t)m * p.K + k);
          if (p.delta) d[r] = *reinterpret_cast<const uint4*>(p.delta + (int64_t)m * p.K + k);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (m0 + r >= p.M) continue;
          if (p.delta) v[r] = add_f16x8(v[r], d[r]);
          if (p.x_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(p.x_out + (int64_t)(m0 + r) * p.K + k) = v[r];
          const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            ss[r] += f.x * f.x + f.y * f.y;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], o);
        if (lane == 0 && m0 + r < p.M) s_part[m0 + r][warp] = ss[r];
      }
    }
  }
  if (PRO == kPrologueRmsNorm) {
    bar_sync(1, kConsumers);
    if (tid < p.M) {
      float tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < CW; ++w2) tot += s_part[tid][w2];
      s_inv[tid] = rsqrtf(tot / (float)p.K + p.eps);
    }
    bar_sync(1, kConsumers);
  }

  // (one K block in this case: the staged row is complete before the loop, the kept registers end here)
  if (PRO == kPrologueRmsNorm && rms_one_pass) {
    const int words = p.kblk >> 3;
    const float inv = s_inv[0];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int j = tid + r * kConsumers;
      if (j >= words) continue;              // (words is a multiple of 32: whole warps leave together)
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j * 8 < p.K) v = scale_f16x8(rms_keep[r], inv, rms_w[r]);
      float psum = stage_word(j, 0, v);
      if (FAST) {
        // a group's four words sit in four consecutive lanes (words are dealt out in order, 32 per warp and round)
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        if ((j & 3) == 0) store_group_sum(j >> 2, psum);
      }
    }
  }
  for (int kb = 0; kb < nkb; ++kb) {
    const int k_lo = kb * p.kblk;
    const int k_hi = min(p.K, k_lo + p.kblk);
    // ---- stage x[:, k_lo .. k_lo + kblk) permuted per 8 k; zero beyond K and beyond M --------------
    if (kb > 0) bar_sync(1, kConsumers);         // everyone is done reading the previous block
    if (FAST && !(PRO == kPrologueRmsNorm && rms_one_pass)) {
      // one batch column: a thread takes a whole scale group (four words, 64 contiguous bytes), so its offset sum
      // needs no exchange; all loads of a thread are issued before the first use
      const int groups = p.kblk >> 5;
      for (int grp = tid; grp < groups; grp += kConsumers) {
        const int k = k_lo + grp * 32;
        uint4 a[4], b[4], c[4];
        const bool live = k < p.K;
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
          a[wd] = b[wd] = c[wd] = make_uint4(0, 0, 0, 0);
          if (live) {
            if (PRO == kPrologueSwiGLU) {
              a[wd] = *reinterpret_cast<const uint4*>(p.x + k + 8 * wd);
              b[wd] = *reinterpret_cast<const uint4*>(p.x + p.K + k + 8 * wd);
            } else {
              a[wd] = *reinterpret_cast<const uint4*>(p.x + k + 8 * wd);
              if (PRO == kPrologueRmsNorm) {
                if (p.delta) b[wd] = *reinterpret_cast<const uint4*>(p.delta + k + 8 * wd);
                c[wd] = *reinterpret_cast<const uint4*>(p.norm_w + k + 8 * wd);
              }
            }
          }
        }
        float psum = 0.f;
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
          uint4 v = a[wd];
          if (live) {
            if (PRO == kPrologueSwiGLU) {
              v = silu_mul_f16x8(a[wd], b[wd]);
            } else if (PRO == kPrologueRmsNorm) {
              if (p.delta) v = add_f16x8(v, b[wd]);
              v = scale_f16x8(v, s_inv[0], c[wd]);
            }
          }
          psum += stage_word(4 * grp + wd, 0, v);
        }
        store_group_sum(grp, psum);
      }
    } else if (!(PRO == kPrologueRmsNorm && rms_one_pass)) {
      // four items per thread and round: all loads of a round are issued before the first use
      const int words = p.kblk >> 3;
      const int items = words * NC;              // a multiple of 32: a warp's 32 items are all inside or all outside
      // (registers: small batches keep two CTAs per SM; without a prologue only one array is live)
      constexpr int R = NC >= 8 ? 4 : (PRO == kPrologueNone ? 4 : (NC == 1 ? 2 : 1));
      for (int i0 = tid; i0 < items; i0 += kConsumers * R) {
        uint4 a[R], b[R], c[R];
        bool live[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = i0 + r * kConsumers;
          const int j = i / NC, m = i - j * NC;
          const int k = k_lo + j * 8;
          live[r] = i < items && m < p.M && k < p.K;
          a[r] = b[r] = c[r] = make_uint4(0, 0, 0, 0);
          if (live[r]) {
            if (PRO == kPrologueSwiGLU) {
              // x is [M, 2K] = gate | up
              a[r] = *reinterpret_cast<const uint4*>(p.x + (int64_t)m * 2 * p.K + k);
              b[r] = *reinterpret_cast<const uint4*>(p.x + (int64_t)m * 2 * p.K + p.K + k);
            } else {
              a[r] = *reinterpret_cast<const uint4*>(p.x + (int64_t)m * p.K + k);
              if (PRO == kPrologueRmsNorm) {
                if (p.delta) b[r] = *reinterpret_cast<const uint4*>(p.delta + (int64_t)m * p.K + k);
                c[r] = *reinterpret_cast<const uint4*>(p.norm_w + k);
              }
            }
          }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = i0 + r * kConsumers;
          if (i >= items) continue;
          const int j = i / NC, m = i - j * NC;
          uint4 v = a[r];
          if (live[r]) {
            if (PRO == kPrologueSwiGLU) {
              v = silu_mul_f16x8(a[r], b[r]);       // fp32 inside, one fp16 rounding
            } else if (PRO == kPrologueRmsNorm) {
              if (p.delta) v = add_f16x8(v, b[r]);
              v = scale_f16x8(v, s_inv[m], c[r]);
            }
          }
          stage_word(j, m, v);
        }
      }
    }
    bar_sync(1, kConsumers);
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[0][mt][i] = acc[1][mt][i] = 0.f;

      const uint4* xk = x_thr;
      const float4* ck = c_thr;
      for (int k0 = k_lo; k0 < k_hi; k0 += KC, xk += kXStage, ck += kCStage, s = (s + 1 == p.nstages ? 0 : s + 1), round += (s == 0)) {
        if (FAST) {
          // (the first stage of the launch is in registers already)
          if (!(kb == 0 && tile == (int)blockIdx.x && k0 == k_lo)) fast_load(s, round, fw, fsc);
          // this warp's chunks of the stage are warp and warp + CW; those past K are skipped
          const int nch = (min(k_hi, k0 + KC) - k0 + 255) >> 8;
          fast_stage((warp < nch) + (warp + CW < nch), fw, fsc, xk, ck);
        } else {
        // On a timeout the kernel keeps going without waiting (results are garbage, the error
        // flag says so) so that every warp still reaches the named barriers and the CTA ends.
        if (!mbar_try_wait(&full[s], round & 1)) {
          if (!*(volatile int*)&s_abort && !mbar_wait_ns(&full[s], round & 1, kConsumerWaitNs)) {
            atomicExch(&g_gemv_pipe_error, 2);
            *(volatile int*)&s_abort = 1;
          }
        }
        const unsigned char* st = ring + (size_t)s * kStageBytes;
        uint4 w[U][2][2];        // [chunk of this warp][row g / g+8][group 2t / 2t+1]
        uint32_t sc[U][2];       // scales of groups (2t, 2t+1) as a half2, rows g / g+8
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const unsigned char* su = st + u * (CW * kRows * 128);
          w[u][0][0] = *reinterpret_cast<const uint4*>(su + w_off);
          w[u][0][1] = *reinterpret_cast<const uint4*>(su + (w_off ^ 16u));
          w[u][1][0] = *reinterpret_cast<const uint4*>(su + w_off + 1024);
          w[u][1][1] = *reinterpret_cast<const uint4*>(su + (w_off ^ 16u) + 1024);
          const unsigned char* ss = st + u * (CW * kRows * 16);
          sc[u][0] = *reinterpret_cast<const uint32_t*>(ss + s_off);
          sc[u][1] = *reinterpret_cast<const uint32_t*>(ss + s_off + 128);
        }
        // the loads must have returned before the stage goes back to the producer
#pragma unroll
        for (int u = 0; u < U; ++u) {
          pin_loaded(w[u][0][0]);
          pin_loaded(w[u][0][1]);
          pin_loaded(w[u][1][0]);
          pin_loaded(w[u][1][1]);
          pin_loaded(sc[u][0]);
          pin_loaded(sc[u][1]);
        }
        fence_proxy_async_smem();   // generic reads ordered before the TMA refill (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);            // all of this warp's share is in registers

        if (k0 + KC <= k_hi) {
          // whole stage inside K: straight-line code over this warp's chunks
#pragma unroll
          for (int u = 0; u < U; ++u) chunk(w[u], sc[u], xk + u * kXUnit);
        } else {
          // chunks past K were zero-filled: nothing to add
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (k0 + (warp + u * CW) * 256 < k_hi) chunk(w[u], sc[u], xk + u * kXUnit);
        }
        }
      }

      // ---- hand this warp's partial sums of the tile to the epilogue warp --------------------------
      if (rround > 0 && !mbar_try_wait(&red_empty[rb], (rround - 1) & 1)) {
        if (!*(volatile int*)&s_abort && !mbar_wait_ns(&red_empty[rb], (rround - 1) & 1, kConsumerWaitNs)) {
          atomicExch(&g_gemv_pipe_error, 8);
          *(volatile int*)&s_abort = 1;
        }
      }
      if (FAST) {
        // lanes t = 0 and t = 1 hold the two halves (groups 0..3 and 4..7 of every chunk) of rows g and g+8
        float lo = acc[0][0][0] + acc[1][0][0], hi = acc[0][0][2] + acc[1][0][2];
        lo += __shfl_xor_sync(0xffffffffu, lo, 1);
        hi += __shfl_xor_sync(0xffffffffu, hi, 1);
        float* rbuf = red + rb * (CW * kOut) + warp * kOut;
        if (t == 0) {
          *reinterpret_cast<float2*>(rbuf + g * NCP) = make_float2(lo, 0.f);
          *reinterpret_cast<float2*>(rbuf + (g + 8) * NCP) = make_float2(hi, 0.f);
        }
      } else {
        float* rbuf = red + rb * (CW * kOut) + warp * kOut + lane;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) rbuf[(mt * 4 + i) * 32] = acc[0][mt][i] + acc[1][mt][i];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_full[rb]);   // release: the stores above are visible to the waiter
      rb = rb + 1 == nred ? 0 : rb + 1;
      rround += (rb == 0);
    }
  }
  }   // (consumer scope)

tail:
  if (p.red.world > 1) {
    // the consumers wait here until the epilogue warp has seen every rank's flag; then the CTA adds
    // up items blockIdx.x, blockIdx.x + gridDim.x, ... (8 outputs each), all peers' loads in flight at once
    bar_sync(3, (CW + 1) * 32);
    const int rt = warp < CW ? tid : CW * 32 + lane;           // 0 .. (CW+1)*32-1 (the TMA warp has left)
    const int n8 = (p.M * p.N) >> 3;                           // N % 8 == 0 is checked by the caller
    for (int i = blockIdx.x + rt * gridDim.x; i < n8; i += (CW + 1) * 32 * gridDim.x) {
      uint4 v[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < p.red.world) v[r] = ld_volatile_v4(p.red.peer_y[r] + (int64_t)i * 8);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.red.world) {
          const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
      *reinterpret_cast<uint4*>(p.red.out + (int64_t)i * 8) = o;
    }
  }
  if (*(volatile int*)&s_abort) {
    // copies may still be in flight into this CTA's shared memory: let them land before exit
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

struct Prologue {
  int kind = kPrologueNone;
  const __half* delta = nullptr;
  const __half* norm_w = nullptr;
  __half* x_out = nullptr;
  float eps = 0.f;
  RopeOut rope;          // rotary embedding + KV append in the epilogue (qkv matmul of a batch-1 step)
};

template <int NC, int CW, int CH, int PRO, bool FAST>
int launch_pipe(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int M, int N, int K,
                cudaStream_t stream, const Prologue& pro, const PeerReduce& red) {
  constexpr int MT = (NC + 7) / 8;
  constexpr int kOut = FAST ? kRows * 2 : MT * 128;
  constexpr int KC = 256 * CH;
  constexpr int kStageBytes = CH * kRows * (128 + 16);
  constexpr int kThreads = (CW + 2) * 32;
  using XL = XLayout<NC>;
  PipeParams p;
  p.rope = pro.rope;
  if (pro.rope.on) {
    // the fast form's epilogue layout, one K block, whole 128-row units
    if (!FAST || NC != 1 || M != 1 || N % 128 != 0 || N != 3 * pro.rope.nh * 128) return B200_ENOTREADY;
    // rows as {dim in half: 64 | half: 2 | unit: N/128}, tile = 8 dims x 2 halves of one unit
    const uint64_t wd[5] = {32, 64, 2, (uint64_t)(N / 128), (uint64_t)(K / 256)};
    const uint64_t ws[4] = {(uint64_t)K / 2, (uint64_t)K / 2 * 64, (uint64_t)K / 2 * 128, 128};
    const uint32_t wb[5] = {32, 8, 2, 1, CH};
    int rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 5, wq, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint64_t rp = (uint64_t)(K / 32) * 2;    // bytes per row of scales
    const uint64_t sd[5] = {8, 64, 2, (uint64_t)(N / 128), (uint64_t)(K / 256)};
    const uint64_t ss[4] = {rp, rp * 64, rp * 128, 16};
    const uint32_t sb[5] = {8, 8, 2, 1, CH};
    rc = make_tmap(&p.tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, scales, sd, ss, sb, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  } else {
    const uint64_t wd[3] = {32, (uint64_t)N, (uint64_t)(K / 256)};
    const uint64_t ws[2] = {(uint64_t)K / 2, 128};
    const uint32_t wb[3] = {32, kRows, CH};
    int rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, wq, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint64_t sd[3] = {8, (uint64_t)N, (uint64_t)(K / 256)};
    const uint64_t ss[2] = {(uint64_t)(K / 32) * 2, 16};
    const uint32_t sb[3] = {8, kRows, CH};
    rc = make_tmap(&p.tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, scales, sd, ss, sb, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  p.x = x; p.y = y;
  p.M = M; p.N = N; p.K = K;
  p.delta = pro.delta; p.norm_w = pro.norm_w; p.x_out = pro.x_out; p.eps = pro.eps;
  p.red = red;
  p.paired = current_layout() == kLayoutPaired;
  p.ntiles = (N + kRows - 1) / kRows;
  const int kpad = ((K + KC - 1) / KC) * KC;
  const int stages_per_tile = kpad / KC;
  const size_t kMaxSmem = 227 * 1024;
  const int sms = sm_count();
  auto kern = q4f16_gemv_pipe_kernel<NC, CW, CH, PRO, FAST>;
  // Ask for the largest shared-memory carve-out: the default picks the smallest that fits ONE CTA,
  // which would keep further CTAs (or the next dependent launch) off the SM.
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  auto fixed_bytes = [&](int stages) {
    return (size_t)1024 /* base alignment slack */ + (4 * kMaxStages + 2) * sizeof(uint64_t) + (size_t)stages * kStageBytes +
           (size_t)(stages + 1) * CW * kOut * sizeof(float);
  };
  auto block_bytes = [&](int k) { return XL::bytes(k) + (FAST ? (size_t)(k / 256) * 32 * sizeof(float) : 0); };
  size_t need = 0;
  int kblk = kpad, grid = 0, stages = (int)options().gemv_stages;
  bool placed = false;
  if (FAST) {
    // Two CTAs per SM, one stage each (registers are the second buffer, as in the exact form): measured fastest
    // for every shape of the 7B decode step.  Deeper rings (up to a CTA's whole share of W resident, one CTA per
    // SM so that the next launch's CTAs prefetch beside this launch's) were measured too: no faster for
    // N = K = 4096 and 10-20 % slower for the large matmuls.  Options gemv.ctas_per_sm and gemv.stages
    // still select them.
    int per_sm = (int)options().gemv_ctas_per_sm;
    if (per_sm <= 0) per_sm = 2;
    if (per_sm > 2) per_sm = 2;
    grid = sms * per_sm;
    if (grid > p.ntiles) grid = p.ntiles;
    p.tiles_per_cta = (p.ntiles + grid - 1) / grid;
    // (an explicit stage count may use up to half an SM, so that two CTAs still fit)
    const size_t budget = stages > 0 ? (228 * 1024 - 2 * 1024) / 2 : 76 * 1024;
    int want = stages > 0 ? stages : p.tiles_per_cta * stages_per_tile;
    if (want > kMaxStages) want = kMaxStages;
    for (int st = want; st >= 1 && !placed; --st) {
      need = fixed_bytes(st) + block_bytes(kpad);
      if (need <= budget || (st == 1 && need <= kMaxSmem)) {
        stages = st;
        placed = true;
      }
    }
  } else {
    // Registers are the second buffer (a stage is handed back as soon as it has been copied out) and
    // two CTAs share an SM, so one stage per CTA measured fastest for one row and for 9..16 rows; with 2..8 rows a
    // second stage measured 0-12 % faster (M = 2: 11.7 -> 10.2 us at N = 4096, K = 11008; 16.7 -> 15.6 at N = 22016).
    if (stages <= 0) stages = (M >= 2 && M <= 8) ? 2 : 1;
    if (stages > kMaxStages) stages = kMaxStages;
    int max_per_sm = (int)options().gemv_ctas_per_sm;
    if (max_per_sm <= 0) max_per_sm = 2;
    // Prefer the whole of x beside the ring; give up ring depth before cutting K into blocks (a
    // shallower ring costs little, K blocks cost a carry array and restaging).
    for (; stages >= 1 && !placed; --stages) {
      need = fixed_bytes(stages) + block_bytes(kpad);
      if (need > kMaxSmem) continue;
      // resident CTAs per SM as the hardware will place them (registers and threads count too);
      // the answer for the last shared-memory size is remembered (per thread, per kernel variant)
      static thread_local size_t cached_need = 0;
      static thread_local int cached_per_sm = 0;
      if (cached_need != need) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
        if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemv: cudaFuncSetAttribute(%zu): %s", need, cudaGetErrorString(e));
        int q = 1;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kern, kThreads, need) != cudaSuccess || q < 1) q = 1;
        cached_need = need;
        cached_per_sm = q;
      }
      int per_sm = cached_per_sm;
      if (per_sm > max_per_sm) per_sm = max_per_sm;
      grid = sms * per_sm;
      if (grid > p.ntiles) grid = p.ntiles;
      p.tiles_per_cta = (p.ntiles + grid - 1) / grid;
      placed = true;
      break;
    }
  }
  if (!placed) {
    // ... otherwise cut K into blocks of as many stages' worth as fit, leaving room for the carries.
    stages = 1;
    grid = sms < p.ntiles ? sms : p.ntiles;
    p.tiles_per_cta = (p.ntiles + grid - 1) / grid;
    const size_t carries = (size_t)p.tiles_per_cta * kOut * sizeof(float);
    const size_t fixed = fixed_bytes(1);
    if (fixed + carries + block_bytes(KC) > kMaxSmem) return B200_ENOTREADY;   // caller falls back
    kblk = (int)((kMaxSmem - fixed - carries) / block_bytes(KC)) * KC;
    need = fixed + carries + block_bytes(kblk);
  }
  {
    static thread_local size_t attr_need = 0;      // (per thread, per kernel variant)
    if (attr_need != need) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
      if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemv: cudaFuncSetAttribute(%zu): %s", need, cudaGetErrorString(e));
      attr_need = need;
    }
  }
  p.nstages = stages;
  p.kblk = kblk;
  if (pro.rope.on && kblk < kpad) return B200_ENOTREADY;   // (K cut into blocks: the rotary epilogue takes one)

  cudaError_t e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = need;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemv launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

template <int CW, int CH, int PRO>
int launch_pipe_m(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int m, int n, int k,
                  cudaStream_t stream, const Prologue& pro, const PeerReduce& red) {
  if (m == 1) {
    // batch 1: the fast form unless the caller asks for the reference's rounding of every weight (gemv.exact = 1)
    // or, by default (gemv.exact = 0), K is short.  The fast form's staging of x also builds the offset sums and the
    // block-diagonal operand, about 0.15 us more per launch, which it wins back from K of about 2500 on: measured at
    // N = 4096, exact / fast = 2.96 / 3.12 us at K = 512, 3.38 / 3.51 at 1536, 3.62 / 3.69 at 2048, 4.16 / 4.13 at
    // 2816, 4.88 / 4.58 at 4096, 7.26 / 6.80 at 8192, 9.16 / 8.72 at 11008 (and 14.3 / 12.9 at N = 22016, K = 4096).
    // gemv.exact = 2 forces the fast form for every K (tests).
    const bool fast = options().gemv_exact == 2 || (options().gemv_exact == 0 && k >= 2560);
    if (fast) return launch_pipe<1, CW, CH, PRO, true>(x, wq, scales, y, m, n, k, stream, pro, red);
    return launch_pipe<1, CW, CH, PRO, false>(x, wq, scales, y, m, n, k, stream, pro, red);
  }
  if (m == 2) return launch_pipe<2, CW, CH, PRO, false>(x, wq, scales, y, m, n, k, stream, pro, red);
  if (m <= 4) return launch_pipe<4, CW, CH, PRO, false>(x, wq, scales, y, m, n, k, stream, pro, red);
  if (m <= 8) return launch_pipe<8, CW, CH, PRO, false>(x, wq, scales, y, m, n, k, stream, pro, red);
  return launch_pipe<16, CW, CH, PRO, false>(x, wq, scales, y, m, n, k, stream, pro, red);
}

template <int PRO>
int dispatch_form(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int m, int n, int k,
                  cudaStream_t stream, const Prologue& pro, const PeerReduce& red) {
  return launch_pipe_m<8, 16, PRO>(x, wq, scales, y, m, n, k, stream, pro, red);
}

int dispatch_pipe(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N, int64_t K,
                  cudaStream_t stream, const Prologue& pro, const PeerReduce& red) {
  if (K % 256 != 0 || (reinterpret_cast<uintptr_t>(scales) & 15u)) return B200_ENOTREADY;
  int m = (int)M, n = (int)N, k = (int)K;
  if (pro.kind == kPrologueRmsNorm) return dispatch_form<kPrologueRmsNorm>(x, wq, scales, y, m, n, k, stream, pro, red);
  if (pro.kind == kPrologueSwiGLU) return dispatch_form<kPrologueSwiGLU>(x, wq, scales, y, m, n, k, stream, pro, red);
  return dispatch_form<kPrologueNone>(x, wq, scales, y, m, n, k, stream, pro, red);
}

// The sum over tensor-parallel ranks as a kernel of its own, for partial results that another kernel produced
// (the mid-batch and prefill matmuls): same protocol as the tail of the skinny kernel above.  The partial result
// peer_y[rank] was written by the launch in front of this one (stream order; with programmatic dependent launch
// the wait below is what orders it).  CTA 0 publishes this rank's flag to every rank, every CTA waits (bounded)
// for all ranks' flags and adds up its share of the `count` values in rank order with plain peer loads.
__global__ void __launch_bounds__(256)
peer_allreduce_kernel(int64_t n8, const PeerReduce red) {
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int e = *red.epoch + 1;
  if (tid < 32) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      if (tid < red.world) st_release_sys(red.peer_flags[tid] + red.flag_base + red.rank, e);
    }
    if (tid < red.world) {
      const int* f = red.peer_flags[red.rank] + red.flag_base + tid;
      const uint64_t t0 = globaltimer_ns();
      while (ld_acquire_sys(f) < e) {
        if (globaltimer_ns() - t0 > red.wait_ns) {     // a rank never published: give up, flag the error
          atomicExch(&g_gemv_pipe_error, 16);
          break;
        }
      }
    }
  }
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + tid; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < red.world) v[r] = ld_volatile_v4(red.peer_y[r] + i * 8);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < red.world) {
        const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(red.out + i * 8) = o;
  }
}

PeerReduce make_reduce(const B200PeerReduce* r) {
  PeerReduce red;
  if (!r || r->world <= 1) return red;
  red.world = r->world;
  red.rank = r->rank;
  for (int i = 0; i < r->world && i < kMaxPeers; ++i) {
    red.peer_y[i] = static_cast<const __half*>(r->peer_y[i]);
    red.peer_flags[i] = static_cast<int*>(r->peer_flags[i]);
  }
  red.flag_base = r->flag_base;
  red.epoch = static_cast<const int*>(r->epoch);
  red.done_counter = static_cast<int*>(r->done_counter);
  red.out = static_cast<__half*>(r->out);
  red.wait_ns = (uint64_t)options().gemv_peer_wait_ms * 1000000ull;
  return red;
}

}  // namespace

int launch_peer_allreduce(int64_t count, const B200PeerReduce* r, cudaStream_t stream) {
  const PeerReduce red = make_reduce(r);
  const int64_t n8 = count >> 3;
  if (n8 == 0) return B200_OK;
  // never more CTAs than can be resident at once (they wait for the other ranks): a quarter of that is plenty for
  // the few hundred KB this moves
  int64_t grid = (n8 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 2;
  if (grid > cap) grid = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, n8, red);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "peer all-reduce launch: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

// Returns B200_ENOTREADY when the shape is outside what this kernel takes (caller falls back to
// the register-streaming kernel).
int launch_gemv_pipe(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                     int64_t K, cudaStream_t stream) {
  return dispatch_pipe(x, wq, scales, y, M, N, K, stream, Prologue{}, PeerReduce{});
}

// y = (rmsnorm(fp16(x + delta)) * norm_w) . decode(W)^T; fp16(x + delta) also goes to x_out (if given).
int launch_gemv_pipe_rmsnorm(const __half* x, const __half* delta, const __half* norm_w, __half* x_out, float eps,
                             const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N, int64_t K,
                             cudaStream_t stream) {
  Prologue pro;
  pro.kind = kPrologueRmsNorm; pro.delta = delta; pro.norm_w = norm_w; pro.x_out = x_out; pro.eps = eps;
  return dispatch_pipe(x, wq, scales, y, M, N, K, stream, pro, PeerReduce{});
}

// qkv = rmsnorm(x + delta) . decode(W)^T for ONE row, with the rotary embedding and the KV append in the epilogue:
// writes the rotated query to q_out and the new token's rotated key and value into the caches at *pos; no qkv
// buffer.  B200_ENOTREADY when the launch would not use the fast form (the epilogue is written for its layout).
int launch_gemv_pipe_rmsnorm_rope(const __half* x, const __half* delta, const __half* norm_w, __half* x_out, float eps,
                                  const uint32_t* wq, const __half* scales, const float* cos_t, const float* sin_t,
                                  const int* pos, __half* q_out, __half* k_cache, __half* v_cache, int64_t nh, int64_t K,
                                  cudaStream_t stream) {
  Prologue pro;
  pro.kind = kPrologueRmsNorm; pro.delta = delta; pro.norm_w = norm_w; pro.x_out = x_out; pro.eps = eps;
  pro.rope.cos_t = cos_t; pro.rope.sin_t = sin_t; pro.rope.pos = pos;
  pro.rope.q_out = q_out; pro.rope.k_cache = k_cache; pro.rope.v_cache = v_cache;
  pro.rope.nh = (int)nh; pro.rope.on = 1;
  return dispatch_pipe(x, wq, scales, q_out /* unused */, 1, 3 * nh * 128, K, stream, pro, PeerReduce{});
}

// y = (silu(gu[:, :K]) * gu[:, K:]) . decode(W)^T
int launch_gemv_pipe_swiglu(const __half* gu, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                            int64_t K, cudaStream_t stream) {
  Prologue pro;
  pro.kind = kPrologueSwiGLU;
  return dispatch_pipe(gu, wq, scales, y, M, N, K, stream, pro, PeerReduce{});
}

// Row-parallel matmul + sum over ranks in one kernel; swiglu != 0 applies the SwiGLU prologue.
int launch_gemv_pipe_allreduce(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                               int64_t K, int swiglu, const B200PeerReduce* red, cudaStream_t stream) {
  Prologue pro;
  pro.kind = swiglu ? kPrologueSwiGLU : kPrologueNone;
  return dispatch_pipe(x, wq, scales, y, M, N, K, stream, pro, make_reduce(red));
}

int gemv_pipe_error_read_and_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_pipe_error, sizeof(int)) != cudaSuccess) return 0xff;
  if (v) cudaMemcpyToSymbol(g_gemv_pipe_error, &zero, sizeof(int));
  return v & 0xff;
}

}  // namespace b200
