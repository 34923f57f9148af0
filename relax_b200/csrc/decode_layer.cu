// One decoder layer of a batch-1 decode step as ONE persistent kernel.
//
// A decode step through separate launches pays, per launch, the hand-over between dependent kernels
// (about a microsecond before the next kernel's wait returns), a cold pipeline, and a tail in which
// most SMs idle; a 7B-shaped layer is seven such launches around 140 MB of weights and KV that need
// 20 microseconds of HBM time.  Here one grid of one CTA per SM walks the layer's five stages
//
//     1  qkv   = Wqkv . rmsnorm(x + delta)            (also writes x_mid = x + delta)
//     2  attn  = attention(rope(q), cache + rope(k), v)  per (head, 128-token chunk), merged per head
//     3  o     = Wo . attn                            (+ sum over tensor-parallel ranks)
//     4  act   = silu(gate) * up,  gate | up = Wgu . rmsnorm(x_mid + o)   (also writes x_out = x_mid + o)
//     5  down  = Wdown . act                          (+ sum over tensor-parallel ranks)
//
// and the stages hand over through arrival counters in global memory (a grid barrier: every CTA adds
// one when its stores are fenced, everyone polls until the count reaches grid * (step + 1); counters
// grow from step to step and are never reset).  The TMA warp does not take part in the barriers: it
// streams the CTA's tiles of all four weight matrices through the shared-memory ring in program order,
// so the next matmul's first tiles arrive while the current stage drains and during the attention.
//
// The four matmuls use the batch-1 fast form of the skinny kernel (gemv_pipe.cu): raw offset nibbles
// into mma.sync, block-diagonal activations, group scales applied to fp32 group sums; RMSNorm and the
// residual adds run inside the staging of the activation vector.  SwiGLU runs where the gate and up rows
// are produced: a CTA takes the gate tile and the up tile of the same 16 outputs one after the other, and
// its epilogue warp stores silu(gate) * up, so nobody has to recompute the 11008 activations per CTA.
//
// Warps: eight consumers (matmuls and attention), one TMA warp, one epilogue warp.
//
// Every wait is bounded by wall time: a wait that runs out sets a bit in the layer kernel's error word
// (b200_device_error_flags), the CTA stops waiting and runs through, nothing hangs.
//
// All CTAs of the grid must be resident together (they wait for each other): the grid is at most one CTA
// per SM and the kernel is launched with one CTA per SM's worth of shared memory.  Launches of this
// kernel follow each other in ONE stream; a launch only starts once every CTA of the launch before it
// has started (programmatic dependent launch) and never waits for anything a later launch does, so two
// launches cannot block each other.
#include "internal.h"
#include "q4_common.cuh"
#include "skinny_common.cuh"
#include "sm100_ptx.cuh"
#include "tmap.h"

namespace b200 {

__device__ int g_layer_error = 0;   // bit 0 producer, 1 stage wait, 2 epilogue, 3 hand-off, 4 peer flags, 5 grid barrier

namespace {

using namespace ptx;
using namespace skinny;

constexpr int kRows = 16;                // rows per stage / row tile
constexpr int CW = 8;                    // consumer warps
constexpr int CH = 16;                   // 256-k chunks per stage
constexpr int U = CH / CW;               // chunks per warp per stage
constexpr int KC = 256 * CH;             // k per stage
constexpr int kWBytes = CH * kRows * 128;
constexpr int kSBytes = CH * kRows * 16;
constexpr int kStageBytes = kWBytes + kSBytes;
constexpr int kMaxStages = 5;
constexpr int kNumRed = 2;               // partial-sum buffers between the consumers and the epilogue warp
constexpr int kAttnHelpers = 0;           // extra warps that only work in the attention stage (8 were measured: the 18-warp CTA
                                          // leaves 96 registers per thread, the matmuls spill and the layer gets 15 % slower)
constexpr int kThreads = (CW + 2 + kAttnHelpers) * 32;
constexpr int kAttnThreads = (CW + kAttnHelpers) * 32;
constexpr int kAttnGroups = (CW + kAttnHelpers) / 4;
constexpr int kConsumers = CW * 32;
constexpr int kOut = kRows * 2;          // one value per row, padded to two
constexpr int kAttnChunk = 128;
constexpr int kTok = 16;                 // tokens per attention round and warp (all loads of a round in flight together)
constexpr uint64_t kProducerWaitNs = 30000000000ull;
using XL = XLayout<1>;

struct LayerPeer {
  int world, rank;                       // world <= 1: no sum over ranks
  const __half* peer_y[kMaxPeers];       // rank r's partial result as mapped on this GPU
  int* peer_flags[kMaxPeers];            // rank r's flag array as mapped on this GPU
  int flag_base;
  __half* y_local;                       // this rank's partial result (= peer_y[rank])
};

struct LayerParams {
  CUtensorMap tm_w[4], tm_s[4];          // qkv, o, gate|up, down
  int N[4], K[4];
  const __half* x_in;                    // residual stream [H]
  const __half* delta_in;                // still to be added to it (previous layer's MLP output) or null
  __half* x_mid;                         // x_in + delta_in
  __half* qkv;                           // [3 * nh * 128]
  __half* attn;                          // [nh * 128]
  __half* o;                             // [H]
  __half* x_out;                         // x_mid + o: the residual stream the next layer gets
  __half* act;                           // [I]: silu(gate) * up
  __half* down;                          // [H]: the next layer's delta
  const __half* norm1;
  const __half* norm2;
  float eps;
  const float* cos_t;
  const float* sin_t;
  const int* pos;
  __half* k_cache;
  __half* v_cache;
  float* attn_scratch;                   // [nh][nsplit][130] floats
  int* attn_counters;                    // [nh], zero between steps
  int nh, max_ctx, nsplit;
  float scale_log2e;
  unsigned* bar;                         // 6 arrival counters of this layer: after stages 1..4, and the two "partial result complete" counts
  const int* step;                       // device scalar that grows by one per decode step
  uint64_t wait_ns;
  int nstages, kmax;
  int paired;                            // nibble order of the packed words (q4_common.cuh)
  LayerPeer peer_o, peer_down;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned atom_add_release_gpu(unsigned* p, unsigned v) {
  unsigned old;
  asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Order in which a CTA takes the row tiles of a matmul.  Plain: cta, cta + grid, ...  Paired (gate | up): the
// gate tile and the up tile of the same 16 outputs one after the other: pair p = cta, cta + grid, ... gives
// tiles p and p + half.
struct TileOrder {
  int count;      // tiles this CTA takes
  int cta, grid, half;
  __device__ TileOrder(int N, bool paired, int cta_, int grid_) : cta(cta_), grid(grid_) {
    const int ntiles = (N + kRows - 1) / kRows;
    half = paired ? ntiles / 2 : 0;
    const int units = paired ? half : ntiles;
    const int mine = cta < units ? (units - cta + grid - 1) / grid : 0;
    count = paired ? 2 * mine : mine;
  }
  __device__ int tile(int i) const { return half ? cta + (i >> 1) * grid + (i & 1) * half : cta + i * grid; }
};

__global__ void __launch_bounds__(kThreads, 1)
q4f16_decode_layer_kernel(const __grid_constant__ LayerParams p) {
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* ring = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)p.nstages * kStageBytes);
  uint64_t* empty = full + kMaxStages;
  uint64_t* red_full = empty + kMaxStages;
  uint64_t* red_empty = red_full + kNumRed;
  uint4* xs = reinterpret_cast<uint4*>(red_empty + kNumRed + (kNumRed & 1));     // 16-byte aligned
  float* negcorr = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + XL::bytes(p.kmax));
  float* red = negcorr + (p.kmax >> 8) * 32;

  __shared__ int s_abort;
  __shared__ uint4 s_zero;
  __shared__ float s_part[CW];
  __shared__ float s_inv;
  __shared__ float sm_m[4][4], sm_l[4][4], sm_acc[4][4][128];
  __shared__ int s_last[4];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int grid = (int)gridDim.x;

  if (tid == 0) {
    s_abort = 0;
    s_zero = make_uint4(0, 0, 0, 0);
    for (int s = 0; s < p.nstages; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], CW);
    }
    for (int s = 0; s < kNumRed; ++s) {
      mbar_init(&red_full[s], CW);
      mbar_init(&red_empty[s], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  // Polls an arrival counter until it reaches `target` (counters only grow; compared wrap-safe).  Bounded.
  auto grid_wait = [&](const unsigned* ctr, unsigned target) {
    if (*(volatile int*)&s_abort) return;
    const uint64_t t0 = globaltimer_ns();
    while ((int)(ld_acquire_gpu(ctr) - target) < 0) {
      if (globaltimer_ns() - t0 > p.wait_ns) {
        atomicOr(&g_layer_error, 32);
        *(volatile int*)&s_abort = 1;
        return;
      }
    }
  };

  // Stage 2.  The attention warps in groups of four; a group takes (head, 128-token chunk) units.  Every lane has
  // the K and V loads of 16 of its warp's tokens in flight at once.  The group that arrives last for a head merges
  // that head's chunks.  `aw` = index among the attention warps.
  auto attention_stage = [&](int aw) {
    const int grp4 = aw >> 2;
    const int wl = aw & 3;
    const int gt = wl * 32 + lane;                 // thread within the group
    const int pos = p.pos[0];
    const int ctx = pos + 1;
    const int used = (ctx + kAttnChunk - 1) / kAttnChunk;
    const int nunits = p.nh * used;
    const int nh = p.nh;
    const int d0 = lane * 4;
    const int r0 = d0 & 63;
    const int64_t tok_stride = (int64_t)nh * 128;
    // (the rotation angles only depend on the position: fetched before the wait)
    const float4 cs = *reinterpret_cast<const float4*>(p.cos_t + (int64_t)pos * 64 + r0);
    const float4 sn = *reinterpret_cast<const float4*>(p.sin_t + (int64_t)pos * 64 + r0);
    const unsigned target = ((unsigned)*p.step + 1u) * (unsigned)grid;
    if (aw == 0 && lane == 0) grid_wait(&p.bar[0], target);
    bar_sync(2, kAttnThreads);
    const float c[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
    const float sign = lane < 16 ? -1.f : 1.f;
    auto rotate = [&](const __half* v, float (&o)[4]) {
      const uint2 raw = *reinterpret_cast<const uint2*>(v + d0);
      const __half2* hh = reinterpret_cast<const __half2*>(&raw);
      const float2 a = __half22float2(hh[0]), e = __half22float2(hh[1]);
      const float mine[4] = {a.x, a.y, e.x, e.y};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, mine[j], 16);
        o[j] = __half2float(__float2half_rn(mine[j] * c[j] + sign * other * sv[j]));
      }
    };
    for (int unit = (int)blockIdx.x * kAttnGroups + grp4; unit < nunits; unit += kAttnGroups * grid) {
      const int h = unit / used, split = unit - h * used;
      const int t0 = split * kAttnChunk;
      const int t1 = min(ctx, t0 + kAttnChunk);
      float* part = p.attn_scratch + ((int64_t)h * p.nsplit + split) * 130;
      const __half* kb = p.k_cache + (int64_t)h * 128 + d0;
      const __half* vb = p.v_cache + (int64_t)h * 128 + d0;
      uint2 kv[kTok], vv[kTok];
      auto load_round = [&](int tb) {
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
          const int tk = min(tb + j, t1 - 1);        // clamped: a token past the end is loaded but not used
          kv[j] = *reinterpret_cast<const uint2*>(kb + tk * tok_stride);
          vv[j] = *reinterpret_cast<const uint2*>(vb + tk * tok_stride);
        }
      };
      const int tb0 = t0 + wl * kTok;
      if (split == used - 1) {
        if (wl == 0) {
          // the new token belongs to this chunk: its rotated k and its v go into the caches first
          float kr[4];
          rotate(p.qkv + (nh + h) * 128, kr);
          const int64_t slot = ((int64_t)pos * nh + h) * 128 + d0;
          uint2 kw;
          __half2* kh2 = reinterpret_cast<__half2*>(&kw);
          kh2[0] = __floats2half2_rn(kr[0], kr[1]);
          kh2[1] = __floats2half2_rn(kr[2], kr[3]);
          *reinterpret_cast<uint2*>(p.k_cache + slot) = kw;
          *reinterpret_cast<uint2*>(p.v_cache + slot) = *reinterpret_cast<const uint2*>(p.qkv + (2 * nh + h) * 128 + d0);
        }
        bar_sync(4 + grp4, 128);                   // the appended token is visible to the group
      }
      if (tb0 < t1) load_round(tb0);               // in flight while q is fetched and rotated
      float qf[4];
      rotate(p.qkv + h * 128, qf);
#pragma unroll
      for (int j = 0; j < 4; ++j) qf[j] *= p.scale_log2e;
      float m = -INFINITY, l = 0.f, av[4] = {0.f, 0.f, 0.f, 0.f};
      for (int tb = tb0; tb < t1; tb += 4 * kTok) {
        if (tb != tb0) load_round(tb);
        float sc[kTok];
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
          const __half2* kh = reinterpret_cast<const __half2*>(&kv[j]);
          const float2 k01 = __half22float2(kh[0]), k23 = __half22float2(kh[1]);
          sc[j] = qf[0] * k01.x + qf[1] * k01.y + qf[2] * k23.x + qf[3] * k23.y;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int j = 0; j < kTok; ++j) sc[j] += __shfl_xor_sync(0xffffffffu, sc[j], o);
        float mn = m;
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
          if (tb + j >= t1) sc[j] = -INFINITY;
          mn = fmaxf(mn, sc[j]);
        }
        const float corr = exp2f(m - mn);
        l *= corr;
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] *= corr;
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
          const float pj = exp2f(sc[j] - mn);
          const __half2* vh = reinterpret_cast<const __half2*>(&vv[j]);
          const float2 v01 = __half22float2(vh[0]), v23 = __half22float2(vh[1]);
          l += pj;
          av[0] += pj * v01.x;
          av[1] += pj * v01.y;
          av[2] += pj * v23.x;
          av[3] += pj * v23.y;
        }
        m = mn;
      }
      if (lane == 0) { sm_m[grp4][wl] = m; sm_l[grp4][wl] = l; }
#pragma unroll
      for (int j = 0; j < 4; ++j) sm_acc[grp4][wl][lane * 4 + j] = av[j];
      bar_sync(4 + grp4, 128);
      {
        const float M = fmaxf(fmaxf(sm_m[grp4][0], sm_m[grp4][1]), fmaxf(sm_m[grp4][2], sm_m[grp4][3]));
        float L = 0.f, A = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < 4; ++w2) {
          const float f = (sm_m[grp4][w2] == -INFINITY) ? 0.f : exp2f(sm_m[grp4][w2] - M);
          L += sm_l[grp4][w2] * f;
          A += sm_acc[grp4][w2][gt] * f;
        }
        part[2 + gt] = A;
        if (gt == 0) { part[0] = M; part[1] = L; }
      }
      // the group that arrives last for this head merges the chunks
      __threadfence();
      bar_sync(4 + grp4, 128);
      if (gt == 0) s_last[grp4] = atomicAdd(&p.attn_counters[h], 1) == used - 1;
      bar_sync(4 + grp4, 128);
      if (s_last[grp4]) {
        __threadfence();
        if (gt == 0) p.attn_counters[h] = 0;
        const float* pp = p.attn_scratch + (int64_t)h * p.nsplit * 130;
        float M = -INFINITY, L = 0.f, A = 0.f;
        for (int s0 = 0; s0 < used; s0 += 16) {
          float Ms[16], Ls[16], As[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int si = min(s0 + j, used - 1);
            Ms[j] = __ldcg(pp + si * 130);
            Ls[j] = __ldcg(pp + si * 130 + 1);
            As[j] = __ldcg(pp + si * 130 + 2 + gt);
          }
          float Mn = M;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (s0 + j < used) Mn = fmaxf(Mn, Ms[j]);
          const float corr = exp2f(M - Mn);
          L *= corr;
          A *= corr;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (s0 + j < used) {
              const float f = exp2f(Ms[j] - Mn);
              L += Ls[j] * f;
              A += As[j] * f;
            }
          }
          M = Mn;
        }
        p.attn[h * 128 + gt] = __float2half_rn(A / L);
      }
      bar_sync(4 + grp4, 128);                     // sm_* and s_last are free for the next unit
    }
    // every attention warp of the CTA is through: the CTA signs off
    __threadfence();
    bar_sync(2, kAttnThreads);
    if (aw == 0 && lane == 0) atom_add_release_gpu(&p.bar[1], 1u);
  };

  if (kAttnHelpers > 0 && warp >= CW + 2) {
    // ------------------------------------------------------------------ attention helpers
    pdl_wait();
    attention_stage(warp - 2);
    return;
  }

  if (warp == CW) {
    // ------------------------------------------------------------------ producer warp
    // lane 0 streams the packed weights, lane 1 the scales of this CTA's tiles of the four matrices, in the
    // order the consumers take them.  It never looks at the activations, so it runs ahead of every barrier.
    const bool is_w = lane == 0;
    if (lane < 2) {
      const uint64_t policy = policy_evict_first();
      int s = 0;
      uint32_t round = 0;
      bool dead = false;
      auto produce = [&](const CUtensorMap* tw, const CUtensorMap* ts, int N, int K, bool paired) {
        if (dead) return;
        prefetch_tmap(is_w ? tw : ts);
        const TileOrder order(N, paired, (int)blockIdx.x, grid);
        const int kpad = ((K + KC - 1) / KC) * KC;
        for (int ti = 0; ti < order.count; ++ti) {
          const int tile = order.tile(ti);
          for (int k0 = 0; k0 < kpad; k0 += KC, s = (s + 1 == p.nstages ? 0 : s + 1), round += (s == 0)) {
            if (round > 0) {
              if (*(volatile int*)&s_abort || !mbar_wait_ns_relaxed(&empty[s], (round - 1) & 1, kProducerWaitNs)) {
                atomicOr(&g_layer_error, 1);
                *(volatile int*)&s_abort = 1;
                dead = true;
                return;
              }
            }
            unsigned char* st = ring + (size_t)s * kStageBytes;
            if (is_w) {
              mbar_arrive_expect_tx(&full[s], kWBytes);
              tma_load_3d_hint(st, tw, 0, tile * kRows, k0 >> 8, &full[s], policy);
            } else {
              mbar_arrive_expect_tx(&full[s], kSBytes);
              tma_load_3d_hint(st + kWBytes, ts, 0, tile * kRows, k0 >> 8, &full[s], policy);
            }
          }
        }
      };
      produce(&p.tm_w[0], &p.tm_s[0], p.N[0], p.K[0], false);
      produce(&p.tm_w[1], &p.tm_s[1], p.N[1], p.K[1], false);
      produce(&p.tm_w[2], &p.tm_s[2], p.N[2], p.K[2], true);
      produce(&p.tm_w[3], &p.tm_s[3], p.N[3], p.K[3], false);
    }
    return;
  }

  if (warp == CW + 1) {
    // ------------------------------------------------------------------ epilogue warp
    // Adds up the consumer warps' partial sums of each finished tile (in warp order), stores fp16, and after
    // the last tile of a matmul signs this CTA off at the stage's counter.  For the two row-parallel matmuls
    // under tensor parallelism it also runs the sum over ranks.
    pdl_wait();
    const unsigned step1 = (unsigned)*p.step + 1u;
    const unsigned target = step1 * (unsigned)grid;
    int rb = 0;
    uint32_t rround = 0;
    // paired: the tiles come as (gate, up) of the same 16 outputs; what is stored is silu(gate) * up, both rounded
    // to fp16 first as the matmul's own output would be
    auto finish = [&](int N, __half* y, bool paired) {
      const TileOrder order(N, paired, (int)blockIdx.x, grid);
      float gate = 0.f;
      for (int ti = 0; ti < order.count; ++ti) {
        const int tile = order.tile(ti);
        if (!mbar_try_wait(&red_full[rb], rround & 1)) {
          if (!*(volatile int*)&s_abort && !mbar_wait_ns_relaxed(&red_full[rb], rround & 1, kProducerWaitNs)) {
            atomicOr(&g_layer_error, 4);
            *(volatile int*)&s_abort = 1;
          }
        }
        const float* rbuf = red + rb * (CW * kOut);
        float sum = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < CW; ++w2) sum += rbuf[w2 * kOut + lane];
        const int row = tile * kRows + (lane >> 1);
        if (!paired) {
          if ((lane & 1) == 0 && row < N) y[row] = __float2half_rn(sum);
        } else if ((ti & 1) == 0) {
          gate = __half2float(__float2half_rn(sum));
        } else {
          const float up = __half2float(__float2half_rn(sum));
          if ((lane & 1) == 0) y[row - order.half * kRows] = __float2half_rn(gate / (1.f + __expf(-gate)) * up);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&red_empty[rb]);
        rb = rb + 1 == kNumRed ? 0 : rb + 1;
        rround += (rb == 0);
      }
      __syncwarp();
    };
    // this CTA's stores are fenced, then it is counted
    auto sign_off = [&](unsigned* ctr) -> unsigned {
      unsigned old = 0;
      __syncwarp();
      if (lane == 0) {
        __threadfence();
        old = atom_add_release_gpu(ctr, 1u);
      }
      return __shfl_sync(0xffffffffu, old, 0);
    };
    // Sum over tensor-parallel ranks of a row-parallel matmul's partial results (N outputs), in rank order, by
    // plain loads from the peers' memory.  The CTA that completes this GPU's partial result tells every rank.
    auto peer_sum = [&](const LayerPeer& pr, unsigned* partial_ctr, int N, __half* out) {
      const unsigned old = sign_off(partial_ctr);
      if (old + 1u == target) {
        __threadfence_system();
        if (lane < pr.world) st_release_sys(pr.peer_flags[lane] + pr.flag_base + pr.rank, (int)step1);
      }
      if (lane < pr.world && !*(volatile int*)&s_abort) {
        const int* f = pr.peer_flags[pr.rank] + pr.flag_base + lane;
        const uint64_t t0 = globaltimer_ns();
        while (ld_acquire_sys(f) < (int)step1) {
          if (globaltimer_ns() - t0 > p.wait_ns) {
            atomicOr(&g_layer_error, 16);
            *(volatile int*)&s_abort = 1;
            break;
          }
        }
      }
      __syncwarp();
      const int n8 = N >> 3;
      for (int i = blockIdx.x + lane * grid; i < n8; i += 32 * grid) {
        uint4 v[kMaxPeers];
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
          if (r < pr.world) v[r] = ld_volatile_v4(pr.peer_y[r] + (int64_t)i * 8);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r) {
          if (r < pr.world) {
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
        *reinterpret_cast<uint4*>(out + (int64_t)i * 8) = o;
      }
    };

    finish(p.N[0], p.qkv, false);
    sign_off(&p.bar[0]);
    if (p.peer_o.world > 1) {
      finish(p.N[1], p.peer_o.y_local, false);
      peer_sum(p.peer_o, &p.bar[4], p.N[1], p.o);
    } else {
      finish(p.N[1], p.o, false);
    }
    sign_off(&p.bar[2]);
    finish(p.N[2], p.act, true);
    sign_off(&p.bar[3]);
    if (p.peer_down.world > 1) {
      finish(p.N[3], p.peer_down.y_local, false);
      peer_sum(p.peer_down, &p.bar[5], p.N[3], p.down);
    } else {
      finish(p.N[3], p.down, false);
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int g = lane >> 2;
  const int t = lane & 3;
  const uint32_t w_off = (uint32_t)((warp * kRows + g) * 128 + (((2 * t) ^ g) << 4));
  const uint32_t s_off = (uint32_t)(kWBytes + (warp * kRows + g) * 16 + (t & 1) * 8);
  const uint4* x_thr = xs + (warp * 36 + 9 * t);
  constexpr int kXStage = CH * XL::kSlotsPerChunk;
  constexpr int kXUnit = CW * XL::kSlotsPerChunk;
  const bool x_own = g == t;
  const int x_mul = x_own ? 1 : 0;
  const float4* c_thr = reinterpret_cast<const float4*>(negcorr) + warp * 8 + (t & 1) * 2;
  constexpr int kCStage = CH * 8;
  constexpr int kCUnit = CW * 8;
  const Q4Consts qc = q4_consts();
  const uint32_t magic_hi = 0x54005400u;

  int s = 0;
  uint32_t round = 0;
  int rb = 0;
  uint32_t rround = 0;
  float acc0, acc1, acc2, acc3;          // row g: even / odd groups, row g+8: even / odd groups

  // the U chunks of one stage (see fast_stage in gemv_pipe.cu)
  auto fast_stage = [&](const uint4 (&w)[U][2][2], const uint2 (&sc)[U][2], const uint4* xu, const float4* cu) {
    float d[U][2][4];
    const uint4* xb = x_own ? xu : &s_zero;
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
      uint32_t a[U][2][8];
      uint4 b[U][2];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t w0 = wd == 0 ? w[u][0][h].x : wd == 1 ? w[u][0][h].y : wd == 2 ? w[u][0][h].z : w[u][0][h].w;
          const uint32_t w1 = wd == 0 ? w[u][1][h].x : wd == 1 ? w[u][1][h].y : wd == 2 ? w[u][1][h].z : w[u][1][h].w;
          b[u][h] = xb[x_mul * (u * kXUnit + 4 * h + wd)];
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
      for (int u = 0; u < U; ++u)
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
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          mma_16x8x16(d[u][h], a[u][h][4], a[u][h][5], a[u][h][6], a[u][h][7], b[u][h].z, b[u][h].w);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float2 g01 = __half22float2(u32_as_h2(sc[u][0].x)), g23 = __half22float2(u32_as_h2(sc[u][0].y));
      const float2 h01 = __half22float2(u32_as_h2(sc[u][1].x)), h23 = __half22float2(u32_as_h2(sc[u][1].y));
      acc0 = fmaf(g01.x, d[u][0][0], acc0);
      acc0 = fmaf(g23.x, d[u][0][1], acc0);
      acc1 = fmaf(g01.y, d[u][1][0], acc1);
      acc1 = fmaf(g23.y, d[u][1][1], acc1);
      acc2 = fmaf(h01.x, d[u][0][2], acc2);
      acc2 = fmaf(h23.x, d[u][0][3], acc2);
      acc3 = fmaf(h01.y, d[u][1][2], acc3);
      acc3 = fmaf(h23.y, d[u][1][3], acc3);
    }
  };
  auto fast_load = [&](uint4 (&w)[U][2][2], uint2 (&sc)[U][2]) {
    if (!mbar_try_wait(&full[s], round & 1)) {
      if (!*(volatile int*)&s_abort && !mbar_wait_ns(&full[s], round & 1, p.wait_ns)) {
        atomicOr(&g_layer_error, 2);
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
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    s = s + 1 == p.nstages ? 0 : s + 1;
    round += (s == 0);
  };
  // one staged word (eight activations) in the order the unpack produces; returns its offset sum
  auto stage_word = [&](int j, const uint4& v) -> float {
    xs[XL::slot(j, 0)] = staged_order(v, p.paired != 0);
    return offset_sum_f16x8(v, p.paired != 0);
  };
  auto store_group_sum = [&](int grp, float psum) {
    const int ci = corr_index(grp);
    negcorr[ci] = -psum;
    negcorr[ci + 2] = -psum;
  };

  // Stages the activation vector of a matmul with K inputs (zero up to the next multiple of a stage's k):
  //   kind 0: src as it is            kind 1: rmsnorm(src + add) * nw, src + add also to `sum_out` (CTA 0)
  //   kind 2: silu(src[0:K]) * src[K:2K]
  // A thread takes whole scale groups (four words), so the offset sums need no exchange.
  auto stage_x = [&](int kind, const __half* src, const __half* add, const __half* nw, __half* sum_out, int K) {
    const int kpad = ((K + KC - 1) / KC) * KC;
    const int groups = kpad >> 5;
    float inv = 1.f;
    if (kind == 1 && K <= kConsumers * 16) {
      // a row of at most 2 * 8 * 256 values: a thread's two 8-value words are the same in the statistics pass and in
      // the staging pass, so the three vectors are loaded once, all loads in flight together, and kept in registers
      uint4 keep[2], nwv[2], dl[2];
      bool live[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int k = (tid + r * kConsumers) * 8;
        live[r] = k < K;
        keep[r] = nwv[r] = dl[r] = make_uint4(0, 0, 0, 0);
        if (live[r]) {
          keep[r] = *reinterpret_cast<const uint4*>(src + k);
          if (add) dl[r] = *reinterpret_cast<const uint4*>(add + k);
          nwv[r] = *reinterpret_cast<const uint4*>(nw + k);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        if (!live[r]) continue;
        const int k = (tid + r * kConsumers) * 8;
        if (add) keep[r] = add_f16x8(keep[r], dl[r]);
        if (sum_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(sum_out + k) = keep[r];
        const __half2* h = reinterpret_cast<const __half2*>(&keep[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) s_part[warp] = ss;
      bar_sync(1, kConsumers);
      float tot = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < CW; ++w2) tot += s_part[w2];
      inv = rsqrtf(tot / (float)K + p.eps);
      const int words = kpad >> 3;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int j = tid + r * kConsumers;
        if (j >= words) continue;                // (words is a multiple of 32: whole warps leave together)
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j * 8 < K) v = scale_f16x8(keep[r], inv, nwv[r]);
        float psum = stage_word(j, v);
        psum += __shfl_xor_sync(0xffffffffu, psum, 1);       // a group's four words sit in four consecutive lanes
        psum += __shfl_xor_sync(0xffffffffu, psum, 2);
        if ((j & 3) == 0) store_group_sum(j >> 2, psum);
      }
      // words beyond the two a thread holds (K < the padded length): zeros
      for (int j = tid + 2 * kConsumers; j < words; j += kConsumers) {
        float psum = stage_word(j, make_uint4(0, 0, 0, 0));
        if ((j & 3) == 0) store_group_sum(j >> 2, psum);
      }
      bar_sync(1, kConsumers);
      return;
    }
    if (kind == 1) {
      float ss = 0.f;
      for (int k = tid * 8; k < K; k += kConsumers * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(src + k);
        if (add) v = add_f16x8(v, *reinterpret_cast<const uint4*>(add + k));
        if (sum_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(sum_out + k) = v;
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) s_part[warp] = ss;
      bar_sync(1, kConsumers);
      if (tid == 0) {
        float tot = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < CW; ++w2) tot += s_part[w2];
        s_inv = rsqrtf(tot / (float)K + p.eps);
      }
      bar_sync(1, kConsumers);
      inv = s_inv;
    }
    for (int grp = tid; grp < groups; grp += kConsumers) {
      const int k = grp * 32;
      const bool live = k < K;
      uint4 a[4], b[4], c[4];
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        a[wd] = b[wd] = c[wd] = make_uint4(0, 0, 0, 0);
        if (live) {
          a[wd] = *reinterpret_cast<const uint4*>(src + k + 8 * wd);
          if (kind == 2) b[wd] = *reinterpret_cast<const uint4*>(src + K + k + 8 * wd);
          if (kind == 1) {
            if (add) b[wd] = *reinterpret_cast<const uint4*>(add + k + 8 * wd);
            c[wd] = *reinterpret_cast<const uint4*>(nw + k + 8 * wd);
          }
        }
      }
      float psum = 0.f;
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        uint4 v = a[wd];
        if (live) {
          if (kind == 2) {
            v = silu_mul_f16x8(a[wd], b[wd]);
          } else if (kind == 1) {
            if (add) v = add_f16x8(v, b[wd]);
            v = scale_f16x8(v, inv, c[wd]);
          }
        }
        psum += stage_word(4 * grp + wd, v);
      }
      store_group_sum(grp, psum);
    }
    bar_sync(1, kConsumers);
  };

  // This CTA's row tiles of one matmul; `have` says that the first stage is already in fw / fsc.
  uint4 fw[U][2][2];
  uint2 fsc[U][2];
  auto gemv_tiles = [&](int N, int K, bool have, bool paired) {
    const TileOrder order(N, paired, (int)blockIdx.x, grid);
    const int kpad = ((K + KC - 1) / KC) * KC;
    for (int ti = 0; ti < order.count; ++ti) {
      acc0 = acc1 = acc2 = acc3 = 0.f;
      const uint4* xk = x_thr;
      const float4* ck = c_thr;
      for (int k0 = 0; k0 < kpad; k0 += KC, xk += kXStage, ck += kCStage) {
        if (!have) fast_load(fw, fsc);
        have = false;
        fast_stage(fw, fsc, xk, ck);
      }
      if (rround > 0 && !mbar_try_wait(&red_empty[rb], (rround - 1) & 1)) {
        if (!*(volatile int*)&s_abort && !mbar_wait_ns(&red_empty[rb], (rround - 1) & 1, p.wait_ns)) {
          atomicOr(&g_layer_error, 8);
          *(volatile int*)&s_abort = 1;
        }
      }
      float lo = acc0 + acc1, hi = acc2 + acc3;
      lo += __shfl_xor_sync(0xffffffffu, lo, 1);
      hi += __shfl_xor_sync(0xffffffffu, hi, 1);
      float* rbuf = red + rb * (CW * kOut) + warp * kOut;
      if (t == 0) {
        *reinterpret_cast<float2*>(rbuf + g * 2) = make_float2(lo, 0.f);
        *reinterpret_cast<float2*>(rbuf + (g + 8) * 2) = make_float2(hi, 0.f);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_full[rb]);
      rb = rb + 1 == kNumRed ? 0 : rb + 1;
      rround += (rb == 0);
    }
  };
  // every consumer warp waits until every CTA has signed off at `ctr`
  auto wait_stage = [&](const unsigned* ctr, unsigned target) {
    if (tid == 0) grid_wait(ctr, target);
    bar_sync(1, kConsumers);
  };

  // ---- stage 1: q | k | v ------------------------------------------------------------------------
  // The weights do not depend on the previous kernel: this warp's share of the first stage is in registers
  // before the wait for the activations returns.
  const bool pre = (int)blockIdx.x < (p.N[0] + kRows - 1) / kRows;
  if (pre) fast_load(fw, fsc);
  pdl_wait();
  const unsigned target = ((unsigned)*p.step + 1u) * (unsigned)grid;
  stage_x(1, p.x_in, p.delta_in, p.norm1, p.x_mid, p.K[0]);
  gemv_tiles(p.N[0], p.K[0], pre, false);

  // ---- stage 2: rotary embedding, KV append, attention over the cache --------------------------------
  attention_stage(warp);

  // ---- stage 3: o projection ------------------------------------------------------------------------
  wait_stage(&p.bar[1], target);
  stage_x(0, p.attn, nullptr, nullptr, nullptr, p.K[1]);
  gemv_tiles(p.N[1], p.K[1], false, false);

  // ---- stage 4: gate | up -----------------------------------------------------------------------------
  wait_stage(&p.bar[2], target);
  stage_x(1, p.x_mid, p.o, p.norm2, p.x_out, p.K[2]);
  gemv_tiles(p.N[2], p.K[2], false, true);

  // ---- stage 5: down projection ------------------------------------------------------------------------
  wait_stage(&p.bar[3], target);
  stage_x(0, p.act, nullptr, nullptr, nullptr, p.K[3]);
  gemv_tiles(p.N[3], p.K[3], false, false);

  if (*(volatile int*)&s_abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

int fill_maps(LayerParams& p, int d, const void* wq, const void* scales, int64_t N, int64_t K) {
  if (K % 256 != 0 || (reinterpret_cast<uintptr_t>(scales) & 15u) || (reinterpret_cast<uintptr_t>(wq) & 15u))
    return fail(B200_EINVAL, "decode_layer: matmul %d needs K %% 256 == 0 and 16-byte aligned weights and scales", d);
  const uint64_t wd[3] = {32, (uint64_t)N, (uint64_t)(K / 256)};
  const uint64_t ws[2] = {(uint64_t)K / 2, 128};
  const uint32_t wb[3] = {32, kRows, CH};
  int rc = make_tmap(&p.tm_w[d], CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, wq, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  const uint64_t sd[3] = {8, (uint64_t)N, (uint64_t)(K / 256)};
  const uint64_t ss[2] = {(uint64_t)(K / 32) * 2, 16};
  const uint32_t sb[3] = {8, kRows, CH};
  rc = make_tmap(&p.tm_s[d], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, scales, sd, ss, sb, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  p.N[d] = (int)N;
  p.K[d] = (int)K;
  return B200_OK;
}

int fill_peer(LayerPeer& lp, const B200PeerReduce* r, const char* what) {
  lp = LayerPeer{};
  if (!r || r->world <= 1) return B200_OK;
  if (r->world > kMaxPeers || r->rank < 0 || r->rank >= r->world) return fail(B200_EINVAL, "decode_layer: %s: world %d / rank %d out of range", what, r->world, r->rank);
  lp.world = r->world;
  lp.rank = r->rank;
  for (int i = 0; i < r->world; ++i) {
    if (!r->peer_y[i] || !r->peer_flags[i] || (reinterpret_cast<uintptr_t>(r->peer_y[i]) & 15u))
      return fail(B200_EINVAL, "decode_layer: %s: peer %d has a null or misaligned buffer", what, i);
    lp.peer_y[i] = static_cast<const __half*>(r->peer_y[i]);
    lp.peer_flags[i] = static_cast<int*>(r->peer_flags[i]);
  }
  lp.flag_base = r->flag_base;
  lp.y_local = const_cast<__half*>(lp.peer_y[r->rank]);
  return B200_OK;
}

}  // namespace

int layer_error_read_and_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_layer_error, sizeof(int)) != cudaSuccess) return 0xff;
  if (v) cudaMemcpyToSymbol(g_layer_error, &zero, sizeof(int));
  return v & 0xff;
}

}  // namespace b200

using namespace b200;

extern "C" {

int64_t b200_decode_layer_scratch_bytes(int64_t nh, int64_t max_ctx) {
  const int64_t nsplit = (max_ctx + kAttnChunk - 1) / kAttnChunk;
  // attention partials, then per-head arrival counters, then the six stage counters
  return nh * nsplit * 130 * (int64_t)sizeof(float) + nh * (int64_t)sizeof(int) + 8 * (int64_t)sizeof(unsigned);
}

int b200_decode_layer(const B200DecodeLayer* a, void* stream) {
  const char* who = "decode_layer";
  if (!a) return fail(B200_EINVAL, "%s: null descriptor", who);
  if (a->hidden <= 0 || a->hidden % 256 != 0 || a->heads <= 0 || a->inter_local <= 0 || a->inter_local % 256 != 0 || a->max_ctx <= 0)
    return fail(B200_EINVAL, "%s: hidden and inter_local must be positive multiples of 256, heads and max_ctx positive", who);
  if (a->world < 1 || a->world > 8 || a->heads % a->world != 0 || a->hidden % (a->world * 256) != 0)
    return fail(B200_EINVAL, "%s: world %d does not divide %d heads / hidden %lld into whole 256-blocks", who, a->world, a->heads, (long long)a->hidden);
  if (a->hidden != (int64_t)a->heads * 128) return fail(B200_EINVAL, "%s: heads of 128 dimensions only (hidden = heads * 128)", who);
  const void* need[] = {a->x_in, a->x_mid, a->qkv, a->attn, a->o, a->x_out, a->act, a->down, a->norm1, a->norm2, a->cos_t, a->sin_t, a->pos,
                        a->k_cache, a->v_cache, a->scratch, a->step, a->wq_qkv, a->s_qkv, a->wq_o, a->s_o, a->wq_gu, a->s_gu, a->wq_down, a->s_down};
  for (const void* ptr : need)
    if (!ptr) return fail(B200_EINVAL, "%s: null pointer in the descriptor", who);
  for (const void* ptr : {a->x_in, (const void*)a->x_mid, (const void*)a->qkv, (const void*)a->attn, (const void*)a->o, (const void*)a->x_out,
                          (const void*)a->act, (const void*)a->down, a->norm1, a->norm2, a->delta_in})
    if (reinterpret_cast<uintptr_t>(ptr) & 15u) return fail(B200_EINVAL, "%s: activation buffers must be 16-byte aligned", who);
  if (a->x_mid == a->x_in || a->x_out == a->x_mid) return fail(B200_EINVAL, "%s: x_mid must not alias x_in, nor x_out x_mid (other CTAs still read them)", who);
  int rc = ensure_device();
  if (rc) return rc;

  LayerParams p{};
  const int64_t H = a->hidden, hl = H / a->world, il = a->inter_local;
  const int nh = a->heads / a->world;
  if ((rc = fill_maps(p, 0, a->wq_qkv, a->s_qkv, 3 * hl, H))) return rc;
  if ((rc = fill_maps(p, 1, a->wq_o, a->s_o, H, hl))) return rc;
  if ((rc = fill_maps(p, 2, a->wq_gu, a->s_gu, 2 * il, H))) return rc;
  if ((rc = fill_maps(p, 3, a->wq_down, a->s_down, H, il))) return rc;
  p.x_in = (const __half*)a->x_in; p.delta_in = (const __half*)a->delta_in; p.x_mid = (__half*)a->x_mid;
  p.qkv = (__half*)a->qkv; p.attn = (__half*)a->attn; p.o = (__half*)a->o; p.x_out = (__half*)a->x_out;
  p.act = (__half*)a->act; p.down = (__half*)a->down;
  p.norm1 = (const __half*)a->norm1; p.norm2 = (const __half*)a->norm2; p.eps = a->eps;
  p.paired = current_layout() == kLayoutPaired;
  p.cos_t = (const float*)a->cos_t; p.sin_t = (const float*)a->sin_t; p.pos = (const int*)a->pos;
  p.k_cache = (__half*)a->k_cache; p.v_cache = (__half*)a->v_cache;
  p.nh = nh; p.max_ctx = (int)a->max_ctx;
  p.nsplit = (int)((a->max_ctx + kAttnChunk - 1) / kAttnChunk);
  p.scale_log2e = 1.4426950408889634f / sqrtf(128.f);
  p.attn_scratch = (float*)a->scratch;
  p.attn_counters = reinterpret_cast<int*>(p.attn_scratch + (int64_t)nh * p.nsplit * 130);
  p.bar = reinterpret_cast<unsigned*>(p.attn_counters + nh);
  p.step = (const int*)a->step;
  p.wait_ns = (uint64_t)options().layer_wait_ms * 1000000ull;
  if ((rc = fill_peer(p.peer_o, a->world > 1 ? &a->reduce_o : nullptr, "o projection"))) return rc;
  if ((rc = fill_peer(p.peer_down, a->world > 1 ? &a->reduce_down : nullptr, "down projection"))) return rc;
  if (a->world > 1 && (p.peer_o.world != a->world || p.peer_down.world != a->world))
    return fail(B200_EINVAL, "%s: world %d needs both reduction descriptors", who, a->world);

  int kmax = 0;
  for (int d = 0; d < 4; ++d) {
    const int kpad = ((p.K[d] + KC - 1) / KC) * KC;
    if (kpad > kmax) kmax = kpad;
  }
  p.kmax = kmax;
  const size_t kMaxSmem = 227 * 1024;
  auto need_bytes = [&](int stages) {
    return (size_t)1024 + (size_t)stages * kStageBytes + (2 * kMaxStages + 2 * kNumRed + 2) * sizeof(uint64_t) + XL::bytes(kmax) +
           (size_t)(kmax / 256) * 32 * sizeof(float) + (size_t)kNumRed * CW * kOut * sizeof(float);
  };
  int stages = (int)options().layer_stages;
  if (stages <= 0 || stages > kMaxStages) stages = kMaxStages;
  while (stages > 1 && need_bytes(stages) > kMaxSmem) --stages;
  const size_t smem = need_bytes(stages);
  if (smem > kMaxSmem) return fail(B200_EINVAL, "%s: activation vectors of %d values do not fit beside the weight ring", who, kmax);
  p.nstages = stages;

  auto kern = q4f16_decode_layer_kernel;
  static thread_local size_t attr_smem = 0;
  if (attr_smem != smem) {
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(B200_ELAUNCH, "%s: cudaFuncSetAttribute(%zu): %s", who, smem, cudaGetErrorString(e));
    attr_smem = smem;
  }
  int grid = sm_count();
  if (options().layer_max_ctas > 0 && grid > options().layer_max_ctas) grid = (int)options().layer_max_ctas;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "%s launch: %s", who, cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

}  // extern "C"
