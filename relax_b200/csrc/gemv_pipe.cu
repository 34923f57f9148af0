// Skinny q4f16 matmul, pipelined form: persistent CTAs fed by TMA.
//
// The register-streaming kernel in gemv.cu can keep only a couple of KB per warp in flight,
// far short of the ~40 KB per SM that HBM3e needs to stay busy, and many small bulk copies are
// bound by the TMA unit's per-instruction cost (measured here: one issuing thread sustains
// about 2.2 tiled loads per microsecond whatever their size, so a load must carry ~32 KB).
// Two producer threads per CTA each issue one tiled TMA load per stage (32 KB of packed
// weights; 4 KB of scales) into a ring of shared-memory stages (~140 KB in flight per CTA)
// and eight consumer warps drain it:
//
//   stage      = 16 rows of W x 4096 k.  The weights are seen through a 3-D tensor map
//                (32 words = 256 k | row | 256-k chunk) so that one box {32,16,16} lands as
//                [chunk][row][128 B] with the 128-byte swizzle: the eight rows a warp reads in
//                one instruction then sit in eight different bank groups.  The scales use the
//                same trick with 16-byte units ([unit of 8 groups][row][16 B]).  Rows past N and
//                chunks past K are zero-filled by the TMA unit (zero scale => zero weight).
//   consumer w = lane (g,t) owns, for rows g and g+8, the 16-byte words (= scale groups) 2t+(w&1)
//                of chunks w/2 + 4j; it dequantises them (exact q-7, one HMUL2 by the scale, as
//                the reference rounds) and feeds mma.sync m16n8k16 with x fragments read from
//                a copy of x kept in shared memory in the matching permuted order
//   row tile   = 16 rows over the whole K range; partial sums of the 8 warps meet in shared
//                memory (double-buffered, one named barrier per tile) and are stored as fp16
//   CTA        = persistent: row tiles blockIdx.x, blockIdx.x + gridDim.x, ...
//
// When x does not fit beside the ring (large M*K) the K range is cut into blocks: x is restaged
// per block and per-tile partial sums are carried in a small shared-memory array.
//
// Programmatic dependent launch: the weights never depend on the previous kernel in the stream,
// so the producer starts copying before griddepcontrol.wait; only the consumers (which read x
// and write y) wait.  At ~110 KB of shared memory two consecutive launches fit on one SM, which
// hides the fill/drain bubble between back-to-back decode matmuls when shared memory allows.
//
// Requires K % 256 == 0 and 16-byte aligned scales (tensor-map stride rules); other shapes use
// the register-streaming kernel.
#include "internal.h"
#include "q4_common.cuh"
#include "sm100_ptx.cuh"
#include "tmap.h"

namespace b200 {

__device__ int g_gemv_pipe_error = 0;   // set when a bounded wait gives up

namespace {

using namespace ptx;

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 2) * 32;   // + one producer warp for weights, one for scales
constexpr int kChunks = 16;              // 256-k chunks per stage
constexpr int KC = 256 * kChunks;        // k per stage (4096)
constexpr int kRows = 16;                // rows per stage / row tile
constexpr int kWBytes = kChunks * kRows * 128;      // 32768: [chunk][row][128 B], 128B-swizzled
constexpr int kSBytes = kRows * (KC / 32) * 2;      // 4096:  [unit = chunk][row][8 scales = 16 B]
constexpr int kStageBytes = kWBytes + kSBytes;      // 36864 (a multiple of 1024, as the swizzle needs)
constexpr int kMaxStages = 6;
constexpr uint64_t kConsumerWaitNs = 2000000000ull;     // 2 s: a stage copy takes microseconds
constexpr uint64_t kProducerWaitNs = 30000000000ull;    // 30 s: may span the previous kernel's whole run

__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Layout of the staged x block: one 16-byte slot per (8-k word jw, batch column).  The four
// lanes t of a row-group read words 8 apart in the same instruction, so the slot index must
// differ mod 8 between them:
//   NC >= 8: NC slots per word, column XOR-ed with 2*((jw>>3)&3)  (= 2t);
//   NC <  8: NC+1 slots per word -- the extra column stays zero and is what lanes whose batch
//            column does not exist read, so the load needs no predicate -- plus 2 slots of padding
//            after every 8 words.
template <int NC>
struct XLayout {
  static constexpr int kSlotsPerWord = NC >= 8 ? NC : NC + 1;
  __device__ __forceinline__ static int slot(int jw, int col) {
    if (NC >= 8) return jw * NC + (col ^ (((jw >> 3) & 3) << 1));
    return jw * kSlotsPerWord + col + 2 * (jw >> 3);
  }
  // bytes for a block of `k` (multiple of 64)
  __host__ __device__ static constexpr size_t bytes(int k) {
    return NC >= 8 ? (size_t)NC * k * 2 : ((size_t)(k / 8) * kSlotsPerWord + 2 * (size_t)(k / 64)) * 16;
  }
};

struct PipeParams {
  CUtensorMap tm_w;   // uint32 {32, N, K/256}, box {32, 16, 16}, 128B swizzle
  CUtensorMap tm_s;   // fp16   {8, N, K/256},  box {8, 16, 16}
  const __half* x;
  __half* y;
  int M, N, K;
  int kblk;        // k per x block (multiple of KC, or >= K)
  int nstages;
  int ntiles;      // ceil(N / 16)
  int tiles_per_cta;
};

// Shared memory carve-up (after rounding the base up to 1024 bytes):
//   ring: nstages * kStageBytes
//   [.., +8*2*kMaxStages)          full / empty mbarriers
//   xs:   NC * kblk * 2            permuted x block
//   red:  2 * 8 * MT*128 * 4       cross-warp partial sums, double buffered
//   accs: tiles_per_cta * MT*128*4 (only when K is cut into several blocks)
template <int NC>
__global__ void __launch_bounds__(kThreads, 1)
q4f16_gemv_pipe_kernel(const __grid_constant__ PipeParams p) {
  constexpr int MT = (NC + 7) / 8;
  constexpr int kOut = MT * 128;           // outputs per row tile held in fragment order
  extern __shared__ unsigned char smem_unaligned[];
  // Round the base up to 1024 bytes by OFFSETTING the shared array (not by casting through an
  // integer): the compiler then still knows these are shared-memory addresses and emits LDS/STS.
  unsigned char* ring = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + (size_t)p.nstages * kStageBytes);
  uint64_t* empty = full + kMaxStages;
  uint4* xs = reinterpret_cast<uint4*>(empty + kMaxStages);
  float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + XLayout<NC>::bytes(p.kblk));
  float* accs = red + 2 * kConsumerWarps * kOut;

  __shared__ int s_abort;                    // set once a bounded wait gives up: later waits are skipped

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int nkb = (p.K + p.kblk - 1) / p.kblk;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < p.nstages; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp >= kConsumerWarps) {
    // ------------------------------------------------------------------ producer warps
    // warp 8 loads the packed weights, warp 9 the scales: one tiled load per stage each.
    const bool is_w = warp == kConsumerWarps;
    if (lane == 0) {
      prefetch_tmap(is_w ? &p.tm_w : &p.tm_s);
      const uint64_t policy = policy_evict_first();
      uint32_t it = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        const int k_lo = kb * p.kblk;
        const int k_hi = min(p.K, k_lo + p.kblk);
        for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
          const int row0 = tile * kRows;
          for (int k0 = k_lo; k0 < k_hi; k0 += KC, ++it) {
            const int s = it % p.nstages;
            const uint32_t round = it / p.nstages;
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
            if (is_w) {
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

  // -------------------------------------------------------------------- consumer warps
  const int g = lane >> 2;
  const int t = lane & 3;
  const int ctid = tid;                          // 0..255
  constexpr int kConsumers = kConsumerWarps * 32;

  pdl_wait();                                    // x may be the previous kernel's output

  uint32_t it = 0;
  uint32_t tile_parity = 0;
  for (int kb = 0; kb < nkb; ++kb) {
    const int k_lo = kb * p.kblk;
    const int k_hi = min(p.K, k_lo + p.kblk);
    // ---- stage x[:, k_lo .. k_lo + kblk) permuted per 8 k; zero beyond K and beyond M --------------
    if (kb > 0) bar_sync(1, kConsumers);         // everyone is done reading the previous block
    {
      const int words = p.kblk >> 3;
      constexpr int SPW = XLayout<NC>::kSlotsPerWord;
      for (int i = ctid; i < words * SPW; i += kConsumers) {
        int j = i / SPW, m = i - j * SPW;
        int k = k_lo + j * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m < p.M && k < p.K) v = *reinterpret_cast<const uint4*>(p.x + (int64_t)m * p.K + k);
        uint4 q;
        q.x = __byte_perm(v.x, v.z, 0x5410);
        q.y = __byte_perm(v.x, v.z, 0x7632);
        q.z = __byte_perm(v.y, v.w, 0x5410);
        q.w = __byte_perm(v.y, v.w, 0x7632);
        xs[XLayout<NC>::slot(j, m)] = q;
      }
    }
    bar_sync(1, kConsumers);

    int slot = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++slot) {
      float acc[2][MT][4];
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[a][mt][i] = 0.f;

      for (int k0 = k_lo; k0 < k_hi; k0 += KC, ++it) {
        const int s = it % p.nstages;
        const uint32_t round = it / p.nstages;
        // On a timeout the kernel keeps going without waiting (results are garbage, the error
        // flag says so) so that every warp still reaches the named barriers and the CTA ends.
        if (!*(volatile int*)&s_abort && !mbar_wait_ns(&full[s], round & 1, kConsumerWaitNs)) {
          atomicExch(&g_gemv_pipe_error, 2);
          *(volatile int*)&s_abort = 1;
        }
        const unsigned char* st = ring + (size_t)s * kStageBytes;
        const int u = 2 * t + (warp & 1);                     // 16-byte word (= group) inside a 256-k chunk
        const int swz = (u ^ g) << 4;                         // 128B swizzle: word index XOR (row % 8)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint4 w0[2], w1[2];
          __half sc0[2], sc1[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int c = (warp >> 1) + 4 * (2 * half + j);   // chunk inside the stage
            w0[j] = *reinterpret_cast<const uint4*>(st + (c * kRows + g) * 128 + swz);
            w1[j] = *reinterpret_cast<const uint4*>(st + (c * kRows + g + 8) * 128 + swz);
            // scales: [chunk c][row][8 groups]; this thread's group is number u of the chunk
            sc0[j] = *reinterpret_cast<const __half*>(st + kWBytes + (c * kRows + g) * 16 + u * 2);
            sc1[j] = *reinterpret_cast<const __half*>(st + kWBytes + (c * kRows + g + 8) * 16 + u * 2);
          }
          if (half == 1) {
            // the loads must have returned before the stage goes back to the producer
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              pin_loaded(w0[j]);
              pin_loaded(w1[j]);
              pin_loaded((uint32_t)__half_as_ushort(sc0[j]) | ((uint32_t)__half_as_ushort(sc1[j]) << 16));
            }
            fence_proxy_async_smem();   // generic reads ordered before the TMA refill (async proxy)
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);            // all of the stage is in registers: hand it back
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int gl = ((warp >> 1) + 4 * (2 * half + j)) * 8 + u;   // group inside the stage
            const __half2 s0 = __half2(sc0[j], sc0[j]), s1 = __half2(sc1[j], sc1[j]);
            const int jbase = (((k0 - k_lo) >> 5) + gl) * 4;  // word index inside the staged x block
            const uint32_t wr0[4] = {w0[j].x, w0[j].y, w0[j].z, w0[j].w};
            const uint32_t wr1[4] = {w1[j].x, w1[j].y, w1[j].z, w1[j].w};
            const uint4* xb = xs + XLayout<NC>::slot(jbase, NC >= 8 ? g : (g < NC ? g : NC));
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
              uint4 b[MT];
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) b[mt] = xb[wd * XLayout<NC>::kSlotsPerWord + 8 * mt];
              uint32_t a_lo[4], a_hi[4];
              q4_dequant_pairs(wr0[wd], s0, a_lo);
              q4_dequant_pairs(wr1[wd], s1, a_hi);
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                mma_16x8x16(acc[0][mt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[mt].x, b[mt].y);
                mma_16x8x16(acc[1][mt], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[mt].z, b[mt].w);
              }
            }
          }
        }
      }

      // ---- cross-warp reduction of this (tile, k block) ---------------------------------------------
      float* rbuf = red + tile_parity * (kConsumerWarps * kOut);
      tile_parity ^= 1;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < 4; ++i) rbuf[warp * kOut + (mt * 4 + i) * 32 + lane] = acc[0][mt][i] + acc[1][mt][i];
      bar_sync(2, kConsumers);
      if (ctid < kOut) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) sum += rbuf[w * kOut + ctid];
        if (nkb > 1) {
          float* a = accs + slot * kOut + ctid;
          if (kb > 0) sum += *a;
          if (kb < nkb - 1) *a = sum;
        }
        if (kb == nkb - 1) {
          const int ln = ctid & 31, q = ctid >> 5;
          const int i = q & 3, mt = q >> 2;
          const int row = tile * kRows + (ln >> 2) + 8 * (i >> 1);
          const int col = mt * 8 + 2 * (ln & 3) + (i & 1);
          if (row < p.N && col < p.M) p.y[(int64_t)col * p.N + row] = __float2half_rn(sum);
        }
      }
    }
  }
  if (*(volatile int*)&s_abort) {
    // copies may still be in flight into this CTA's shared memory: let them land before exit
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

template <int NC>
int launch_pipe(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int M, int N, int K,
                cudaStream_t stream) {
  constexpr int MT = (NC + 7) / 8;
  constexpr int kOut = MT * 128;
  PipeParams p;
  {
    const uint64_t wd[3] = {32, (uint64_t)N, (uint64_t)(K / 256)};
    const uint64_t ws[2] = {(uint64_t)K / 2, 128};
    const uint32_t wb[3] = {32, kRows, kChunks};
    int rc = make_tmap(&p.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, wq, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint64_t sd[3] = {8, (uint64_t)N, (uint64_t)(K / 256)};
    const uint64_t ss[2] = {(uint64_t)(K / 32) * 2, 16};
    const uint32_t sb[3] = {8, kRows, kChunks};
    rc = make_tmap(&p.tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, scales, sd, ss, sb, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
  }
  p.x = x; p.y = y;
  p.M = M; p.N = N; p.K = K;
  p.ntiles = (N + kRows - 1) / kRows;
  int stages = (int)options().gemv_stages;
  if (stages <= 0) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  const size_t kMaxSmem = 227 * 1024;
  const int kpad = ((K + KC - 1) / KC) * KC;
  const int sms = sm_count();
  size_t need = 0;
  int kblk = 0, grid = 0;
  // Prefer a deep ring with the whole of x beside it; give up ring depth before cutting K into
  // blocks (a shallower ring costs bandwidth, K blocks cost a carry array and restaging).
  for (;; --stages) {
    const size_t fixed = 1024 /* base alignment slack */ + 2 * kMaxStages * sizeof(uint64_t) +
                         (size_t)stages * kStageBytes + 2 * kConsumerWarps * kOut * sizeof(float);
    // Two CTAs per SM when everything fits twice (a dependent launch can then move in early).
    const int per_sm = (2 * (fixed + XLayout<NC>::bytes(kpad) + 1024) <= 228 * 1024) ? 2 : 1;
    grid = sms * per_sm;
    if (grid > p.ntiles) grid = p.ntiles;
    p.tiles_per_cta = (p.ntiles + grid - 1) / grid;
    need = fixed + XLayout<NC>::bytes(kpad);
    kblk = kpad;
    if (need <= kMaxSmem) break;
    if (stages > 2) continue;
    // ... otherwise cut K into blocks of as many stages' worth as fit, leaving room for the carries.
    const size_t carries = (size_t)p.tiles_per_cta * kOut * sizeof(float);
    if (fixed + carries + XLayout<NC>::bytes(KC) > kMaxSmem) return B200_ENOTREADY;   // caller falls back
    kblk = (int)((kMaxSmem - fixed - carries) / XLayout<NC>::bytes(KC)) * KC;
    need = fixed + carries + XLayout<NC>::bytes(kblk);
    break;
  }
  p.nstages = stages;
  p.kblk = kblk;

  auto kern = q4f16_gemv_pipe_kernel<NC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "gemv: cudaFuncSetAttribute(%zu): %s", need, cudaGetErrorString(e));
  // Ask for the largest shared-memory carve-out: the default picks the smallest that fits ONE CTA,
  // which would keep a second CTA (or the next dependent launch) off the SM.
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
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

}  // namespace

// Returns B200_ENOTREADY when the shape is outside what this kernel takes (caller falls back to
// the register-streaming kernel).
int launch_gemv_pipe(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                     int64_t K, cudaStream_t stream) {
  if (K % 256 != 0 || (reinterpret_cast<uintptr_t>(scales) & 15u)) return B200_ENOTREADY;
  int m = (int)M, n = (int)N, k = (int)K;
  if (m == 1) return launch_pipe<1>(x, wq, scales, y, m, n, k, stream);
  if (m == 2) return launch_pipe<2>(x, wq, scales, y, m, n, k, stream);
  if (m <= 4) return launch_pipe<4>(x, wq, scales, y, m, n, k, stream);
  if (m <= 8) return launch_pipe<8>(x, wq, scales, y, m, n, k, stream);
  return launch_pipe<16>(x, wq, scales, y, m, n, k, stream);
}

int gemv_pipe_error_read_and_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemv_pipe_error, sizeof(int)) != cudaSuccess) return 0xff;
  if (v) cudaMemcpyToSymbol(g_gemv_pipe_error, &zero, sizeof(int));
  return v & 0xff;
}

}  // namespace b200
