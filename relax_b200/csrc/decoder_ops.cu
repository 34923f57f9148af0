// Glue kernels of one Llama-style decode step around the quantised matmuls: RMSNorm (with the
// residual add fused), rotary embedding + KV-cache append, single-query attention over the fp16
// cache (split over the context, partials combined by a second kernel) and SwiGLU.
//
// The reference has no op for RMSNorm, RoPE or attention (its op list stops at mean / sqrt /
// divide / multiply / strided_slice / concat / softmax / silu, python/tvm/relax/transform/
// legalize_ops.py:378-381,506-514); the semantics here are the composition of those ops with
// statistics in fp32 and one fp16 rounding at each kernel's output, which is what the oracle's
// decoder restatement does too.
//
// All of them are HBM/latency bound and tiny next to the weight streams, except the attention,
// which reads 2 * ctx * heads * 128 fp16 per sequence.
#include "internal.h"
#include "sm100_ptx.cuh"

namespace b200 {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// y[b,:] = fp16( f32(x) * rsqrt(mean(f32(x)^2) + eps) * f32(w) ); optionally x += delta first (the
// updated x is written back: it is the residual stream).  One CTA per row, H % 8 == 0.
template <bool kAdd>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(__half* __restrict__ x, const __half* __restrict__ delta, const __half* __restrict__ w,
               __half* __restrict__ y, int H, float eps) {
  ptx::pdl_wait();
  extern __shared__ float xs[];                 // H floats
  __shared__ float red[8];
  const int b = blockIdx.x;
  __half* xr = x + (int64_t)b * H;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    __half2* h = reinterpret_cast<__half2*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __half22float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
    if (kAdd) {
      uint4 dv = *reinterpret_cast<const uint4*>(delta + (int64_t)b * H + i);
      __half2* dh = reinterpret_cast<__half2*>(&dv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __half22float2(dh[j]);
        // the residual stream is stored in fp16: round the sum once, then normalise what was stored
        __half2 r = __floats2half2_rn(f[2 * j] + t.x, f[2 * j + 1] + t.y);
        h[j] = r;
        float2 rf = __half22float2(r);
        f[2 * j] = rf.x;
        f[2 * j + 1] = rf.y;
      }
      *reinterpret_cast<uint4*>(xr + i) = v;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      xs[i + j] = f[j];
      ss += f[j] * f[j];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)H + eps);
  ptx::pdl_launch_dependents();
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const __half2* wh = reinterpret_cast<const __half2*>(&wv);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 wf = __half22float2(wh[j]);
      oh[j] = __floats2half2_rn(xs[i + 2 * j] * inv * wf.x, xs[i + 2 * j + 1] * inv * wf.y);
    }
    *reinterpret_cast<uint4*>(y + (int64_t)b * H + i) = o;
  }
}

// Rotary embedding (rotate-half pairing i <-> i+64 inside a 128-wide head) of q and k, then k and v
// go to the cache at position pos[0].  qkv row layout: [q heads | k heads | v heads], nh heads each.
// cos/sin tables fp32 [max_pos, 64].  grid (nh, B), 64 threads.
__global__ void __launch_bounds__(64)
rope_kv_append_kernel(const __half* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      const int* __restrict__ pos_ptr, __half* __restrict__ q_out, __half* __restrict__ k_cache,
                      __half* __restrict__ v_cache, int nh, int max_ctx) {
  ptx::pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y, i = threadIdx.x;
  const int pos = pos_ptr[0];
  const float c = cos_t[(int64_t)pos * 64 + i], s = sin_t[(int64_t)pos * 64 + i];
  const __half* row = qkv + (int64_t)b * 3 * nh * 128;
  const __half* q = row + h * 128;
  const __half* k = row + (nh + h) * 128;
  const __half* v = row + (2 * nh + h) * 128;
  const float q0 = __half2float(q[i]), q1 = __half2float(q[i + 64]);
  const float k0 = __half2float(k[i]), k1 = __half2float(k[i + 64]);
  __half* qo = q_out + ((int64_t)b * nh + h) * 128;
  qo[i] = __float2half_rn(q0 * c - q1 * s);
  qo[i + 64] = __float2half_rn(q1 * c + q0 * s);
  const int64_t slot = (((int64_t)b * max_ctx + pos) * nh + h) * 128;
  k_cache[slot + i] = __float2half_rn(k0 * c - k1 * s);
  k_cache[slot + i + 64] = __float2half_rn(k1 * c + k0 * s);
  v_cache[slot + i] = v[i];
  v_cache[slot + i + 64] = v[i + 64];
  ptx::pdl_launch_dependents();
}

// Single-query attention, split over the context: CTA (split, head, batch) handles tokens
// [split*chunk, min(ctx, (split+1)*chunk)) with an online softmax in fp32 and writes the partial
// (max, sum, acc[128]) to scratch [B, nh, nsplit, 130] floats.  4 warps; lane owns 4 of the 128 dims.
constexpr int kAttnChunk = 128;
template <int kTok>
__global__ void __launch_bounds__(128)
attn_decode_partial_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache,
                           const __half* __restrict__ v_cache, const int* __restrict__ pos_ptr,
                           float* __restrict__ scratch, int nh, int max_ctx, int nsplit, float scale_log2e,
                           int early_ok) {
  // early_ok: the caller promises that the position and the cache entries older than the new token were
  // complete before the launch in front of this one BEGAN (see B200_ATTN_EARLY_KV_LOADS).  Then
  // everything up to the wait reads only finished data, and the first round of K/V loads of a chunk
  // that does not hold the new token is in flight while the kernel before this one finishes.
  // Without the promise nothing is read before the wait.
  if (!early_ok) ptx::pdl_wait();
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int ctx = pos_ptr[0] + 1;
  const int t0 = split * kAttnChunk;
  const int t1 = min(ctx, t0 + kAttnChunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* out = scratch + (((int64_t)b * nh + h) * nsplit + split) * 130;
  __shared__ float sm_m[4], sm_l[4], sm_acc[4][128];
  const int64_t tok_stride = (int64_t)nh * 128;
  const __half* kb = k_cache + ((int64_t)b * max_ctx * nh + h) * 128 + lane * 4;
  const __half* vb = v_cache + ((int64_t)b * max_ctx * nh + h) * 128 + lane * 4;
  uint2 kv[kTok], vv[kTok];
  auto load_round = [&](int tb) {
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      const int t = min(tb + j, t1 - 1);             // clamped: a token past the end is loaded but not used
      kv[j] = *reinterpret_cast<const uint2*>(kb + t * tok_stride);
      vv[j] = *reinterpret_cast<const uint2*>(vb + t * tok_stride);
    }
  };
  int tb = t0 + warp * kTok;
  const bool early = early_ok && t1 < ctx;           // the new token (position ctx - 1) is not in this chunk
  if (early && tb < t1) load_round(tb);
  if (early_ok) ptx::pdl_wait();
  if (!early && tb < t1) load_round(tb);
  float qf[4];
  {
    uint2 qv = *reinterpret_cast<const uint2*>(q + ((int64_t)b * nh + h) * 128 + lane * 4);
    const __half2* qh = reinterpret_cast<const __half2*>(&qv);
    float2 a = __half22float2(qh[0]), c = __half22float2(qh[1]);
    qf[0] = a.x * scale_log2e; qf[1] = a.y * scale_log2e; qf[2] = c.x * scale_log2e; qf[3] = c.y * scale_log2e;
  }
  float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  // kTok tokens per round: all 2*kTok loads are issued before the first use (a single query has
  // no other parallelism to cover the memory latency), then one online-softmax update per round.
  // 16 tokens (two rounds per warp and chunk) when the grid is small and latency decides, 8 when
  // the batch fills the GPU and the kernel streams at the HBM rate anyway.
  for (; tb < t1; tb += 4 * kTok) {
    if (tb != t0 + warp * kTok) load_round(tb);      // (the first round is already in flight)
    float s[kTok];
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      const __half2* kh = reinterpret_cast<const __half2*>(&kv[j]);
      const float2 k01 = __half22float2(kh[0]), k23 = __half22float2(kh[1]);
      s[j] = qf[0] * k01.x + qf[1] * k01.y + qf[2] * k23.x + qf[3] * k23.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int j = 0; j < kTok; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o);
    float mn = m;
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      if (tb + j >= t1) s[j] = -INFINITY;            // log2-domain scores; masked tokens get weight 0
      mn = fmaxf(mn, s[j]);
    }
    const float corr = exp2f(m - mn);                // m = -inf on the first round: exp2f(-inf) = 0
    l *= corr;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] *= corr;
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      const float pj = exp2f(s[j] - mn);
      const __half2* vh = reinterpret_cast<const __half2*>(&vv[j]);
      const float2 v01 = __half22float2(vh[0]), v23 = __half22float2(vh[1]);
      l += pj;
      acc[0] += pj * v01.x;
      acc[1] += pj * v01.y;
      acc[2] += pj * v23.x;
      acc[3] += pj * v23.y;
    }
    m = mn;
  }
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int j = 0; j < 4; ++j) sm_acc[warp][lane * 4 + j] = acc[j];
  __syncthreads();
  ptx::pdl_launch_dependents();
  // combine the 4 warps: thread d owns output dim d
  const int d = threadIdx.x;
  float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
  float L = 0.f, A = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float f = (sm_m[w] == -INFINITY) ? 0.f : exp2f(sm_m[w] - M);
    L += sm_l[w] * f;
    A += sm_acc[w][d] * f;
  }
  out[2 + d] = A;
  if (d == 0) { out[0] = M; out[1] = L; }
}

// Rotary embedding + KV append + attention + merge of the partials in ONE launch.
// grid (nsplit, nh, B), 128 threads.  CTA (split, h, b):
//   * rotates q of head h itself (lane owns dims 4*lane..+3; its rotate-half partner is lane ^ 16);
//   * if its chunk holds the new token, rotates k, writes k and v into the caches at *pos first;
//   * runs the online softmax over its chunk as attn_decode_partial_kernel does;
//   * bumps a per-(b, h) counter; the CTA that arrives last merges all chunks' partials and stores
//     fp16.  The counters live after the partials in `scratch`, must be zero before the first call
//     and are left zero.
template <int kTok>
__global__ void __launch_bounds__(128)
attn_decode_fused_kernel(const __half* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         const int* __restrict__ pos_ptr, __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                         __half* __restrict__ out, float* __restrict__ scratch, int nh, int max_ctx, int nsplit,
                         float scale_log2e, int merge) {
  ptx::pdl_wait();
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int pos = pos_ptr[0];
  const int ctx = pos + 1;
  const int used = (ctx + kAttnChunk - 1) / kAttnChunk;
  if (split >= used) return;
  const int t0 = split * kAttnChunk;
  const int t1 = min(ctx, t0 + kAttnChunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* part = scratch + (((int64_t)b * nh + h) * nsplit + split) * 130;
  int* counters = reinterpret_cast<int*>(scratch + (int64_t)gridDim.z * nh * nsplit * 130);
  __shared__ float sm_m[4], sm_l[4], sm_acc[4][128];
  __shared__ int s_last;

  const __half* row = qkv + (int64_t)b * 3 * nh * 128;
  const int d0 = lane * 4;                         // this lane's dims
  const int r0 = d0 & 63;                          // their rotation index (pairs i <-> i + 64)
  const float4 cs = *reinterpret_cast<const float4*>(cos_t + (int64_t)pos * 64 + r0);
  const float4 sn = *reinterpret_cast<const float4*>(sin_t + (int64_t)pos * 64 + r0);
  const float c[4] = {cs.x, cs.y, cs.z, cs.w}, s[4] = {sn.x, sn.y, sn.z, sn.w};
  const float sign = lane < 16 ? -1.f : 1.f;       // first half: a*c - b*s, second half: b*c + a*s
  auto rotate = [&](const __half* v, float (&o)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(v + d0);
    const __half2* hh = reinterpret_cast<const __half2*>(&raw);
    const float2 a = __half22float2(hh[0]), e = __half22float2(hh[1]);
    const float mine[4] = {a.x, a.y, e.x, e.y};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, mine[j], 16);
      // round to fp16 as the stand-alone rotary kernel does (q and k are fp16 tensors in the layer)
      o[j] = __half2float(__float2half_rn(mine[j] * c[j] + sign * other * s[j]));
    }
  };

  if (split == used - 1 && warp == 0) {
    // the new token belongs to this chunk: put its rotated k and its v into the caches first
    float kr[4];
    rotate(row + (nh + h) * 128, kr);
    const int64_t slot = (((int64_t)b * max_ctx + pos) * nh + h) * 128 + d0;
    uint2 kw;
    __half2* kh2 = reinterpret_cast<__half2*>(&kw);
    kh2[0] = __floats2half2_rn(kr[0], kr[1]);
    kh2[1] = __floats2half2_rn(kr[2], kr[3]);
    *reinterpret_cast<uint2*>(k_cache + slot) = kw;
    *reinterpret_cast<uint2*>(v_cache + slot) = *reinterpret_cast<const uint2*>(row + (2 * nh + h) * 128 + d0);
  }
  float qf[4];
  rotate(row + h * 128, qf);
#pragma unroll
  for (int j = 0; j < 4; ++j) qf[j] *= scale_log2e;
  __syncthreads();                                 // the appended token is visible to the whole CTA

  float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int64_t tok_stride = (int64_t)nh * 128;
  const __half* kb = k_cache + ((int64_t)b * max_ctx * nh + h) * 128 + d0;
  const __half* vb = v_cache + ((int64_t)b * max_ctx * nh + h) * 128 + d0;
  for (int tb = t0 + warp * kTok; tb < t1; tb += 4 * kTok) {
    uint2 kv[kTok], vv[kTok];
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      const int t = min(tb + j, t1 - 1);
      kv[j] = *reinterpret_cast<const uint2*>(kb + t * tok_stride);
      vv[j] = *reinterpret_cast<const uint2*>(vb + t * tok_stride);
    }
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
    for (int i = 0; i < 4; ++i) acc[i] *= corr;
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      const float pj = exp2f(sc[j] - mn);
      const __half2* vh = reinterpret_cast<const __half2*>(&vv[j]);
      const float2 v01 = __half22float2(vh[0]), v23 = __half22float2(vh[1]);
      l += pj;
      acc[0] += pj * v01.x;
      acc[1] += pj * v01.y;
      acc[2] += pj * v23.x;
      acc[3] += pj * v23.y;
    }
    m = mn;
  }
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int j = 0; j < 4; ++j) sm_acc[warp][lane * 4 + j] = acc[j];
  __syncthreads();
  ptx::pdl_launch_dependents();
  const int d = threadIdx.x;
  {
    const float M = fmaxf(fmaxf(sm_m[0], sm_m[1]), fmaxf(sm_m[2], sm_m[3]));
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = (sm_m[w] == -INFINITY) ? 0.f : exp2f(sm_m[w] - M);
      L += sm_l[w] * f;
      A += sm_acc[w][d] * f;
    }
    part[2 + d] = A;
    if (d == 0) { part[0] = M; part[1] = L; }
  }
  if (!merge) return;                              // the merge kernel follows as its own launch
  // ---- the CTA that arrives last for this (b, h) merges the chunks ---------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&counters[b * nh + h], 1) == used - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) counters[b * nh + h] = 0;
  const float* p = scratch + ((int64_t)b * nh + h) * nsplit * 130;
  // sixteen chunks per round, all loads of a round issued together (the partials sit in L2)
  float M = -INFINITY, L = 0.f, A = 0.f;
  for (int s0 = 0; s0 < used; s0 += 16) {
    float Ms[16], Ls[16], As[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int si = min(s0 + j, used - 1);
      Ms[j] = __ldcg(p + si * 130);
      Ls[j] = __ldcg(p + si * 130 + 1);
      As[j] = __ldcg(p + si * 130 + 2 + d);
    }
    float Mn = M;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (s0 + j < used) Mn = fmaxf(Mn, Ms[j]);
    const float corr = exp2f(M - Mn);            // first round: exp2f(-inf) = 0
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
  out[((int64_t)b * nh + h) * 128 + d] = __float2half_rn(A / L);
}

// Merges the nsplit partials of one (batch, head) and writes fp16 [B, nh*128].  grid (nh, B), 128 threads.
__global__ void __launch_bounds__(128)
attn_decode_combine_kernel(const float* __restrict__ scratch, const int* __restrict__ pos_ptr, __half* __restrict__ out,
                           int nh, int nsplit) {
  ptx::pdl_wait();
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int ctx = pos_ptr[0] + 1;
  const int used = (ctx + kAttnChunk - 1) / kAttnChunk;
  const float* p = scratch + ((int64_t)b * nh + h) * nsplit * 130;
  // sixteen chunks per round, all 48 loads of a round issued together (the partials sit in L2), one
  // online-softmax update per round
  float M = -INFINITY, L = 0.f, A = 0.f;
  for (int s0 = 0; s0 < used; s0 += 16) {
    float Ms[16], Ls[16], As[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int si = min(s0 + j, used - 1);
      Ms[j] = p[si * 130];
      Ls[j] = p[si * 130 + 1];
      As[j] = p[si * 130 + 2 + d];
    }
    float Mn = M;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (s0 + j < used) Mn = fmaxf(Mn, Ms[j]);
    const float corr = exp2f(M - Mn);            // first round: exp2f(-inf) = 0
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
  ptx::pdl_launch_dependents();
  out[((int64_t)b * nh + h) * 128 + d] = __float2half_rn(A / L);
}

// out[b,i] = fp16( silu(f32(g)) * f32(u) ), gu row = [gate (I) | up (I)].  I % 8 == 0.
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ out, int I, int64_t total8) {
  ptx::pdl_wait();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total8) return;
  const int per_row = I / 8;
  const int64_t b = idx / per_row;
  const int i = (int)(idx - b * per_row) * 8;
  uint4 gv = *reinterpret_cast<const uint4*>(gu + b * 2 * I + i);
  uint4 uv = *reinterpret_cast<const uint4*>(gu + b * 2 * I + I + i);
  const __half2* gh = reinterpret_cast<const __half2*>(&gv);
  const __half2* uh = reinterpret_cast<const __half2*>(&uv);
  uint4 o;
  __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 g = __half22float2(gh[j]), u = __half22float2(uh[j]);
    float a = g.x / (1.f + __expf(-g.x)) * u.x;
    float c = g.y / (1.f + __expf(-g.y)) * u.y;
    oh[j] = __floats2half2_rn(a, c);
  }
  ptx::pdl_launch_dependents();
  *reinterpret_cast<uint4*>(out + b * I + i) = o;
}

// out[b,:] = table[ids[b],:] (fp16 rows of H, H % 8 == 0).  grid (B), 128 threads.
__global__ void __launch_bounds__(128)
embed_rows_kernel(const __half* __restrict__ table, const int* __restrict__ ids, __half* __restrict__ out, int H,
                  int vocab) {
  ptx::pdl_wait();
  const int b = blockIdx.x;
  int id = ids[b];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);          // clamp: never read outside the table
  const uint4* src = reinterpret_cast<const uint4*>(table + (int64_t)id * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)b * H);
  ptx::pdl_launch_dependents();
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// *pos += delta (one thread): advances the decode position on the device so that a captured
// graph can be replayed token after token.
__global__ void advance_pos_kernel(int* pos, int delta) {
  ptx::pdl_wait();
  ptx::pdl_launch_dependents();
  if (threadIdx.x == 0 && blockIdx.x == 0) *pos += delta;
}

template <typename K, typename... A>
int launch(const char* what, K kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemv_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "%s launch: %s", what, cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int b200_rmsnorm(void* x, const void* delta, const void* w, void* y, int64_t B, int64_t H, float eps, void* stream) {
  if (B < 0 || H <= 0 || H % 8 != 0 || H > 16384) return fail(B200_EINVAL, "rmsnorm: need 0 < H <= 16384, H %% 8 == 0");
  if (B == 0) return B200_OK;
  if (!x || !w || !y) return fail(B200_EINVAL, "rmsnorm: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  auto s = static_cast<cudaStream_t>(stream);
  if (delta)
    return launch("add_rmsnorm", rmsnorm_kernel<true>, dim3((unsigned)B), dim3(256), (size_t)H * 4, s, (__half*)x,
                  (const __half*)delta, (const __half*)w, (__half*)y, (int)H, eps);
  return launch("rmsnorm", rmsnorm_kernel<false>, dim3((unsigned)B), dim3(256), (size_t)H * 4, s, (__half*)x,
                (const __half*)nullptr, (const __half*)w, (__half*)y, (int)H, eps);
}

int b200_rope_kv_append(const void* qkv, const void* cos_t, const void* sin_t, const void* pos, void* q_out,
                        void* k_cache, void* v_cache, int64_t B, int64_t nh, int64_t max_ctx, void* stream) {
  if (B <= 0 || nh <= 0 || max_ctx <= 0) return fail(B200_EINVAL, "rope_kv_append: bad sizes");
  if (!qkv || !cos_t || !sin_t || !pos || !q_out || !k_cache || !v_cache) return fail(B200_EINVAL, "rope_kv_append: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  return launch("rope_kv_append", rope_kv_append_kernel, dim3((unsigned)nh, (unsigned)B), dim3(64), 0,
                static_cast<cudaStream_t>(stream), (const __half*)qkv, (const float*)cos_t, (const float*)sin_t,
                (const int*)pos, (__half*)q_out, (__half*)k_cache, (__half*)v_cache, (int)nh, (int)max_ctx);
}

int64_t b200_attn_decode_scratch_bytes(int64_t B, int64_t nh, int64_t max_ctx) {
  int64_t nsplit = (max_ctx + kAttnChunk - 1) / kAttnChunk;
  return B * nh * nsplit * 130 * (int64_t)sizeof(float);
}

int64_t b200_attn_decode_fused_scratch_bytes(int64_t B, int64_t nh, int64_t max_ctx) {
  return b200_attn_decode_scratch_bytes(B, nh, max_ctx) + B * nh * (int64_t)sizeof(int);
}

int b200_attn_decode_fused(const void* qkv, const void* cos_t, const void* sin_t, const void* pos, void* k_cache, void* v_cache,
                           void* out, void* scratch, int64_t B, int64_t nh, int64_t max_ctx, void* stream) {
  if (B <= 0 || nh <= 0 || max_ctx <= 0 || B > 65535 || nh > 65535) return fail(B200_EINVAL, "attn_decode_fused: bad sizes");
  if (!qkv || !cos_t || !sin_t || !pos || !k_cache || !v_cache || !out || !scratch)
    return fail(B200_EINVAL, "attn_decode_fused: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  const int nsplit = (int)((max_ctx + kAttnChunk - 1) / kAttnChunk);
  const float scale_log2e = 1.4426950408889634f / sqrtf(128.f);
  return launch("attn_decode_fused", attn_decode_fused_kernel<8>, dim3((unsigned)nsplit, (unsigned)nh, (unsigned)B), dim3(128), 0,
                static_cast<cudaStream_t>(stream), (const __half*)qkv, (const float*)cos_t, (const float*)sin_t,
                (const int*)pos, (__half*)k_cache, (__half*)v_cache, (__half*)out, (float*)scratch, (int)nh, (int)max_ctx,
                nsplit, scale_log2e, 1);
}

int b200_attn_decode_rope(const void* qkv, const void* cos_t, const void* sin_t, const void* pos, void* k_cache, void* v_cache,
                          void* out, void* scratch, int64_t B, int64_t nh, int64_t max_ctx, void* stream) {
  if (B <= 0 || nh <= 0 || max_ctx <= 0 || B > 65535 || nh > 65535) return fail(B200_EINVAL, "attn_decode_rope: bad sizes");
  if (!qkv || !cos_t || !sin_t || !pos || !k_cache || !v_cache || !out || !scratch)
    return fail(B200_EINVAL, "attn_decode_rope: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  const int nsplit = (int)((max_ctx + kAttnChunk - 1) / kAttnChunk);
  const float scale_log2e = 1.4426950408889634f / sqrtf(128.f);
  auto s = static_cast<cudaStream_t>(stream);
  const bool small_grid = (int64_t)nsplit * nh * B < 2048;
  rc = launch("attn_decode_rope", small_grid ? attn_decode_fused_kernel<16> : attn_decode_fused_kernel<8>,
              dim3((unsigned)nsplit, (unsigned)nh, (unsigned)B), dim3(128), 0, s, (const __half*)qkv, (const float*)cos_t,
              (const float*)sin_t, (const int*)pos, (__half*)k_cache, (__half*)v_cache, (__half*)out, (float*)scratch, (int)nh,
              (int)max_ctx, nsplit, scale_log2e, 0);
  if (rc) return rc;
  return launch("attn_decode_combine", attn_decode_combine_kernel, dim3((unsigned)nh, (unsigned)B), dim3(128), 0, s,
                (const float*)scratch, (const int*)pos, (__half*)out, (int)nh, nsplit);
}

int b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const void* pos, void* out, void* scratch,
                     int64_t B, int64_t nh, int64_t max_ctx, uint32_t flags, void* stream) {
  if (B <= 0 || nh <= 0 || max_ctx <= 0) return fail(B200_EINVAL, "attn_decode: bad sizes");
  if (B > 65535 || nh > 65535 || max_ctx > 0x3fffffffLL)
    return fail(B200_EINVAL, "attn_decode: batch and heads are limited to 65535 (grid dimensions), max_ctx to 2^30");
  if (flags & ~(uint32_t)B200_ATTN_EARLY_KV_LOADS) return fail(B200_EINVAL, "attn_decode: unknown flag bits %#x", flags);
  if (!q || !k_cache || !v_cache || !pos || !out || !scratch) return fail(B200_EINVAL, "attn_decode: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  const int nsplit = (int)((max_ctx + kAttnChunk - 1) / kAttnChunk);
  auto s = static_cast<cudaStream_t>(stream);
  const float scale_log2e = 1.4426950408889634f / sqrtf(128.f);
  // few CTAs (small batch): latency bound, more loads in flight per warp (measured: 7B shape, context
  // 2048, batch 1: -2 us per layer; batch 16: no gain, so the 8-token form stays there)
  const bool small_grid = (int64_t)nsplit * nh * B < 2048;
  rc = launch("attn_decode_partial", small_grid ? attn_decode_partial_kernel<16> : attn_decode_partial_kernel<8>,
              dim3((unsigned)nsplit, (unsigned)nh, (unsigned)B),
              dim3(128), 0, s, (const __half*)q, (const __half*)k_cache, (const __half*)v_cache, (const int*)pos,
              (float*)scratch, (int)nh, (int)max_ctx, nsplit, scale_log2e, (int)(flags & B200_ATTN_EARLY_KV_LOADS));
  if (rc) return rc;
  return launch("attn_decode_combine", attn_decode_combine_kernel, dim3((unsigned)nh, (unsigned)B), dim3(128), 0, s,
                (const float*)scratch, (const int*)pos, (__half*)out, (int)nh, nsplit);
}

int b200_embed_rows(const void* table, const void* ids, void* out, int64_t B, int64_t H, int64_t vocab, void* stream) {
  if (B < 0 || H <= 0 || H % 8 != 0 || vocab <= 0) return fail(B200_EINVAL, "embed_rows: need H %% 8 == 0, vocab > 0");
  if (B == 0) return B200_OK;
  if (!table || !ids || !out) return fail(B200_EINVAL, "embed_rows: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  return launch("embed_rows", embed_rows_kernel, dim3((unsigned)B), dim3(128), 0, static_cast<cudaStream_t>(stream),
                (const __half*)table, (const int*)ids, (__half*)out, (int)H, (int)vocab);
}

int b200_advance_pos(void* pos, int64_t delta, void* stream) {
  if (!pos) return fail(B200_EINVAL, "advance_pos: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  return launch("advance_pos", advance_pos_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), (int*)pos,
                (int)delta);
}

// ---- attention without caller-provided scratch ------------------------------------------------
// Partial results live in a fixed array inside the library image instead of a buffer the caller
// allocates.  kStaticAttnSlots (batch * heads * 128-token chunks) bounds what fits.
constexpr int64_t kStaticAttnSlots = 8192;                       // e.g. 16 sequences x 32 heads x 2048 tokens
static __device__ __align__(256) float g_attn_static_scratch[kStaticAttnSlots * 130];   // 4.26 MB per GPU

int b200_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, const void* pos, void* out, int64_t B,
                            int64_t nh, int64_t max_ctx, uint32_t flags, void* stream) {
  if (B <= 0 || nh <= 0 || max_ctx <= 0) return fail(B200_EINVAL, "attn_decode_static: bad sizes");
  if (B > 65535 || nh > 65535 || max_ctx > 0x3fffffffLL)
    return fail(B200_EINVAL, "attn_decode_static: batch and heads are limited to 65535 (grid dimensions), max_ctx to 2^30");
  if (!q || !k_cache || !v_cache || !pos || !out) return fail(B200_EINVAL, "attn_decode_static: null pointer");
  const int64_t nsplit = (max_ctx + kAttnChunk - 1) / kAttnChunk;
  // (B, nh <= 65535 and nsplit <= 2^23: the product below cannot overflow 64 bits)
  if (B * nh * nsplit > kStaticAttnSlots)
    return fail(B200_EINVAL,
                "attn_decode_static: batch %lld x heads %lld x %lld chunks of 128 tokens = %lld partial results, the built-in "
                "scratch holds %lld; use b200_attn_decode with a caller-owned buffer",
                (long long)B, (long long)nh, (long long)nsplit, (long long)(B * nh * nsplit), (long long)kStaticAttnSlots);
  int rc = ensure_device();
  if (rc) return rc;
  // The array's name is only a handle on the host: its device address is looked up once per
  // device, with that device current, and handed to the kernels like any other buffer.
  static float* scratch_of_device[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(B200_ENODEVICE, "attn_decode_static: no current device");
  if (!scratch_of_device[dev]) {
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_attn_static_scratch);
    if (e != cudaSuccess || !ptr)
      return fail(B200_ELAUNCH, "attn_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    scratch_of_device[dev] = ptr;
  }
  return b200_attn_decode(q, k_cache, v_cache, pos, out, scratch_of_device[dev], B, nh, max_ctx, flags, stream);
}

int b200_silu_mul(const void* gu, void* out, int64_t B, int64_t I, void* stream) {
  if (B < 0 || I <= 0 || I % 8 != 0) return fail(B200_EINVAL, "silu_mul: need I %% 8 == 0");
  if (B == 0) return B200_OK;
  if (!gu || !out) return fail(B200_EINVAL, "silu_mul: null pointer");
  int rc = ensure_device();
  if (rc) return rc;
  const int64_t total8 = B * (I / 8);
  return launch("silu_mul", silu_mul_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0,
                static_cast<cudaStream_t>(stream), (const __half*)gu, (__half*)out, (int)I, total8);
}

}  // extern "C"
