/*
 * b200_q4f16.h -- C ABI of the B200 (sm_100a) q4f16 dequantize+matmul kernel library.
 *
 * This is the drop-in boundary for ONE path of tlc-pack/relax: the group-quantized
 * matmul that its fusion pipeline leaves as a fused `decode -> matmul -> astype`
 * PrimFunc (uint32-packed int4 weights, fp16 scales per 32 elements of K, zero point 7).
 * Every entry point is `extern "C"`, takes plain pointers and sizes (or DLPack tensors,
 * which are plain C structs), never allocates device memory unless stated, launches on
 * the stream it is given and returns without synchronising.
 *
 * Data layout (all row-major, contiguous):
 *     x       fp16   [M, K]
 *     wq      uint32 [N, K/8]    element k of row n sits in bits 4*(k%8).. of word k/8
 *     scales  fp16   [N, K/32]
 *     y       fp16   [M, N]      y = x . w^T,  w[n,k] = fp16(q[n,k]-7) * scales[n,k/32]
 * fp32 accumulation; the dequantised weight is rounded to fp16 exactly once, as the
 * reference's TIR does, so `b200_q4f16_dequantize` is bit-exact against it.
 *
 * Error convention (mirrors the reference's packed-function convention,
 * include/tvm/runtime/c_runtime_api.h:238,355-363): 0 on success; a negative B200_E*
 * code after storing a thread-local message readable with b200_last_error().  Nothing
 * is launched when validation fails.  There is no CPU fallback: without a CUDA device
 * of compute capability 10.x every compute entry point returns B200_ENODEVICE.
 */
#ifndef B200_Q4F16_H_
#define B200_Q4F16_H_

#include <stdint.h>

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)     /* bad shape, dtype, alignment, null pointer */
#define B200_ENODEVICE (-2)  /* no sm_100 device / CUDA runtime error before launch */
#define B200_ELAUNCH (-3)    /* the launch itself was rejected by the CUDA runtime */
#define B200_EDEVICE (-4)    /* a kernel reported a device-side error flag (bounded wait ran out) */
#define B200_ENOTREADY (-5)  /* communicator / workspace not initialised */

/* ---- DLPack tensor view (binary compatible with DLTensor of dlpack.h v0.x/1.x) ------------
 * The reference passes tensors to packed functions as DLTensor* / NDArray handles
 * (include/tvm/runtime/ndarray.h:85-188, include/tvm/runtime/packed_func.h:577-586). */
typedef struct {
  int32_t device_type; /* 2 = kDLCUDA, 1 = kDLCPU, 3 = kDLCUDAHost */
  int32_t device_id;
} B200DLDevice;
typedef struct {
  uint8_t code; /* 0 int, 1 uint, 2 float */
  uint8_t bits;
  uint16_t lanes;
} B200DLDataType;
typedef struct {
  void* data;
  B200DLDevice device;
  int32_t ndim;
  B200DLDataType dtype;
  int64_t* shape;
  int64_t* strides; /* NULL = compact row-major */
  uint64_t byte_offset;
} B200DLTensor;

/* ---- library state --------------------------------------------------------------------- */

/* Message of the last failing call on this thread ("" if none).  Replaces TVMGetLastError
 * (include/tvm/runtime/c_runtime_api.h:229-238) for callers outside TVM. */
B200_API const char* b200_last_error(void);

/* ABI version of this header: major*100 + minor. */
B200_API int b200_abi_version(void);

/* Sets / reads the stream that the DLPack and packed entry points launch on for the calling
 * thread.  Mirrors CUDAThreadEntry::ThreadLocal()->stream set through TVMSetStream
 * (src/runtime/cuda/cuda_common.h:55-66, src/runtime/cuda/cuda_device_api.cc:209-211).
 * NULL is the legacy default stream, as in the reference. */
B200_API int b200_set_stream(void* cuda_stream);
B200_API void* b200_get_stream(void);

/* ---- kernels on raw device pointers ---------------------------------------------------- */

/* w_out fp16 [N,K] = decode(wq, scales).  Replaces the `decode` PrimFunc the reference
 * compiles from generic TIR ops (src/tir/op/op.cc:564 right_shift, :606 bitwise_and, :282
 * cast) when decode and matmul stay two kernels.  Bit-exact.  K % 32 == 0. */
B200_API int b200_q4f16_dequantize(const void* wq, const void* scales, void* w_out, int64_t N, int64_t K,
                          void* cuda_stream);

/* y = x . decode(wq, scales)^T.  Replaces the fused decode+matmul+astype PrimFunc
 * (FuseTIR output, src/relax/transform/fuse_tir.cc:708-711; matmul semantics
 * python/tvm/relax/transform/legalize_ops.py:203-264; astype :157-162).
 * Picks the kernel family from M: the streaming skinny kernel for M <= 16, the tcgen05 /
 * TMEM tensor-core kernel above that.  K % 32 == 0; pointers 16-byte aligned. */
B200_API int b200_q4f16_matmul(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                      int64_t K, void* cuda_stream);

/* The two families, callable directly (same contract as b200_q4f16_matmul).
 * b200_q4f16_gemv requires 1 <= M <= 16. */
B200_API int b200_q4f16_gemv(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                    int64_t K, void* cuda_stream);
B200_API int b200_q4f16_gemm(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                    int64_t K, void* cuda_stream);
/* Weight-stationary tensor-core kernel for mid-sized batches (1 <= M <= 128, K % 256 == 0, scales
 * 16-byte aligned): 128 weight rows are the MMA's M, the batch its N, K is split over a thread-block
 * cluster whose partial tiles are added through distributed shared memory.  b200_q4f16_matmul picks
 * it for 16 < M <= 128. */
B200_API int b200_q4f16_gemm_ws(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                                int64_t K, void* cuda_stream);

/* Same matmul with the activation and the result in HOST memory (pinned memory makes the
 * copies asynchronous): copies x to `x_dev`, runs the kernel, copies `y_dev` back to y_host,
 * all on `cuda_stream`.  x_dev / y_dev are caller-owned device staging buffers of M*K and M*N
 * fp16.  The weights stay on the device, as parameters do in the reference's VM
 * (python/tvm/relax/vm.py:620-629).  Transfers of up to 256 KB from or to page-locked host
 * buffers (16-byte aligned) are done by small kernels through the buffer's device mapping instead
 * of the copy engine, the result copy as a programmatic dependent of the matmul; pageable
 * buffers and larger transfers use cudaMemcpyAsync.  Either way the call returns after enqueueing. */
B200_API int b200_q4f16_matmul_host(const void* x_host, void* x_dev, const void* wq, const void* scales, void* y_dev,
                           void* y_host, int64_t M, int64_t N, int64_t K, void* cuda_stream);

/* ---- DLPack entry points (destination-passing style) ------------------------------------
 * What a `R.call_tir("b200.q4f16_matmul", (x, wq, scales), out_sinfo)` call reaches: inputs
 * first, pre-allocated output last (src/relax/transform/call_tir_rewrite.cc:94-110).  They
 * validate dtype, rank, shape agreement, compactness, device and alignment exactly as a
 * contrib library must (cf. src/runtime/contrib/cublas/cublas.cc:211-267) and launch on the
 * thread's current stream (b200_set_stream). */
B200_API int b200_q4f16_matmul_dl(const B200DLTensor* x, const B200DLTensor* wq, const B200DLTensor* scales,
                         B200DLTensor* y);
B200_API int b200_q4f16_dequantize_dl(const B200DLTensor* wq, const B200DLTensor* scales, B200DLTensor* w_out);
/* b200_q4f16_matmul_dl with the kernel family chosen by the caller instead of by M: what the BYOC
 * codegen's option {"family": ...} selects (options reach a codegen through RunCodegen's map,
 * src/relax/transform/run_codegen.cc:42,155).  B200_FAMILY_GEMV requires 1 <= M <= 16. */
#define B200_FAMILY_AUTO 0
#define B200_FAMILY_GEMV 1
#define B200_FAMILY_GEMM 2
/* `family` bits 0-7: B200_FAMILY_*; bits 8-15: 0 = the process-wide weight layout (option "weights.layout"),
 * else B200_LAYOUT_* + 1 for this call (B200_FAMILY_WITH_LAYOUT). */
#define B200_FAMILY_WITH_LAYOUT(family, layout) ((family) | (((layout) + 1) << 8))
B200_API int b200_q4f16_matmul_dl_family(const B200DLTensor* x, const B200DLTensor* wq, const B200DLTensor* scales,
                                         B200DLTensor* y, int32_t family);

/* ---- output projection of a decode step -------------------------------------------------
 * logits fp16 [B, V] = h fp16 [B, H] . w fp16 [V, H]^T, fp32 accumulation, one RN-even rounding: the reference's
 * generic matmul + astype (python/tvm/relax/transform/legalize_ops.py:203-264, 157-162) on an unquantised
 * table, for 1 <= B <= 16 rows (above that a library GEMM is the right tool).  H % 32 == 0, 16-byte aligned
 * pointers.  `logits` may be NULL when only the tokens are wanted.  With `tokens` != NULL the kernel also
 * writes the greedy choice of every row, token_offset + argmax over the V rows of THIS table (ties: the lowest
 * index), which needs `scratch`: b200_lm_head_scratch_bytes() bytes of device memory, zeroed once by the caller
 * and left zeroed-where-it-matters by every call; calls that share a scratch buffer must be ordered (one stream).
 * Allocates nothing. */
B200_API int64_t b200_lm_head_scratch_bytes(void);
B200_API int b200_lm_head(const void* h, const void* w, void* logits, int32_t* tokens, void* scratch, int64_t B,
                          int64_t V, int64_t H, int64_t token_offset, void* stream);

/* ---- offline weight repack --------------------------------------------------------------
 * The reference binds weights into the executable as constants when it builds
 * (python/tvm/relax/vm.py:620-629 hands `const_name_to_constant` to the external codegen's modules), so a
 * backend is free to store them in the order its kernels prefer.  B200_LAYOUT_REFERENCE is what the
 * reference's encoder writes: nibble j of word i of a row is k = 8 i + j.  B200_LAYOUT_PAIRED keeps shape,
 * dtype and scales and permutes the nibbles inside every 32-bit word to k0,k2,k4,k6,k1,k3,k5,k7: the kernels'
 * mask-and-or unpack then yields (k0,k1)(k2,k3)(k4,k5)(k6,k7) directly, which saves the tensor-core kernels'
 * dequantisers four byte permutes per word and the skinny kernels the permutation of x.
 * repack: reference order -> `layout`; unpack: `layout` -> reference order; each is the other's exact
 * inverse (bit for bit).  `out` may be the same buffer as `in` (in place) but must not otherwise overlap it.
 * Every matmul and dequantise entry point reads its weights in the process-wide layout (option
 * "weights.layout", default B200_LAYOUT_REFERENCE) unless the call names one (the *_layout entry points,
 * B200_FAMILY_WITH_LAYOUT). */
#define B200_LAYOUT_REFERENCE 0
#define B200_LAYOUT_PAIRED 1
B200_API int b200_q4f16_repack(const void* wq, void* packed_out, int64_t N, int64_t K, int32_t layout, void* stream);
B200_API int b200_q4f16_unpack(const void* packed, void* wq_out, int64_t N, int64_t K, int32_t layout, void* stream);
B200_API int b200_q4f16_matmul_layout(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                                      int64_t K, int32_t layout, void* stream);
B200_API int b200_q4f16_dequantize_layout(const void* wq, const void* scales, void* w_out, int64_t N, int64_t K,
                                          int32_t layout, void* stream);

/* ---- packed-function symbols of the reference's C backend ABI ---------------------------
 * Signature TVMBackendPackedCFunc (include/tvm/runtime/c_backend_api.h:49-51); the form the
 * reference's BYOC C wrapper emits (src/relay/backend/contrib/codegen_c/codegen_c.h:101-112).
 * `args` is an array of 8-byte TVMValue unions, tensors arrive as v_handle with type code
 * 7 (kTVMDLTensorHandle) or 13 (kTVMNDArrayHandle).  Arguments: (x, wq, scales, y) and
 * (wq, scales, w_out).  Return 0, or -1 with the message available from b200_last_error()
 * (a TVM build forwards it with TVMAPISetLastError). */
B200_API int32_t b200_q4f16_matmul_packed(void* args, int* type_codes, int num_args, void* out_value,
                                 int* out_type_code, void* resource_handle);
B200_API int32_t b200_q4f16_dequantize_packed(void* args, int* type_codes, int num_args, void* out_value,
                                     int* out_type_code, void* resource_handle);

/* ---- skinny matmul with a neighbour of the decoder layer fused in (1 <= M <= 16, K % 256 == 0,
 * scales 16-byte aligned).  The reference reaches the same effect when FuseOps folds elementwise
 * producers/consumers into the matmul group (src/relay/analysis/graph_partitioner.cc:285-296).
 *
 * gemv_rmsnorm:  r = fp16(x + delta)  (delta may be NULL);  if x_out != NULL, x_out = r (the updated
 *                residual stream; must not alias x);  y = (r * rsqrt(mean(r^2) + eps) * norm_w) . W^T
 * gemv_swiglu:   gu fp16 [M, 2K] = gate | up;  y = (silu(gate) * up) . W^T
 * Statistics and products in fp32, one fp16 rounding of the activation, as the stand-alone kernels. */
B200_API int b200_q4f16_gemv_rmsnorm(const void* x, const void* delta, const void* norm_w, void* x_out, float eps,
                                     const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                                     void* cuda_stream);
/* gemv_rmsnorm for the qkv projection of ONE decode row, with b200_rope_kv_append in its epilogue: the matmul's
 * rows are [q heads | k heads | v heads] (heads of 128); q is rotated (rotate-half pairing d <-> d+64, tables fp32
 * [max_pos, 64], position *pos) into q_out fp16 [heads*128], the rotated key and the value of the new token go
 * into k_cache / v_cache fp16 [max_ctx, heads, 128] at slot *pos; there is no qkv buffer.  Same arithmetic as the
 * two separate kernels (the rotation works on the fp16-rounded matmul results).  Returns B200_ENOTREADY, with
 * nothing launched, when this launch would not use the skinny kernel's fast form (option gemv.exact = 1, or K below
 * 2560): call the two separate entry points then. */
B200_API int b200_q4f16_gemv_rmsnorm_rope(const void* x, const void* delta, const void* norm_w, void* x_out, float eps,
                                          const void* wq, const void* scales, const void* cos_t, const void* sin_t,
                                          const void* pos, void* q_out, void* k_cache, void* v_cache, int64_t heads,
                                          int64_t K, void* cuda_stream);
B200_API int b200_q4f16_gemv_swiglu(const void* gu, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                                    int64_t K, void* cuda_stream);

/* ---- row-parallel skinny matmul with the sum over tensor-parallel ranks fused in ------------------
 * The reference has no sharding or collective; this is the row-parallel half of the tensor-parallel
 * layout: every rank multiplies its K slice, the partial results are added over ranks.  Here the sum
 * is the tail of the matmul kernel itself, over NVLink peer memory, instead of a separate collective:
 * the CTA that finishes last on a GPU publishes a flag to every peer, waits (bounded, 2 s) for theirs,
 * then adds the `world` partial results in rank order (same bits on every rank) into `out`.
 *
 *   y            this rank's partial result [M,N] fp16; must be peer_y[rank], i.e. memory every peer maps
 *   peer_y[r]    rank r's y as mapped on this GPU; peer_flags[r]: rank r's int32 flag array likewise
 *   flag_base    first of `world` consecutive flag slots reserved for this call site
 *   epoch        device int32 that grows by one per step; flags carry *epoch + 1, so slots are never reset
 *   done_counter device int32, zero before the first launch (the kernel leaves it zero)
 *   out          [M,N] fp16 local result
 * A call site may reuse y / its flag slots in the next step only after another reduction of this kind
 * has completed in between (two alternating call sites, as o-proj and down-proj of a decoder layer,
 * satisfy this).  1 <= M <= 16, K % 256 == 0, N % 8 == 0, scales 16-byte aligned, world <= 8.
 * swiglu != 0: x is gate|up [M,2K] and silu(gate)*up is applied first (see b200_q4f16_gemv_swiglu).
 * A wait that runs out (after option "gemv.peer_wait_ms", default 2000) sets bit 4 of the skinny kernel's
 * byte in b200_device_error_flags(); the kernel still finishes and writes `out` from whatever the peers'
 * buffers hold. */
typedef struct {
  int32_t world, rank;
  const void* peer_y[8];
  void* peer_flags[8];
  int32_t flag_base;
  const void* epoch;
  void* done_counter;
  void* out;
} B200PeerReduce;
B200_API int b200_q4f16_gemv_allreduce(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N,
                                       int64_t K, int32_t swiglu, const B200PeerReduce* red, void* cuda_stream);

/* The same sum as a kernel of its own, for partial results that another kernel of this library wrote (the
 * mid-batch and prefill matmuls have no fused tail): out = sum over ranks of peer_y[r][0..count), fp16, in rank
 * order.  The partial result peer_y[rank] must have been written by work that precedes this call in `stream`.
 * Same descriptor and the same rules for flag slots and buffer reuse as above (`done_counter` is not used);
 * count % 8 == 0; a wait that runs out sets the same error bit.  Every rank must make the matching call. */
B200_API int b200_allreduce_peer(int64_t count, const B200PeerReduce* red, void* cuda_stream);

/* ---- one decoder layer of a batch-1 decode step as ONE persistent kernel -----------------------------
 * The reference reaches a comparable effect when FuseOps folds a matmul's elementwise neighbours into its
 * group (src/relay/analysis/graph_partitioner.cc:285-296); it has no kernel that spans several matmuls.
 * Here a grid of one CTA per SM walks
 *     qkv = Wqkv . rmsnorm(x_in + delta_in)        x_mid = x_in + delta_in
 *     attn = attention(rope(q), cache + rope(k), v)    (rotary embedding, KV append at *pos, softmax over 0..*pos)
 *     o = Wo . attn  (+ sum over ranks)            x_out = x_mid + o
 *     act = silu(gate) * up,  gate | up = Wgu . rmsnorm(x_out)       down = Wdown . act  (+ sum over ranks)
 * handing over between the stages through arrival counters in `scratch` (bounded waits; a wait that runs out
 * sets a bit of byte 3 of b200_device_error_flags and the kernel runs through).  The caller adds `down` to
 * x_out (the next layer does it as its delta_in).  Batch 1; heads of 128; hidden, hidden / world and
 * inter_local multiples of 256; weights in the layout of this header (qkv rows = q heads | k heads | v heads of
 * this rank, gu rows = gate | up).  KV caches fp16 [max_ctx, heads / world, 128].
 *   scratch   b200_decode_layer_scratch_bytes(heads / world, max_ctx) bytes PER LAYER, zero before the first step
 *             (the kernel leaves its counters consistent from step to step; do not share it between layers)
 *   step      device int32 that grows by exactly one between two decode steps (the counters count arrivals up
 *             to grid * (*step + 1)); all layers of a step see the same value
 *   world > 1 reduce_o / reduce_down: as B200PeerReduce of b200_q4f16_gemv_allreduce, with `epoch`, `done_counter`
 *             and `out` unused (flags carry *step + 1; results go to o / down); the partial results live in
 *             peer_y[rank].  The two reductions must use different buffers and flag slots (a buffer is written
 *             again only after another reduction has completed in between).
 * Launches of this kernel must follow each other in one stream: all its CTAs wait for each other, so they must
 * be resident together, which holds when nothing else competes for the SMs at that moment. */
typedef struct {
  int32_t world, rank;
  int64_t hidden, inter_local, max_ctx;
  int32_t heads;                  /* of the whole model; this rank takes heads / world */
  float eps;
  const void* x_in; const void* delta_in;      /* delta_in may be NULL */
  void* x_mid; void* qkv; void* attn; void* o; void* x_out; void* act; void* down;   /* fp16: [hidden] [3*hidden/world] [hidden/world] [hidden] [hidden] [inter_local] [hidden] */
  const void* norm1; const void* norm2;
  const void* cos_t; const void* sin_t; const void* pos;
  void* k_cache; void* v_cache;
  void* scratch; const void* step;
  const void* wq_qkv; const void* s_qkv; const void* wq_o; const void* s_o;
  const void* wq_gu; const void* s_gu; const void* wq_down; const void* s_down;
  B200PeerReduce reduce_o, reduce_down;
} B200DecodeLayer;
B200_API int64_t b200_decode_layer_scratch_bytes(int64_t heads_local, int64_t max_ctx);
B200_API int b200_decode_layer(const B200DecodeLayer* layer, void* cuda_stream);

/* ---- glue kernels of a decode step (around the quantised matmuls) --------------------------
 * The reference has no RMSNorm / RoPE / attention op; these compute the composition of its
 * elementwise ops (mean, sqrt, divide, multiply, softmax, silu: python/tvm/relax/transform/
 * legalize_ops.py:378-381,506-514) with fp32 statistics and one fp16 rounding at each output.
 * All pointers are device pointers; `pos` points at one int32 (the position of the token being
 * decoded, read on the device so that a captured CUDA graph can be replayed for every position). */

/* y[b,:] = rmsnorm(x[b,:]) * w.  If delta != NULL, x += delta first (x is updated in place: the
 * residual stream).  x, delta, y fp16 [B,H]; w fp16 [H]; H % 8 == 0, H <= 16384. */
B200_API int b200_rmsnorm(void* x, const void* delta, const void* w, void* y, int64_t B, int64_t H, float eps,
                          void* cuda_stream);

/* Rotary embedding of q and k (pairs i, i+64 of a 128-wide head; cos/sin fp32 [max_pos,64]), then k
 * and v are stored in the caches at position *pos.  qkv fp16 [B, 3*nh*128] = [q | k | v];
 * q_out fp16 [B, nh, 128]; caches fp16 [B, max_ctx, nh, 128]. */
B200_API int b200_rope_kv_append(const void* qkv, const void* cos_t, const void* sin_t, const void* pos, void* q_out,
                                 void* k_cache, void* v_cache, int64_t B, int64_t nh, int64_t max_ctx,
                                 void* cuda_stream);

/* out fp16 [B, nh*128] = softmax(q.K^T / sqrt(128)) . V over positions 0..*pos.  `scratch` is
 * caller-owned device memory of b200_attn_decode_scratch_bytes(B, nh, max_ctx) bytes holding the
 * per-chunk partial results (two launches: partials over 128-token chunks, then the merge).
 * B, nh <= 65535.
 *
 * flags = 0: every input is read after the kernel has synchronised with the launch in front of it in
 * the stream; any sequence of launches is safe.
 * flags = B200_ATTN_EARLY_KV_LOADS: *pos and the cache entries at positions BELOW *pos are read before
 * that synchronisation, so that the first K/V loads overlap the tail of the preceding kernel.  The
 * attention kernel may then start while the kernel TWO launches back is still running, unless the
 * launch directly in front of it waits for its own predecessor before it lets its dependents start.
 * So set the flag only when both hold:
 *   (1) the launch directly in front of this call writes neither *pos nor a cache entry below *pos, and
 *       it is either not a programmatic-dependent launch or one that executes griddepcontrol.wait before
 *       griddepcontrol.launch_dependents (b200_rope_kv_append, b200_rmsnorm, b200_silu_mul,
 *       b200_embed_rows and b200_advance_pos of this library do; the q4f16 matmul entry points do NOT:
 *       they release their dependents first, so with one of them directly in front, leave the flag clear);
 *   (2) whatever last wrote *pos or those cache entries was launched before that launch.
 * The entry at *pos itself and q may be written by the launch directly in front (that is what
 * b200_rope_kv_append does; the decode engine of this repository calls it there and sets the flag). */
#define B200_ATTN_EARLY_KV_LOADS 1u
B200_API int64_t b200_attn_decode_scratch_bytes(int64_t B, int64_t nh, int64_t max_ctx);
B200_API int b200_attn_decode(const void* q, const void* k_cache, const void* v_cache, const void* pos, void* out,
                              void* scratch, int64_t B, int64_t nh, int64_t max_ctx, uint32_t flags, void* cuda_stream);

/* Rotary embedding of q and k, KV append at *pos, attention over positions 0..*pos and the merge of
 * the per-chunk partials in one launch (what b200_rope_kv_append + b200_attn_decode do in three).
 * qkv fp16 [B, 3*nh*128] = [q | k | v] of the new token; out fp16 [B, nh*128].  `scratch`:
 * b200_attn_decode_fused_scratch_bytes(B, nh, max_ctx) bytes of caller-owned device memory whose last
 * B*nh int32 (the arrival counters) must be ZERO before the first call; the kernel leaves them zero. */
B200_API int64_t b200_attn_decode_fused_scratch_bytes(int64_t B, int64_t nh, int64_t max_ctx);
B200_API int b200_attn_decode_fused(const void* qkv, const void* cos_t, const void* sin_t, const void* pos, void* k_cache,
                                    void* v_cache, void* out, void* scratch, int64_t B, int64_t nh, int64_t max_ctx,
                                    void* cuda_stream);

/* The same in two launches: rotary embedding, KV append and the per-chunk attention in the first, the
 * merge of the partials in the second (no arrival counters).  Arguments as b200_attn_decode_fused;
 * `scratch` needs b200_attn_decode_scratch_bytes(B, nh, max_ctx) bytes and no initialisation. */
B200_API int b200_attn_decode_rope(const void* qkv, const void* cos_t, const void* sin_t, const void* pos, void* k_cache,
                                   void* v_cache, void* out, void* scratch, int64_t B, int64_t nh, int64_t max_ctx,
                                   void* cuda_stream);

/* Same attention for callers that cannot hand over scratch memory.  (No counterpart in the
 * reference.)  Some hosts of this library are not allowed to allocate device memory at the point
 * where they call it: a runtime whose memory planner has already fixed every buffer of the step,
 * or a plugin running under a host that forbids cudaMalloc on its threads.  This entry point
 * allocates nothing, neither here nor in anything it calls: the partial results of the two-pass
 * attention go to a 4.26 MB array that is part of the library image on every GPU that loads it.
 *   - Limit: B * nh * ceil(max_ctx / 128) <= 8192 (e.g. 16 sequences x 32 heads x 2048 tokens);
 *     larger problems are refused with B200_EINVAL and a message, nothing is launched.
 *   - The first call on each device looks up the array's device address (make that device current;
 *     do this first call outside any stream capture).
 *   - All calls on a device share the one array: two calls that overlap on the GPU (different
 *     streams) overwrite each other's partial results.  Calls ordered on one stream are safe; every
 *     slot that is read has been written by the same call, so nothing needs clearing in between.
 *   - `flags` as for b200_attn_decode (0 is always safe). */
B200_API int b200_attn_decode_static(const void* q, const void* k_cache, const void* v_cache, const void* pos, void* out,
                                     int64_t B, int64_t nh, int64_t max_ctx, uint32_t flags, void* cuda_stream);

/* out[b,:] = table[ids[b],:]: fp16 table [vocab,H], int32 ids [B] on the device (ids are clamped
 * to the table).  H % 8 == 0.  (reference: relax.take, python/tvm/relax/transform/legalize_ops.py:168) */
B200_API int b200_embed_rows(const void* table, const void* ids, void* out, int64_t B, int64_t H, int64_t vocab,
                             void* cuda_stream);

/* *pos += delta on the device (pos: one int32). */
B200_API int b200_advance_pos(void* pos, int64_t delta, void* cuda_stream);

/* out[b,i] = silu(gu[b,i]) * gu[b,I+i]; gu fp16 [B,2I], out fp16 [B,I]; I % 8 == 0. */
B200_API int b200_silu_mul(const void* gu, void* out, int64_t B, int64_t I, void* cuda_stream);

/* ---- introspection used by tests and the benchmark --------------------------------------- */

/* Number of kernels this library has launched on the calling thread since the last reset. */
B200_API int64_t b200_launch_count(void);
B200_API void b200_reset_launch_count(void);

/* Reads (and clears) the device-side error word: non-zero when a kernel's bounded wait ran
 * out and it gave up instead of spinning.  Synchronises the device; for tests and diagnosis.
 * Returns the flag bits (>= 0) or a negative B200_E* code. */
B200_API int b200_device_error_flags(void);

/* Selects a kernel variant / tuning knob by name (e.g. "gemv.warps", "gemv.peer_wait_ms"); returns B200_EINVAL for
 * an unknown name or value.  Intended for benchmarking sweeps; defaults are the tuned ones. */
B200_API int b200_set_option(const char* name, int64_t value);
B200_API int64_t b200_get_option(const char* name);

#ifdef __cplusplus
}
#endif
#endif /* B200_Q4F16_H_ */
