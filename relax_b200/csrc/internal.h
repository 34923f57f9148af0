// Host-side declarations shared by the translation units of the kernel library.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_q4f16.h"

namespace b200 {

// Stores a printf-formatted message for b200_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void count_launch(int n = 1);

// Tuning knobs (b200_set_option).  Plain ints; read at launch time.
struct Options {
  int64_t gemv_variant = 0;   // 0 = auto, 1 = register-streaming kernel, 2 = bulk-copy pipelined kernel
  int64_t gemv_warps = 0;     // 0 = auto
  int64_t gemv_stages = 0;    // 0 = auto (bulk-copy pipeline depth)
  int64_t gemv_pdl = 1;       // programmatic dependent launch on the streaming kernels
  int64_t gemv_ctas_per_sm = 0;  // 0 = auto: cap on resident CTAs per SM used to size the grid
  int64_t gemv_exact = 0;     // batch-1 form of the skinny kernel: 0 = fast form where K fills its stages, exact form otherwise;
                              // 1 = always round every weight to fp16 as the reference does (exact form); 2 = always the fast form
  int64_t gemv_peer_wait_ms = 2000;  // how long the fused sum over ranks waits for the other GPUs' flags
  int64_t layer_wait_ms = 2000; // layer kernel: how long a CTA waits at a stage counter, a peer flag or a weight stage
  int64_t layer_stages = 0;     // layer kernel: depth of the weight ring (0 = as many as fit, at most 5)
  int64_t layer_max_ctas = 0;   // layer kernel: cap on the grid (0 = one CTA per SM); tests use small grids
  int64_t gemm_max_ctas = 0;  // 0 = one per SM; smaller values force several tiles per CTA (tests)
  int64_t gemm_ws_ksplit = 0; // 0 = auto: K slices (= cluster size) of the weight-stationary kernel
  int64_t weights_layout = 0; // B200_LAYOUT_*: the nibble order every matmul entry point assumes unless the call names one
  int64_t gemm_ws_x_stages = 0; // 0 = auto: cap on the depth of the weight-stationary kernel's x ring
  int64_t gemm_ws_w_stages = 0; // 0 = auto (2): depth of its dequantised-weight ring
  int64_t gemm_ws_r_stages = 0; // 0 = auto: cap on the depth of its packed-weight ring (>= 2)
  int64_t gemm_ws_xk = 0;       // 0 = auto: K blocks per stage of its x and dequantised rings (2 or 4)
  int64_t gemm_ws_max_m = 128; // largest M the automatic dispatch gives to the weight-stationary kernel (0 = never)
};
Options& options();

// Weight layout of the matmul being launched on this thread: the call's own (entry points that carry a layout
// set it for their duration through LayoutScope), else the process-wide option.
int current_layout();
struct LayoutScope {
  explicit LayoutScope(int layout);   // layout < 0: keep the option's
  ~LayoutScope();
  int saved;
};

// Kernel launchers: arguments validated by the caller, pointers are device pointers.
int launch_dequantize(const uint32_t* wq, const __half* scales, __half* w, int64_t N, int64_t K,
                      cudaStream_t stream);
// Word-wise permutation between the reference's nibble order and `layout` (to_layout = true: reference -> layout).
int launch_repack(const uint32_t* in, uint32_t* out, int64_t n_words, int layout, bool to_layout, cudaStream_t stream);
int launch_gemv(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                int64_t K, cudaStream_t stream);
// Skinny matmul with a neighbour of the decoder layer fused into the staging of x (1 <= M <= 16,
// K % 256 == 0, 16-byte aligned scales; B200_ENOTREADY otherwise).
int launch_gemv_pipe_rmsnorm(const __half* x, const __half* delta, const __half* norm_w, __half* x_out, float eps,
                             const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N, int64_t K,
                             cudaStream_t stream);
int launch_gemv_pipe_rmsnorm_rope(const __half* x, const __half* delta, const __half* norm_w, __half* x_out, float eps,
                                  const uint32_t* wq, const __half* scales, const float* cos_t, const float* sin_t,
                                  const int* pos, __half* q_out, __half* k_cache, __half* v_cache, int64_t nh, int64_t K,
                                  cudaStream_t stream);
int launch_gemv_pipe_swiglu(const __half* gu, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                            int64_t K, cudaStream_t stream);
int launch_gemv_pipe_allreduce(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                               int64_t K, int swiglu, const B200PeerReduce* red, cudaStream_t stream);
// Sum over tensor-parallel ranks of `count` fp16 values whose per-rank partial results sit in peer-mapped buffers
// (protocol of B200PeerReduce).
int launch_peer_allreduce(int64_t count, const B200PeerReduce* red, cudaStream_t stream);
int launch_gemm_ws(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                   int64_t K, cudaStream_t stream);
int launch_gemm(const __half* x, const uint32_t* wq, const __half* scales, __half* y, int64_t M, int64_t N,
                int64_t K, cudaStream_t stream);

// fp16 output projection of a decode step (1 <= B <= 16) with optional greedy sampling; B200_ENOTREADY when the
// activations do not fit in shared memory.
int launch_lm_head(const __half* x, const __half* w, __half* logits, int* tokens, float* scratch, int64_t B, int64_t V,
                   int64_t H, int64_t token_offset, cudaStream_t stream);
int64_t lm_head_scratch_bytes();

// Reads and clears the per-kernel device error words (bit 0-7: skinny pipeline, 8-15: tensor-core GEMM, 16-23: weight-stationary GEMM,
// 24-30: decoder-layer kernel).
int device_error_flags_read_and_clear();
int gemv_pipe_error_read_and_clear();
int gemm_error_read_and_clear();
int gemm_ws_error_read_and_clear();
int layer_error_read_and_clear();

// Device capability check, cached per device; 0 when the current device is sm_100.
int ensure_device();
int sm_count();

}  // namespace b200
