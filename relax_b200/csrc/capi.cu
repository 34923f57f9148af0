// C ABI of the kernel library: argument validation, kernel-family dispatch, error state.
// Everything a caller outside this library may bind is declared in include/b200_q4f16.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "internal.h"

namespace b200 {

namespace {
thread_local char g_err[512] = {0};
thread_local int64_t g_launches = 0;
thread_local cudaStream_t g_stream = nullptr;
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches += n; }

Options& options() {
  static Options o;
  return o;
}

thread_local int g_call_layout = -1;
int current_layout() { return g_call_layout >= 0 ? g_call_layout : (int)options().weights_layout; }
LayoutScope::LayoutScope(int layout) : saved(g_call_layout) {
  if (layout >= 0) g_call_layout = layout;
}
LayoutScope::~LayoutScope() { g_call_layout = saved; }

// Per-process cache of "device d is usable" (index = device ordinal).
int ensure_device() {
  static int ok[64] = {0};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200_ENODEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (dev >= 0 && dev < 64 && ok[dev]) return B200_OK;
  cudaDeviceProp p;
  e = cudaGetDeviceProperties(&p, dev);
  if (e != cudaSuccess) return fail(B200_ENODEVICE, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (p.major != 10)
    return fail(B200_ENODEVICE, "device %d is sm_%d%d; this library is built for sm_100a only and has no fallback",
                dev, p.major, p.minor);
  if (dev >= 0 && dev < 64) ok[dev] = 1;
  return B200_OK;
}

int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(const char* who, const void* wq, const void* scales, int64_t N, int64_t K) {
  if (N < 0 || K < 0) return fail(B200_EINVAL, "%s: negative size N=%lld K=%lld", who, (long long)N, (long long)K);
  if (K % 32 != 0) return fail(B200_EINVAL, "%s: K=%lld is not a multiple of the group size 32", who, (long long)K);
  if (N > 0x7fffffffLL / 32 || K > 0x3fffffffLL)
    return fail(B200_EINVAL, "%s: N=%lld K=%lld exceeds the supported range", who, (long long)N, (long long)K);
  if (N > 0 && K > 0) {
    if (!wq || !scales) return fail(B200_EINVAL, "%s: null weight or scale pointer", who);
    if (!aligned16(wq)) return fail(B200_EINVAL, "%s: packed weights must be 16-byte aligned", who);
    if (reinterpret_cast<uintptr_t>(scales) & 1u) return fail(B200_EINVAL, "%s: scales must be 2-byte aligned", who);
  }
  return B200_OK;
}

int check_matmul(const char* who, const void* x, const void* wq, const void* scales, const void* y, int64_t M,
                 int64_t N, int64_t K) {
  if (M < 0) return fail(B200_EINVAL, "%s: negative M=%lld", who, (long long)M);
  int rc = check_common(who, wq, scales, N, K);
  if (rc) return rc;
  if (M > 0x7fffffffLL / 64) return fail(B200_EINVAL, "%s: M=%lld exceeds the supported range", who, (long long)M);
  if (M > 0 && K > 0 && (!x || !aligned16(x))) return fail(B200_EINVAL, "%s: x must be non-null and 16-byte aligned", who);
  if (M > 0 && N > 0 && (!y || (reinterpret_cast<uintptr_t>(y) & 1u)))
    return fail(B200_EINVAL, "%s: y must be non-null and 2-byte aligned", who);
  return B200_OK;
}

// y = 0 when the reduction is empty (K == 0): the sum over no terms.
int zero_output(void* y, int64_t M, int64_t N, cudaStream_t s) {
  if (M * N == 0) return B200_OK;
  cudaError_t e = cudaMemsetAsync(y, 0, (size_t)(M * N) * 2, s);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  return B200_OK;
}

enum Family { kAuto, kGemv, kGemm, kGemmWs };

int matmul_impl(Family fam, const char* who, const void* x, const void* wq, const void* scales, void* y, int64_t M,
                int64_t N, int64_t K, void* stream) {
  int rc = check_matmul(who, x, wq, scales, y, M, N, K);
  if (rc) return rc;
  if (fam == kGemv && (M < 1 || M > 16))
    return fail(B200_EINVAL, "%s: the skinny kernel takes 1 <= M <= 16, got %lld", who, (long long)M);
  rc = ensure_device();
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (M == 0 || N == 0) return B200_OK;
  if (K == 0) return zero_output(y, M, N, s);
  bool use_gemv = fam == kGemv || (fam == kAuto && M <= 16);
  // 9..16 batch rows: the skinny kernel stages all of x in every CTA (and restages it in K blocks once 16 rows x K
  // no longer fit beside its ring); the weight-stationary kernel streams x through a ring instead.  Measured on
  // B200 it is the faster one wherever its K split is in use (N up to about 8192: 9.8 against 12.1 us at
  // N = K = 4096, 16.4 against 29.5 at K = 11008) and always when x does not fit; with many row tiles the skinny
  // kernel wins (24.8 against 39 us at N = 22016).
  if (fam == kAuto && M >= 9 && M <= 16 && (N <= 8192 || M * K * 2 > 160 * 1024) && K % 256 == 0 && options().gemm_ws_max_m >= M) {
    rc = launch_gemm_ws(static_cast<const __half*>(x), static_cast<const uint32_t*>(wq), static_cast<const __half*>(scales),
                        static_cast<__half*>(y), M, N, K, s);
    if (rc != B200_ENOTREADY) return rc;
  }
  auto xh = static_cast<const __half*>(x);
  auto wh = static_cast<const uint32_t*>(wq);
  auto sh = static_cast<const __half*>(scales);
  auto yh = static_cast<__half*>(y);
  if (use_gemv) return launch_gemv(xh, wh, sh, yh, M, N, K, s);
  // Mid-sized batches (up to 128 rows): the weights stream once whatever the batch, which the prefill kernel's
  // 256-token tiles would waste (measured at M = 64: 23.7 against 51 us at N = 12288, 46 against 51 at N = 22016).
  if (fam == kGemmWs || (fam == kAuto && M <= options().gemm_ws_max_m)) {
    rc = launch_gemm_ws(xh, wh, sh, yh, M, N, K, s);
    if (rc != B200_ENOTREADY) return rc;
    if (fam == kGemmWs) return fail(B200_EINVAL, "%s: the weight-stationary kernel takes 1 <= M <= 128, K %% 256 == 0, 16-byte aligned scales", who);
  }
  return launch_gemm(xh, wh, sh, yh, M, N, K, s);
}

// ---- DLPack validation -------------------------------------------------------------------
bool is_dtype(const B200DLTensor* t, int code, int bits) {
  return t->dtype.code == code && t->dtype.bits == bits && t->dtype.lanes == 1;
}

int check_tensor(const char* who, const char* name, const B200DLTensor* t, int code, int bits, int* dev) {
  if (!t) return fail(B200_EINVAL, "%s: %s is null", who, name);
  if (t->ndim != 2) return fail(B200_EINVAL, "%s: %s must have 2 dimensions, has %d", who, name, t->ndim);
  if (!t->shape) return fail(B200_EINVAL, "%s: %s has no shape", who, name);
  if (!is_dtype(t, code, bits))
    return fail(B200_EINVAL, "%s: %s must be %s%d, got code=%d bits=%d lanes=%d", who, name,
                code == 2 ? "float" : "uint", bits, t->dtype.code, t->dtype.bits, t->dtype.lanes);
  if (t->device.device_type != 2 /* kDLCUDA */)
    return fail(B200_EINVAL, "%s: %s is not on a CUDA device (device_type=%d)", who, name, t->device.device_type);
  if (*dev < 0) *dev = t->device.device_id;
  else if (*dev != t->device.device_id)
    return fail(B200_EINVAL, "%s: %s is on device %d, other arguments on device %d", who, name, t->device.device_id, *dev);
  if (t->strides && t->shape[0] != 0 && t->shape[1] != 0) {  // compact row-major only (strides of size-1 dimensions are free)
    int64_t expect = 1;
    for (int i = 1; i >= 0; --i) {
      if (t->shape[i] != 1 && t->strides[i] != expect)
        return fail(B200_EINVAL, "%s: %s is not contiguous", who, name);
      expect *= t->shape[i];
    }
  }
  if (t->shape[0] < 0 || t->shape[1] < 0) return fail(B200_EINVAL, "%s: %s has a negative extent", who, name);
  return B200_OK;
}

void* data_ptr(const B200DLTensor* t) { return static_cast<char*>(t->data) + t->byte_offset; }

int check_current_device(const char* who, int dev) {
  int cur = -1;
  cudaError_t e = cudaGetDevice(&cur);
  if (e != cudaSuccess) return fail(B200_ENODEVICE, "%s: no CUDA device: %s", who, cudaGetErrorString(e));
  if (cur != dev)
    return fail(B200_EINVAL, "%s: tensors live on device %d but the current device is %d", who, dev, cur);
  return B200_OK;
}

}  // namespace
}  // namespace b200

using namespace b200;

// Small host transfers as kernels.  A copy-engine transfer on either side of a 5 us matmul costs
// more than the matmul (each switch between the copy engine and the SMs is a few microseconds), so
// activations and results up to kHostKernelBytes travel by a one-CTA-per-16-KB kernel that reads or
// writes the pinned host buffer through its device mapping; the result copy is launched as a
// programmatic dependent of the matmul.  Pageable host memory and larger transfers use cudaMemcpyAsync.
namespace b200 {
namespace {
constexpr size_t kHostKernelBytes = 256 * 1024;

__global__ void __launch_bounds__(256) host_copy_kernel(const unsigned char* __restrict__ src, unsigned char* __restrict__ dst,
                                                        size_t bytes, int wait_for_primary) {
  if (wait_for_primary) asm volatile("griddepcontrol.wait;" ::: "memory");
  const size_t n16 = bytes >> 4;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  if (blockIdx.x == 0)
    for (size_t i = (n16 << 4) + threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
}

// Device-side address of a pinned (page-locked, mapped) host buffer, or null for anything else.
void* mapped_host_pointer(const void* host) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (a.type != cudaMemoryTypeHost) return nullptr;
  return a.devicePointer;
}

// dst <- src (one of them a mapped host buffer) on `s`; dependent = launch as a programmatic dependent
// of the kernel before it in the stream (the copy waits for that kernel's completion itself).
int host_copy(const void* src, void* dst, size_t bytes, bool dependent, cudaStream_t s) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((bytes + 16383) / 16384));
  cfg.blockDim = dim3(256);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, host_copy_kernel, static_cast<const unsigned char*>(src),
                                     static_cast<unsigned char*>(dst), bytes, dependent ? 1 : 0);
  if (e != cudaSuccess) return fail(B200_ELAUNCH, "q4f16_matmul_host: copy kernel: %s", cudaGetErrorString(e));
  count_launch();
  return B200_OK;
}
}  // namespace
}  // namespace b200

extern "C" {

const char* b200_last_error(void) { return g_err; }
int b200_abi_version(void) { return 102; }

int b200_set_stream(void* s) {
  g_stream = static_cast<cudaStream_t>(s);
  return B200_OK;
}
void* b200_get_stream(void) { return g_stream; }

int64_t b200_launch_count(void) { return g_launches; }
void b200_reset_launch_count(void) { g_launches = 0; }

int b200_device_error_flags(void) {
  int rc = ensure_device();
  if (rc) return rc;
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(B200_EDEVICE, "device_error_flags: %s", cudaGetErrorString(cudaGetLastError()));
  return device_error_flags_read_and_clear();
}

int b200_set_option(const char* name, int64_t v) {
  if (!name) return fail(B200_EINVAL, "set_option: null name");
  Options& o = options();
  if (!strcmp(name, "gemv.variant")) { if (v < 0 || v > 2) return fail(B200_EINVAL, "gemv.variant in 0..2"); o.gemv_variant = v; }
  else if (!strcmp(name, "gemv.warps")) { if (v < 0 || v > 16) return fail(B200_EINVAL, "gemv.warps in 0..16"); o.gemv_warps = v; }
  else if (!strcmp(name, "gemv.stages")) { if (v < 0 || v > 16) return fail(B200_EINVAL, "gemv.stages in 0..16"); o.gemv_stages = v; }
  else if (!strcmp(name, "gemv.pdl")) { o.gemv_pdl = v != 0; }
  else if (!strcmp(name, "gemv.ctas_per_sm")) { if (v < 0 || v > 8) return fail(B200_EINVAL, "gemv.ctas_per_sm in 0..8"); o.gemv_ctas_per_sm = v; }
  else if (!strcmp(name, "gemv.exact")) { if (v < 0 || v > 2) return fail(B200_EINVAL, "gemv.exact is 0 (by shape), 1 (exact form) or 2 (fast form)"); o.gemv_exact = v; }
  else if (!strcmp(name, "gemv.peer_wait_ms")) { if (v < 1 || v > 60000) return fail(B200_EINVAL, "gemv.peer_wait_ms in 1..60000"); o.gemv_peer_wait_ms = v; }
  else if (!strcmp(name, "layer.wait_ms")) { if (v < 1 || v > 60000) return fail(B200_EINVAL, "layer.wait_ms in 1..60000"); o.layer_wait_ms = v; }
  else if (!strcmp(name, "layer.stages")) { if (v < 0 || v > 5) return fail(B200_EINVAL, "layer.stages in 0..5"); o.layer_stages = v; }
  else if (!strcmp(name, "layer.max_ctas")) { if (v < 0 || v > 1024) return fail(B200_EINVAL, "layer.max_ctas in 0..1024"); o.layer_max_ctas = v; }
  else if (!strcmp(name, "gemm.ws_ksplit")) { if (v < 0 || v > 8 || (v & (v - 1))) return fail(B200_EINVAL, "gemm.ws_ksplit is 0, 1, 2, 4 or 8"); o.gemm_ws_ksplit = v; }
  else if (!strcmp(name, "gemm.ws_x_stages")) { if (v < 0 || v > 8) return fail(B200_EINVAL, "gemm.ws_x_stages in 0..8"); o.gemm_ws_x_stages = v; }
  else if (!strcmp(name, "gemm.ws_w_stages")) { if (v < 0 || v > 8) return fail(B200_EINVAL, "gemm.ws_w_stages in 0..8"); o.gemm_ws_w_stages = v; }
  else if (!strcmp(name, "gemm.ws_r_stages")) { if (v < 0 || v == 1 || v > 8) return fail(B200_EINVAL, "gemm.ws_r_stages is 0 or in 2..8"); o.gemm_ws_r_stages = v; }
  else if (!strcmp(name, "gemm.ws_xk")) { if (v != 0 && v != 2 && v != 4) return fail(B200_EINVAL, "gemm.ws_xk is 0, 2 or 4"); o.gemm_ws_xk = v; }
  else if (!strcmp(name, "gemm.ws_max_m")) { if (v < 0 || v > 128) return fail(B200_EINVAL, "gemm.ws_max_m in 0..128"); o.gemm_ws_max_m = v; }
  else if (!strcmp(name, "weights.layout")) { if (v != B200_LAYOUT_REFERENCE && v != B200_LAYOUT_PAIRED) return fail(B200_EINVAL, "weights.layout is 0 (reference) or 1 (paired)"); o.weights_layout = v; }
  else if (!strcmp(name, "gemm.max_ctas")) { if (v < 0 || v > 1024) return fail(B200_EINVAL, "gemm.max_ctas in 0..1024"); o.gemm_max_ctas = v; }
  else return fail(B200_EINVAL, "set_option: unknown option '%s'", name);
  return B200_OK;
}

int64_t b200_get_option(const char* name) {
  if (!name) return -1;
  Options& o = options();
  if (!strcmp(name, "gemv.variant")) return o.gemv_variant;
  if (!strcmp(name, "gemv.warps")) return o.gemv_warps;
  if (!strcmp(name, "gemv.stages")) return o.gemv_stages;
  if (!strcmp(name, "gemv.pdl")) return o.gemv_pdl;
  if (!strcmp(name, "gemv.ctas_per_sm")) return o.gemv_ctas_per_sm;
  if (!strcmp(name, "gemv.exact")) return o.gemv_exact;
  if (!strcmp(name, "gemv.peer_wait_ms")) return o.gemv_peer_wait_ms;
  if (!strcmp(name, "gemm.max_ctas")) return o.gemm_max_ctas;
  if (!strcmp(name, "layer.wait_ms")) return o.layer_wait_ms;
  if (!strcmp(name, "layer.stages")) return o.layer_stages;
  if (!strcmp(name, "layer.max_ctas")) return o.layer_max_ctas;
  if (!strcmp(name, "gemm.ws_ksplit")) return o.gemm_ws_ksplit;
  if (!strcmp(name, "gemm.ws_max_m")) return o.gemm_ws_max_m;
  if (!strcmp(name, "gemm.ws_x_stages")) return o.gemm_ws_x_stages;
  if (!strcmp(name, "gemm.ws_w_stages")) return o.gemm_ws_w_stages;
  if (!strcmp(name, "gemm.ws_xk")) return o.gemm_ws_xk;
  if (!strcmp(name, "gemm.ws_r_stages")) return o.gemm_ws_r_stages;
  if (!strcmp(name, "weights.layout")) return o.weights_layout;
  return -1;
}

int b200_q4f16_dequantize(const void* wq, const void* scales, void* w_out, int64_t N, int64_t K, void* stream) {
  int rc = check_common("q4f16_dequantize", wq, scales, N, K);
  if (rc) return rc;
  if (N > 0 && K > 0 && (!w_out || !aligned16(w_out)))
    return fail(B200_EINVAL, "q4f16_dequantize: output must be non-null and 16-byte aligned");
  rc = ensure_device();
  if (rc) return rc;
  return launch_dequantize(static_cast<const uint32_t*>(wq), static_cast<const __half*>(scales),
                           static_cast<__half*>(w_out), N, K, static_cast<cudaStream_t>(stream));
}

static int check_layout(const char* who, int32_t layout) {
  if (layout != B200_LAYOUT_REFERENCE && layout != B200_LAYOUT_PAIRED)
    return fail(B200_EINVAL, "%s: unknown weight layout %d (0 reference, 1 paired)", who, (int)layout);
  return B200_OK;
}

static int repack_impl(const char* who, const void* in, void* out, int64_t N, int64_t K, int32_t layout, bool to_layout,
                       void* stream) {
  int rc = check_layout(who, layout);
  if (rc) return rc;
  if (N < 0 || K < 0) return fail(B200_EINVAL, "%s: negative shape N=%lld K=%lld", who, (long long)N, (long long)K);
  if (K % 32 != 0) return fail(B200_EINVAL, "%s: K=%lld is not a multiple of the group size 32", who, (long long)K);
  if (N > 0 && K > 0 && (!in || !out)) return fail(B200_EINVAL, "%s: null pointer", who);
  if (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 3u) != 0)
    return fail(B200_EINVAL, "%s: buffers must be 4-byte aligned", who);
  if (N > 0 && K > 0 && in != out) {
    const char* a = static_cast<const char*>(in);
    const char* b = static_cast<const char*>(out);
    const int64_t bytes = N * (K / 2);
    if (a < b + bytes && b < a + bytes) return fail(B200_EINVAL, "%s: input and output overlap without being the same buffer", who);
  }
  if ((rc = ensure_device())) return rc;
  return launch_repack(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), N * (K / 8), layout, to_layout,
                       static_cast<cudaStream_t>(stream));
}

int64_t b200_lm_head_scratch_bytes(void) {
  if (ensure_device()) return -1;
  return lm_head_scratch_bytes();
}

int b200_lm_head(const void* h, const void* w, void* logits, int32_t* tokens, void* scratch, int64_t B, int64_t V,
                 int64_t H, int64_t token_offset, void* stream) {
  if (B < 1 || B > 16) return fail(B200_EINVAL, "lm_head: takes 1 <= B <= 16 rows, got %lld", (long long)B);
  if (V < 1 || V > 0x7fffff00LL || H < 32 || H % 32 != 0)
    return fail(B200_EINVAL, "lm_head: need 1 <= V < 2^31, H >= 32 and H %% 32 == 0 (V=%lld H=%lld)", (long long)V, (long long)H);
  if (!h || !w || (!logits && !tokens)) return fail(B200_EINVAL, "lm_head: null pointer (h, w, and one of logits / tokens are required)");
  if (tokens && !scratch) return fail(B200_EINVAL, "lm_head: tokens need the scratch buffer (b200_lm_head_scratch_bytes)");
  if (!aligned16(h) || !aligned16(w) || (scratch && !aligned16(scratch)) || (reinterpret_cast<uintptr_t>(logits) & 1u) ||
      (reinterpret_cast<uintptr_t>(tokens) & 3u))
    return fail(B200_EINVAL, "lm_head: h, w and scratch must be 16-byte aligned");
  if (token_offset < 0 || token_offset + V > 0x7fffffffLL) return fail(B200_EINVAL, "lm_head: token_offset + V overflows int32");
  int rc = ensure_device();
  if (rc) return rc;
  rc = launch_lm_head(static_cast<const __half*>(h), static_cast<const __half*>(w), static_cast<__half*>(logits), tokens,
                      static_cast<float*>(scratch), B, V, H, token_offset, static_cast<cudaStream_t>(stream));
  if (rc == B200_ENOTREADY) return fail(B200_EINVAL, "lm_head: %lld rows of H=%lld do not fit in shared memory", (long long)B, (long long)H);
  return rc;
}

int b200_q4f16_repack(const void* wq, void* packed_out, int64_t N, int64_t K, int32_t layout, void* stream) {
  return repack_impl("q4f16_repack", wq, packed_out, N, K, layout, true, stream);
}

int b200_q4f16_unpack(const void* packed, void* wq_out, int64_t N, int64_t K, int32_t layout, void* stream) {
  return repack_impl("q4f16_unpack", packed, wq_out, N, K, layout, false, stream);
}

int b200_q4f16_matmul_layout(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                             int32_t layout, void* stream) {
  int rc = check_layout("q4f16_matmul_layout", layout);
  if (rc) return rc;
  LayoutScope scope(layout);
  return matmul_impl(kAuto, "q4f16_matmul_layout", x, wq, scales, y, M, N, K, stream);
}

int b200_q4f16_dequantize_layout(const void* wq, const void* scales, void* w_out, int64_t N, int64_t K, int32_t layout,
                                 void* stream) {
  int rc = check_layout("q4f16_dequantize_layout", layout);
  if (rc) return rc;
  LayoutScope scope(layout);
  return b200_q4f16_dequantize(wq, scales, w_out, N, K, stream);
}

int b200_q4f16_matmul(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                      void* stream) {
  return matmul_impl(kAuto, "q4f16_matmul", x, wq, scales, y, M, N, K, stream);
}
int b200_q4f16_gemv(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                    void* stream) {
  return matmul_impl(kGemv, "q4f16_gemv", x, wq, scales, y, M, N, K, stream);
}
int b200_q4f16_gemm(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                    void* stream) {
  return matmul_impl(kGemm, "q4f16_gemm", x, wq, scales, y, M, N, K, stream);
}

int b200_q4f16_gemv_rmsnorm(const void* x, const void* delta, const void* norm_w, void* x_out, float eps, const void* wq,
                            const void* scales, void* y, int64_t M, int64_t N, int64_t K, void* stream) {
  const char* who = "q4f16_gemv_rmsnorm";
  int rc = check_matmul(who, x, wq, scales, y, M, N, K);
  if (rc) return rc;
  if (M < 1 || M > 16) return fail(B200_EINVAL, "%s: takes 1 <= M <= 16, got %lld", who, (long long)M);
  if (N < 1 || K < 256 || K % 256 != 0) return fail(B200_EINVAL, "%s: needs N >= 1 and K a positive multiple of 256", who);
  if (!aligned16(scales)) return fail(B200_EINVAL, "%s: scales must be 16-byte aligned", who);
  if (!norm_w || !aligned16(norm_w)) return fail(B200_EINVAL, "%s: norm weight must be non-null and 16-byte aligned", who);
  if ((delta && !aligned16(delta)) || (x_out && !aligned16(x_out))) return fail(B200_EINVAL, "%s: delta / x_out must be 16-byte aligned", who);
  if (x_out == x) return fail(B200_EINVAL, "%s: x_out must not alias x (other CTAs still read x)", who);
  rc = ensure_device();
  if (rc) return rc;
  rc = launch_gemv_pipe_rmsnorm(static_cast<const __half*>(x), static_cast<const __half*>(delta), static_cast<const __half*>(norm_w),
                                static_cast<__half*>(x_out), eps, static_cast<const uint32_t*>(wq),
                                static_cast<const __half*>(scales), static_cast<__half*>(y), M, N, K,
                                static_cast<cudaStream_t>(stream));
  if (rc == B200_ENOTREADY) return fail(B200_EINVAL, "%s: shape outside the fused kernel's domain", who);
  return rc;
}

int b200_q4f16_gemv_rmsnorm_rope(const void* x, const void* delta, const void* norm_w, void* x_out, float eps, const void* wq,
                                 const void* scales, const void* cos_t, const void* sin_t, const void* pos, void* q_out,
                                 void* k_cache, void* v_cache, int64_t heads, int64_t K, void* stream) {
  const char* who = "q4f16_gemv_rmsnorm_rope";
  if (heads < 1 || heads > 4096) return fail(B200_EINVAL, "%s: heads %lld out of range", who, (long long)heads);
  const int64_t N = 3 * heads * 128;
  int rc = check_matmul(who, x, wq, scales, q_out, 1, N, K);
  if (rc) return rc;
  if (K < 256 || K % 256 != 0) return fail(B200_EINVAL, "%s: needs K a positive multiple of 256", who);
  if (!aligned16(scales)) return fail(B200_EINVAL, "%s: scales must be 16-byte aligned", who);
  if (!norm_w || !aligned16(norm_w)) return fail(B200_EINVAL, "%s: norm weight must be non-null and 16-byte aligned", who);
  if ((delta && !aligned16(delta)) || (x_out && !aligned16(x_out))) return fail(B200_EINVAL, "%s: delta / x_out must be 16-byte aligned", who);
  if (x_out == x) return fail(B200_EINVAL, "%s: x_out must not alias x (other CTAs still read x)", who);
  if (!cos_t || !sin_t || !pos || !k_cache || !v_cache) return fail(B200_EINVAL, "%s: null table, position or cache pointer", who);
  rc = ensure_device();
  if (rc) return rc;
  // B200_ENOTREADY (no message): the launch would not use the fast form; the caller runs b200_q4f16_gemv_rmsnorm and
  // b200_rope_kv_append instead
  return launch_gemv_pipe_rmsnorm_rope(static_cast<const __half*>(x), static_cast<const __half*>(delta),
                                       static_cast<const __half*>(norm_w), static_cast<__half*>(x_out), eps,
                                       static_cast<const uint32_t*>(wq), static_cast<const __half*>(scales),
                                       static_cast<const float*>(cos_t), static_cast<const float*>(sin_t),
                                       static_cast<const int*>(pos), static_cast<__half*>(q_out), static_cast<__half*>(k_cache),
                                       static_cast<__half*>(v_cache), heads, K, static_cast<cudaStream_t>(stream));
}

int b200_q4f16_gemv_swiglu(const void* gu, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                           void* stream) {
  const char* who = "q4f16_gemv_swiglu";
  int rc = check_matmul(who, gu, wq, scales, y, M, N, K);
  if (rc) return rc;
  if (M < 1 || M > 16) return fail(B200_EINVAL, "%s: takes 1 <= M <= 16, got %lld", who, (long long)M);
  if (N < 1 || K < 256 || K % 256 != 0) return fail(B200_EINVAL, "%s: needs N >= 1 and K a positive multiple of 256", who);
  if (!aligned16(scales)) return fail(B200_EINVAL, "%s: scales must be 16-byte aligned", who);
  rc = ensure_device();
  if (rc) return rc;
  rc = launch_gemv_pipe_swiglu(static_cast<const __half*>(gu), static_cast<const uint32_t*>(wq), static_cast<const __half*>(scales),
                               static_cast<__half*>(y), M, N, K, static_cast<cudaStream_t>(stream));
  if (rc == B200_ENOTREADY) return fail(B200_EINVAL, "%s: shape outside the fused kernel's domain", who);
  return rc;
}

int b200_q4f16_gemv_allreduce(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                              int32_t swiglu, const B200PeerReduce* red, void* stream) {
  const char* who = "q4f16_gemv_allreduce";
  int rc = check_matmul(who, x, wq, scales, y, M, N, K);
  if (rc) return rc;
  if (M < 1 || M > 16) return fail(B200_EINVAL, "%s: takes 1 <= M <= 16, got %lld", who, (long long)M);
  if (N < 8 || N % 8 != 0 || K < 256 || K % 256 != 0)
    return fail(B200_EINVAL, "%s: needs N a positive multiple of 8 and K a positive multiple of 256", who);
  if (!aligned16(scales) || !aligned16(y)) return fail(B200_EINVAL, "%s: scales and y must be 16-byte aligned", who);
  if (!red) return fail(B200_EINVAL, "%s: null reduction descriptor", who);
  if (red->world < 1 || red->world > 8 || red->rank < 0 || red->rank >= red->world)
    return fail(B200_EINVAL, "%s: world %d / rank %d out of range (1..8)", who, red->world, red->rank);
  if (red->world > 1) {
    if (!red->epoch || !red->done_counter || !red->out || !aligned16(red->out) || red->flag_base < 0)
      return fail(B200_EINVAL, "%s: epoch, done_counter and a 16-byte aligned out are required", who);
    for (int r = 0; r < red->world; ++r)
      if (!red->peer_y[r] || !aligned16(red->peer_y[r]) || !red->peer_flags[r])
        return fail(B200_EINVAL, "%s: peer %d has a null or misaligned buffer", who, r);
    if (red->peer_y[red->rank] != y) return fail(B200_EINVAL, "%s: y must be this rank's entry of peer_y", who);
  }
  rc = ensure_device();
  if (rc) return rc;
  rc = launch_gemv_pipe_allreduce(static_cast<const __half*>(x), static_cast<const uint32_t*>(wq),
                                  static_cast<const __half*>(scales), static_cast<__half*>(y), M, N, K, swiglu, red,
                                  static_cast<cudaStream_t>(stream));
  if (rc == B200_ENOTREADY) return fail(B200_EINVAL, "%s: shape outside the fused kernel's domain", who);
  return rc;
}

int b200_allreduce_peer(int64_t count, const B200PeerReduce* red, void* stream) {
  const char* who = "allreduce_peer";
  if (count < 0 || count % 8 != 0) return fail(B200_EINVAL, "%s: count must be a non-negative multiple of 8, got %lld", who, (long long)count);
  if (!red) return fail(B200_EINVAL, "%s: null reduction descriptor", who);
  if (red->world < 2 || red->world > 8 || red->rank < 0 || red->rank >= red->world)
    return fail(B200_EINVAL, "%s: world %d / rank %d out of range (2..8)", who, red->world, red->rank);
  if (!red->epoch || !red->out || !aligned16(red->out) || red->flag_base < 0)
    return fail(B200_EINVAL, "%s: epoch and a 16-byte aligned out are required", who);
  for (int r = 0; r < red->world; ++r)
    if (!red->peer_y[r] || !aligned16(red->peer_y[r]) || !red->peer_flags[r])
      return fail(B200_EINVAL, "%s: peer %d has a null or misaligned buffer", who, r);
  int rc = ensure_device();
  if (rc) return rc;
  return launch_peer_allreduce(count, red, static_cast<cudaStream_t>(stream));
}

int b200_q4f16_gemm_ws(const void* x, const void* wq, const void* scales, void* y, int64_t M, int64_t N, int64_t K,
                       void* stream) {
  return matmul_impl(kGemmWs, "q4f16_gemm_ws", x, wq, scales, y, M, N, K, stream);
}

int b200_q4f16_matmul_host(const void* x_host, void* x_dev, const void* wq, const void* scales, void* y_dev,
                           void* y_host, int64_t M, int64_t N, int64_t K, void* stream) {
  if (M < 0 || N < 0 || K < 0) return fail(B200_EINVAL, "q4f16_matmul_host: negative size");
  if ((M * K > 0 && (!x_host || !x_dev)) || (M * N > 0 && (!y_host || !y_dev)))
    return fail(B200_EINVAL, "q4f16_matmul_host: null host or staging buffer");
  int rc = check_matmul("q4f16_matmul_host", x_dev, wq, scales, y_dev, M, N, K);
  if (rc) return rc;
  rc = ensure_device();
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  const size_t xb = (size_t)(M * K) * 2, yb = (size_t)(M * N) * 2;
  if (xb > 0) {
    void* xm = xb <= kHostKernelBytes && !(reinterpret_cast<uintptr_t>(x_host) & 15) ? mapped_host_pointer(x_host) : nullptr;
    if (xm) {
      if ((rc = host_copy(xm, x_dev, xb, false, s))) return rc;
    } else {
      e = cudaMemcpyAsync(x_dev, x_host, xb, cudaMemcpyHostToDevice, s);
      if (e != cudaSuccess) return fail(B200_ELAUNCH, "q4f16_matmul_host: H2D copy: %s", cudaGetErrorString(e));
    }
  }
  rc = matmul_impl(kAuto, "q4f16_matmul_host", x_dev, wq, scales, y_dev, M, N, K, stream);
  if (rc) return rc;
  if (yb > 0) {
    void* ym = yb <= kHostKernelBytes && !(reinterpret_cast<uintptr_t>(y_host) & 15) ? mapped_host_pointer(y_host) : nullptr;
    if (ym) {
      if ((rc = host_copy(y_dev, ym, yb, true, s))) return rc;
    } else {
      e = cudaMemcpyAsync(y_host, y_dev, yb, cudaMemcpyDeviceToHost, s);
      if (e != cudaSuccess) return fail(B200_ELAUNCH, "q4f16_matmul_host: D2H copy: %s", cudaGetErrorString(e));
    }
  }
  return B200_OK;
}

int b200_q4f16_matmul_dl(const B200DLTensor* x, const B200DLTensor* wq, const B200DLTensor* scales, B200DLTensor* y) {
  return b200_q4f16_matmul_dl_family(x, wq, scales, y, B200_FAMILY_AUTO);
}

int b200_q4f16_matmul_dl_family(const B200DLTensor* x, const B200DLTensor* wq, const B200DLTensor* scales, B200DLTensor* y,
                                int32_t family) {
  const char* who = "b200.q4f16_matmul";
  int dev = -1, rc;
  // bits 0-7: kernel family; bits 8-15: weight layout + 1 (0 = the process-wide option)
  const int32_t layout_code = (family >> 8) & 0xff;
  if ((family & ~0xffff) != 0 || layout_code > 2)
    return fail(B200_EINVAL, "%s: malformed family/layout code 0x%x", who, (unsigned)family);
  family &= 0xff;
  if (family != B200_FAMILY_AUTO && family != B200_FAMILY_GEMV && family != B200_FAMILY_GEMM)
    return fail(B200_EINVAL, "%s: unknown kernel family %d (0 auto, 1 skinny, 2 tensor-core)", who, (int)family);
  LayoutScope scope(layout_code - 1);
  if ((rc = check_tensor(who, "x", x, 2, 16, &dev))) return rc;
  if ((rc = check_tensor(who, "wq", wq, 1, 32, &dev))) return rc;
  if ((rc = check_tensor(who, "scales", scales, 2, 16, &dev))) return rc;
  if ((rc = check_tensor(who, "y", y, 2, 16, &dev))) return rc;
  int64_t M = x->shape[0], K = x->shape[1], N = wq->shape[0];
  if (K % 32 != 0) return fail(B200_EINVAL, "%s: K=%lld is not a multiple of the group size 32", who, (long long)K);
  if (wq->shape[1] != K / 8)
    return fail(B200_EINVAL, "%s: wq is [%lld,%lld], expected [N,%lld] for K=%lld", who, (long long)wq->shape[0],
                (long long)wq->shape[1], (long long)(K / 8), (long long)K);
  if (scales->shape[0] != N || scales->shape[1] != K / 32)
    return fail(B200_EINVAL, "%s: scales is [%lld,%lld], expected [%lld,%lld]", who, (long long)scales->shape[0],
                (long long)scales->shape[1], (long long)N, (long long)(K / 32));
  if (y->shape[0] != M || y->shape[1] != N)
    return fail(B200_EINVAL, "%s: y is [%lld,%lld], expected [%lld,%lld]", who, (long long)y->shape[0],
                (long long)y->shape[1], (long long)M, (long long)N);
  if ((rc = check_current_device(who, dev))) return rc;
  const Family fam = family == B200_FAMILY_GEMV ? kGemv : family == B200_FAMILY_GEMM ? kGemm : kAuto;
  return matmul_impl(fam, who, data_ptr(x), data_ptr(wq), data_ptr(scales), data_ptr(y), M, N, K, g_stream);
}

int b200_q4f16_dequantize_dl(const B200DLTensor* wq, const B200DLTensor* scales, B200DLTensor* w_out) {
  const char* who = "b200.q4f16_dequantize";
  int dev = -1, rc;
  if ((rc = check_tensor(who, "wq", wq, 1, 32, &dev))) return rc;
  if ((rc = check_tensor(who, "scales", scales, 2, 16, &dev))) return rc;
  if ((rc = check_tensor(who, "w", w_out, 2, 16, &dev))) return rc;
  int64_t N = wq->shape[0], K = wq->shape[1] * 8;
  if (K % 32 != 0) return fail(B200_EINVAL, "%s: K=%lld is not a multiple of the group size 32", who, (long long)K);
  if (scales->shape[0] != N || scales->shape[1] != K / 32)
    return fail(B200_EINVAL, "%s: scales is [%lld,%lld], expected [%lld,%lld]", who, (long long)scales->shape[0],
                (long long)scales->shape[1], (long long)N, (long long)(K / 32));
  if (w_out->shape[0] != N || w_out->shape[1] != K)
    return fail(B200_EINVAL, "%s: output is [%lld,%lld], expected [%lld,%lld]", who, (long long)w_out->shape[0],
                (long long)w_out->shape[1], (long long)N, (long long)K);
  if ((rc = check_current_device(who, dev))) return rc;
  return b200_q4f16_dequantize(data_ptr(wq), data_ptr(scales), data_ptr(w_out), N, K, g_stream);
}

// ---- packed-function symbols (legacy TVM C backend ABI) ------------------------------------
// TVMValue is an 8-byte union; tensors come as v_handle with type code 7 or 13.
static int packed_tensors(const char* who, void* args, int* type_codes, int num_args, int want,
                          const B200DLTensor** out) {
  if (num_args != want) return fail(B200_EINVAL, "%s: expected %d arguments, got %d", who, want, num_args);
  if (!args || !type_codes) return fail(B200_EINVAL, "%s: null argument array", who);
  void** vals = static_cast<void**>(args);
  for (int i = 0; i < want; ++i) {
    if (type_codes[i] != 7 && type_codes[i] != 13)
      return fail(B200_EINVAL, "%s: argument %d has type code %d, expected a tensor (7 or 13)", who, i, type_codes[i]);
    out[i] = static_cast<const B200DLTensor*>(vals[i]);
  }
  return B200_OK;
}

int32_t b200_q4f16_matmul_packed(void* args, int* type_codes, int num_args, void* out_value, int* out_type_code,
                                 void* resource_handle) {
  (void)out_value; (void)resource_handle;
  const B200DLTensor* t[4];
  if (packed_tensors("b200.q4f16_matmul", args, type_codes, num_args, 4, t)) return -1;
  if (b200_q4f16_matmul_dl(t[0], t[1], t[2], const_cast<B200DLTensor*>(t[3]))) return -1;
  if (out_type_code) *out_type_code = 4;  // kTVMNullptr: DPS functions return nothing
  return 0;
}

int32_t b200_q4f16_dequantize_packed(void* args, int* type_codes, int num_args, void* out_value, int* out_type_code,
                                     void* resource_handle) {
  (void)out_value; (void)resource_handle;
  const B200DLTensor* t[3];
  if (packed_tensors("b200.q4f16_dequantize", args, type_codes, num_args, 3, t)) return -1;
  if (b200_q4f16_dequantize_dl(t[0], t[1], const_cast<B200DLTensor*>(t[2]))) return -1;
  if (out_type_code) *out_type_code = 4;
  return 0;
}

}  // extern "C"
