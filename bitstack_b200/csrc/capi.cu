// extern "C" entry points declared in include/bitstack_b200.h: argument checks,
// kernel choice, workspace carving.  No device allocation, no host sync (except the
// *_host variant, whose contract is to return finished host data).
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace bsb {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static unsigned long long g_launches = 0;
void count_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }

// profiling hook: a bounded list of event pairs recorded around the tcgen05 decode kernel
int g_pdl_enabled = 1;   // programmatic dependent launch between the library's kernels (bsb_set_dependent_launch)
static const int kMaxProfile = 4096;
static cudaEvent_t g_prof_ev[2 * kMaxProfile];
static int g_prof_cap = 0, g_prof_n = 0;
static bool g_prof_on = false;
void profile_mark(cudaStream_t s, bool after) {
  if (!g_prof_on) return;
  if (!after) {
    if (g_prof_n >= g_prof_cap) return;
    cudaEventRecord(g_prof_ev[2 * g_prof_n], s);
  } else {
    if (g_prof_n >= g_prof_cap) return;
    cudaEventRecord(g_prof_ev[2 * g_prof_n + 1], s);
    ++g_prof_n;
  }
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- sticky device status -----------------------------------------------------------------------
// One word per device, in the library image (zero when the library is loaded).  Kernels store into it only with
// atomicCAS(word, 0, code), so the first event stays until bsb_read_status() fetches and clears it.
static __device__ int g_status_word;

int* device_status_word() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("no usable current device for the status word");
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_status_word);
    if (e != cudaSuccess) {
      set_error("cudaGetSymbolAddress(status word) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = (int*)p;
  }
  return cached[dev];
}

int check_weight(const bsb_weight* w) {
  BSB_CHECK_ARG(w != nullptr, "weight is NULL");
  BSB_CHECK_ARG(w->out_features >= 0 && w->in_features >= 0 && w->k >= 1 && w->blocks >= 0,
                "bad weight dims out=%d in=%d k=%d blocks=%d", w->out_features, w->in_features, w->k, w->blocks);
  if (w->blocks > 0 && (int64_t)w->out_features * w->in_features > 0) {
    BSB_CHECK_ARG(w->qweight && w->u && w->vt, "weight has NULL qweight/u/vt");
    const int64_t e = (int64_t)w->out_features * w->in_features;
    BSB_CHECK_ARG(w->blocks == 1 || w->q_block_stride >= (e + 7) / 8, "q_block_stride %lld too small", (long long)w->q_block_stride);
    BSB_CHECK_ARG(w->blocks == 1 || w->u_block_stride >= (int64_t)w->out_features * w->k, "u_block_stride too small");
    BSB_CHECK_ARG(w->blocks == 1 || w->vt_block_stride >= (int64_t)w->in_features * w->k, "vt_block_stride too small");
  }
  return BSB_OK;
}

// largest batch that goes through the decode kernel (pairs of rows); above it the weight is rebuilt once and
// multiplied by the GEMM
static const int kDecodeRowsMax = 6;
static const int kFusedRowsMax = 16;

static int pick_algo(const bsb_weight& w, int64_t rows, int algo) {
  if (algo != BSB_ALGO_AUTO) return algo;
  if (rows <= kDecodeRowsMax && gemv_tc5_supported(w)) {
    // two rows per pass: cheaper than anything else up to here, except on small weights, where the fixed cost of
    // every pass dominates and one fused sign-GEMM call serves all rows (measured with 8 blocks, L2 flushed:
    // 4096 x 4096 at 6 rows 101 -> 63 us, at 4 rows 68 -> 63; 1024 x 4096 at 4 rows 58 -> 34)
    const int64_t signs = (int64_t)w.out_features * w.in_features * w.blocks;
    const bool small = (rows >= 3 && signs <= (64ll << 20)) || (rows >= 5 && signs <= (160ll << 20));
    if (small && signgemm_mma_supported(w, rows)) return BSB_ALGO_SIGN_GEMM_MMA;
    return BSB_ALGO_GEMV_TC5;
  }
  // 7 .. 16 rows: the fused sign-GEMM (W never leaves the multiprocessor) beats rebuilding W; above that the sign stage,
  // which is paid per block and per 16-row tile of the batch in the register variant, loses to rebuild + GEMM
  // (measured on 14336 x 4096, 8 blocks: 159 us against 199 at 16 rows, 214 against 200 at 32)
  if (rows <= kFusedRowsMax && signgemm_mma_supported(w, rows)) return BSB_ALGO_SIGN_GEMM_MMA;
  if (rebuild_supported(w) && gemm_supported(rows, w.out_features, w.in_features)) return BSB_ALGO_REBUILD_GEMM;
  return BSB_ALGO_GENERAL;
}

static int64_t workspace_for(const bsb_weight& w, int64_t rows, int algo) {
  switch (pick_algo(w, rows, algo)) {
    case BSB_ALGO_GEMV_TC5:
      return gemv_tc5_workspace_bytes(&w, 1, rows >= 2 ? 2 : 1);
    case BSB_ALGO_SIGN_GEMM:
      return signgemm_workspace_bytes(w, rows);
    case BSB_ALGO_SIGN_GEMM_MMA:
      return signgemm_mma_workspace_bytes(w, rows);
    case BSB_ALGO_REBUILD_GEMM:
      return align_up64((int64_t)w.out_features * w.in_features * 2, 256);   // the rebuilt fp16 W
    default:
      return 0;
  }
}

// fp16 zero / bias fill for weights with no active block
__global__ void fill_bias_kernel(__half* y, float* y32, int64_t rows, int64_t y_stride, int M, const __half* bias) {
  const int64_t total = rows * M;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / M;
    const int m = (int)(i % M);
    const __half v = bias ? bias[m] : __float2half(0.f);
    if (y32) y32[r * y_stride + m] = __half2float(v);
    else y[r * y_stride + m] = v;
  }
}

// exactly one of y (fp16 output) and y32 (fp32 partial sums, the tensor-parallel variant) is non-null
static int forward_one(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride, __half* y, float* y32,
                       int64_t y_stride, void* workspace, int64_t workspace_bytes, int algo, cudaStream_t s) {
  if (rows == 0 || w.out_features == 0) return BSB_OK;
  BSB_CHECK_ARG(x != nullptr && (y != nullptr) != (y32 != nullptr), "x or y is NULL");
  BSB_CHECK_ARG(x_stride >= w.in_features && y_stride >= w.out_features, "row stride smaller than the row");
  if (w.blocks == 0 || w.in_features == 0) {
    const int64_t total = rows * w.out_features;
    fill_bias_kernel<<<(unsigned)min((int64_t)1024, ceil_div64(total, 256)), 256, 0, s>>>(
        y, y32, rows, y_stride, w.out_features, reinterpret_cast<const __half*>(w.bias));
    return check_launch("fill_bias_kernel");
  }
  const int a = pick_algo(w, rows, algo);
  const int64_t need = workspace_for(w, rows, a);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
    set_error("workspace of %lld bytes needed, %lld given", (long long)need, (long long)workspace_bytes);
    return BSB_EWORKSPACE;
  }
  switch (a) {
    case BSB_ALGO_GENERAL:
      return launch_general_forward(w, x, rows, x_stride, y, y32, y_stride, s);
    case BSB_ALGO_GEMV_TC5: {
      BSB_CHECK_ARG(gemv_tc5_supported(w), "GEMV_TC5: unsupported shape/alignment (out=%d in=%d k=%d)",
                    w.out_features, w.in_features, w.k);
      // rows go through the kernel two at a time (one MMA serves both), a last odd row alone
      for (int64_t r = 0; r < rows;) {
        const int nr = (rows - r >= 2 && x_stride % 8 == 0) ? 2 : 1;
        __half* yr = y32 ? reinterpret_cast<__half*>(y32 + r * y_stride) : y + r * y_stride;
        if (int rc = launch_gemv_tc5(&w, 1, x + r * x_stride, x_stride, nr, &yr, &y_stride, workspace, workspace_bytes, s, y32 != nullptr)) return rc;
        r += nr;
      }
      return BSB_OK;
    }
    case BSB_ALGO_SIGN_GEMM:
      return launch_signgemm(w, x, rows, x_stride, y, y32, y_stride, workspace, workspace_bytes, s);
    case BSB_ALGO_SIGN_GEMM_MMA:
      return launch_signgemm_mma(w, x, rows, x_stride, y, y32, y_stride, workspace, workspace_bytes, s);
    case BSB_ALGO_REBUILD_GEMM: {
      BSB_CHECK_ARG(rebuild_supported(w) && gemm_supported(rows, w.out_features, w.in_features),
                    "REBUILD_GEMM: unsupported shape/alignment (out=%d in=%d k=%d)", w.out_features,
                    w.in_features, w.k);
      BSB_CHECK_ARG((uintptr_t)workspace % 16 == 0, "workspace must be 16-byte aligned");
      __half* wbuf = (__half*)workspace;
      if (int rc = launch_rebuild_weight(w, wbuf, s)) return rc;
      if (gemm_tc5_supported(rows, w.out_features, w.in_features) && ((uintptr_t)y | (uintptr_t)y32) % 16 == 0 && y_stride % 8 == 0 &&
          (uintptr_t)x % 16 == 0 && x_stride % 8 == 0)
        return launch_gemm_tc5(x, rows, x_stride, wbuf, w.out_features, w.in_features,
                               reinterpret_cast<const __half*>(w.bias), y, y32, y_stride, s);
      BSB_CHECK_ARG(y32 == nullptr, "partial-sum output needs 16-byte aligned rows (x, y and their strides)");
      // outputs that are not 16-byte aligned: the warp-level (mma.sync) kernel
      return launch_gemm_xwt(x, rows, x_stride, wbuf, w.out_features, w.in_features,
                             reinterpret_cast<const __half*>(w.bias), y, y_stride, s);
    }
    default:
      set_error("unknown or unavailable algo %d", a);
      return BSB_EINVAL;
  }
}

}  // namespace bsb

using namespace bsb;

extern "C" {

int bsb_version(void) { return 100; }

const char* bsb_last_error(void) { return g_err; }

int bsb_device_info(int* sm, int* major, int* minor) {
  int dev = 0;
  BSB_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp p;
  BSB_CUDA(cudaGetDeviceProperties(&p, dev));
  if (sm) *sm = p.multiProcessorCount;
  if (major) *major = p.major;
  if (minor) *minor = p.minor;
  return BSB_OK;
}

int bsb_pack_sign(const int8_t* sign, int64_t n, uint8_t* packed, int32_t* bad_count, void* stream) {
  BSB_CHECK_ARG(n >= 0, "negative element count");
  BSB_CHECK_ARG(n == 0 || (sign && packed), "NULL buffer");
  return launch_pack_sign(sign, n, packed, bad_count, (cudaStream_t)stream);
}

int bsb_unpack_sign(const uint8_t* packed, int64_t n, int8_t* out, void* stream) {
  BSB_CHECK_ARG(n >= 0, "negative element count");
  BSB_CHECK_ARG(n == 0 || (packed && out), "NULL buffer");
  return launch_unpack_sign(packed, n, out, (cudaStream_t)stream);
}

int bsb_reconstruct_weight(const bsb_weight* w, uint16_t* w_out, void* stream) {
  if (int rc = check_weight(w)) return rc;
  if ((int64_t)w->out_features * w->in_features == 0) return BSB_OK;
  BSB_CHECK_ARG(w_out != nullptr, "output is NULL");
  if (w->blocks > 0 && rebuild_supported(*w)) return launch_rebuild_weight(*w, (__half*)w_out, (cudaStream_t)stream);
  return launch_general_reconstruct(*w, (__half*)w_out, (cudaStream_t)stream);
}

int bsb_vt_absmax(const bsb_weight* w, float* out, void* stream) {
  if (int rc = check_weight(w)) return rc;
  BSB_CHECK_ARG(out != nullptr, "output is NULL");
  return launch_vt_absmax(*w, out, (cudaStream_t)stream);
}

int64_t bsb_linear_workspace_bytes(const bsb_weight* w, int64_t rows, int algo) {
  if (check_weight(w) != BSB_OK || rows < 0) return -1;
  if (w->blocks == 0 || rows == 0) return 0;
  return workspace_for(*w, rows, algo);
}

int bsb_linear_forward(const bsb_weight* w, const uint16_t* x, int64_t rows, int64_t x_stride, uint16_t* y,
                       int64_t y_stride, void* workspace, int64_t workspace_bytes, int algo, void* stream) {
  if (int rc = check_weight(w)) return rc;
  BSB_CHECK_ARG(rows >= 0, "negative row count");
  return forward_one(*w, (const __half*)x, rows, x_stride, (__half*)y, nullptr, y_stride, workspace, workspace_bytes,
                     algo, (cudaStream_t)stream);
}

int bsb_linear_forward_partial(const bsb_weight* w, const uint16_t* x, int64_t rows, int64_t x_stride, float* y,
                               int64_t y_stride, void* workspace, int64_t workspace_bytes, int algo, void* stream) {
  if (int rc = check_weight(w)) return rc;
  BSB_CHECK_ARG(rows >= 0, "negative row count");
  return forward_one(*w, (const __half*)x, rows, x_stride, nullptr, y, y_stride, workspace, workspace_bytes, algo,
                     (cudaStream_t)stream);
}

int bsb_linear_forward_grouped(const bsb_weight* ws, int32_t n_weights, const uint16_t* x, int64_t rows,
                               int64_t x_stride, uint16_t* const* ys, const int64_t* y_strides, void* workspace,
                               int64_t workspace_bytes, int algo, void* stream) {
  BSB_CHECK_ARG(n_weights >= 1 && ws && ys && y_strides, "bad group arguments");
  BSB_CHECK_ARG(rows >= 0, "negative row count");
  for (int i = 0; i < n_weights; ++i) {
    if (int rc = check_weight(&ws[i])) return rc;
    BSB_CHECK_ARG(ws[i].in_features == ws[0].in_features, "grouped weights must share in_features");
  }
  cudaStream_t s = (cudaStream_t)stream;
  // one fused launch sequence when every member qualifies for the decode kernel
  bool fused = (algo == BSB_ALGO_AUTO || algo == BSB_ALGO_GEMV_TC5) && rows >= 1 && rows <= kDecodeRowsMax && n_weights <= 4;
  for (int i = 0; i < n_weights && fused; ++i) fused = ws[i].blocks > 0 && ws[i].out_features > 0 && gemv_tc5_supported(ws[i]);
  if (fused) {
    const int64_t need = gemv_tc5_workspace_bytes(ws, n_weights, rows >= 2 ? 2 : 1);
    if (workspace == nullptr || workspace_bytes < need) {
      set_error("workspace of %lld bytes needed, %lld given", (long long)need, (long long)workspace_bytes);
      return BSB_EWORKSPACE;
    }
    for (int64_t r = 0; r < rows;) {
      const int nr = (rows - r >= 2 && x_stride % 8 == 0) ? 2 : 1;   // two rows per pass of the decode kernel
      __half* yr[4];
      for (int i = 0; i < n_weights; ++i) yr[i] = (__half*)ys[i] + r * y_strides[i];
      if (int rc = launch_gemv_tc5(ws, n_weights, (const __half*)x + r * x_stride, x_stride, nr, yr, y_strides, workspace, workspace_bytes, s))
        return rc;
      r += nr;
    }
    return BSB_OK;
  }
  for (int i = 0; i < n_weights; ++i) {
    if (int rc = forward_one(ws[i], (const __half*)x, rows, x_stride, (__half*)ys[i], nullptr, y_strides[i], workspace,
                             workspace_bytes, algo, s))
      return rc;
  }
  return BSB_OK;
}

int bsb_linear_forward_grouped_ex(const bsb_weight* ws, int32_t n_weights, const uint16_t* x, int64_t rows, int64_t x_stride,
                                  const float* x_absmax, uint16_t* const* ys, const int64_t* y_strides,
                                  void* workspace, int64_t workspace_bytes, void* stream) {
  BSB_CHECK_ARG(n_weights >= 1 && n_weights <= 4 && ws && ys && y_strides && x, "bad group arguments");
  BSB_CHECK_ARG(rows >= 1 && rows <= kDecodeRowsMax, "the extended call runs on the decode path: 1..%d rows (got %lld)",
                kDecodeRowsMax, (long long)rows);
  for (int i = 0; i < n_weights; ++i) {
    if (int rc = check_weight(&ws[i])) return rc;
    BSB_CHECK_ARG(ws[i].in_features == ws[0].in_features, "grouped weights must share in_features");
    BSB_CHECK_ARG(ws[i].blocks > 0 && ws[i].out_features > 0 && gemv_tc5_supported(ws[i]),
                  "the extended call needs the decode kernel: weight %d has no active block or an unsupported shape/alignment", i);
  }
  BSB_CHECK_ARG(rows == 1 || x_stride % 8 == 0, "x rows must be 16-byte aligned");
  const int64_t need = gemv_tc5_workspace_bytes(ws, n_weights, rows >= 2 ? 2 : 1);
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("workspace of %lld bytes needed, %lld given", (long long)need, (long long)workspace_bytes);
    return BSB_EWORKSPACE;
  }
  for (int64_t r = 0; r < rows;) {
    const int nr = (rows - r >= 2) ? 2 : 1;
    __half* yr[4];
    for (int i = 0; i < n_weights; ++i) yr[i] = (__half*)ys[i] + r * y_strides[i];
    if (int rc = launch_gemv_tc5(ws, n_weights, (const __half*)x + r * x_stride, x_stride, nr, yr, y_strides, workspace,
                                 workspace_bytes, (cudaStream_t)stream, false, x_absmax ? x_absmax + r : nullptr))
      return rc;
    r += nr;
  }
  return BSB_OK;
}

int64_t bsb_linear_grouped_workspace_bytes(const bsb_weight* ws, int32_t n_weights, int64_t rows, int algo) {
  if (!ws || n_weights < 1 || rows < 0) return -1;
  int64_t need = 0;
  bool fused = (algo == BSB_ALGO_AUTO || algo == BSB_ALGO_GEMV_TC5) && rows >= 1 && rows <= kDecodeRowsMax && n_weights <= 4;
  for (int i = 0; i < n_weights; ++i) {
    if (check_weight(&ws[i]) != BSB_OK) return -1;
    fused = fused && ws[i].blocks > 0 && ws[i].out_features > 0 && gemv_tc5_supported(ws[i]);
    if (ws[i].blocks > 0 && rows > 0) need = max(need, workspace_for(ws[i], rows, algo));
  }
  if (fused) need = max(need, gemv_tc5_workspace_bytes(ws, n_weights, rows >= 2 ? 2 : 1));
  return need;
}

int bsb_read_status(int32_t* code_out, int32_t clear) {
  BSB_CHECK_ARG(code_out != nullptr, "NULL argument");
  int* word = device_status_word();
  if (word == nullptr) return BSB_ECUDA;
  BSB_CUDA(cudaDeviceSynchronize());   // every stream of the device: the word is shared by all of them
  BSB_CUDA(cudaMemcpy(code_out, word, 4, cudaMemcpyDeviceToHost));
  if (clear && *code_out != 0) BSB_CUDA(cudaMemset(word, 0, 4));
  if (*code_out != 0) {
    set_error("a time-bounded wait gave up on the device (code %d): the outputs of that call are NaN", *code_out);
    return BSB_ETIMEOUT;
  }
  return BSB_OK;
}

int bsb_set_wait_limit_ms(int32_t ms) {
  BSB_CHECK_ARG(ms >= 1 && ms <= 60000, "wait limit must be 1..60000 ms");
  gemv_tc5_set_wait_limit_ns((unsigned long long)ms * 1000000ull);
  signgemm_set_wait_limit_ns((unsigned long long)ms * 1000000ull);
  return BSB_OK;
}

int bsb_set_dependent_launch(int32_t on) {
  g_pdl_enabled = on ? 1 : 0;
  return BSB_OK;
}

#ifdef BSB_TUNING
// tuning build only (not declared in the public header): timing experiments and the cycle trace of the decode kernel
int bsb_tuning_set_trace(void* device_buffer) {
  gemv_tc5_set_trace((unsigned long long*)device_buffer);
  return BSB_OK;
}
int bsb_tuning_set_mode(int32_t mode) {
  gemv_tc5_set_dbg(mode);
  return BSB_OK;
}
int bsb_tuning_set_timeline(void* device_buffer, int32_t records) {
  gemv_tc5_set_timeline((unsigned long long*)device_buffer, records);
  return BSB_OK;
}
int bsb_tuning_mma_rate(int32_t n_cols, int32_t per_commit, int32_t iters, int32_t issuers, int32_t ctas_per_sm, float* ns_per_mma_per_sm) {
  return gemv_tc5_mma_rate(n_cols, per_commit, iters, issuers, ctas_per_sm, ns_per_mma_per_sm);
}
#endif

int64_t bsb_debug_launch_count(void) { return (int64_t)g_launches; }

int bsb_debug_profile_start(int32_t max_launches) {
  BSB_CHECK_ARG(max_launches >= 1 && max_launches <= kMaxProfile, "1..%d launches can be profiled", kMaxProfile);
  BSB_CHECK_ARG(!g_prof_on, "profiling already on");
  for (int i = g_prof_cap * 2; i < max_launches * 2; ++i) BSB_CUDA(cudaEventCreate(&g_prof_ev[i]));
  if (max_launches > g_prof_cap) g_prof_cap = max_launches;
  g_prof_n = 0;
  g_prof_on = true;
  return BSB_OK;
}

int bsb_debug_profile_stop(float* ms_out, int32_t capacity, int32_t* n_out) {
  BSB_CHECK_ARG(g_prof_on, "profiling is not on");
  g_prof_on = false;
  BSB_CHECK_ARG(ms_out && n_out, "NULL output");
  const int n = g_prof_n < capacity ? g_prof_n : capacity;
  for (int i = 0; i < n; ++i) {
    BSB_CUDA(cudaEventSynchronize(g_prof_ev[2 * i + 1]));
    BSB_CUDA(cudaEventElapsedTime(&ms_out[i], g_prof_ev[2 * i], g_prof_ev[2 * i + 1]));
  }
  *n_out = n;
  return BSB_OK;
}

int bsb_linear_forward_host(const bsb_weight* w, const uint16_t* host_x, int64_t rows, uint16_t* host_y,
                            uint16_t* dev_x, uint16_t* dev_y, void* workspace, int64_t workspace_bytes, int algo,
                            void* stream) {
  if (int rc = check_weight(w)) return rc;
  BSB_CHECK_ARG(rows >= 0, "negative row count");
  if (rows == 0) return BSB_OK;
  BSB_CHECK_ARG(host_x && host_y && dev_x && dev_y, "NULL buffer");
  cudaStream_t s = (cudaStream_t)stream;
  BSB_CUDA(cudaMemcpyAsync(dev_x, host_x, (size_t)rows * w->in_features * 2, cudaMemcpyHostToDevice, s));
  if (int rc = forward_one(*w, (const __half*)dev_x, rows, w->in_features, (__half*)dev_y, nullptr, w->out_features,
                           workspace, workspace_bytes, algo, s))
    return rc;
  BSB_CUDA(cudaMemcpyAsync(host_y, dev_y, (size_t)rows * w->out_features * 2, cudaMemcpyDeviceToHost, s));
  int32_t code = 0;
  BSB_CUDA(cudaMemcpyAsync(&code, device_status_word(), 4, cudaMemcpyDeviceToHost, s));
  BSB_CUDA(cudaStreamSynchronize(s));
  if (code != 0) {   // the call's outputs are NaN; the word stays set until bsb_read_status() clears it
    set_error("a time-bounded wait gave up on the device (code %d)", code);
    return BSB_ETIMEOUT;
  }
  return BSB_OK;
}

}  // extern "C"
