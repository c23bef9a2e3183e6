// Shared helpers for the bitstack_b200 kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/bitstack_b200.h"

namespace bsb {

// thread-local error text returned by bsb_last_error()
void set_error(const char* fmt, ...);

#define BSB_CHECK_ARG(cond, ...)      \
  do {                                \
    if (!(cond)) {                    \
      ::bsb::set_error(__VA_ARGS__);  \
      return BSB_EINVAL;              \
    }                                 \
  } while (0)

#define BSB_CUDA(call)                                                        \
  do {                                                                        \
    cudaError_t e__ = (call);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      ::bsb::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), \
                       __FILE__, __LINE__);                                   \
      return BSB_ECUDA;                                                       \
    }                                                                         \
  } while (0)

// number of kernels this library has launched from the calling process
void count_launch();
// optional timing of the dominant decode kernel: events around each of its launches
void profile_mark(cudaStream_t s, bool after);

inline int check_launch(const char* what) {
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return BSB_ECUDA;
  }
  return BSB_OK;
}

// Programmatic dependent launch.  Every kernel of the decode step starts with pdl_enter(): wait until the kernels
// before it in the stream have completed and their writes are visible (a no-op for a normal launch), then let the
// NEXT kernel be scheduled, which will sit in its own wait.  Launch latency overlaps; constants of a weight may be
// fetched before the wait, nothing that another kernel writes is touched before it.
extern int g_pdl_enabled;
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
#ifdef BSB_PDL_EARLY   // measurement variant: the successor is released before this kernel's own wait (a whole chain of
  pdl_trigger();       // kernels becomes resident ahead of time); measured 7 % slower on a full decode step
  pdl_wait();
#else
  pdl_wait();
  pdl_trigger();
#endif
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int64_t align_up64(int64_t a, int64_t b) { return ceil_div64(a, b) * b; }

// number of multiprocessors of the current device (cached per device)
int sm_count();

// dimension and block-stride checks shared by every entry point that takes a weight
int check_weight(const bsb_weight* w);

// Device address of the library's sticky status word for the current device (looked up once per device with
// cudaGetSymbolAddress; nullptr + error text when that fails).  A kernel whose time-bounded wait gives up stores
// a non-zero code there with atomicCAS(word, 0, code): the first event stays until bsb_read_status() clears it.
int* device_status_word();

// ---- launchers implemented in the kernel translation units -------------------
int launch_pack_sign(const int8_t* sign, int64_t n, uint8_t* packed, int32_t* bad, cudaStream_t s);
int launch_unpack_sign(const uint8_t* packed, int64_t n, int8_t* out, cudaStream_t s);

// exactly one of y (fp16 output) and y32 (fp32 partial sums of a tensor-parallel shard) is non-null here and below
int launch_general_forward(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride,
                           __half* y, float* y32, int64_t y_stride, cudaStream_t s);
int launch_general_reconstruct(const bsb_weight& w, __half* w_out, cudaStream_t s);

// fast reconstruction (k == 16, in % 32 == 0, out % 16 == 0)
bool rebuild_supported(const bsb_weight& w);
int launch_rebuild_weight(const bsb_weight& w, __half* w_out, cudaStream_t s);

// y[rows][out] = x[rows][in] . W[out][in]^T (+bias), fp16 in, fp32 accumulate
bool gemm_supported(int64_t rows, int out_features, int in_features);
int launch_gemm_xwt(const __half* x, int64_t rows, int64_t x_stride, const __half* w,
                    int out_features, int in_features, const __half* bias, __half* y,
                    int64_t y_stride, cudaStream_t s);

// the same product on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory)
bool gemm_tc5_supported(int64_t rows, int out_features, int in_features);
int launch_gemm_tc5(const __half* x, int64_t rows, int64_t x_stride, const __half* w, int out_features,
                    int in_features, const __half* bias, __half* y, float* y32, int64_t y_stride, cudaStream_t s);

// small-batch path (7 .. 64 rows): signs expanded inside the multiprocessor into the fp16 operand of a tcgen05 MMA
bool signgemm_supported(const bsb_weight& w, int64_t rows);
int64_t signgemm_workspace_bytes(const bsb_weight& w, int64_t rows);
void signgemm_set_wait_limit_ns(unsigned long long ns);
int launch_signgemm(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride, __half* y, float* y32, int64_t y_stride,
                    void* workspace, int64_t workspace_bytes, cudaStream_t s);

// the same with warp-level MMAs and everything between the two MMAs in registers
bool signgemm_mma_supported(const bsb_weight& w, int64_t rows);
int64_t signgemm_mma_workspace_bytes(const bsb_weight& w, int64_t rows);
int launch_signgemm_mma(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride, __half* y, float* y32, int64_t y_stride,
                        void* workspace, int64_t workspace_bytes, cudaStream_t s);

// decode path (tcgen05: sign operand expanded into tensor memory)
int launch_vt_absmax(const bsb_weight& w, float* out, cudaStream_t s);
bool gemv_tc5_supported(const bsb_weight& w);
int64_t gemv_tc5_workspace_bytes(const bsb_weight* ws, int n_weights, int rows_per_pass);   // rows_per_pass: 1 or 2
void gemv_tc5_set_wait_limit_ns(unsigned long long ns);
#ifdef BSB_TUNING
void gemv_tc5_set_trace(unsigned long long* device_buffer);
void gemv_tc5_set_dbg(int mode);
void gemv_tc5_set_timeline(unsigned long long* device_buffer, int records);
int gemv_tc5_mma_rate(int n_cols, int per_commit, int iters, int issuers, int ctas_per_sm, float* ns_per_mma_per_sm);
#endif
// out_f32: the ys point at fp32 rows (partial sums of a tensor-parallel shard) instead of fp16 ones;
// x_absmax: optional max |x| per row of this pass
int launch_gemv_tc5(const bsb_weight* ws, int n_weights, const __half* x, int64_t x_stride, int rows, __half* const* ys,
                    const int64_t* y_strides, void* workspace, int64_t workspace_bytes, cudaStream_t s, bool out_f32 = false,
                    const float* x_absmax = nullptr);

}  // namespace bsb
