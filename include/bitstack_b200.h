/*
 * bitstack_b200 -- C ABI of the B200 (sm_100a) BitStack linear hot path.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on
 * the CUDA stream it is given (a cudaStream_t passed as void*, NULL = the legacy
 * default stream), never synchronises the host and never allocates device
 * memory: scratch space is passed in by the caller.  Return value: 0 on
 * success, a negative BSB_E* code otherwise; bsb_last_error() then returns a
 * text describing the failure for the calling thread.
 *
 * Storage layout (identical to what the reference module keeps after
 * stack_blocks(), bitstack/modules/BitStackLinear.py:183-195):
 *   qweight  uint8  [blocks][out*in/8]   sign bits, 8 per byte, first sign in the
 *                                         most significant bit, row-major over
 *                                         (out, in), +1 -> 1, -1 -> 0
 *   u        fp16   [blocks][out][k]
 *   vt       fp16   [blocks][k][in]
 *   bias     fp16   [out] or NULL
 * Only k == 16 is accelerated (the reference's operating point); other k values
 * run on the general kernel.
 */
#ifndef BITSTACK_B200_H
#define BITSTACK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BSB_OK 0
#define BSB_EINVAL (-1)    /* bad argument (shape, alignment, null pointer) */
#define BSB_ECUDA (-2)     /* a CUDA runtime call or launch failed */
#define BSB_EWORKSPACE (-3)/* scratch buffer missing or too small */
#define BSB_ELIMIT (-4)    /* size beyond a documented maximum */
#define BSB_ETIMEOUT (-5)  /* a time-bounded wait inside a kernel gave up; that call's outputs are NaN */

/* One stacked BitStack weight.  Strides are between consecutive blocks:
 * q_block_stride in bytes, u/vt_block_stride in fp16 elements.  `blocks` is the
 * number of ACTIVE blocks (the reference's w_bit); changing it needs no repack
 * (bitstack/modules/BitStackLinear.py:173-181). */
typedef struct bsb_weight {
  const uint8_t* qweight;
  const uint16_t* u;
  const uint16_t* vt;
  const uint16_t* bias; /* may be NULL */
  const float* vt_absmax; /* optional fp32 [blocks][k]: max |vt| per (block, rank), as
                             bsb_vt_absmax() writes it; NULL = recomputed on every call */
  int64_t q_block_stride;
  int64_t u_block_stride;
  int64_t vt_block_stride;
  int32_t out_features;
  int32_t in_features;
  int32_t k;
  int32_t blocks;
} bsb_weight;

/* Kernel choice for bsb_linear_forward.  AUTO picks by shape and row count. */
enum {
  BSB_ALGO_AUTO = 0,
  BSB_ALGO_GENERAL = 1,   /* any shape, CUDA cores, fp32 */
  BSB_ALGO_REBUILD_GEMM = 3, /* batch/prefill: rebuild fp16 W, then the tcgen05 GEMM */
  BSB_ALGO_GEMV_TC5 = 4,  /* decode (1-6 rows): packed signs expanded into tensor memory, tcgen05 fp8 MMAs */
  BSB_ALGO_SIGN_GEMM = 5, /* small batch (up to 64 rows): signs applied to tcgen05 rank-16 products inside the
                             multiprocessor and fed to the tcgen05 GEMM from shared memory; W is never written */
  BSB_ALGO_SIGN_GEMM_MMA = 6 /* the same fusion with warp-level MMAs, everything between the two MMAs in registers */
};

int bsb_version(void);
const char* bsb_last_error(void);

/* Multiprocessor count etc. of the current device; fills nothing and returns
 * BSB_ECUDA when there is no usable device. */
int bsb_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* Replaces pack_sign (bitstack/utils/pack_utils.py:5-18).  sign: n int8 values,
 * each +1 or -1.  packed: (n+7)/8 bytes; padding bits are written as 0.
 * If bad_count is not NULL the number of values that are neither +1 nor -1 is
 * ADDED to *bad_count (device int32; the caller zeroes it) -- the reference
 * asserts on such input. */
int bsb_pack_sign(const int8_t* sign, int64_t n, uint8_t* packed, int32_t* bad_count, void* stream);

/* Replaces unpack_sign / unpack_sign_v2 / unpack_sign_triton
 * (bitstack/utils/pack_utils.py:20-26, 50-82, 84-138, 177-204).
 * out: n int8 values +1/-1; padding bits are never written. */
int bsb_unpack_sign(const uint8_t* packed, int64_t n, int8_t* out, void* stream);

/* Replaces the weight reconstruction of the fused levels:
 * reconstruct_w_triton, unpack_and_reconstruct_w_triton{,_v2,_v3}
 * (bitstack/utils/inference_utils.py:135-156, 371-387, 465-488, 571-595) and the
 * per-block loop of forward_l0 (bitstack/modules/BitStackLinear.py:107-113).
 * w: fp16 [out][in] = sum over active blocks of sign * (u @ vt), accumulated in
 * fp32 and rounded once. */
int bsb_reconstruct_weight(const bsb_weight* w, uint16_t* w_out, void* stream);

/* One-time helper for the decode kernels: out[j*k + r] = max_n |vt[j][r][n]| over
 * the first w->blocks blocks.  No reference counterpart (the reference has no
 * quantised intermediate); the result only sets the scale of an internal fp8
 * operand and is a pure function of the stored factors. */
int bsb_vt_absmax(const bsb_weight* w, float* out, void* stream);

/* Scratch bytes bsb_linear_forward needs for this weight / row count / algo. */
int64_t bsb_linear_workspace_bytes(const bsb_weight* w, int64_t rows, int algo);

/* Replaces BitStackLinear.forward for every fused level
 * (bitstack/modules/BitStackLinear.py:88-157): y = x @ W^T (+ bias), fp32
 * accumulation, fp16 output.  x: [rows][in] fp16 with row stride x_stride
 * (elements); y: [rows][out] fp16 with row stride y_stride. */
int bsb_linear_forward(const bsb_weight* w, const uint16_t* x, int64_t rows, int64_t x_stride,
                       uint16_t* y, int64_t y_stride, void* workspace, int64_t workspace_bytes,
                       int algo, void* stream);

/* Tensor-parallel variant of bsb_linear_forward: the same product written as fp32 PARTIAL SUMS, not rounded to
 * fp16.  A projection whose input columns are sharded over P devices (the o / down projections of a decoder layer)
 * yields one partial per device; the caller adds them (one all-reduce) and rounds ONCE, as a single device would.
 * No counterpart in the reference, which has no tensor parallelism (its forward is
 * bitstack/modules/BitStackLinear.py:88-157 on one device).  y: fp32 [rows][out], row stride y_stride elements,
 * 16-byte aligned rows; a bias, if the weight has one, is added (give it to one shard only).  Same scratch as
 * bsb_linear_forward. */
int bsb_linear_forward_partial(const bsb_weight* w, const uint16_t* x, int64_t rows, int64_t x_stride,
                               float* y, int64_t y_stride, void* workspace, int64_t workspace_bytes,
                               int algo, void* stream);

/* Several weights applied to the SAME x in one launch sequence (q/k/v, gate/up
 * of a decoder layer; the reference calls the module once per projection,
 * bitstack/modules/BitStackLinear.py:88-103).  All weights share in_features.
 * ys[i]: [rows][w[i].out_features], row stride y_strides[i]. */
int bsb_linear_forward_grouped(const bsb_weight* ws, int32_t n_weights, const uint16_t* x,
                               int64_t rows, int64_t x_stride, uint16_t* const* ys,
                               const int64_t* y_strides, void* workspace, int64_t workspace_bytes,
                               int algo, void* stream);

/* bsb_linear_forward_grouped for a decode step (rows <= 6) whose input comes with its row maxima.  No counterpart
 * in the reference.  x_absmax: fp32 [rows], max |x| of every input row as the operation that produced x delivered
 * it (bsb_add_rmsnorm, bsb_silu_mul): the decode kernel's operand preparation needs that number for the scale of
 * its fp8 operand and then does not have to scan x for it (NULL = computed inside, as bsb_linear_forward_grouped
 * does).  A value smaller than the true maximum would clip the operand: pass what the producer computed.
 * Needs the decode path: rows <= 6 and every weight with k == 16, in_features % 128 == 0, 16-byte aligned tensors
 * and at least one active block; otherwise BSB_EINVAL. */
int bsb_linear_forward_grouped_ex(const bsb_weight* ws, int32_t n_weights, const uint16_t* x, int64_t rows,
                                  int64_t x_stride, const float* x_absmax, uint16_t* const* ys,
                                  const int64_t* y_strides, void* workspace, int64_t workspace_bytes, void* stream);

/* Scratch bytes bsb_linear_forward_grouped needs. */
int64_t bsb_linear_grouped_workspace_bytes(const bsb_weight* ws, int32_t n_weights, int64_t rows, int algo);

/* ---- decode-time glue (no counterpart in the reference, which leaves these ops to the Hugging
 * Face Llama modules; bitstack/utils/scale_utils.py:3-5 names the classes it wraps) ------------
 * bsb_add_rmsnorm: h[rows][hidden] += delta (if delta != NULL; fp16 residual stream, written
 *   back), then y = h * rsqrt(mean(h^2) + eps) * weight with fp32 arithmetic; y_absmax (fp32 [rows], may be
 *   NULL) receives max |y| per row.  hidden % 8 == 0, hidden <= 16384, 16-byte aligned buffers.
 * bsb_rope_cache: rotary embedding at position *pos (device scalar) on q[batch][q_heads*dim] in
 *   place and on k, which is written with v into caches [batch][kv_heads][max_len][dim];
 *   cos/sin tables are [max_len][dim] in the "rotate half" convention.
 * bsb_decode_attention: the same rotary embedding and cache write as bsb_rope_cache (q is NOT
 *   modified) followed by softmax(q.K^T / sqrt(dim)).V over cache positions 0..*pos for one new
 *   token per batch row, grouped-query heads, fp32 softmax; out[batch][q_heads*dim].  head_dim 64 or 128,
 *   max_len <= 8192.  `scratch` (bsb_decode_attention_scratch_bytes, 16-byte aligned) must be ZERO before its
 *   first use and is left ready for the next call; calls sharing a scratch must be stream-ordered.
 *   *pos and the cache rows below it are read before the kernel waits for the work in front of it: they must not be
 *   written by the kernel launched directly before this call (bsb_rope_cache and bsb_greedy_step, which write them,
 *   never release their successor early, so calling those directly before is fine).
 * bsb_greedy_step: tokens[b] = first index of the maximum of logits[b][0..vocab) (fp16 rows row_stride apart), then
 *   *pos += 1 (pos may be NULL): the sampling and bookkeeping of a greedy decode step in one launch.
 * bsb_silu_mul: out = silu(gate) * up on [rows][n] fp16 (n % 8 == 0, 16-byte aligned); out_absmax (fp32 [rows], may be
 *   NULL) receives max |out| per row. */
int bsb_add_rmsnorm(uint16_t* h, const uint16_t* delta, const uint16_t* weight, float eps, uint16_t* y, float* y_absmax,
                    int64_t rows, int32_t hidden, void* stream);
int bsb_rope_cache(uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* cos_table, const uint16_t* sin_table,
                   const int64_t* pos, uint16_t* k_cache, uint16_t* v_cache, int32_t batch, int32_t q_heads,
                   int32_t kv_heads, int32_t head_dim, int32_t max_len, void* stream);
int bsb_decode_attention(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* cos_table,
                         const uint16_t* sin_table, const int64_t* pos, uint16_t* k_cache, uint16_t* v_cache, uint16_t* out,
                         int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_len, void* scratch,
                         int64_t scratch_bytes, void* stream);
int64_t bsb_decode_attention_scratch_bytes(int32_t batch, int32_t q_heads, int32_t head_dim);
int bsb_greedy_step(const uint16_t* logits, int64_t batch, int64_t vocab, int64_t row_stride, int64_t* tokens, int64_t* pos,
                    void* stream);
int bsb_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, float* out_absmax, int64_t rows, int32_t n,
                 void* stream);

/* ---- tensor parallelism: one-shot all-reduce over NVLink peer memory, fused with the add + RMSNorm that follows a
 * column-sharded projection.  No counterpart in the reference (single-device forward,
 * bitstack/modules/BitStackLinear.py:88-157).  One process per GPU; every rank owns an AREA of device memory that
 * all ranks map (CUDA inter-process handles) and calls bsb_peer_allreduce_add_rmsnorm with its fp32 partial sums
 * (bsb_linear_forward_partial): the kernel stores them into the peers' areas with plain stores over NVLink, waits
 * -- time-bounded, status word + NaN outputs on a give-up -- for the peers' partials, adds all of them in rank order
 * (bit-identical on every rank), rounds once to fp16 and continues as bsb_add_rmsnorm does: h += sum,
 * x_out = rmsnorm(h) * norm_weight, x_absmax = max |x_out| per row.  It replaces ncclAllReduce + a conversion + the
 * add/norm kernel; NCCL stays the fallback where peer mapping is not available.
 *   bsb_peer_area_bytes   size of an area for `world` ranks and up to max_rows x max_width fp32 partials.
 *   bsb_peer_alloc        set-up only (this one allocates): a zeroed area on the current device + its 64-byte handle.
 *   bsb_peer_open         set-up only: maps the area behind a peer's handle into this process.
 *   bsb_peer_close        releases an area (own != 0) or a mapping.
 *   areas[p]              the area of rank p as mapped in the calling process (areas[rank] = its own).
 * Every rank must make the same sequence of calls with the same rows / width.  width % 8 == 0, width <= 16384,
 * 16-byte aligned buffers, world <= 8. */
int64_t bsb_peer_area_bytes(int32_t world, int32_t max_rows, int32_t max_width);
int bsb_peer_alloc(int64_t bytes, void** area_out, uint8_t* handle_out);
int bsb_peer_open(const uint8_t* handle, void** area_out);
int bsb_peer_close(void* area, int32_t own);
int bsb_peer_allreduce_add_rmsnorm(void* const* areas, int32_t rank, int32_t world, int32_t max_rows, int32_t max_width,
                                   const float* partial, int64_t partial_stride, int32_t rows, int32_t width, uint16_t* h,
                                   const uint16_t* norm_weight, float eps, uint16_t* x_out, float* x_absmax, void* stream);

/* Forward for callers that may not allocate device memory.  It has no counterpart in the
 * reference.  Some hosts hand a plug-in a fixed set of buffers and forbid any device
 * allocation once they are running -- an inference server with a frozen memory plan, a
 * framework whose own pool already owns the whole GPU, a latency-critical loop that must not
 * take the driver's allocator lock (cudaMalloc stalls the device) -- and such a host has no
 * workspace to lend either.  This entry point therefore brings its scratch with it: a
 * 16 MiB array inside the library image (bsb_noalloc_scratch_bytes()), which every GPU that
 * loads the library keeps until the process ends.  Same math and kernel as the single-row
 * decode path of bsb_linear_forward (rows are processed one after another); it calls no
 * cudaMalloc, cudaFree or allocating library routine.
 *   - Weights whose scratch need exceeds the built-in area (more than 16 MiB: about 32 active
 *     blocks x 16384 input features) are rejected with BSB_ELIMIT; so are shapes the decode
 *     kernel does not take (k != 16, in_features % 128 != 0, unaligned tensors) with BSB_EINVAL.
 *   - The first call on each device looks up the device address of the built-in area (with
 *     that device current); make that first call before starting any stream capture.
 *   - All calls share the one area, which keeps whatever the last call left there; the kernels
 *     re-initialise the counters they depend on at the start of every call.
 *     Two calls that overlap on the GPU (different streams, or different host threads without
 *     ordering) would overwrite each other's scratch: serialise them. */
int64_t bsb_noalloc_scratch_bytes(void);
int bsb_linear_forward_noalloc(const bsb_weight* w, const uint16_t* x, int64_t rows, int64_t x_stride,
                               uint16_t* y, int64_t y_stride, void* stream);

/* Device-side failures (no reference counterpart; the reference fails loudly on the host,
 * bitstack/modules/BitStackLinear.py:103,120,152, and so must this).  Every wait inside the tcgen05 kernels is
 * time-bounded.  A wait that gives up (a hardware or driver fault, never expected in a healthy run) makes its
 * CTA write NaN to every output it was responsible for and stores a code in a per-device status word that
 * stays set until it is read -- later calls do not clear it.
 *   bsb_read_status: synchronises the current device, copies the word to *code_out and, if `clear` is non-zero,
 *     resets it.  Returns BSB_OK when the word is 0, BSB_ETIMEOUT otherwise.  Codes: 1-8 decode kernel (1 Z' ring,
 *     2 Z' slab, 3/4 operand stage full/empty, 5/6 accumulator full/empty, 7/8 sign ring), 21-24 GEMM, 31-37 fused
 *     sign-GEMM, 51 peer all-reduce.
 *     Call it wherever the host synchronises anyway (bsb_linear_forward_host does).
 *   bsb_set_wait_limit_ms: the time limit of every such wait (default 200 ms), for kernels launched afterwards. */
int bsb_read_status(int32_t* code_out, int32_t clear);
int bsb_set_wait_limit_ms(int32_t ms);

/* Programmatic dependent launch between the library's kernels (default on): every kernel allows its successor in
 * the stream to be scheduled early and waits itself for its predecessors before touching memory, so launch
 * latencies overlap.  0 switches it off (plain stream order), e.g. to time a kernel alone. */
int bsb_set_dependent_launch(int32_t on);

/* Measurement aids (no reference counterpart).  bsb_debug_launch_count: kernels this
 * library has launched so far in the process.  bsb_debug_profile_start/stop: while
 * on, a CUDA event pair is recorded on the launching stream around every launch of
 * the tcgen05 decode kernel (at most max_launches); stop waits for them and writes
 * the per-launch durations in milliseconds. */
int64_t bsb_debug_launch_count(void);
int bsb_debug_profile_start(int32_t max_launches);
int bsb_debug_profile_stop(float* ms_out, int32_t capacity, int32_t* n_out);

/* Same forward with HOST x and y buffers: copies x to the device, runs the
 * forward, copies y back and waits for it -- the call a host-only user makes.
 * dev_x / dev_y are caller-provided device staging buffers of rows*in and
 * rows*out fp16 elements.  Returns BSB_ETIMEOUT if the device status word is set when the
 * outputs arrive (see bsb_read_status). */
int bsb_linear_forward_host(const bsb_weight* w, const uint16_t* host_x, int64_t rows,
                            uint16_t* host_y, uint16_t* dev_x, uint16_t* dev_y, void* workspace,
                            int64_t workspace_bytes, int algo, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BITSTACK_B200_H */
