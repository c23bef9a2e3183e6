// One-shot all-reduce over NVLink peer memory, fused with the residual add + RMSNorm that follows a column-sharded
// projection (o / down) of a tensor-parallel decoder layer.
//
// The reference has no tensor parallelism (its forward runs on one device, bitstack/modules/BitStackLinear.py:88-157);
// with the projections sharded by input columns every rank holds fp32 PARTIAL sums of the projection output.  Instead
// of ncclAllReduce + a conversion + the add/norm kernel (three launches, ~20 us of latency at batch 1), one kernel per
// rank
//   1. stores its partial rows into every peer's receive area with plain 16-byte stores over NVLink (peer pointers
//      from cudaIpcOpenMemHandle; no multicast, no TMA),
//   2. publishes a per-(sender, row) flag with a system-scope release store,
//   3. waits -- time-bounded -- for the flags of all peers, adds the partials IN RANK ORDER (every rank computes the
//      same bits), rounds the sum to fp16 once, and
//   4. does h += sum, x = rmsnorm(h) * weight, max |x| with the same code as the stand-alone kernel (rowops.cuh).
// Receive areas and flags are double buffered by call parity: a rank can only be one call ahead of a peer (it needs
// that peer's partial of the current call to finish it), so the call after next never meets unread data.  The call
// counter lives in device memory and is advanced by the last CTA of each call: a captured graph replays correctly.
// A wait that runs out raises the status word and fills x / h with NaN; it never spins forever.
#include "common.cuh"
#include "rowops.cuh"

namespace bsb {

namespace {

constexpr int kMaxWorld = 8;
constexpr unsigned long long kDefaultWaitNs = 2000ull * 1000 * 1000;   // peers may be a whole kernel behind: 2 s

struct PeerParams {
  float* recv[kMaxWorld];        // receive area of every rank as mapped here: [2 parities][world senders][max_rows][max_width]
  int* flags[kMaxWorld];         // flags of every rank: [2][world][max_rows]
  int* local;                    // this rank's control words: [0] call counter, [1] CTAs finished
  __half* scratch;               // [max_rows][max_width] fp16: the rounded sum of a row
  int rank, world, max_rows, max_width;
  const float* partial;          // [rows][width], row stride partial_stride
  int64_t partial_stride;
  int rows, width;
  __half* h;                     // residual stream [rows][width], updated in place
  const __half* norm_w;
  float eps;
  __half* x_out;                 // [rows][width]
  float* x_absmax;               // [rows] or nullptr
  int* status;
  unsigned long long wait_ns;
};

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// one CTA per row
__global__ void __launch_bounds__(kRowThreads) peer_allreduce_add_rmsnorm_kernel(const PeerParams P) {
  __shared__ float red[32];
  __shared__ int s_epoch, s_ok;
  // the norm weight (a constant, evicted by the weight stream since the last step) is asked into L2 during the wait
  if ((int)threadIdx.x * 64 < P.width) asm volatile("prefetch.global.L2 [%0];" ::"l"(P.norm_w + threadIdx.x * 64));
  pdl_enter();
  const int r = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) { s_epoch = *reinterpret_cast<volatile int*>(P.local); s_ok = 1; }
  __syncthreads();
  const int e = s_epoch, par = e & 1;
  const int64_t area = (int64_t)P.max_rows * P.max_width;               // floats per (parity, sender)
  const int nvec = P.width / 4;
  const float4* mine = reinterpret_cast<const float4*>(P.partial + (int64_t)r * P.partial_stride);
  // 1. this rank's row into every peer's receive area
  for (int p = 0; p < P.world; ++p) {
    if (p == P.rank) continue;
    float4* dst = reinterpret_cast<float4*>(P.recv[p] + ((int64_t)par * P.world + P.rank) * area + (int64_t)r * P.max_width);
    for (int i = tid; i < nvec; i += kRowThreads) dst[i] = mine[i];
  }
  __threadfence_system();
  __syncthreads();
  // 2. flags: one per (receiver, sender = this rank, row)
  if (tid < P.world && tid != P.rank)
    st_release_sys(P.flags[tid] + ((int64_t)par * P.world + P.rank) * P.max_rows + r, e + 1);
  // 3. wait for every peer's row (time-bounded)
  if (tid < P.world && tid != P.rank) {
    const int* f = P.flags[P.rank] + ((int64_t)par * P.world + tid) * P.max_rows + r;
    const uint64_t t0 = global_ns();
    bool ok = true;
    while (ld_acquire_sys(f) != e + 1) {
      __nanosleep(100);
      if (global_ns() - t0 > P.wait_ns) { ok = false; break; }
    }
    if (!ok) { atomicCAS(P.status, 0, 51); s_ok = 0; }
  }
  __syncthreads();
  __half* srow = P.scratch + (int64_t)r * P.max_width;
  if (s_ok) {
    // the sum in rank order, rounded to fp16 once (what a single device's fp16 projection output would be)
    for (int i = tid; i < nvec; i += kRowThreads) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < P.world; ++p) {
        const float4 v = (p == P.rank) ? mine[i]
                                       : __ldcv(reinterpret_cast<const float4*>(P.recv[P.rank] + ((int64_t)par * P.world + p) * area +
                                                                                (int64_t)r * P.max_width) + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      reinterpret_cast<__half2*>(srow)[2 * i] = __floats2half2_rn(s.x, s.y);
      reinterpret_cast<__half2*>(srow)[2 * i + 1] = __floats2half2_rn(s.z, s.w);
    }
    __threadfence_block();
    __syncthreads();
    // 4. h += sum; x = rmsnorm(h) * weight; max |x|
    add_rmsnorm_row<true>(P.h + (int64_t)r * P.width, srow, P.norm_w, P.eps, P.x_out + (int64_t)r * P.width, P.width, red,
                          P.x_absmax ? P.x_absmax + r : nullptr);
  } else {
    const __half nan = __float2half_rn(__int_as_float(0x7FC00000));
    for (int i = tid; i < P.width; i += kRowThreads) {
      P.h[(int64_t)r * P.width + i] = nan;
      P.x_out[(int64_t)r * P.width + i] = nan;
    }
    if (tid == 0 && P.x_absmax) P.x_absmax[r] = __int_as_float(0x7FC00000);
  }
  // the last CTA of the call advances the call counter (every CTA has read it by now)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(P.local + 1, 1) == (int)gridDim.x - 1) {
      P.local[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(P.local) = e + 1;
    }
  }
}

unsigned long long g_peer_wait_ns = kDefaultWaitNs;

}  // namespace
}  // namespace bsb

using namespace bsb;

extern "C" {

int64_t bsb_peer_area_bytes(int32_t world, int32_t max_rows, int32_t max_width) {
  if (world < 1 || world > kMaxWorld || max_rows < 1 || max_width < 8 || max_width % 8) return -1;
  const int64_t recv = 2ll * world * max_rows * max_width * 4;
  const int64_t flags = align_up64(2ll * world * max_rows * 4, 256);
  const int64_t local = 256;
  const int64_t scratch = align_up64((int64_t)max_rows * max_width * 2, 256);
  return align_up64(recv, 256) + flags + local + scratch;
}

// Set-up (NOT for the hot path: these two allocate / map device memory).  bsb_peer_alloc: a zeroed area of `bytes` on the
// current device and the 64-byte inter-process handle other ranks open.  bsb_peer_open: maps a peer's area here.
int bsb_peer_alloc(int64_t bytes, void** area_out, uint8_t* handle_out) {
  BSB_CHECK_ARG(bytes > 0 && area_out && handle_out, "bad arguments");
  void* p = nullptr;
  BSB_CUDA(cudaMalloc(&p, (size_t)bytes));
  BSB_CUDA(cudaMemset(p, 0, (size_t)bytes));
  cudaIpcMemHandle_t h;
  BSB_CUDA(cudaIpcGetMemHandle(&h, p));
  static_assert(sizeof(h) == 64, "handle size");
  memcpy(handle_out, &h, 64);
  *area_out = p;
  return BSB_OK;
}

int bsb_peer_open(const uint8_t* handle, void** area_out) {
  BSB_CHECK_ARG(handle && area_out, "bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  BSB_CUDA(cudaIpcOpenMemHandle(area_out, h, cudaIpcMemLazyEnablePeerAccess));
  return BSB_OK;
}

int bsb_peer_close(void* area, int32_t own) {
  if (area == nullptr) return BSB_OK;
  if (own) BSB_CUDA(cudaFree(area));
  else BSB_CUDA(cudaIpcCloseMemHandle(area));
  return BSB_OK;
}

int bsb_peer_allreduce_add_rmsnorm(void* const* areas, int32_t rank, int32_t world, int32_t max_rows, int32_t max_width,
                                   const float* partial, int64_t partial_stride, int32_t rows, int32_t width, uint16_t* h,
                                   const uint16_t* norm_weight, float eps, uint16_t* x_out, float* x_absmax, void* stream) {
  BSB_CHECK_ARG(areas && partial && h && norm_weight && x_out, "NULL argument");
  BSB_CHECK_ARG(world >= 2 && world <= kMaxWorld && rank >= 0 && rank < world, "rank %d / world %d", rank, world);
  BSB_CHECK_ARG(rows >= 1 && rows <= max_rows && width >= 8 && width <= max_width && width % 8 == 0 && max_width % 8 == 0 &&
                width <= kRowThreads * kRowVecs * 8, "rows %d (max %d), width %d (max %d, multiple of 8, <= 16384)", rows, max_rows,
                width, max_width);
  BSB_CHECK_ARG(((uintptr_t)partial | (uintptr_t)h | (uintptr_t)norm_weight | (uintptr_t)x_out) % 16 == 0 && partial_stride % 4 == 0,
                "buffers must be 16-byte aligned");
  PeerParams P;
  memset(&P, 0, sizeof(P));
  const int64_t recv_bytes = align_up64(2ll * world * max_rows * max_width * 4, 256);
  const int64_t flag_bytes = align_up64(2ll * world * max_rows * 4, 256);
  for (int p = 0; p < world; ++p) {
    BSB_CHECK_ARG(areas[p] != nullptr, "area of rank %d is NULL", p);
    P.recv[p] = reinterpret_cast<float*>(areas[p]);
    P.flags[p] = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(areas[p]) + recv_bytes);
  }
  uint8_t* own = reinterpret_cast<uint8_t*>(areas[rank]);
  P.local = reinterpret_cast<int*>(own + recv_bytes + flag_bytes);
  P.scratch = reinterpret_cast<__half*>(own + recv_bytes + flag_bytes + 256);
  P.rank = rank;
  P.world = world;
  P.max_rows = max_rows;
  P.max_width = max_width;
  P.partial = partial;
  P.partial_stride = partial_stride;
  P.rows = rows;
  P.width = width;
  P.h = reinterpret_cast<__half*>(h);
  P.norm_w = reinterpret_cast<const __half*>(norm_weight);
  P.eps = eps;
  P.x_out = reinterpret_cast<__half*>(x_out);
  P.x_absmax = x_absmax;
  P.status = device_status_word();
  if (P.status == nullptr) return BSB_ECUDA;
  P.wait_ns = g_peer_wait_ns;
  BSB_CUDA(launch_pdl(peer_allreduce_add_rmsnorm_kernel, dim3((unsigned)rows), dim3(kRowThreads), 0, (cudaStream_t)stream, P));
  return check_launch("peer_allreduce_add_rmsnorm_kernel");
}

}  // extern "C"
