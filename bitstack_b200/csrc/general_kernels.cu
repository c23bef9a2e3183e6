// Shape-agnostic CUDA-core kernels: any out/in/k, fp32 arithmetic.  They are the
// path for ragged shapes (in_features not a multiple of 128, rank != 16) and the
// on-device cross-check for the tensor-core kernels.
//
// Math (bitstack/modules/BitStackLinear.py:7-15,105-114 of the reference):
//   W = sum_j S_j * (U_j Vt_j),   y = x W^T + bias
// evaluated here as  y[m] = sum_j sum_r U_j[m,r] * sum_n S_j[m,n] Vt_j[r,n] x[n].
#include "common.cuh"

namespace bsb {

namespace {

__device__ __forceinline__ float sign_at(const uint8_t* __restrict__ q, int64_t e) {
  const uint32_t b = q[e >> 3];
  return ((b >> (7 - (int)(e & 7))) & 1u) ? 1.0f : -1.0f;
}

constexpr int kRankChunk = 16;

// one warp per (x row, output feature)
__global__ void __launch_bounds__(256) general_forward_kernel(bsb_weight w, const __half* __restrict__ x,
                                                              int64_t rows, int64_t x_stride,
                                                              __half* __restrict__ y, float* __restrict__ y32,
                                                              int64_t y_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t total = rows * (int64_t)w.out_features;
  if (warp >= total) return;
  const int64_t row = warp / w.out_features;
  const int m = (int)(warp % w.out_features);
  const int N = w.in_features;
  const __half* xr = x + row * x_stride;
  const __half* u_all = reinterpret_cast<const __half*>(w.u);
  const __half* vt_all = reinterpret_cast<const __half*>(w.vt);

  float acc = 0.f;
  for (int j = 0; j < w.blocks; ++j) {
    const uint8_t* q = w.qweight + (int64_t)j * w.q_block_stride;
    const __half* u = u_all + (int64_t)j * w.u_block_stride + (int64_t)m * w.k;
    const __half* vt = vt_all + (int64_t)j * w.vt_block_stride;
    for (int r0 = 0; r0 < w.k; r0 += kRankChunk) {
      float t[kRankChunk];
#pragma unroll
      for (int r = 0; r < kRankChunk; ++r) t[r] = 0.f;
      for (int n = lane; n < N; n += 32) {
        const float sx = sign_at(q, (int64_t)m * N + n) * __half2float(xr[n]);
#pragma unroll
        for (int r = 0; r < kRankChunk; ++r) {
          if (r0 + r < w.k) t[r] = fmaf(sx, __half2float(vt[(int64_t)(r0 + r) * N + n]), t[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < kRankChunk; ++r) {
        float v = t[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (r0 + r < w.k) acc = fmaf(__half2float(u[r0 + r]), v, acc);
      }
    }
  }
  if (lane == 0) {
    if (w.bias) acc += __half2float(reinterpret_cast<const __half*>(w.bias)[m]);
    if (y32) y32[row * y_stride + m] = acc;   // partial-sum output of a tensor-parallel shard: no rounding
    else y[row * y_stride + m] = __float2half_rn(acc);
  }
}

// one thread per weight element
__global__ void __launch_bounds__(256) general_reconstruct_kernel(bsb_weight w, __half* __restrict__ out) {
  const int64_t total = (int64_t)w.out_features * w.in_features;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const __half* u_all = reinterpret_cast<const __half*>(w.u);
  const __half* vt_all = reinterpret_cast<const __half*>(w.vt);
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const int m = (int)(e / w.in_features);
    const int n = (int)(e % w.in_features);
    float acc = 0.f;
    for (int j = 0; j < w.blocks; ++j) {
      const __half* u = u_all + (int64_t)j * w.u_block_stride + (int64_t)m * w.k;
      const __half* vt = vt_all + (int64_t)j * w.vt_block_stride + n;
      float a = 0.f;
      for (int r = 0; r < w.k; ++r)
        a = fmaf(__half2float(u[r]), __half2float(vt[(int64_t)r * w.in_features]), a);
      acc += sign_at(w.qweight + (int64_t)j * w.q_block_stride, e) * a;
    }
    out[e] = __float2half_rn(acc);
  }
}

}  // namespace

int launch_general_forward(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride,
                           __half* y, float* y32, int64_t y_stride, cudaStream_t s) {
  const int64_t warps = rows * (int64_t)w.out_features;
  if (warps == 0) return BSB_OK;
  const int64_t blocks = ceil_div64(warps, 8);
  BSB_CHECK_ARG(blocks < (1ll << 31), "general forward: too many output elements (%lld)", (long long)warps);
  general_forward_kernel<<<(unsigned)blocks, 256, 0, s>>>(w, x, rows, x_stride, y, y32, y_stride);
  return check_launch("general_forward_kernel");
}

int launch_general_reconstruct(const bsb_weight& w, __half* w_out, cudaStream_t s) {
  const int64_t total = (int64_t)w.out_features * w.in_features;
  if (total == 0) return BSB_OK;
  int64_t blocks = ceil_div64(total, 256);
  const int64_t cap = (int64_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  general_reconstruct_kernel<<<(unsigned)blocks, 256, 0, s>>>(w, w_out);
  return check_launch("general_reconstruct_kernel");
}

}  // namespace bsb
