// Row operations of a decoder layer around the projections, shared by the stand-alone glue kernels and by the
// output stage of the decode kernel so that both produce bit-identical results:
//   add + RMSNorm:  h (+= delta);  y = h * rsqrt(mean(h^2) + eps) * weight      (fp32 inside, fp16 residual stream)
//   SiLU * up:      out = silu(gate) * up                                        (fp16 SiLU, as torch rounds it)
// Both also deliver max |result| of the row, which the next projection's operand preparation needs.
// One CTA works on one row (add + RMSNorm: kRowThreads threads; SiLU * up: any multiple of 32); `red` is shared
// scratch of 32 floats.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace bsb {

constexpr int kRowThreads = 512;
constexpr int kRowVecs = 4;   // 16-byte vectors per thread: rows up to 512 * 4 * 8 = 16384 elements

// COHERENT: delta was written by other CTAs of the running kernel (read through L2, not the read-only path)
template <bool COHERENT>
__device__ __forceinline__ uint4 row_load(const uint4* p) {
  return COHERENT ? __ldcg(p) : __ldg(p);
}

// reduction over the CTA (any multiple of 32 threads up to 1024; `red` holds 32 floats)
__device__ __forceinline__ float row_block_reduce(float v, float* red, bool is_max) {
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  __syncthreads();   // `red` may still be read from a previous reduction
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  const int nw = (int)blockDim.x >> 5;
  float tot = 0.f;
  for (int i = 0; i < nw; ++i) tot = is_max ? fmaxf(tot, red[i]) : tot + red[i];
  return tot;
}

// hidden % 8 == 0, hidden <= 16384, 16-byte aligned rows.  absmax_out may be nullptr.
template <bool COHERENT>
__device__ __forceinline__ void add_rmsnorm_row(__half* __restrict__ h, const __half* __restrict__ delta,
                                                const __half* __restrict__ weight, float eps, __half* __restrict__ y,
                                                int hidden, float* red, float* absmax_out) {
  uint4* hr = reinterpret_cast<uint4*>(h);
  const uint4* dr = reinterpret_cast<const uint4*>(delta);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  const int nvec = hidden / 8;
  uint4 hv[kRowVecs], dv[kRowVecs], wv[kRowVecs];
#pragma unroll
  for (int k = 0; k < kRowVecs; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i < nvec) {
      hv[k] = hr[i];
      if (dr) dv[k] = row_load<COHERENT>(dr + i);
      wv[k] = __ldg(wr + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kRowVecs; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i < nvec) {
      __half2* hp = reinterpret_cast<__half2*>(&hv[k]);
      if (dr) {
        const __half2* dp = reinterpret_cast<const __half2*>(&dv[k]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 a = __half22float2(hp[q]), d = __half22float2(dp[q]);
          hp[q] = __floats2half2_rn(a.x + d.x, a.y + d.y);   // the residual stream stays fp16
        }
        hr[i] = hv[k];
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __half22float2(hp[q]);
        ss += a.x * a.x + a.y * a.y;
      }
    }
  }
  const float tot = row_block_reduce(ss, red, false);
  const float inv = rsqrtf(tot / (float)hidden + eps);
  uint4* yr = reinterpret_cast<uint4*>(y);
  float am = 0.f;
#pragma unroll
  for (int k = 0; k < kRowVecs; ++k) {
    const int i = threadIdx.x + k * kRowThreads;
    if (i < nvec) {
      const __half2* hp = reinterpret_cast<const __half2*>(&hv[k]);
      const __half2* wp = reinterpret_cast<const __half2*>(&wv[k]);
      uint4 out;
      __half2* op = reinterpret_cast<__half2*>(&out);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __half22float2(hp[q]), wq = __half22float2(wp[q]);
        op[q] = __floats2half2_rn(a.x * inv * wq.x, a.y * inv * wq.y);
        const float2 f = __half22float2(__habs2(op[q]));
        am = fmaxf(am, fmaxf(f.x, f.y));
      }
      yr[i] = out;
    }
  }
  if (absmax_out != nullptr) {   // uniform for the CTA
    am = row_block_reduce(am, red, true);
    if (threadIdx.x == 0) *absmax_out = am;
  }
}

// n % 8 == 0, 16-byte aligned rows, any n (threads stride over the row).  absmax_out may be nullptr.
template <bool COHERENT>
__device__ __forceinline__ void silu_mul_row(const __half* __restrict__ gate, const __half* __restrict__ up,
                                             __half* __restrict__ out, int n, float* red, float* absmax_out) {
  const uint4* gr = reinterpret_cast<const uint4*>(gate);
  const uint4* ur = reinterpret_cast<const uint4*>(up);
  uint4* orow = reinterpret_cast<uint4*>(out);
  float am = 0.f;
  auto one = [&](const uint4& gv, const uint4& uv, int i) {
    const __half2* gp = reinterpret_cast<const __half2*>(&gv);
    const __half2* up2 = reinterpret_cast<const __half2*>(&uv);
    uint4 o;
    __half2* op = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = __half22float2(gp[q]), b = __half22float2(up2[q]);
      const __half2 s = __floats2half2_rn(__fdividef(a.x, 1.f + __expf(-a.x)), __fdividef(a.y, 1.f + __expf(-a.y)));   // fp16 SiLU
      const float2 sf = __half22float2(s);
      op[q] = __floats2half2_rn(sf.x * b.x, sf.y * b.y);
      const float2 f = __half22float2(__habs2(op[q]));
      am = fmaxf(am, fmaxf(f.x, f.y));
    }
    orow[i] = o;
  };
  // two vectors per thread and array are in flight at a time (a 14336-wide row is 1.75 vectors per thread of a
  // 1024-thread CTA: all of its loads go out together)
  const int nvec = n / 8, stride = (int)blockDim.x;
  for (int i0 = threadIdx.x; i0 < nvec; i0 += 2 * stride) {
    const int i1 = i0 + stride;
    const bool two = i1 < nvec;
    const uint4 g0 = row_load<COHERENT>(gr + i0), u0 = row_load<COHERENT>(ur + i0);
    uint4 g1 = make_uint4(0, 0, 0, 0), u1 = g1;
    if (two) {
      g1 = row_load<COHERENT>(gr + i1);
      u1 = row_load<COHERENT>(ur + i1);
    }
    one(g0, u0, i0);
    if (two) one(g1, u1, i1);
  }
  if (absmax_out != nullptr) {
    am = row_block_reduce(am, red, true);
    if (threadIdx.x == 0) *absmax_out = am;
  }
}

}  // namespace bsb
