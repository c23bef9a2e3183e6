// Small fused kernels around the BitStack projections of a decoder layer at decode time
// (a handful of rows): residual add + RMSNorm, rotary embedding + KV-cache write, SiLU*up.
// The reference delegates these to the Hugging Face Llama modules (one PyTorch launch per
// elementary op); at batch 1 the launches cost more than the math, hence the fusion.
#include "common.cuh"

namespace bsb {
namespace {

// h[row] (+= delta[row]) ; y[row] = h[row] * rsqrt(mean(h^2) + eps) * weight      (fp32 inside)
// one CTA per row; a thread keeps its 8-element vectors (16-byte loads) in registers, so the row is
// read once, the norm weight is fetched before the reduction and nothing is staged in shared memory
constexpr int kNormThreads = 512;
constexpr int kNormVecs = 4;   // vectors per thread: rows up to 512 * 4 * 8 = 16384 elements
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(__half* __restrict__ h, const __half* __restrict__ delta,
                                                                   const __half* __restrict__ weight, float eps,
                                                                   __half* __restrict__ y, int hidden) {
  __shared__ float red[kNormThreads / 32];
  const int64_t row = blockIdx.x;
  uint4* hr = reinterpret_cast<uint4*>(h + row * hidden);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * hidden) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  const int nvec = hidden / 8;
  uint4 hv[kNormVecs], dv[kNormVecs], wv[kNormVecs];
#pragma unroll
  for (int k = 0; k < kNormVecs; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
      hv[k] = hr[i];
      if (dr) dv[k] = __ldg(dr + i);
      wv[k] = __ldg(wr + i);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < kNormVecs; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
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
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)hidden + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * hidden);
#pragma unroll
  for (int k = 0; k < kNormVecs; ++k) {
    const int i = threadIdx.x + k * kNormThreads;
    if (i < nvec) {
      const __half2* hp = reinterpret_cast<const __half2*>(&hv[k]);
      const __half2* wp = reinterpret_cast<const __half2*>(&wv[k]);
      uint4 out;
      __half2* op = reinterpret_cast<__half2*>(&out);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __half22float2(hp[q]), wq = __half22float2(wp[q]);
        op[q] = __floats2half2_rn(a.x * inv * wq.x, a.y * inv * wq.y);
      }
      yr[i] = out;
    }
  }
}

// one CTA per (batch row, head); heads [0, Hq) are query heads (rotated in place), then Hkv key
// heads (rotated into the cache), then Hkv value heads (copied into the cache)
__global__ void __launch_bounds__(128) rope_cache_kernel(__half* __restrict__ q, const __half* __restrict__ k,
                                                         const __half* __restrict__ v, const __half* __restrict__ cos_t,
                                                         const __half* __restrict__ sin_t, const int64_t* __restrict__ pos_p,
                                                         __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                                         int Hq, int Hkv, int D, int max_len) {
  const int b = blockIdx.y, head = blockIdx.x;
  const int64_t pos = *pos_p;
  if (pos < 0 || pos >= max_len) return;   // out of the cache: nothing is written
  const int half_d = D / 2;
  const __half* cs = cos_t + pos * D;
  const __half* sn = sin_t + pos * D;
  if (head < Hq + Hkv) {
    const bool is_q = head < Hq;
    const __half* src = is_q ? q + ((int64_t)b * Hq + head) * D : k + ((int64_t)b * Hkv + (head - Hq)) * D;
    __half* dst = is_q ? q + ((int64_t)b * Hq + head) * D
                       : k_cache + (((int64_t)b * Hkv + (head - Hq)) * max_len + pos) * D;
    for (int i = threadIdx.x; i < half_d; i += blockDim.x) {
      const float x0 = __half2float(src[i]), x1 = __half2float(src[i + half_d]);
      const float c0 = __half2float(cs[i]), c1 = __half2float(cs[i + half_d]);
      const float s0 = __half2float(sn[i]), s1 = __half2float(sn[i + half_d]);
      // x*cos + rotate_half(x)*sin with rotate_half(x) = [-x1, x0]
      const float o0 = x0 * c0 - x1 * s0, o1 = x1 * c1 + x0 * s1;
      dst[i] = __float2half_rn(o0);
      dst[i + half_d] = __float2half_rn(o1);
    }
  } else {
    const int hv = head - Hq - Hkv;
    const __half* src = v + ((int64_t)b * Hkv + hv) * D;
    __half* dst = v_cache + (((int64_t)b * Hkv + hv) * max_len + pos) * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
  }
}

__global__ void __launch_bounds__(256) silu_mul_kernel(const __half2* __restrict__ g, const __half2* __restrict__ u,
                                                       __half2* __restrict__ out, int64_t n2) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += (int64_t)gridDim.x * blockDim.x) {
    const float2 a = __half22float2(g[i]), b = __half22float2(u[i]);
    const __half2 s = __floats2half2_rn(a.x / (1.f + __expf(-a.x)), a.y / (1.f + __expf(-a.y)));   // fp16 SiLU, as torch rounds it
    const float2 sf = __half22float2(s);
    out[i] = __floats2half2_rn(sf.x * b.x, sf.y * b.y);
  }
}

}  // namespace
}  // namespace bsb

using namespace bsb;

extern "C" {

int bsb_add_rmsnorm(uint16_t* h, const uint16_t* delta, const uint16_t* weight, float eps, uint16_t* y, int64_t rows,
                    int32_t hidden, void* stream) {
  BSB_CHECK_ARG(h && weight && y, "NULL buffer");
  BSB_CHECK_ARG(rows >= 0 && hidden > 0 && hidden % 8 == 0 && hidden <= kNormThreads * kNormVecs * 8,
                "hidden must be a multiple of 8 and <= 16384");
  BSB_CHECK_ARG(((uintptr_t)h | (uintptr_t)weight | (uintptr_t)y | (uintptr_t)delta) % 16 == 0, "buffers must be 16-byte aligned");
  if (rows == 0) return BSB_OK;
  BSB_CHECK_ARG(rows <= 65535 * 32, "too many rows");
  add_rmsnorm_kernel<<<(unsigned)rows, kNormThreads, 0, (cudaStream_t)stream>>>(
      (__half*)h, (const __half*)delta, (const __half*)weight, eps, (__half*)y, hidden);
  return check_launch("add_rmsnorm_kernel");
}

int bsb_rope_cache(uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* cos_table, const uint16_t* sin_table,
                   const int64_t* pos, uint16_t* k_cache, uint16_t* v_cache, int32_t batch, int32_t q_heads,
                   int32_t kv_heads, int32_t head_dim, int32_t max_len, void* stream) {
  BSB_CHECK_ARG(q && k && v && cos_table && sin_table && pos && k_cache && v_cache, "NULL buffer");
  BSB_CHECK_ARG(batch >= 1 && q_heads >= 1 && kv_heads >= 1 && head_dim >= 2 && head_dim % 2 == 0 && max_len >= 1,
                "bad attention shape");
  dim3 grid(q_heads + 2 * kv_heads, batch);
  rope_cache_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((__half*)q, (const __half*)k, (const __half*)v,
                                                            (const __half*)cos_table, (const __half*)sin_table, pos,
                                                            (__half*)k_cache, (__half*)v_cache, q_heads, kv_heads,
                                                            head_dim, max_len);
  return check_launch("rope_cache_kernel");
}

int bsb_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t n, void* stream) {
  BSB_CHECK_ARG(gate && up && out, "NULL buffer");
  BSB_CHECK_ARG(n >= 0 && n % 2 == 0, "element count must be even");
  BSB_CHECK_ARG(((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) % 4 == 0, "buffers must be 4-byte aligned");
  if (n == 0) return BSB_OK;
  int64_t blocks = ceil_div64(n / 2, 256);
  if (blocks > 1184) blocks = 1184;
  silu_mul_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __half2*)gate, (const __half2*)up, (__half2*)out, n / 2);
  return check_launch("silu_mul_kernel");
}

}  // extern "C"
