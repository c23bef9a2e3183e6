// Small fused kernels around the BitStack projections of a decoder layer at decode time
// (a handful of rows): residual add + RMSNorm, rotary embedding + KV-cache write, SiLU*up.
// The reference delegates these to the Hugging Face Llama modules (one PyTorch launch per
// elementary op); at batch 1 the launches cost more than the math, hence the fusion.
#include <cstdint>

#include "common.cuh"
#include "rowops.cuh"

namespace bsb {
namespace {

// h[row] (+= delta[row]) ; y[row] = h[row] * rsqrt(mean(h^2) + eps) * weight; optionally max |y[row]|.
// One CTA per row (rowops.cuh).
__global__ void __launch_bounds__(kRowThreads) add_rmsnorm_kernel(__half* __restrict__ h, const __half* __restrict__ delta,
                                                                  const __half* __restrict__ weight, float eps,
                                                                  __half* __restrict__ y, int hidden, float* __restrict__ absmax) {
  __shared__ float red[32];
  // the norm weight is a constant that the projections' weight stream has evicted since the last step: it is
  // asked into L2 while this kernel still waits for the one in front
  if ((int)threadIdx.x * 64 < hidden) asm volatile("prefetch.global.L2 [%0];" ::"l"(weight + threadIdx.x * 64));
  pdl_enter();
  const int64_t row = blockIdx.x;
  add_rmsnorm_row<false>(h + row * hidden, delta ? delta + row * hidden : nullptr, weight, eps, y + row * hidden, hidden, red,
                         absmax ? absmax + row : nullptr);
}

// one CTA per (batch row, head); heads [0, Hq) are query heads (rotated in place), then Hkv key
// heads (rotated into the cache), then Hkv value heads (copied into the cache)
__global__ void __launch_bounds__(128) rope_cache_kernel(__half* __restrict__ q, const __half* __restrict__ k,
                                                         const __half* __restrict__ v, const __half* __restrict__ cos_t,
                                                         const __half* __restrict__ sin_t, const int64_t* __restrict__ pos_p,
                                                         __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                                         int Hq, int Hkv, int D, int max_len) {
  // no early release of the kernel behind this one: decode_attention_kernel reads cache rows in front of its own wait,
  // which is only safe for rows whose writer has finished before it starts
  pdl_wait();
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

// ---- single-token attention with the rotary embedding and the KV-cache write folded in --------
// kAttSplits CTAs per (query head, batch row), each over a contiguous share of the cache positions
// (one CTA alone pays every memory latency of its phases in sequence; the cache of a layer is cold);
// 256 threads; caches [batch][kv_heads][max_len][D] fp16.
//   A. q and the new k are rotated in fp32 and rounded to fp16 (what a separate rotary kernel would
//      have stored); the new k and v go into the caches (every CTA of a KV group writes the same
//      bytes), q stays in shared memory as fp32.
//   B. scores: one THREAD per cache position -- its whole K row is D/8 independent 16-byte loads, so
//      a CTA keeps tens of KB in flight instead of paying one memory latency per position.
//   C. softmax statistics over the scores in shared memory (fp32).
//   D. P.V: thread (r, c) adds rows r, r+16, ... of V for the c-th 8-element vector, eight rows in
//      flight; the 16 partial sums per element are merged in shared memory.
//   E. every CTA leaves (max, sum, unnormalised output) in `partial`; the last one to arrive on the
//      head's counter merges the kAttSplits results, writes `out` and resets the counter to 0.
#ifndef BSB_ATT_SPLITS
#define BSB_ATT_SPLITS 4
#endif
constexpr int kAttSplits = BSB_ATT_SPLITS;
template <int D>
__global__ void __launch_bounds__(256) decode_attention_kernel(const __half* __restrict__ q, const __half* __restrict__ k,
                                                               const __half* __restrict__ v, const __half* __restrict__ cos_t,
                                                               const __half* __restrict__ sin_t, const int64_t* __restrict__ pos_p,
                                                               __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                                                               __half* __restrict__ out, int Hq, int Hkv, int max_len, float scale,
                                                               float* __restrict__ partial, int* __restrict__ counters) {
  constexpr int kVec = D / 8;            // 16-byte vectors per row
  constexpr int kRowsPerPass = 256 / kVec;
  extern __shared__ float s_score[];     // [pos + 1]
  __shared__ float s_q[D];
  __shared__ float s_red[8];
  __shared__ float s_part[kRowsPerPass][D];
  __shared__ int s_last;
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // The position and the cache rows below it were written by kernels that finished before the kernel in front of
  // this one started (every kernel of the chain waits for its predecessor before it ends), so they may be read
  // before this kernel's own wait: the first K row of every thread is in flight while the projection kernel drains.
  const int64_t pos = *pos_p;
  if (pos < 0 || pos >= max_len) {   // out of the cache: nothing is written (the kernel still takes its place in the chain of waits)
    pdl_enter();
    return;
  }
  const int hk = h / (Hq / Hkv);
  __half* kc = k_cache + ((int64_t)b * Hkv + hk) * (int64_t)max_len * D;
  __half* vc = v_cache + ((int64_t)b * Hkv + hk) * (int64_t)max_len * D;
  const int n_all = (int)pos + 1;
  const int share = (n_all + kAttSplits - 1) / kAttSplits;
  const int p_lo = min(split * share, n_all);
  const int n = min(share, n_all - p_lo);
  uint4 k_first[kVec];
  const bool have_first = tid < n && p_lo + tid != (int)pos;   // the row of this step's own position is written below
  if (have_first) {
    const uint4* row = reinterpret_cast<const uint4*>(kc + (int64_t)(p_lo + tid) * D);
#pragma unroll
    for (int c = 0; c < kVec; ++c) k_first[c] = row[c];
  }
  // the V rows of the share: asked into L2 now, read after the softmax weights are known
  for (int p = tid; p < 2 * n; p += 256) {
    const __half* line = vc + (int64_t)(p_lo + (p >> 1)) * D + (p & 1) * (D / 2);   // both halves of a row: two 128-byte lines at D = 128
    asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
  }
  pdl_enter();

  // ---- A ----
  if (tid < D / 2) {
    const int i = tid;
    const float c0 = __half2float(cos_t[pos * D + i]), c1 = __half2float(cos_t[pos * D + i + D / 2]);
    const float s0 = __half2float(sin_t[pos * D + i]), s1 = __half2float(sin_t[pos * D + i + D / 2]);
    // x*cos + rotate_half(x)*sin with rotate_half(x) = [-x1, x0]
    const __half* qs = q + ((int64_t)b * Hq + h) * D;
    float x0 = __half2float(qs[i]), x1 = __half2float(qs[i + D / 2]);
    s_q[i] = __half2float(__float2half_rn(x0 * c0 - x1 * s0));
    s_q[i + D / 2] = __half2float(__float2half_rn(x1 * c1 + x0 * s1));
    const __half* ks = k + ((int64_t)b * Hkv + hk) * D;
    x0 = __half2float(ks[i]);
    x1 = __half2float(ks[i + D / 2]);
    kc[pos * D + i] = __float2half_rn(x0 * c0 - x1 * s0);
    kc[pos * D + i + D / 2] = __float2half_rn(x1 * c1 + x0 * s1);
  } else if (tid < D / 2 + D / 8) {
    const int c = tid - D / 2;
    reinterpret_cast<uint4*>(vc + pos * D)[c] = reinterpret_cast<const uint4*>(v + ((int64_t)b * Hkv + hk) * D)[c];
  }
  __syncthreads();

  // ---- B ----  (positions [p_lo, p_lo + n) of the pos + 1 in the cache; scores are indexed from p_lo)
  kc += (int64_t)p_lo * D;
  vc += (int64_t)p_lo * D;
  float m_loc = -INFINITY;
  for (int p = tid; p < n; p += 256) {
    const uint4* row = reinterpret_cast<const uint4*>(kc + (int64_t)p * D);
    uint4 raw[kVec];
#pragma unroll
    for (int c = 0; c < kVec; ++c) raw[c] = (p == tid && have_first) ? k_first[c] : row[c];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < kVec; ++c) {
      const __half2* h2 = reinterpret_cast<const __half2*>(&raw[c]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h2[e]);
        dot = fmaf(f.x, s_q[c * 8 + 2 * e], dot);
        dot = fmaf(f.y, s_q[c * 8 + 2 * e + 1], dot);
      }
    }
    const float sc = dot * scale;
    s_score[p] = sc;
    m_loc = fmaxf(m_loc, sc);
  }
  // ---- C ----
  for (int o = 16; o > 0; o >>= 1) m_loc = fmaxf(m_loc, __shfl_xor_sync(0xFFFFFFFFu, m_loc, o));
  if (lane == 0) s_red[warp] = m_loc;
  __syncthreads();
  float m = s_red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, s_red[w]);
  __syncthreads();
  float l_loc = 0.f;
  for (int p = tid; p < n; p += 256) {
    const float e = __expf(s_score[p] - m);
    s_score[p] = e;
    l_loc += e;
  }
  for (int o = 16; o > 0; o >>= 1) l_loc += __shfl_xor_sync(0xFFFFFFFFu, l_loc, o);
  if (lane == 0) s_red[warp] = l_loc;
  __syncthreads();
  float l = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) l += s_red[w];

  // ---- D ----
  const int r = tid / kVec, c = tid % kVec;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int p = r; p < n; p += 8 * kRowsPerPass) {
    uint4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {          // rows past the end: no load, weight 0
      const int pu = p + u * kRowsPerPass;
      raw[u] = pu < n ? reinterpret_cast<const uint4*>(vc + (int64_t)pu * D)[c] : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int pu = p + u * kRowsPerPass;
      const float w = pu < n ? s_score[pu] : 0.f;
      const __half2* h2 = reinterpret_cast<const __half2*>(&raw[u]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h2[e]);
        acc[2 * e] = fmaf(w, f.x, acc[2 * e]);
        acc[2 * e + 1] = fmaf(w, f.y, acc[2 * e + 1]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_part[r][c * 8 + e] = acc[e];
  __syncthreads();
  // ---- E ----
  float* mine = partial + (((int64_t)b * Hq + h) * kAttSplits + split) * (D + 2);
  if (tid < D) {
    float o = 0.f;
#pragma unroll
    for (int rr = 0; rr < kRowsPerPass; ++rr) o += s_part[rr][tid];
    mine[2 + tid] = o;
  }
  if (tid == 0) { mine[0] = m; mine[1] = l; }
  __syncthreads();
  if (tid == 0) {
    // the barrier ordered every thread's stores before this release, which orders them before the count; the
    // acquiring count and the barrier below order the other shares' results before the loads (from L2)
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(counters + b * Hq + h) : "memory");
    s_last = (old == kAttSplits - 1);
    if (s_last) counters[b * Hq + h] = 0;   // ready for the next call
  }
  __syncthreads();
  if (!s_last) return;
  if (tid < D) {
    const float* all = partial + ((int64_t)b * Hq + h) * kAttSplits * (D + 2);
    float mm = -INFINITY;
#pragma unroll
    for (int sidx = 0; sidx < kAttSplits; ++sidx) mm = fmaxf(mm, __ldcg(all + sidx * (D + 2)));
    float ll = 0.f, o = 0.f;
#pragma unroll
    for (int sidx = 0; sidx < kAttSplits; ++sidx) {
      const float f = __expf(__ldcg(all + sidx * (D + 2)) - mm);   // an empty share has max -inf, sum 0: weight 0
      ll += __ldcg(all + sidx * (D + 2) + 1) * f;
      o += __ldcg(all + sidx * (D + 2) + 2 + tid) * f;
    }
    out[((int64_t)b * Hq + h) * D + tid] = __float2half_rn(o / ll);
  }
}

// greedy sampling step: tokens[b] = index of the first maximum of logits[b][0..V), then *pos += 1.
// One CTA per batch row, 16-byte loads; ties go to the lowest index (torch.argmax's rule).
__global__ void __launch_bounds__(1024) greedy_step_kernel(const __half* __restrict__ logits, int64_t V, int64_t stride,
                                                           int64_t* __restrict__ tokens, int64_t* __restrict__ pos) {
  __shared__ float s_val[32];
  __shared__ int64_t s_idx[32];
  pdl_wait();   // no early release: this kernel writes *pos, which decode_attention_kernel reads in front of its own wait
  const __half* row = logits + (int64_t)blockIdx.x * stride;
  float best = -INFINITY;
  int64_t best_i = INT64_MAX;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) % 16 == 0);
  const int64_t n8 = vec_ok ? V / 8 : 0;
  for (int64_t i = threadIdx.x; i < n8; i += blockDim.x) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row) + i);
    const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float f = __half2float(h[e]);
      if (f > best) { best = f; best_i = i * 8 + e; }   // ascending index within a thread: the first maximum stays
    }
  }
  for (int64_t i = n8 * 8 + threadIdx.x; i < V; i += blockDim.x) {
    const float f = __half2float(row[i]);
    if (f > best || (f == best && i < best_i)) { best = f; best_i = i; }
  }
  auto better = [](float a, int64_t ai, float b, int64_t bi) { return a > b || (a == b && ai < bi); };
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
    const int64_t oi = __shfl_xor_sync(0xFFFFFFFFu, best_i, o);
    if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = (blockDim.x + 31) / 32;
    best = threadIdx.x < nw ? s_val[threadIdx.x] : -INFINITY;
    best_i = threadIdx.x < nw ? s_idx[threadIdx.x] : INT64_MAX;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int64_t oi = __shfl_xor_sync(0xFFFFFFFFu, best_i, o);
      if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) {
      tokens[blockIdx.x] = best_i == INT64_MAX ? 0 : best_i;   // a row of NaNs: token 0
      if (blockIdx.x == 0 && pos != nullptr) *pos += 1;
    }
  }
}

// out[row] = silu(gate[row]) * up[row]; optionally max |out[row]|.  One CTA per row (rowops.cuh).
constexpr int kSiluThreads = 1024;
__global__ void __launch_bounds__(kSiluThreads) silu_mul_kernel(const __half* __restrict__ g, const __half* __restrict__ u,
                                                                __half* __restrict__ out, int n, float* __restrict__ absmax) {
  __shared__ float red[32];
  pdl_enter();
  const int64_t row = blockIdx.x;
  silu_mul_row<false>(g + row * n, u + row * n, out + row * n, n, red, absmax ? absmax + row : nullptr);
}

}  // namespace
}  // namespace bsb

using namespace bsb;

extern "C" {

int bsb_add_rmsnorm(uint16_t* h, const uint16_t* delta, const uint16_t* weight, float eps, uint16_t* y, float* y_absmax,
                    int64_t rows, int32_t hidden, void* stream) {
  BSB_CHECK_ARG(h && weight && y, "NULL buffer");
  BSB_CHECK_ARG(rows >= 0 && hidden > 0 && hidden % 8 == 0 && hidden <= kRowThreads * kRowVecs * 8,
                "hidden must be a multiple of 8 and <= 16384");
  BSB_CHECK_ARG(((uintptr_t)h | (uintptr_t)weight | (uintptr_t)y | (uintptr_t)delta) % 16 == 0, "buffers must be 16-byte aligned");
  if (rows == 0) return BSB_OK;
  BSB_CHECK_ARG(rows <= 65535 * 32, "too many rows");
  BSB_CUDA(launch_pdl(add_rmsnorm_kernel, dim3((unsigned)rows), dim3(kRowThreads), 0, (cudaStream_t)stream,
                      (__half*)h, (const __half*)delta, (const __half*)weight, eps, (__half*)y, hidden, y_absmax));
  return check_launch("add_rmsnorm_kernel");
}

int bsb_rope_cache(uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* cos_table, const uint16_t* sin_table,
                   const int64_t* pos, uint16_t* k_cache, uint16_t* v_cache, int32_t batch, int32_t q_heads,
                   int32_t kv_heads, int32_t head_dim, int32_t max_len, void* stream) {
  BSB_CHECK_ARG(q && k && v && cos_table && sin_table && pos && k_cache && v_cache, "NULL buffer");
  BSB_CHECK_ARG(batch >= 1 && q_heads >= 1 && kv_heads >= 1 && head_dim >= 2 && head_dim % 2 == 0 && max_len >= 1,
                "bad attention shape");
  dim3 grid(q_heads + 2 * kv_heads, batch);
  BSB_CUDA(launch_pdl(rope_cache_kernel, grid, dim3(128), 0, (cudaStream_t)stream, (__half*)q, (const __half*)k, (const __half*)v,
                      (const __half*)cos_table, (const __half*)sin_table, pos, (__half*)k_cache, (__half*)v_cache, q_heads,
                      kv_heads, head_dim, max_len));
  return check_launch("rope_cache_kernel");
}

int64_t bsb_decode_attention_scratch_bytes(int32_t batch, int32_t q_heads, int32_t head_dim) {
  if (batch < 1 || q_heads < 1 || head_dim < 1) return -1;
  return align_up64((int64_t)batch * q_heads * 4, 256) + (int64_t)batch * q_heads * kAttSplits * (head_dim + 2) * 4;
}

int bsb_decode_attention(const uint16_t* q, const uint16_t* k, const uint16_t* v, const uint16_t* cos_table,
                         const uint16_t* sin_table, const int64_t* pos, uint16_t* k_cache, uint16_t* v_cache, uint16_t* out,
                         int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_len, void* scratch,
                         int64_t scratch_bytes, void* stream) {
  BSB_CHECK_ARG(q && k && v && cos_table && sin_table && pos && k_cache && v_cache && out && scratch, "NULL buffer");
  BSB_CHECK_ARG(batch >= 1 && q_heads >= 1 && head_dim >= 1 && scratch_bytes >= bsb_decode_attention_scratch_bytes(batch, q_heads, head_dim) &&
                (uintptr_t)scratch % 16 == 0, "scratch too small or not 16-byte aligned");
  BSB_CHECK_ARG(batch >= 1 && batch <= 65535 && q_heads >= 1 && kv_heads >= 1 && q_heads % kv_heads == 0 && max_len >= 1,
                "bad attention shape");
  BSB_CHECK_ARG(head_dim == 128 || head_dim == 64, "decode attention is built for head_dim 64 and 128 (got %d)", head_dim);
  BSB_CHECK_ARG(((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16 == 0,
                "buffers must be 16-byte aligned");
  BSB_CHECK_ARG(max_len <= 8192, "decode attention keeps one fp32 score per cache position in shared memory: max_len <= 8192 (got %d)", max_len);
  const float scale = 1.0f / sqrtf((float)head_dim);
  dim3 grid(q_heads, batch, kAttSplits);
  const size_t smem = (size_t)((max_len + kAttSplits - 1) / kAttSplits + 1) * sizeof(float);
  int* counters = reinterpret_cast<int*>(scratch);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(scratch) + align_up64((int64_t)batch * q_heads * 4, 256));
  if (head_dim == 128)
    BSB_CUDA(launch_pdl(decode_attention_kernel<128>, grid, dim3(256), smem, (cudaStream_t)stream,
                        (const __half*)q, (const __half*)k, (const __half*)v, (const __half*)cos_table, (const __half*)sin_table, pos,
                        (__half*)k_cache, (__half*)v_cache, (__half*)out, q_heads, kv_heads, max_len, scale, partial, counters));
  else
    BSB_CUDA(launch_pdl(decode_attention_kernel<64>, grid, dim3(256), smem, (cudaStream_t)stream,
                        (const __half*)q, (const __half*)k, (const __half*)v, (const __half*)cos_table, (const __half*)sin_table, pos,
                        (__half*)k_cache, (__half*)v_cache, (__half*)out, q_heads, kv_heads, max_len, scale, partial, counters));
  return check_launch("decode_attention_kernel");
}

int bsb_greedy_step(const uint16_t* logits, int64_t batch, int64_t vocab, int64_t row_stride, int64_t* tokens, int64_t* pos,
                    void* stream) {
  BSB_CHECK_ARG(logits && tokens, "NULL buffer");
  BSB_CHECK_ARG(batch >= 1 && batch <= 65535 && vocab >= 1 && row_stride >= vocab, "bad shape");
  BSB_CUDA(launch_pdl(greedy_step_kernel, dim3((unsigned)batch), dim3(1024), 0, (cudaStream_t)stream, (const __half*)logits,
                      vocab, row_stride, tokens, pos));
  return check_launch("greedy_step_kernel");
}

int bsb_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, float* out_absmax, int64_t rows, int32_t n,
                 void* stream) {
  BSB_CHECK_ARG(gate && up && out, "NULL buffer");
  BSB_CHECK_ARG(rows >= 0 && n >= 0 && n % 8 == 0, "row length must be a multiple of 8");
  BSB_CHECK_ARG(((uintptr_t)gate | (uintptr_t)up | (uintptr_t)out) % 16 == 0, "buffers must be 16-byte aligned");
  if (rows == 0 || n == 0) return BSB_OK;
  BSB_CHECK_ARG(rows <= 65535 * 32, "too many rows");
  BSB_CUDA(launch_pdl(silu_mul_kernel, dim3((unsigned)rows), dim3(kSiluThreads), 0, (cudaStream_t)stream, (const __half*)gate,
                      (const __half*)up, (__half*)out, n, out_absmax));
  return check_launch("silu_mul_kernel");
}

}  // extern "C"
