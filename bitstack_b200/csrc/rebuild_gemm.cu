// Batch / prefill path, first generation: rebuild the fp16 weight from the packed
// blocks (rank-16 products on the tensor cores, signs applied in registers, fp32
// accumulation over blocks, ONE fp16 rounding), then a dense x.W^T contraction.
//
// Replaces, for rows > 4, what the reference does with an unpack kernel, a
// reconstruct kernel and cuBLAS (bitstack/modules/BitStackLinear.py:116-148,
// bitstack/utils/inference_utils.py:42-156,286-488).
#include "common.cuh"

namespace bsb {

namespace {

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// same with a zero C operand: D = A.B (no register tuple to clear before every MMA)
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// a ^ (~b & 0x80000000): flips the sign of the fp32 pattern `a` when bit 31 of `b` is clear
__device__ __forceinline__ uint32_t flip_if_clear(uint32_t a, uint32_t b) {
  uint32_t out;
  // minterms of a ^ (~b & c) over (a, b, c) with a = 0xF0, b = 0xCC, c = 0xAA: 0xF0 ^ (0x33 & 0xAA) = 0xD2
  asm("lop3.b32 %0, %1, %2, %3, 0xD2;" : "=r"(out) : "r"(a), "r"(b), "r"(0x80000000u));
  return out;
}

// ---------------------------------------------------------------------------
// rebuild: CTA = 8 warps = 128 rows x 64 columns of W; warp = 16 rows x 64 cols
// ---------------------------------------------------------------------------
constexpr int kRbCols = 64;
constexpr int kRbRowsPerCta = 128;
constexpr int kRbRowTiles = 4;             // 128-row tiles per CTA
constexpr int kRbBlockGroup = 16;          // residual blocks staged in shared memory at once
constexpr int kRbVtStride = kRbCols + 8;   // halves; +16 B keeps ldmatrix rows on distinct banks

__global__ void __launch_bounds__(256) rebuild_weight_kernel(bsb_weight w, __half* __restrict__ out) {
  __shared__ __align__(16) __half vt_s[kRbBlockGroup][16][kRbVtStride];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int N = w.in_features, M = w.out_features;
  const int n0 = blockIdx.x * kRbCols;
  const __half* u_all = reinterpret_cast<const __half*>(w.u);
  const __half* vt_all = reinterpret_cast<const __half*>(w.vt);
  // a CTA walks kRbRowTiles 128-row tiles of the same 64 columns: with at most kRbBlockGroup
  // blocks the staged Vt slab is loaded once and reused by all of them
  const bool one_group = w.blocks <= kRbBlockGroup;

  for (int rt = 0; rt < kRbRowTiles; ++rt) {
  const int m0 = (blockIdx.y * kRbRowTiles + rt) * kRbRowsPerCta + warp * 16;
  if ((blockIdx.y * kRbRowTiles + rt) * kRbRowsPerCta >= M) break;   // uniform for the CTA
  const bool active = m0 < M;  // out_features is a multiple of 16

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;

  for (int j0 = 0; j0 < w.blocks; j0 += kRbBlockGroup) {
    const int nj = min(kRbBlockGroup, w.blocks - j0);
    if (rt == 0 || !one_group) {
    __syncthreads();  // previous group fully consumed
    // stage Vt[j0..j0+nj)[0..16)[n0..n0+64): 16 B per thread per step
    for (int i = threadIdx.x; i < nj * 16 * (kRbCols / 8); i += blockDim.x) {
      const int jj = i / (16 * (kRbCols / 8));
      const int rem = i % (16 * (kRbCols / 8));
      const int r = rem / (kRbCols / 8), c8 = rem % (kRbCols / 8);
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(
          vt_all + (int64_t)(j0 + jj) * w.vt_block_stride + (int64_t)r * N + n0 + c8 * 8));
      *reinterpret_cast<uint4*>(&vt_s[jj][r][c8 * 8]) = v;
    }
    __syncthreads();
    }
    if (!active) continue;

    // operands of a block that come straight from global memory (A fragment of U_j: rows m0+g /
    // m0+g+8, ranks 2t,2t+1 / 2t+8,2t+9; 64 sign bits of the two rows) are fetched one block ahead
    auto fetch = [&](int j, uint32_t (&af)[4], uint2& lo, uint2& hi) {
      const __half* u = u_all + (int64_t)j * w.u_block_stride;
      af[0] = __ldg(reinterpret_cast<const uint32_t*>(u + (int64_t)(m0 + g) * 16 + 2 * t));
      af[1] = __ldg(reinterpret_cast<const uint32_t*>(u + (int64_t)(m0 + g + 8) * 16 + 2 * t));
      af[2] = __ldg(reinterpret_cast<const uint32_t*>(u + (int64_t)(m0 + g) * 16 + 2 * t + 8));
      af[3] = __ldg(reinterpret_cast<const uint32_t*>(u + (int64_t)(m0 + g + 8) * 16 + 2 * t + 8));
      const uint8_t* q = w.qweight + (int64_t)j * w.q_block_stride;
      lo = __ldg(reinterpret_cast<const uint2*>(q + ((int64_t)(m0 + g) * N + n0) / 8));
      hi = __ldg(reinterpret_cast<const uint2*>(q + ((int64_t)(m0 + g + 8) * N + n0) / 8));
    };
    uint32_t a_next[4];
    uint2 lo_next, hi_next;
    fetch(j0, a_next, lo_next, hi_next);
    for (int jj = 0; jj < nj; ++jj) {
      uint32_t a[4] = {a_next[0], a_next[1], a_next[2], a_next[3]};
      const uint2 lo_t = make_uint2(lo_next.x << (2 * t), lo_next.y << (2 * t));
      const uint2 hi_t = make_uint2(hi_next.x << (2 * t), hi_next.y << (2 * t));
      if (jj + 1 < nj) fetch(j0 + jj + 1, a_next, lo_next, hi_next);
#pragma unroll
      for (int pair = 0; pair < 4; ++pair) {  // two 8-column tiles per ldmatrix.x4
        uint32_t b[4];
        // lanes 0-7: ranks 0-7 @ tile 2*pair; 8-15: ranks 8-15 @ same tile;
        // 16-23 / 24-31: the same for tile 2*pair+1
        const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int col = (2 * pair + (lane >> 4)) * 8;
        ldmatrix_x4_trans(b, &vt_s[jj][row][col]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = 2 * pair + h;
          float d[4];
          mma_f16_16816_zero(d, a, b[2 * h], b[2 * h + 1]);
          // column 8i+2t is bit 7-2t of byte i: the words were shifted left by 2t once per block, so the
          // shift that brings an element's bit to bit 31 is a compile-time constant (the compiler is free to
          // place it on the multiply pipe); d is flipped when the bit is clear, one LOP3 per element
          const uint32_t wlo = (i < 4) ? lo_t.x : lo_t.y;
          const uint32_t whi = (i < 4) ? hi_t.x : hi_t.y;
          constexpr int kBase = 24;
          const int sh = kBase - 8 * (i & 3);
          acc[i][0] += __uint_as_float(flip_if_clear(__float_as_uint(d[0]), wlo << sh));
          acc[i][1] += __uint_as_float(flip_if_clear(__float_as_uint(d[1]), wlo << (sh + 1)));
          acc[i][2] += __uint_as_float(flip_if_clear(__float_as_uint(d[2]), whi << sh));
          acc[i][3] += __uint_as_float(flip_if_clear(__float_as_uint(d[3]), whi << (sh + 1)));
        }
      }
    }
  }
  if (!active) continue;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int n = n0 + 8 * i + 2 * t;
    *reinterpret_cast<__half2*>(out + (int64_t)(m0 + g) * N + n) = __floats2half2_rn(acc[i][0], acc[i][1]);
    *reinterpret_cast<__half2*>(out + (int64_t)(m0 + g + 8) * N + n) = __floats2half2_rn(acc[i][2], acc[i][3]);
  }
  }
}

// ---------------------------------------------------------------------------
// dense contraction  y[rows][M] = x[rows][K] . W[M][K]^T (+bias)
// CTA tile 128 x 128 x 32, 8 warps as 2 x 4, warp tile 64 x 32, two-stage cp.async
// ---------------------------------------------------------------------------
constexpr int kGmBM = 128, kGmBN = 128, kGmBK = 32;
constexpr int kGmStride = kGmBK + 8;  // halves per shared-memory row (80 B: conflict-free fragment reads)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0 source bytes => 16 zero bytes written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__global__ void __launch_bounds__(256) gemm_xwt_kernel(const __half* __restrict__ x, int64_t rows,
                                                       int64_t x_stride, const __half* __restrict__ wt,
                                                       int M, int K, const __half* __restrict__ bias,
                                                       __half* __restrict__ y, int64_t y_stride) {
  __shared__ __align__(16) __half xs[2][kGmBM][kGmStride];
  __shared__ __align__(16) __half ws[2][kGmBN][kGmStride];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wr = warp >> 2, wc = warp & 3;  // 2 x 4 warps
  const int64_t row0 = (int64_t)blockIdx.y * kGmBM;
  const int col0 = blockIdx.x * kGmBN;

  float acc[4][4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

  auto load_stage = [&](int stage, int k0) {
    // 128 rows x 32 halves = 128 x 4 chunks of 16 B for each operand; 256 threads -> 2 + 2 chunks
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int idx = threadIdx.x + it * 256;
      const int r = idx >> 2, c = (idx & 3) * 8;
      const int64_t xr = row0 + r;
      const bool vx = xr < rows;
      cp_async16(&xs[stage][r][c], x + (vx ? xr : 0) * x_stride + k0 + c, vx);
      const int wrow = col0 + r;
      const bool vw = wrow < M;
      cp_async16(&ws[stage][r][c], wt + (int64_t)(vw ? wrow : 0) * K + k0 + c, vw);
    }
    cp_async_commit();
  };

  const int n_k = K / kGmBK;
  load_stage(0, 0);
  for (int kt = 0; kt < n_k; ++kt) {
    const int cur = kt & 1;
    if (kt + 1 < n_k) {
      load_stage(cur ^ 1, (kt + 1) * kGmBK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGmBK; kk += 16) {
      uint32_t a[4][4], b[4][2];
#pragma unroll
      for (int mi = 0; mi < 4; ++mi) {
        const int r = wr * 64 + mi * 16;
        a[mi][0] = *reinterpret_cast<const uint32_t*>(&xs[cur][r + g][kk + 2 * t]);
        a[mi][1] = *reinterpret_cast<const uint32_t*>(&xs[cur][r + g + 8][kk + 2 * t]);
        a[mi][2] = *reinterpret_cast<const uint32_t*>(&xs[cur][r + g][kk + 2 * t + 8]);
        a[mi][3] = *reinterpret_cast<const uint32_t*>(&xs[cur][r + g + 8][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int c = wc * 32 + ni * 8;
        b[ni][0] = *reinterpret_cast<const uint32_t*>(&ws[cur][c + g][kk + 2 * t]);
        b[ni][1] = *reinterpret_cast<const uint32_t*>(&ws[cur][c + g][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int mi = 0; mi < 4; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) mma_f16_16816(acc[mi][ni], a[mi], b[ni][0], b[ni][1]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int mi = 0; mi < 4; ++mi) {
#pragma unroll
    for (int ni = 0; ni < 4; ++ni) {
      const int c = col0 + wc * 32 + ni * 8 + 2 * t;
      if (c >= M) continue;  // M is a multiple of 8, so c+1 < M as well
      float b0 = 0.f, b1 = 0.f;
      if (bias) {
        b0 = __half2float(bias[c]);
        b1 = __half2float(bias[c + 1]);
      }
      const int64_t r_lo = row0 + wr * 64 + mi * 16 + g;
      if (r_lo < rows)
        *reinterpret_cast<__half2*>(y + r_lo * y_stride + c) =
            __floats2half2_rn(acc[mi][ni][0] + b0, acc[mi][ni][1] + b1);
      if (r_lo + 8 < rows)
        *reinterpret_cast<__half2*>(y + (r_lo + 8) * y_stride + c) =
            __floats2half2_rn(acc[mi][ni][2] + b0, acc[mi][ni][3] + b1);
    }
  }
}

}  // namespace

bool rebuild_supported(const bsb_weight& w) {
  return w.k == 16 && w.in_features % kRbCols == 0 && w.out_features % 16 == 0 &&
         ((uintptr_t)w.qweight % 8 == 0) && (w.q_block_stride % 8 == 0) &&
         ((uintptr_t)w.vt % 16 == 0) && (w.vt_block_stride % 8 == 0) &&
         ((uintptr_t)w.u % 4 == 0) && (w.u_block_stride % 2 == 0);
}

int launch_rebuild_weight(const bsb_weight& w, __half* w_out, cudaStream_t s) {
  BSB_CHECK_ARG(rebuild_supported(w), "rebuild: unsupported shape/alignment (out=%d in=%d k=%d)",
                w.out_features, w.in_features, w.k);
  BSB_CHECK_ARG((uintptr_t)w_out % 4 == 0, "rebuild: output must be 4-byte aligned");
  dim3 grid(w.in_features / kRbCols, (unsigned)ceil_div64(w.out_features, kRbRowsPerCta * kRbRowTiles));
  rebuild_weight_kernel<<<grid, 256, 0, s>>>(w, w_out);
  return check_launch("rebuild_weight_kernel");
}

bool gemm_supported(int64_t rows, int out_features, int in_features) {
  return rows > 0 && in_features % kGmBK == 0 && out_features % 8 == 0;
}

int launch_gemm_xwt(const __half* x, int64_t rows, int64_t x_stride, const __half* w, int out_features,
                    int in_features, const __half* bias, __half* y, int64_t y_stride, cudaStream_t s) {
  BSB_CHECK_ARG(gemm_supported(rows, out_features, in_features), "gemm: unsupported shape");
  BSB_CHECK_ARG((uintptr_t)x % 16 == 0 && x_stride % 8 == 0 && (uintptr_t)w % 16 == 0,
                "gemm: x and W must be 16-byte aligned with row strides that are multiples of 8");
  BSB_CHECK_ARG((uintptr_t)y % 4 == 0 && y_stride % 2 == 0, "gemm: y must be 4-byte aligned, even stride");
  const int64_t gy = ceil_div64(rows, kGmBM);
  BSB_CHECK_ARG(gy <= 65535, "gemm: too many rows (%lld)", (long long)rows);
  dim3 grid((unsigned)ceil_div64(out_features, kGmBN), (unsigned)gy);
  gemm_xwt_kernel<<<grid, 256, 0, s>>>(x, rows, x_stride, w, out_features, in_features, bias, y, y_stride);
  return check_launch("gemm_xwt_kernel");
}

}  // namespace bsb
