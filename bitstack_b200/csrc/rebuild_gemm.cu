// Batch / prefill path, first generation: rebuild the fp16 weight from the packed
// blocks (rank-16 products on the tensor cores rounded to fp16, signs applied to packed
// pairs in registers, fp16 sum over blocks like the reference), then a dense x.W^T contraction.
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

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// rank-16 product with fp16 accumulators, from zero: the two result registers are the rounded products of rows g and
// g + 8, columns 2t, 2t+1 of the 8-column tile, packed as pairs
__device__ __forceinline__ void mma_f16_16816_h(uint32_t (&d)[2], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8};\n"
      : "=r"(d[0]), "=r"(d[1])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0u));
}

// p ^ (~bits & 0x80008000): flips the signs of the packed pair `p` where bit 31 / bit 15 of `bits` is clear
__device__ __forceinline__ uint32_t sign_pair(uint32_t p, uint32_t bits) {
  uint32_t out;
  // minterms of a ^ (~b & c) over (a, b, c) with a = 0xF0, b = 0xCC, c = 0xAA: 0xF0 ^ (0x33 & 0xAA) = 0xD2
  asm("lop3.b32 %0, %1, %2, %3, 0xD2;" : "=r"(out) : "r"(p), "r"(bits), "r"(0x80008000u));
  return out;
}

// ---------------------------------------------------------------------------
// rebuild: CTA = 8 warps = 128 rows x 64 columns of W; warp = 16 rows x 64 cols
// ---------------------------------------------------------------------------
// The sign stage works on PAIRS: the staged Vt slab has the columns of every 32-group in the order
// (16, 0, 17, 1, ..., 31, 15), so an accumulator register of the product holds columns 16 + k (low half) and k (high
// half) of the group; the byte-swapped sign word of the group shifted left by k has exactly those two sign bits at
// bits 15 and 31: one shift, one LOP3 and one packed add per pair and block.  The sum over blocks is taken in fp16,
// block after block, as the reference's own reconstruction does (bitstack/modules/BitStackLinear.py:7-15,88-100).
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

  __half2 acc[8][2];           // [8-position tile of the permuted order][row g / g + 8]
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = __float2half2_rn(0.f);

  // blocks are added from the last to the first: later blocks approximate ever smaller residuals, so the fp16
  // running sum stays small until the dominant first blocks arrive and is rounded at full magnitude only then
  for (int j0 = ((w.blocks - 1) / kRbBlockGroup) * kRbBlockGroup; j0 >= 0; j0 -= kRbBlockGroup) {
    const int nj = min(kRbBlockGroup, w.blocks - j0);
    if (nj <= 0) break;   // no active block: W = 0
    if (rt == 0 || !one_group) {
    __syncthreads();  // previous group fully consumed
    // stage Vt[j0..j0+nj)[0..16)[n0..n0+64) in the pair order: a thread takes columns 8h..8h+7 and 16+8h..16+8h+7 of
    // a 32-group and writes them interleaved (positions 16h .. 16h+15 of the group)
    for (int i = threadIdx.x; i < nj * 16 * 4; i += blockDim.x) {
      const int jj = i / 64, rem = i % 64;
      const int r = rem / 4, grp = (rem >> 1) & 1, h = rem & 1;
      const __half* src = vt_all + (int64_t)(j0 + jj) * w.vt_block_stride + (int64_t)r * N + n0 + grp * 32 + h * 8;
      const uint4 lo = __ldg(reinterpret_cast<const uint4*>(src));        // columns k = 8h .. 8h+7      -> odd positions
      const uint4 hi = __ldg(reinterpret_cast<const uint4*>(src + 16));   // columns 16 + k              -> even positions
      uint4 o0, o1;
      o0.x = __byte_perm(hi.x, lo.x, 0x5410); o0.y = __byte_perm(hi.x, lo.x, 0x7632);
      o0.z = __byte_perm(hi.y, lo.y, 0x5410); o0.w = __byte_perm(hi.y, lo.y, 0x7632);
      o1.x = __byte_perm(hi.z, lo.z, 0x5410); o1.y = __byte_perm(hi.z, lo.z, 0x7632);
      o1.z = __byte_perm(hi.w, lo.w, 0x5410); o1.w = __byte_perm(hi.w, lo.w, 0x7632);
      uint4* dst = reinterpret_cast<uint4*>(&vt_s[jj][r][grp * 32 + h * 16]);
      dst[0] = o0;
      dst[1] = o1;
    }
    __syncthreads();
    }
    if (!active) continue;

    // operands of a block that come straight from global memory (A fragment of U_j: rows m0+g /
    // m0+g+8, ranks 2t,2t+1 / 2t+8,2t+9; 64 sign bits of the two rows) are fetched one block ahead
    const __half* u_j = u_all + (int64_t)(j0 + nj - 1) * w.u_block_stride + (int64_t)(m0 + g) * 16 + 2 * t;
    const uint8_t* q_j = w.qweight + (int64_t)(j0 + nj - 1) * w.q_block_stride + ((int64_t)(m0 + g) * N + n0) / 8;
    auto fetch = [&](const __half* u, const uint8_t* q, uint32_t (&af)[4], uint2& lo, uint2& hi) {
      af[0] = __ldg(reinterpret_cast<const uint32_t*>(u));
      af[1] = __ldg(reinterpret_cast<const uint32_t*>(u + 8 * 16));
      af[2] = __ldg(reinterpret_cast<const uint32_t*>(u + 8));
      af[3] = __ldg(reinterpret_cast<const uint32_t*>(u + 8 * 16 + 8));
      lo = __ldg(reinterpret_cast<const uint2*>(q));
      hi = __ldg(reinterpret_cast<const uint2*>(q + N));   // 8 rows further
    };
    uint32_t a_next[4];
    uint2 lo_next, hi_next;
    fetch(u_j, q_j, a_next, lo_next, hi_next);
#pragma unroll 1
    for (int jj = nj - 1; jj >= 0; --jj) {
      const uint32_t a[4] = {a_next[0], a_next[1], a_next[2], a_next[3]};
      // byte swap: column c of a 32-group -> bit 31 - c; the shift by t selects this thread's pair of every tile
      const uint32_t wg[2] = {__byte_perm(lo_next.x, 0, 0x0123) << t, __byte_perm(lo_next.y, 0, 0x0123) << t};
      const uint32_t wh[2] = {__byte_perm(hi_next.x, 0, 0x0123) << t, __byte_perm(hi_next.y, 0, 0x0123) << t};
      u_j -= w.u_block_stride;
      q_j -= w.q_block_stride;
      if (jj > 0) fetch(u_j, q_j, a_next, lo_next, hi_next);
#pragma unroll
      for (int pair = 0; pair < 4; ++pair) {  // two 8-position tiles per ldmatrix.x4
        uint32_t b[4];
        // lanes 0-7: ranks 0-7 @ tile 2*pair; 8-15: ranks 8-15 @ same tile;
        // 16-23 / 24-31: the same for tile 2*pair+1
        const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int col = (2 * pair + (lane >> 4)) * 8;
        ldmatrix_x4_trans(b, &vt_s[jj][row][col]);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int i = 2 * pair + h;          // tile i: positions 8i + 2t, 8i + 2t + 1 = pair k = 4 (i % 4) + t of group i / 4
          uint32_t d[2];
          mma_f16_16816_h(d, a, b[2 * h], b[2 * h + 1]);
          const int sh = 4 * (i & 3);
          const uint32_t s0 = sign_pair(d[0], wg[i >> 2] << sh), s1 = sign_pair(d[1], wh[i >> 2] << sh);
          acc[i][0] = __hadd2(acc[i][0], *reinterpret_cast<const __half2*>(&s0));
          acc[i][1] = __hadd2(acc[i][1], *reinterpret_cast<const __half2*>(&s1));
        }
      }
    }
  }
  if (!active) continue;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // a register holds column 16 + k (low half) and column k (high half) of the 32-group, k = 4 (i % 4) + t.  Lanes
    // t and t ^ 1 swap halves so that the even lane ends up with columns k, k + 1 and the odd one with 16 + k - 1,
    // 16 + k: every store is an aligned pair of adjacent columns again
    const int k = 4 * (i & 3) + t;
    const int n = n0 + (i >> 2) * 32 + ((t & 1) ? 16 + k - 1 : k);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(&acc[i][h]);
      const uint32_t p = __shfl_xor_sync(0xFFFFFFFFu, v, 1);
      const uint32_t o = (t & 1) ? __byte_perm(v, p, 0x1054) : __byte_perm(v, p, 0x7632);
      *reinterpret_cast<uint32_t*>(out + (int64_t)(m0 + g + 8 * h) * N + n) = o;
    }
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
