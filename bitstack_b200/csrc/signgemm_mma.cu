// Batch path for 7 .. 64 input rows, register-resident variant of the fused sign-GEMM (signgemm_tc5.cu has the
// math and the tcgen05 variant): the weight is never written to memory.
//
// Replaces, for small batches, the reconstruct-then-multiply structure of the reference's fused levels
// (bitstack/modules/BitStackLinear.py:116-148; bitstack/utils/inference_utils.py:286-387).
//
// Per warp: 16 rows of W.  Per (64-column chunk, block j):
//   MMA 1   P = U_j[16 rows] . Vt_j[chunk]            warp-level m16n8k16 MMAs with fp16 accumulators: the result is
//           the fp16 W tile the reference rounds its products to, as packed pairs in registers
//   sign    the accumulator fragment of MMA 1 IS the A fragment of the next MMA; each pair is signed with one LOP3
//           against the shifted sign word (pairing trick: the K order inside every 32-column group is
//           (16, 0, 17, 1, ..., 31, 15), so the two sign bits of a pair sit 16 apart in the byte-swapped word)
//   MMA 2   D[16 rows][T] += A . x'[chunk]^T          fp32 accumulation over chunks and blocks in registers
// Nothing goes through shared or tensor memory between the two MMAs, which is what the step needs: it is bound by
// the instructions per (element, block) of the sign stage and the legacy tensor pipe, not by memory -- the
// tcgen05 variant pays a tensor-memory round trip per step and is slower on these shapes (measured, see the
// batch-path notes).  Vt (column-permuted) and x' chunks are staged in shared memory with cp.async, double buffered.
// A CTA = 8 warps = 128 rows x a K range (split-K over CTAs); fp32 partials are added in split order by a last
// kernel (deterministic), which adds the bias and rounds once.
#include "common.cuh"

namespace bsb {

namespace {

constexpr int kRowsPerCta = 128;
constexpr int kChunk = 64;
constexpr int kPad = 8;                      // halves of padding per staged row: conflict-free fragment reads
constexpr int kRowHalves = kChunk + kPad;
constexpr int kMaxRows = 64;
constexpr int kSmemLimit = 200 * 1024;

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// a rank-16 product with fp16 accumulators, from zero: the two result registers are the rounded pairs (row g | row g + 8,
// columns 2t, 2t+1), i.e. already one half of the next MMA's A fragment
__device__ __forceinline__ void mma_f16_16816_h(uint32_t (&d)[2], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%8,%8};\n"
      : "=r"(d[0]), "=r"(d[1])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0u));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(addr), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
// a packed pair with both signs flipped where bit 31 / bit 15 of `bits` is CLEAR
__device__ __forceinline__ uint32_t sign_pair(uint32_t p, uint32_t bits) {
  uint32_t out;
  asm("lop3.b32 %0, %1, %2, %3, 0xD2;" : "=r"(out) : "r"(p), "r"(bits), "r"(0x80008000u));   // p ^ (~bits & mask)
  return out;
}

struct SgmParams {
  bsb_weight w;
  const __half* vtp;     // [blocks][16][in], columns of every 32-group in the order (16, 0, 17, 1, ..., 31, 15)
  const __half* xp;      // [tpad][in], same column order; rows past the batch are zero
  float* partials;       // [splits][tpad][out]
  int n_chunks, splits, tpad;
};

// VtP and x' (the column order of the pairing trick)
__global__ void __launch_bounds__(256) sgm_prep_kernel(bsb_weight w, const __half* __restrict__ x, int64_t x_stride, int rows, int tpad,
                                                       __half* __restrict__ vtp, __half* __restrict__ xp) {
  const int N = w.in_features;
  const __half* vt = reinterpret_cast<const __half*>(w.vt);
  const int64_t pairs_row = N / 2;
  const int64_t total_v = (int64_t)w.blocks * 16 * pairs_row, total_x = (int64_t)tpad * pairs_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_v + total_x; i += stride) {
    const bool is_v = i < total_v;
    const int64_t k = is_v ? i : i - total_v;
    const int64_t r = k / pairs_row;                       // (block, rank) row of Vt, or input row
    const int pr = (int)(k % pairs_row), grp = pr / 16, ii = pr % 16;
    __half lo = __float2half(0.f), hi = lo;
    if (is_v) {
      const int j = (int)(r / 16), rank = (int)(r % 16);
      const __half* src = vt + (int64_t)j * w.vt_block_stride + (int64_t)rank * N + grp * 32 + ii;
      lo = src[16];
      hi = src[0];
      reinterpret_cast<__half2*>(vtp + r * N)[pr] = __halves2half2(lo, hi);
    } else {
      if (r < rows) {
        const __half* src = x + r * x_stride + grp * 32 + ii;
        lo = src[16];
        hi = src[0];
      }
      reinterpret_cast<__half2*>(xp + r * N)[pr] = __halves2half2(lo, hi);
    }
  }
}

// TN = 8-token tiles of the batch (tpad / 8)
template <int TN>
__global__ void __launch_bounds__(256) signgemm_mma_kernel(const SgmParams P) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const bsb_weight& w = P.w;
  const int nb = w.blocks, N = w.in_features, M = w.out_features;
  const int vt_buf_halves = nb * 16 * kRowHalves, x_buf_halves = P.tpad * kRowHalves;
  __half* vt_s = reinterpret_cast<__half*>(smem_raw);                 // [2][nb][16][72]
  __half* x_s = vt_s + 2 * vt_buf_halves;                             // [2][tpad][72]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int m0 = blockIdx.x * kRowsPerCta + warp * 16;
  const bool active = m0 < M;                                         // out_features is a multiple of 16
  const int c_begin = (int)((int64_t)P.n_chunks * blockIdx.y / P.splits);
  const int c_end = (int)((int64_t)P.n_chunks * (blockIdx.y + 1) / P.splits);

  auto load_chunk = [&](int buf, int c) {
    __half* vd = vt_s + buf * vt_buf_halves;
    for (int i = threadIdx.x; i < nb * 16 * 8; i += blockDim.x) {
      const int row = i >> 3, c8 = i & 7;                             // row = block * 16 + rank
      cp_async16(vd + row * kRowHalves + c8 * 8, P.vtp + (int64_t)row * N + c * kChunk + c8 * 8);
    }
    __half* xd = x_s + buf * x_buf_halves;
    for (int i = threadIdx.x; i < P.tpad * 8; i += blockDim.x) {
      const int row = i >> 3, c8 = i & 7;
      cp_async16(xd + row * kRowHalves + c8 * 8, P.xp + (int64_t)row * N + c * kChunk + c8 * 8);
    }
    cp_async_commit();
  };

  float acc[TN][4];
#pragma unroll
  for (int i = 0; i < TN; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = 0.f;

  const __half* u_all = reinterpret_cast<const __half*>(w.u);
  // operands of a block that come straight from global memory: the A fragment of U_j (rows m0+g / m0+g+8, ranks
  // 2t,2t+1 / 2t+8,2t+9) and the 64 sign bits of the two rows for this chunk
  const __half* u_thr = u_all + (int64_t)(m0 + g) * 16 + 2 * t;          // this thread's first U pair of block 0
  const uint8_t* q_thr = w.qweight + (int64_t)(m0 + g) * (N / 8);          // this thread's first sign row of block 0
  auto fetch = [&](const __half* u, const uint8_t* q, uint32_t (&af)[4], uint2& lo, uint2& hi) {
    af[0] = __ldg(reinterpret_cast<const uint32_t*>(u));
    af[1] = __ldg(reinterpret_cast<const uint32_t*>(u + 8 * 16));
    af[2] = __ldg(reinterpret_cast<const uint32_t*>(u + 8));
    af[3] = __ldg(reinterpret_cast<const uint32_t*>(u + 8 * 16 + 8));
    lo = __ldg(reinterpret_cast<const uint2*>(q));
    hi = __ldg(reinterpret_cast<const uint2*>(q + N));                     // 8 rows further: 8 * N / 8 bytes
  };

  if (c_begin < c_end) load_chunk(0, c_begin);
  for (int c = c_begin; c < c_end; ++c) {
    const int cur = (c - c_begin) & 1;
    if (c + 1 < c_end) {
      load_chunk(cur ^ 1, c + 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (active) {
      const __half* vs = vt_s + cur * vt_buf_halves;
      const __half* xs = x_s + cur * x_buf_halves;
      // B fragments of x' for the whole chunk when they fit in registers (<= 16 tokens), else fetched per slab
      uint32_t xb[TN <= 2 ? 4 : 1][TN][2];
      if (TN <= 2) {
#pragma unroll
        for (int p = 0; p < 4; ++p)
#pragma unroll
          for (int nt = 0; nt < TN; ++nt) {
            xb[p][nt][0] = *reinterpret_cast<const uint32_t*>(xs + (8 * nt + g) * kRowHalves + 16 * p + 2 * t);
            xb[p][nt][1] = *reinterpret_cast<const uint32_t*>(xs + (8 * nt + g) * kRowHalves + 16 * p + 2 * t + 8);
          }
      }
      uint32_t a_next[4];
      uint2 lo_next, hi_next;
      const __half* u_j = u_thr;
      const uint8_t* q_j = q_thr + c * (kChunk / 8);
      fetch(u_j, q_j, a_next, lo_next, hi_next);
#pragma unroll 1
      for (int j = 0; j < nb; ++j) {
        const uint32_t a[4] = {a_next[0], a_next[1], a_next[2], a_next[3]};
        // byte swap: column c of a 32-group -> bit 31 - c; the shift by t selects this thread's pair of every 8-column tile
        const uint32_t wg[2] = {__byte_perm(lo_next.x, 0, 0x0123) << t, __byte_perm(lo_next.y, 0, 0x0123) << t};
        const uint32_t wh[2] = {__byte_perm(hi_next.x, 0, 0x0123) << t, __byte_perm(hi_next.y, 0, 0x0123) << t};
        u_j += w.u_block_stride;
        q_j += w.q_block_stride;
        if (j + 1 < nb) fetch(u_j, q_j, a_next, lo_next, hi_next);
        const __half* vj = vs + j * 16 * kRowHalves;
#pragma unroll
        for (int p = 0; p < 4; ++p) {   // 16 K positions of MMA 2 = two 8-column tiles of MMA 1
          uint32_t b[4];
          // lanes 0-7: ranks 0-7 @ tile 2p; 8-15: ranks 8-15 @ same tile; 16-23 / 24-31: the same for tile 2p+1
          ldmatrix_x4_trans(b, vj + ((lane & 7) + ((lane >> 3) & 1) * 8) * kRowHalves + (2 * p + (lane >> 4)) * 8);
          uint32_t d0[2], d1[2];
          mma_f16_16816_h(d0, a, b[0], b[1]);
          mma_f16_16816_h(d1, a, b[2], b[3]);
          // pair index inside the 32-group = 4 (tile % 4) + t: the words are pre-shifted by t
          const int sh = (p & 1) * 8;
          const uint32_t sg = wg[p >> 1], sh2 = wh[p >> 1];
          uint32_t a2[4];
          a2[0] = sign_pair(d0[0], sg << sh);          // row g,     K 2t, 2t+1
          a2[1] = sign_pair(d0[1], sh2 << sh);         // row g + 8
          a2[2] = sign_pair(d1[0], sg << (sh + 4));    // row g,     K 2t+8, 2t+9
          a2[3] = sign_pair(d1[1], sh2 << (sh + 4));   // row g + 8
#pragma unroll
          for (int nt = 0; nt < TN; ++nt) {
            uint32_t b0, b1;
            if (TN <= 2) {
              b0 = xb[p][nt][0];
              b1 = xb[p][nt][1];
            } else {
              b0 = *reinterpret_cast<const uint32_t*>(xs + (8 * nt + g) * kRowHalves + 16 * p + 2 * t);
              b1 = *reinterpret_cast<const uint32_t*>(xs + (8 * nt + g) * kRowHalves + 16 * p + 2 * t + 8);
            }
            mma_f16_16816(acc[nt], a2, b0, b1);
          }
        }
      }
    }
    __syncthreads();
  }
  if (!active) return;
  float* part = P.partials + (int64_t)blockIdx.y * P.tpad * M;
#pragma unroll
  for (int nt = 0; nt < TN; ++nt) {
    const int tok = 8 * nt + 2 * t;
    part[(int64_t)tok * M + m0 + g] = acc[nt][0];
    part[(int64_t)(tok + 1) * M + m0 + g] = acc[nt][1];
    part[(int64_t)tok * M + m0 + g + 8] = acc[nt][2];
    part[(int64_t)(tok + 1) * M + m0 + g + 8] = acc[nt][3];
  }
}

__global__ void __launch_bounds__(256) sgm_reduce_kernel(const float* __restrict__ partials, int splits, int tpad, int M, int rows,
                                                         const __half* __restrict__ bias, __half* __restrict__ y, float* __restrict__ y32,
                                                         int64_t y_stride) {
  const int64_t total = (int64_t)rows * M;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / M), m = (int)(i % M);
    float s = 0.f;
    for (int q = 0; q < splits; ++q) s += partials[((int64_t)q * tpad + t) * M + m];
    if (bias) s += __half2float(bias[m]);
    if (y32) y32[(int64_t)t * y_stride + m] = s;
    else y[(int64_t)t * y_stride + m] = __float2half_rn(s);
  }
}

struct SgmPlan {
  int tpad, tn, tiles, n_chunks, splits, smem;
  int64_t vtp_off, x_off, part_off, bytes;
};

void make_plan(const bsb_weight& w, int64_t rows, SgmPlan& pl) {
  pl.tpad = rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
  pl.tn = pl.tpad / 8;
  pl.tiles = (int)ceil_div64(w.out_features, kRowsPerCta);
  pl.n_chunks = w.in_features / kChunk;
  // about five CTAs per multiprocessor's worth of work items when the K extent allows: CTAs are small (8 warps)
  int s = (int)ceil_div64((int64_t)sm_count() * 5, pl.tiles);
  if (s > pl.n_chunks / 2) s = pl.n_chunks / 2;
  if (s < 1) s = 1;
  pl.splits = s;
  pl.smem = 2 * (w.blocks * 16 + pl.tpad) * kRowHalves * 2;
  int64_t off = 0;
  pl.vtp_off = off;
  off = align_up64(off + (int64_t)w.blocks * 16 * w.in_features * 2, 256);
  pl.x_off = off;
  off = align_up64(off + (int64_t)pl.tpad * w.in_features * 2, 256);
  pl.part_off = off;
  off = align_up64(off + (int64_t)pl.splits * pl.tpad * w.out_features * 4, 256);
  pl.bytes = off;
}

}  // namespace

bool signgemm_mma_supported(const bsb_weight& w, int64_t rows) {
  if (!(rows >= 1 && rows <= kMaxRows && w.k == 16 && w.blocks >= 1 && w.in_features >= 64 && w.in_features % 64 == 0 &&
        w.out_features >= 16 && w.out_features % 16 == 0 && ((uintptr_t)w.qweight % 8 == 0) &&
        (w.blocks == 1 || w.q_block_stride % 8 == 0) && ((uintptr_t)w.u % 4 == 0) && (w.blocks == 1 || w.u_block_stride % 2 == 0)))
    return false;
  SgmPlan pl;
  make_plan(w, rows, pl);
  return pl.smem <= kSmemLimit;
}

int64_t signgemm_mma_workspace_bytes(const bsb_weight& w, int64_t rows) {
  SgmPlan pl;
  make_plan(w, rows, pl);
  return pl.bytes;
}

// exactly one of y (fp16) and y32 (fp32 partial sums of a tensor-parallel shard) is non-null
int launch_signgemm_mma(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride, __half* y, float* y32, int64_t y_stride,
                        void* workspace, int64_t workspace_bytes, cudaStream_t s) {
  BSB_CHECK_ARG(signgemm_mma_supported(w, rows), "fused sign-GEMM: unsupported shape/alignment (out=%d in=%d k=%d blocks=%d rows=%lld)",
                w.out_features, w.in_features, w.k, w.blocks, (long long)rows);
  BSB_CHECK_ARG((y != nullptr) != (y32 != nullptr), "fused sign-GEMM: exactly one of the fp16 and the fp32 output");
  SgmPlan pl;
  make_plan(w, rows, pl);
  if (workspace == nullptr || workspace_bytes < pl.bytes) {
    set_error("fused sign-GEMM: workspace of %lld bytes needed, %lld given", (long long)pl.bytes, (long long)workspace_bytes);
    return BSB_EWORKSPACE;
  }
  BSB_CHECK_ARG((uintptr_t)workspace % 256 == 0, "fused sign-GEMM: workspace must be 256-byte aligned");
  uint8_t* base = (uint8_t*)workspace;
  SgmParams P;
  P.w = w;
  P.vtp = (const __half*)(base + pl.vtp_off);
  P.xp = (const __half*)(base + pl.x_off);
  P.partials = (float*)(base + pl.part_off);
  P.n_chunks = pl.n_chunks;
  P.splits = pl.splits;
  P.tpad = pl.tpad;
  {
    const int64_t work = ((int64_t)w.blocks * 16 + pl.tpad) * (w.in_features / 2);
    const int blocks = (int)min((int64_t)sm_count() * 8, ceil_div64(work, 256));
    sgm_prep_kernel<<<blocks, 256, 0, s>>>(w, x, x_stride, (int)rows, pl.tpad, (__half*)(base + pl.vtp_off), (__half*)(base + pl.x_off));
    if (int rc = check_launch("sgm_prep_kernel")) return rc;
  }
  static bool attr_set[64] = {false};
  int dev = 0;
  BSB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    BSB_CUDA(cudaFuncSetAttribute(signgemm_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    BSB_CUDA(cudaFuncSetAttribute(signgemm_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    BSB_CUDA(cudaFuncSetAttribute(signgemm_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    attr_set[dev] = true;
  }
  const dim3 grid(pl.tiles, pl.splits);
  if (pl.tn == 2) signgemm_mma_kernel<2><<<grid, 256, pl.smem, s>>>(P);
  else if (pl.tn == 4) signgemm_mma_kernel<4><<<grid, 256, pl.smem, s>>>(P);
  else signgemm_mma_kernel<8><<<grid, 256, pl.smem, s>>>(P);
  if (int rc = check_launch("signgemm_mma_kernel")) return rc;
  {
    const int64_t total = rows * w.out_features;
    const int blocks = (int)min((int64_t)sm_count() * 8, ceil_div64(total, 256));
    sgm_reduce_kernel<<<blocks, 256, 0, s>>>(P.partials, pl.splits, pl.tpad, w.out_features, (int)rows,
                                             reinterpret_cast<const __half*>(w.bias), y, y32, y_stride);
  }
  return check_launch("sgm_reduce_kernel");
}

}  // namespace bsb
