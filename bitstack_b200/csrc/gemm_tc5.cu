// Batch / prefill GEMM on the 5th-generation tensor cores:
//     y[rows][out] = x[rows][in] . W[out][in]^T (+ bias),  fp16 operands, fp32 accumulation.
// W is the fp16 weight rebuilt from the BitStack blocks (rebuild_gemm.cu); this replaces the
// F.linear call of the reference's non-fused forward (bitstack/modules/BitStackLinear.py:105-114)
// for inputs of more than a few rows.
//
// CTA tile: 128 input rows (MMA M, one tensor-memory lane per row) x BN output features (MMA N,
// one fp32 tensor-memory column each), K in steps of 64 (128 bytes of fp16 = one swizzle span).
// Both operands are K-major in global memory, so each stage is two tiled TMA loads
// (cp.async.bulk.tensor.2d, 128-byte swizzle, no multicast) straight into the UMMA canonical
// layout.  Roles: warp 0 = TMA producer (one lane), warp 1 = tensor-memory allocation + MMA issue
// (tcgen05.mma.kind::f16, one elected lane, tcgen05.commit releases stages), warps 2-5 =
// epilogue (tcgen05.ld -> bias -> fp16 -> 16-byte stores; y is row-major with the token row on
// the tensor-memory lane, so every thread writes contiguous bytes of its own row).  CTAs are
// persistent (one per multiprocessor) with two accumulator buffers in tensor memory, so the
// epilogue of a tile overlaps the main loop of the next one.
// All waits are time-bounded; a wait that gives up sets the status word and the CTA leaves.
#include <cuda.h>

#include "common.cuh"

namespace bsb {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;                       // fp16 elements per K step (128 bytes)
constexpr int kThreads = 192;
constexpr int kSmemBudget = 200 * 1024;
constexpr uint64_t kWaitLimitNs = 200ull * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// time-bounded wait; false = gave up
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity) {
  const uint64_t t0 = global_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_test(bar, parity)) return true;
      __nanosleep(64);
    }
    if (global_ns() - t0 > kWaitLimitNs) return false;
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 128; ++i)
    if (mbar_test(bar, parity)) return true;
  return mbar_wait_slow(bar, parity);
}
__device__ __forceinline__ bool elect_one() {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xFFFFFFFF;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok));
  return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]^T, fp16 x fp16 -> fp32, M = 128, K = 16
__device__ __forceinline__ void mma_ss_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                       // leading byte offset: unused with a swizzled K-major tile
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                       // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

struct alignas(64) GemmParams {
  CUtensorMap map_x;   // fp16 [rows][in], box 64 x 128
  CUtensorMap map_w;   // fp16 [out][in], box 64 x BN
  const __half* bias;
  __half* y;           // fp16 output, or
  float* y32;          // fp32 output (partial sums of a tensor-parallel shard): exactly one of the two is set
  int64_t y_stride;
  int rows, out_features, in_features;
  int* status;         // the library's sticky status word: the first wait that gives up leaves its code there
};

template <int BN>
struct GemmSmem {
  static constexpr int kStageBytes = kBM * kBK * 2 + BN * kBK * 2;
  static constexpr int kStages = (kSmemBudget / kStageBytes) > 8 ? 8 : (kSmemBudget / kStageBytes);
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc5_kernel(const __grid_constant__ GemmParams P) {
  constexpr int kStages = GemmSmem<BN>::kStages;
  constexpr int kABytes = kBM * kBK * 2, kBBytes = BN * kBK * 2;
  constexpr int kAcc = (2 * BN <= 512) ? 2 : 1;      // accumulator buffers in tensor memory
  constexpr int kTmemCols = (kAcc * BN < 32) ? 32 : kAcc * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sa = base;                               // [stage][128 rows][128 B]
  uint8_t* sb = base + kStages * kABytes;            // [stage][BN rows][128 B]
  uint64_t* full = reinterpret_cast<uint64_t*>(sb + kStages * kBBytes);
  uint64_t* empty = full + kStages;
  uint64_t* dfull = empty + kStages;                 // [kAcc] accumulator complete
  uint64_t* dempty = dfull + 2;                      // [kAcc] accumulator read out by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dempty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int k_steps = (P.in_features + kBK - 1) / kBK;
  // Persistent CTAs walk the tiles output-column-major: consecutive tiles (and the CTAs of one wave)
  // share a W tile and differ in the row tile, so W comes from DRAM once and x stays in L2.
  const int row_tiles = (P.rows + kBM - 1) / kBM;
  const int col_tiles = (P.out_features + BN - 1) / BN;
  const int n_tiles = row_tiles * col_tiles;

  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < kAcc; ++i) { mbar_init(&dfull[i], 1); mbar_init(&dempty[i], 128); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ------------------------------------------------------------------
    if (lane == 0) {
      int it = 0;                                    // stages filled so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % row_tiles) * kBM, n0 = (tile / row_tiles) * BN;
        for (int k = 0; k < k_steps; ++k, ++it) {
          const int s = it % kStages, n = it / kStages;
          if (n >= 1 && !mbar_wait(&empty[s], (n - 1) & 1)) { if (P.status) atomicCAS(P.status, 0, 21); ok = false; break; }
          mbar_expect_tx(&full[s], kABytes + kBBytes);
          // rows and K past the end of a tensor read as zeros
          tma_load_2d(sa + s * kABytes, &P.map_x, k * kBK, m0, &full[s]);
          tma_load_2d(sb + s * kBBytes, &P.map_w, k * kBK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the warp runs the loop uniformly, one elected lane issues -------------
    const bool leader = elect_one();
    const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);   // f16 x f16 -> f32, K-major
    bool ok = true;
    int it = 0, t_idx = 0;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t_idx) {
      const int ab = t_idx % kAcc, use = t_idx / kAcc;
      // the epilogue must have emptied this accumulator (its use before this one)
      if (use >= 1 && !mbar_wait(&dempty[ab], (use - 1) & 1)) { if (leader && P.status) atomicCAS(P.status, 0, 24); ok = false; break; }
      tc_fence_after();
      const uint32_t dcol = tbase + ab * BN;
      for (int k = 0; k < k_steps; ++k, ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&full[s], (it / kStages) & 1)) { if (leader && P.status) atomicCAS(P.status, 0, 22); ok = false; break; }
        tc_fence_after();
        if (leader) {
          const uint64_t adesc = make_desc_sw128(smem_u32(sa + s * kABytes));
          const uint64_t bdesc = make_desc_sw128(smem_u32(sb + s * kBBytes));
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk)   // 16 elements = 32 bytes further along the swizzled row
            mma_ss_f16(dcol, adesc + 2 * kk, bdesc + 2 * kk, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          mma_commit(&empty[s]);
        }
      }
      if (leader && ok) mma_commit(&dfull[ab]);
    }
  } else {
    // ---- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. +31 = input rows -----------
    const int quarter = warp & 3;
    const uint32_t lane_base = tbase + ((uint32_t)(quarter * 32) << 16);
    int t_idx = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t_idx) {
      const int m0 = (tile % row_tiles) * kBM, n0 = (tile / row_tiles) * BN;
      const int ab = t_idx % kAcc, use = t_idx / kAcc;
      const int row = m0 + quarter * 32 + lane;
      bool ok = mbar_wait(&dfull[ab], use & 1);
      ok = __all_sync(0xFFFFFFFFu, ok ? 1 : 0) != 0;
      if (!ok) {
        if (lane == 0 && P.status) atomicCAS(P.status, 0, 23);
        // this tile and the CTA's remaining ones are marked NaN: a timed-out call must not pass for a result
        const uint32_t nan2 = 0x7E007E00u;
        for (int t2 = tile; t2 < n_tiles; t2 += gridDim.x) {
          const int r2 = (t2 % row_tiles) * kBM + quarter * 32 + lane, c2 = (t2 / row_tiles) * BN;
          if (r2 < P.rows)
            for (int n = c2; n < min(c2 + BN, P.out_features); n += 8) {
              if (P.y32) {
                const float qn = __int_as_float(0x7FC00000);
                *reinterpret_cast<float4*>(P.y32 + (int64_t)r2 * P.y_stride + n) = make_float4(qn, qn, qn, qn);
                *reinterpret_cast<float4*>(P.y32 + (int64_t)r2 * P.y_stride + n + 4) = make_float4(qn, qn, qn, qn);
              } else {
                *reinterpret_cast<uint4*>(P.y + (int64_t)r2 * P.y_stride + n) = make_uint4(nan2, nan2, nan2, nan2);
              }
            }
        }
        break;
      }
      tc_fence_after();
      __half* yrow = P.y + (int64_t)row * P.y_stride;
      float* yrow32 = P.y32 + (int64_t)row * P.y_stride;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t d[32];
        tmem_ld32(lane_base + ab * BN + c, d);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (row < P.rows) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {          // 8 output features = one 16-byte store
            const int n = n0 + c + v * 8;
            if (n < P.out_features) {           // out_features is a multiple of 8
              uint4 out;
              __half2* o = reinterpret_cast<__half2*>(&out);
              float f[8];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float a = __uint_as_float(d[v * 8 + 2 * q]), b = __uint_as_float(d[v * 8 + 2 * q + 1]);
                if (P.bias) {
                  a += __half2float(P.bias[n + 2 * q]);
                  b += __half2float(P.bias[n + 2 * q + 1]);
                }
                o[q] = __floats2half2_rn(a, b);
                f[2 * q] = a;
                f[2 * q + 1] = b;
              }
              if (P.y32) {
                *reinterpret_cast<float4*>(yrow32 + n) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(yrow32 + n + 4) = make_float4(f[4], f[5], f[6], f[7]);
              } else {
                *reinterpret_cast<uint4*>(yrow + n) = out;
              }
            }
          }
        }
      }
      // the accumulator may be overwritten by the tile after next
      tc_fence_before();
      mbar_arrive(&dempty[ab]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(kTmemCols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// fp16 matrix [n_rows][n_cols] with row stride `ld` elements; box = 64 columns x box_rows rows
int make_map(CUtensorMap* map, const __half* ptr, int64_t n_rows, int n_cols, int64_t ld, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return BSB_ECUDA;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)n_cols, (cuuint64_t)n_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%d ld=%lld)", (int)r, (long long)n_rows, n_cols, (long long)ld);
    return BSB_ECUDA;
  }
  return BSB_OK;
}

template <int BN>
int launch_bn(GemmParams& P, const __half* x, int64_t x_stride, const __half* w, cudaStream_t s) {
  constexpr int kStages = GemmSmem<BN>::kStages;
  constexpr int smem = kStages * GemmSmem<BN>::kStageBytes + (2 * kStages + 4) * 8 + 16 + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  BSB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    BSB_CUDA(cudaFuncSetAttribute(gemm_tc5_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set[dev] = true;
  }
  if (int rc = make_map(&P.map_x, x, P.rows, P.in_features, x_stride, kBM)) return rc;
  if (int rc = make_map(&P.map_w, w, P.out_features, P.in_features, P.in_features, BN)) return rc;
  const int64_t n_tiles = ceil_div64(P.out_features, BN) * ceil_div64(P.rows, kBM);
  dim3 grid((unsigned)(n_tiles < sm_count() ? n_tiles : sm_count()));   // persistent: one CTA per multiprocessor
  profile_mark(s, false);
  gemm_tc5_kernel<BN><<<grid, kThreads, smem, s>>>(P);
  profile_mark(s, true);
  return check_launch("gemm_tc5_kernel");
}

}  // namespace

bool gemm_tc5_supported(int64_t rows, int out_features, int in_features) {
  return rows > 0 && rows <= 65535ll * kBM && in_features % 8 == 0 && in_features >= 8 && out_features % 8 == 0 && out_features >= 8;
}

int launch_gemm_tc5(const __half* x, int64_t rows, int64_t x_stride, const __half* w, int out_features,
                    int in_features, const __half* bias, __half* y, float* y32, int64_t y_stride, cudaStream_t s) {
  BSB_CHECK_ARG(gemm_tc5_supported(rows, out_features, in_features), "gemm: unsupported shape (rows=%lld out=%d in=%d)",
                (long long)rows, out_features, in_features);
  BSB_CHECK_ARG((uintptr_t)x % 16 == 0 && x_stride % 8 == 0 && (uintptr_t)w % 16 == 0,
                "gemm: x and W must be 16-byte aligned with row strides that are multiples of 8");
  BSB_CHECK_ARG((y != nullptr) != (y32 != nullptr), "gemm: exactly one of the fp16 and the fp32 output");
  BSB_CHECK_ARG(((uintptr_t)y | (uintptr_t)y32) % 16 == 0 && y_stride % 8 == 0, "gemm: y must be 16-byte aligned with a row stride that is a multiple of 8");
  GemmParams P;
  memset(&P, 0, sizeof(P));
  P.bias = bias;
  P.y = y;
  P.y32 = y32;
  P.y_stride = y_stride;
  P.rows = (int)rows;
  P.out_features = out_features;
  P.in_features = in_features;
  P.status = device_status_word();
  if (P.status == nullptr) return BSB_ECUDA;
  // wide tiles when they still give every multiprocessor a CTA; narrower ones for small problems,
  // which are bound by streaming W and want many CTAs in flight
  const int64_t row_tiles = ceil_div64(rows, kBM);
  const int sms = sm_count();
  if (row_tiles * ceil_div64(out_features, 256) >= sms) return launch_bn<256>(P, x, x_stride, w, s);
  if (row_tiles * ceil_div64(out_features, 128) >= sms) return launch_bn<128>(P, x, x_stride, w, s);
  return launch_bn<64>(P, x, x_stride, w, s);
}

}  // namespace bsb
