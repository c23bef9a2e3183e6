// Batch path for 7 .. 64 input rows, fused: the packed signs are expanded INSIDE the multiprocessor into the fp16
// operand of a tcgen05 MMA, the weight is never written to memory.
//
// Replaces, for small batches, the reconstruct-then-multiply structure of the reference's fused levels
// (bitstack/modules/BitStackLinear.py:116-148: unpack / reconstruct kernel -> fp16 W in memory -> F.linear;
// bitstack/utils/inference_utils.py:286-387 is its packed -> W kernel).
//
// Math.  y[t, m] = sum_n x[t, n] W[m, n],  W = sum_j S_j * (U_j Vt_j).  With A_j = S_j * (U_j Vt_j) rounded to fp16,
//     y = sum_j x A_j^T
// is a chain of fp16 MMAs with ONE fp32 accumulator: the sum over the blocks is taken by the tensor core in fp32.
//
// A CTA owns a 128-row tile of W and walks K in chunks of 64 columns; a STEP is (chunk, block j):
//   MMA 1   P = U_j[tile] (128 x 16) . VtT_j[chunk] (64 x 16)^T   -> tensor memory, fp32          (tcgen05, K = 16)
//   expand  a producer thread per row reads its 64 products (tcgen05.ld), rounds pairs of them to fp16x2, flips
//           the signs of a pair with one LOP3 against the shifted sign word, and stores the row into the A stage
//           (shared memory, the 128-byte-swizzled K-major layout the MMA reads)
//   MMA 2   D (128 x T) += A (128 x 64) . x'[chunk] (T x 64)^T                                    (tcgen05, 4 x K = 16)
// Four producer groups (4 warps each) work on four steps at a time; one thread issues all MMAs.
//
// Pairing trick.  cvt.rn.f16x2 packs two products into one register whose sign bits are bits 31 and 15.  The sign
// word of 32 columns, byte-swapped so that column c is bit 31 - c and shifted left by i, has column i at bit 31 and
// column i + 16 at bit 15: one shift and one LOP3 sign two elements.  So the K order inside every 32-column group
// is (16, 0, 17, 1, ..., 31, 15); a small preparation kernel writes x in that order (x') and Vt transposed
// (VtT [block][in][16], the K-major B operand of MMA 1) into the scratch.
//
// Work is the sequence of UNITS (row tile, 512-column super-chunk); a CTA takes a contiguous range of units, all
// blocks of each.  A run = the units of one row tile inside one CTA = one accumulator; runs write fp32 partial
// tiles, a last kernel adds the runs of a row tile in order (deterministic), adds the bias and rounds once.
// Every wait is time-bounded (status word, NaN outputs on a give-up).
#include <cuda.h>

#include "common.cuh"

namespace bsb {

namespace {

constexpr int kTile = 128;          // W rows per CTA tile (MMA M)
constexpr int kChunk = 64;          // columns per step (one 128-byte swizzle span of fp16)
constexpr int kSuper = 512;         // columns per unit = per staged sign tile (64 bytes per row)
constexpr int kSubs = kSuper / kChunk;
constexpr int kGroups = 4;          // producer groups
constexpr int kStages = 3;          // (super-chunk, block) stages resident
constexpr int kSignBytes = kTile * 64;
constexpr int kVttBytes = kSuper * 32;
constexpr int kUBytes = kTile * 32;
constexpr int kStageBytes = kSignBytes + kVttBytes + kUBytes;   // 28 KB
constexpr int kABytes = kTile * kChunk * 2;                      // 16 KB
constexpr int kMaxRows = 64;
constexpr int kProducerWarps = 4 * kGroups;
constexpr int kWarpStage = kProducerWarps;        // stage loader (signs, VtT, U)
constexpr int kWarpX = kProducerWarps + 1;        // x' loader
constexpr int kWarpMma = kProducerWarps + 2;      // tensor-memory allocation + issue of every MMA 1
constexpr int kWarpMma2 = kProducerWarps + 3;     // two warps: issue of MMA 2 for the even / the odd producer groups
constexpr int kWarpEpi = kProducerWarps + 5;      // 4 epilogue warps
constexpr int kThreads = (kProducerWarps + 9) * 32;
static_assert(kThreads == (kWarpEpi + 4) * 32, "the four epilogue warps are the last ones (they cover the four tensor-memory lane quarters)");
// A single thread issues a tcgen05.mma every ~28 ns and a commit costs it ~60 ns; a step needs one MMA 1 and four
// MMA 2 plus two commits, so the issue is spread over three threads: one for MMA 1, and one each for the MMA 2 of the
// even and of the odd producer groups, which accumulate into their own halves (the epilogue adds the two).
constexpr int kTmemCols = 512;                    // D: 2 halves x 2 buffers x 64, P: 4 x 64
constexpr uint32_t kColD = 0, kColP = 256;
constexpr unsigned long long kDefaultWaitNs = 200ull * 1000 * 1000;

struct alignas(64) SgParams {
  CUtensorMap map_sign;   // u8  [blocks][out][in/8],  box 64 x 128 x 1, 64-byte swizzle
  CUtensorMap map_u;      // f16 [blocks][out][16],    box 16 x 128 x 1, 32-byte swizzle
  CUtensorMap map_vtt;    // f16 [blocks][in][16],     box 16 x 256 x 1, 32-byte swizzle
  CUtensorMap map_x;      // f16 [tpad][in] (x'),      box 64 x tpad,    128-byte swizzle
  int M, N, nb, n_sc, tpad;
  int units_total, units_per_cta, lcm_units;   // lcm(units_per_cta, n_sc): run numbering
  float* partials;        // [run][tpad][128]
  int* status;
  unsigned long long wait_ns;
};

// ------------------------------------------------------------------ PTX helpers
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
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// time-bounded wait; false = gave up
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = global_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
      if (mbar_try(bar, parity)) return true;
    if (global_ns() - t0 > limit_ns) return false;
  }
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
__device__ __forceinline__ void tma_load_3d(void* smem, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
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
// K-major operand tiles as TMA writes them: rows of 128 bytes (8-row groups 1024 bytes apart, 128-byte swizzle) or
// rows of 32 bytes (8-row groups 256 bytes apart, 32-byte swizzle)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t sbo_bytes, uint64_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                       // leading byte offset: unused with a swizzled K-major tile
  d |= (uint64_t)(sbo_bytes >> 4) << 32;        // stride between 8-row groups
  d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
  d |= layout << 61;                            // 2 = 128-byte swizzle, 6 = 32-byte swizzle
  return d;
}
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N) {
  return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);   // f16 x f16 -> f32, both K-major
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// two products -> fp16x2 (hi = a, lo = b), both signs flipped where the matching bit (31 / 15) of `bits` is CLEAR
template <int SHIFT>
__device__ __forceinline__ uint32_t pack_signed(float a, float b, uint32_t word) {
  uint32_t p, out;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(a), "f"(b));
  // p ^ (~(word << SHIFT) & 0x80008000): minterms of a ^ (~b & c) = 0xD2
  asm("lop3.b32 %0, %1, %2, %3, 0xD2;" : "=r"(out) : "r"(p), "r"(word << SHIFT), "r"(0x80008000u));
  return out;
}
// 32 products of one row (columns 0..31 of a 32-column group) -> 16 registers in the K order (16, 0, 17, 1, ...)
__device__ __forceinline__ void expand_half(const uint32_t (&r)[32], uint32_t word, uint32_t* out) {
#define BSB_PS(i) out[i] = pack_signed<i>(__uint_as_float(r[i]), __uint_as_float(r[i + 16]), word)
  BSB_PS(0); BSB_PS(1); BSB_PS(2); BSB_PS(3); BSB_PS(4); BSB_PS(5); BSB_PS(6); BSB_PS(7);
  BSB_PS(8); BSB_PS(9); BSB_PS(10); BSB_PS(11); BSB_PS(12); BSB_PS(13); BSB_PS(14); BSB_PS(15);
#undef BSB_PS
}

// ------------------------------------------------------------------ preparation
// VtT[j][n][r] = Vt[j][r][n] and x'[t][n'] (K order of the pairing trick; rows >= `rows` are zero)
__global__ void __launch_bounds__(256) sg_prep_kernel(bsb_weight w, const __half* __restrict__ x, int64_t x_stride, int rows, int tpad,
                                                      __half* __restrict__ vtt, __half* __restrict__ xp) {
  const int N = w.in_features;
  const __half* vt = reinterpret_cast<const __half*>(w.vt);
  const int64_t total_v = (int64_t)w.blocks * N;           // one thread per (block, column): 16 ranks
  const int64_t total_x = (int64_t)tpad * (N / 2);         // one thread per pair of x'
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_v + total_x; i += stride) {
    if (i < total_v) {
      const int j = (int)(i / N), n = (int)(i % N);
      const __half* src = vt + (int64_t)j * w.vt_block_stride + n;
      __align__(16) __half v[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) v[r] = src[(int64_t)r * N];
      uint4* dst = reinterpret_cast<uint4*>(vtt + ((int64_t)j * N + n) * 16);
      dst[0] = *reinterpret_cast<const uint4*>(&v[0]);
      dst[1] = *reinterpret_cast<const uint4*>(&v[8]);
    } else {
      const int64_t k = i - total_x * 0 - total_v;
      const int t = (int)(k / (N / 2)), pr = (int)(k % (N / 2));
      const int grp = pr / 16, ii = pr % 16;               // pair ii of 32-column group grp
      __half lo = __float2half(0.f), hi = lo;
      if (t < rows) {
        lo = x[(int64_t)t * x_stride + grp * 32 + ii + 16];
        hi = x[(int64_t)t * x_stride + grp * 32 + ii];
      }
      reinterpret_cast<__half2*>(xp + (int64_t)t * N)[pr] = __halves2half2(lo, hi);
    }
  }
}

// ------------------------------------------------------------------ main kernel
struct Step {   // position of a step inside a CTA's range
  int unit, tile, sc, j, sub;
};

__device__ __forceinline__ int run_id_of_unit(const SgParams& P, int u) {
  return u / P.units_per_cta + u / P.n_sc - u / P.lcm_units;
}

__global__ void __launch_bounds__(kThreads, 1) signgemm_tc5_kernel(const __grid_constant__ SgParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int x_bytes = P.tpad * 128;                       // one x' chunk tile
  uint8_t* s_stage = base;                                // [kStages][sign 8 KB | VtT 16 KB | U 4 KB]
  uint8_t* s_a = s_stage + kStages * kStageBytes;         // [kGroups][16 KB]
  uint8_t* s_x = s_a + kGroups * kABytes;                 // [kSubs][tpad * 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_x + kSubs * x_bytes);
  uint64_t* stage_full = bars;                  // [kStages]
  uint64_t* stage_empty = stage_full + kStages; // [kStages]
  uint64_t* x_full = stage_empty + kStages;     // [kSubs]
  uint64_t* x_empty = x_full + kSubs;           // [kSubs]
  uint64_t* p_full = x_empty + kSubs;           // [kGroups]
  uint64_t* p_empty = p_full + kGroups;         // [kGroups]
  uint64_t* a_full = p_empty + kGroups;         // [kGroups]
  uint64_t* a_empty = a_full + kGroups;         // [kGroups]
  uint64_t* d_full = a_empty + kGroups;         // [2]
  uint64_t* d_empty = d_full + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_empty + 2);
  int* failed = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned long long wait_ns = P.wait_ns;
  const int u0 = blockIdx.x * P.units_per_cta;
  const int u1 = min(u0 + P.units_per_cta, P.units_total);
  const int n_units = u1 - u0;
  const int nb = P.nb;
  const int steps_per_unit = nb * kSubs;
  const int total = n_units * steps_per_unit;             // steps of this CTA

  if (warp == kWarpMma) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    *failed = 0;
    for (int i = 0; i < kStages; ++i) { mbar_init(&stage_full[i], 1); mbar_init(&stage_empty[i], 1 + kSubs * kTile); }
    for (int i = 0; i < kSubs; ++i) { mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1); }
    for (int i = 0; i < kGroups; ++i) {
      mbar_init(&p_full[i], 1);
      mbar_init(&p_empty[i], kTile);
      mbar_init(&a_full[i], kTile);
      mbar_init(&a_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&d_full[i], 2); mbar_init(&d_empty[i], kTile); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tmem_slot;
#define SG_GIVE_UP(code) do { atomicCAS(P.status, 0, (code)); *failed = 1; } while (0)

  if (warp == kWarpStage) {
    // ---- stage loader: signs, VtT and U of (unit, block) --------------------------------------------
    if (lane == 0) {
      int k = 0;
      bool ok = true;
      for (int ui = 0; ui < n_units && ok; ++ui) {
        const int unit = u0 + ui, tile = unit / P.n_sc, sc = unit % P.n_sc;
        for (int j = 0; j < nb; ++j, ++k) {
          const int slot = k % kStages, n = k / kStages;
          if (n >= 1 && !mbar_wait(&stage_empty[slot], (n - 1) & 1, wait_ns)) { SG_GIVE_UP(31); ok = false; break; }
          uint8_t* st = s_stage + slot * kStageBytes;
          mbar_expect_tx(&stage_full[slot], kStageBytes);
          tma_load_3d(st, &P.map_sign, sc * 64, tile * kTile, j, &stage_full[slot]);                       // rows / bytes past the end read 0
          tma_load_3d(st + kSignBytes, &P.map_vtt, 0, sc * kSuper, j, &stage_full[slot]);
          tma_load_3d(st + kSignBytes + kVttBytes / 2, &P.map_vtt, 0, sc * kSuper + 256, j, &stage_full[slot]);
          tma_load_3d(st + kSignBytes + kVttBytes, &P.map_u, 0, tile * kTile, j, &stage_full[slot]);
        }
      }
    }
  } else if (warp == kWarpX) {
    // ---- x' loader: the eight 64-column chunks of a unit's super-chunk, kept for all its blocks ------
    if (lane == 0) {
      bool ok = true;
      for (int ui = 0; ui < n_units && ok; ++ui) {
        const int sc = (u0 + ui) % P.n_sc;
        for (int sub = 0; sub < kSubs; ++sub) {
          if (ui >= 1 && !mbar_wait(&x_empty[sub], (ui - 1) & 1, wait_ns)) { SG_GIVE_UP(32); ok = false; break; }
          mbar_expect_tx(&x_full[sub], x_bytes);
          tma_load_2d(s_x + sub * x_bytes, &P.map_x, sc * kSuper + sub * kChunk, 0, &x_full[sub]);
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ---- issuer of MMA 1 (rank product of every step, into the step's producer group's columns).  The warp runs
    //      the loop uniformly, one elected lane issues. -----------------------------------------------------------
    const bool leader = elect_one();
    const uint32_t idesc1 = make_idesc_f16(kTile, kChunk);
    bool ok = true;
#pragma unroll 1
    for (int a = 0; a < total && ok; ++a) {
      const int in_unit = a % steps_per_unit, j = in_unit / kSubs, sub = in_unit % kSubs;
      const int k = (a / steps_per_unit) * nb + j;                       // stage index
      const int slot = k % kStages, g = a % kGroups, use = a / kGroups;
      if (sub == 0 && !mbar_wait(&stage_full[slot], (k / kStages) & 1, wait_ns)) { if (leader) SG_GIVE_UP(33); ok = false; break; }
      if (use >= 1 && !mbar_wait(&p_empty[g], (use - 1) & 1, wait_ns)) { if (leader) SG_GIVE_UP(38); ok = false; break; }
      tc_fence_after();
      if (leader) {
        const uint32_t st = smem_u32(s_stage + slot * kStageBytes);
        const uint64_t adesc = make_desc(st + kSignBytes + kVttBytes, 256, 6);                      // U tile
        const uint64_t bdesc = make_desc(st + kSignBytes + sub * (kChunk * 32), 256, 6);            // 64 rows of VtT
        mma_ss_f16(tbase + kColP + g * 64, adesc, bdesc, idesc1, 0u);
        mma_commit(&p_full[g]);
        if (sub == kSubs - 1) mma_commit(&stage_empty[slot]);   // every MMA 1 of the stage has read it
      }
    }
  } else if (warp == kWarpMma2 || warp == kWarpMma2 + 1) {
    // ---- issuer h of MMA 2: the steps of the producer groups g with g % 2 == h (a group's steps all have the
    //      parity of g), accumulated into half h of the run's accumulator ------------------------------------------
    const int h = warp - kWarpMma2;
    const bool leader = elect_one();
    const uint32_t idesc2 = make_idesc_f16(kTile, P.tpad);
    bool ok = true;
    bool first_of_run = true;
#pragma unroll 1
    for (int b = h; b < total && ok; b += 2) {
      const int ui = b / steps_per_unit, in_unit = b % steps_per_unit, j = in_unit / kSubs, sub = in_unit % kSubs;
      const int unit = u0 + ui, tile = unit / P.n_sc;
      const int g = b % kGroups, use = b / kGroups;
      // runs of this CTA: a new one starts at the CTA's first unit and at every first super-chunk of a row tile
      const int run = tile - u0 / P.n_sc;                  // local run index (tiles are consecutive)
      const bool unit_starts_run = (ui == 0 || unit % P.n_sc == 0);
      const bool unit_ends_run = (ui == n_units - 1 || (unit + 1) % P.n_sc == 0);
      if (unit_starts_run && in_unit == h) first_of_run = true;          // this issuer's first step of the run
      const bool last_of_run = unit_ends_run && in_unit == steps_per_unit - 2 + h;
      const int db = run & 1;
      if (first_of_run && run >= 2 && !mbar_wait(&d_empty[db], ((run >> 1) - 1) & 1, wait_ns)) { if (leader) SG_GIVE_UP(39); ok = false; break; }
      if (!mbar_wait(&a_full[g], use & 1, wait_ns)) { if (leader) SG_GIVE_UP(40); ok = false; break; }
      if (j == 0 && !mbar_wait(&x_full[sub], ui & 1, wait_ns)) { if (leader) SG_GIVE_UP(41); ok = false; break; }
      tc_fence_after();
      if (leader) {
        const uint64_t adesc = make_desc(smem_u32(s_a + g * kABytes), 1024, 2);
        const uint64_t bdesc = make_desc(smem_u32(s_x + sub * x_bytes), 1024, 2);
        const uint32_t dcol = tbase + kColD + h * 128 + db * 64;
#pragma unroll
        for (int kk = 0; kk < kChunk / 16; ++kk)        // 16 elements = 32 bytes further along the swizzled row
          mma_ss_f16(dcol, adesc + 2 * kk, bdesc + 2 * kk, idesc2, (first_of_run && kk == 0) ? 0u : 1u);
        mma_commit(&a_empty[g]);
        if (j == nb - 1) mma_commit(&x_empty[sub]);
        if (last_of_run) mma_commit(&d_full[db]);
      }
      first_of_run = false;
    }
  } else if (warp < kProducerWarps) {
    // ---- producer group g: steps g, g + 4, ...; thread = row of the tile ---------------------------------
    const int g = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tbase + ((uint32_t)(quarter * 32) << 16) + kColP + g * 64;
    uint8_t* arow = s_a + g * kABytes + row * 128;
    const int sw_a = row & 7;                    // 128-byte swizzle of the A stage
    const int sw_s = (row >> 1) & 3;             // 64-byte swizzle of the sign tile
    bool ok = true;
    int use = 0;
#pragma unroll 1
    for (int s = g; s < total && ok; s += kGroups, ++use) {
      const int in_unit = s % steps_per_unit, j = in_unit / kSubs, sub = in_unit % kSubs;
      const int k = (s / steps_per_unit) * nb + j;
      const int slot = k % kStages;
      // the stage's sign tile (visibility of the TMA write needs this thread's own observation of the barrier)
      if (!mbar_wait(&stage_full[slot], (k / kStages) & 1, wait_ns)) { SG_GIVE_UP(34); ok = false; break; }
      const uint8_t* srow = s_stage + slot * kStageBytes + row * 64 + (((sub >> 1) ^ sw_s) << 4) + (sub & 1) * 8;
      const uint2 sw = *reinterpret_cast<const uint2*>(srow);
      mbar_arrive(&stage_empty[slot]);
      const uint32_t w0 = __byte_perm(sw.x, 0, 0x0123), w1 = __byte_perm(sw.y, 0, 0x0123);   // column c -> bit 31 - c
      if (!mbar_wait(&p_full[g], use & 1, wait_ns)) { SG_GIVE_UP(35); ok = false; break; }
      tc_fence_after();
      uint32_t out[32];
      {
        uint32_t r[32];
        tmem_ld32(lane_base, r);
        tmem_wait_ld();
        expand_half(r, w0, out);
        tmem_ld32(lane_base + 32, r);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&p_empty[g]);               // the rank product of this group's next step may be written
        expand_half(r, w1, out + 16);
      }
      if (use >= 1 && !mbar_wait(&a_empty[g], (use - 1) & 1, wait_ns)) { SG_GIVE_UP(36); ok = false; break; }
#pragma unroll
      for (int c = 0; c < 8; ++c)               // 16-byte piece c = K positions 8c .. 8c+7 = registers 4c .. 4c+3
        *reinterpret_cast<uint4*>(arow + ((c ^ sw_a) << 4)) = make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the stores must be visible to the MMA's reads
      mbar_arrive(&a_full[g]);
    }
  } else {
    // ---- epilogue: a run's accumulator -> fp32 partial tile [tpad][128] ------------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tbase + ((uint32_t)(quarter * 32) << 16) + kColD;
    const int first_tile = u0 / P.n_sc, last_tile = (u1 - 1) / P.n_sc;
    for (int tile = first_tile; tile <= last_tile && n_units > 0; ++tile) {
      const int run = tile - first_tile, db = run & 1;
      const int first_unit = max(u0, tile * P.n_sc);
      float* part = P.partials + (int64_t)run_id_of_unit(P, first_unit) * P.tpad * kTile;
      bool ok = mbar_wait(&d_full[db], (run >> 1) & 1, wait_ns);
      ok = __all_sync(0xFFFFFFFFu, ok ? 1 : 0) != 0;
      if (!ok) {
        if (lane == 0) SG_GIVE_UP(37);
        break;
      }
      tc_fence_after();
      for (int c = 0; c < P.tpad; c += 16) {
        uint32_t d0[16], d1[16];
        tmem_ld16(lane_base + db * 64 + c, d0);          // half of the even producer groups
        tmem_ld16(lane_base + 128 + db * 64 + c, d1);    // half of the odd ones
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) part[(c + i) * kTile + row] = __uint_as_float(d0[i]) + __uint_as_float(d1[i]);
      }
      tc_fence_before();
      mbar_arrive(&d_empty[db]);
    }
  }

  // ---- tear-down ----------------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpMma) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(kTmemCols) : "memory");
  }
  if (*failed && n_units > 0) {
    // a wait gave up: every partial tile of this CTA becomes NaN, so the outputs it feeds are NaN
    const float nan = __int_as_float(0x7FC00000);
    const int first_tile = u0 / P.n_sc, last_tile = (u1 - 1) / P.n_sc;
    for (int tile = first_tile; tile <= last_tile; ++tile) {
      float* part = P.partials + (int64_t)run_id_of_unit(P, max(u0, tile * P.n_sc)) * P.tpad * kTile;
      for (int i = tid; i < P.tpad * kTile; i += kThreads) part[i] = nan;
    }
  }
#undef SG_GIVE_UP
}

// y[t][m] = sum over the runs of m's row tile (in run order) + bias, rounded once (or fp32 for partial-sum outputs)
__global__ void __launch_bounds__(256) sg_reduce_kernel(SgParams P, const __half* __restrict__ bias, int rows, __half* __restrict__ y,
                                                        float* __restrict__ y32, int64_t y_stride) {
  const int64_t total = (int64_t)rows * P.M;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / P.M), m = (int)(i % P.M);
    const int tile = m / kTile, r = m % kTile;
    const int r0 = run_id_of_unit(P, tile * P.n_sc), r1 = run_id_of_unit(P, (tile + 1) * P.n_sc - 1);
    float s = 0.f;
    for (int q = r0; q <= r1; ++q) s += P.partials[((int64_t)q * P.tpad + t) * kTile + r];
    if (bias) s += __half2float(bias[m]);
    if (y32) y32[(int64_t)t * y_stride + m] = s;
    else y[(int64_t)t * y_stride + m] = __float2half_rn(s);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn sg_encode_fn() {
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

int encode(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* ptr, const cuuint64_t* dims, const cuuint64_t* strides,
           const cuuint32_t* box, CUtensorMapSwizzle sw, const char* what) {
  EncodeTiledFn enc = sg_encode_fn();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return BSB_ECUDA;
  }
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, dt, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled(%s) failed with code %d", what, (int)r);
    return BSB_ECUDA;
  }
  return BSB_OK;
}

int64_t gcd64(int64_t a, int64_t b) { return b == 0 ? a : gcd64(b, a % b); }

struct SgPlan {
  int tpad, tiles, n_sc, units, upc, grid, runs;
  int64_t vtt_off, x_off, part_off, bytes;
};

void make_plan(const bsb_weight& w, int64_t rows, SgPlan& pl) {
  pl.tpad = (int)ceil_div64(rows, 16) * 16;
  pl.tiles = (int)ceil_div64(w.out_features, kTile);
  pl.n_sc = (int)ceil_div64(w.in_features, kSuper);
  pl.units = pl.tiles * pl.n_sc;
  pl.upc = (int)ceil_div64(pl.units, sm_count());
  pl.grid = (int)ceil_div64(pl.units, pl.upc);
  const int64_t lcm = (int64_t)pl.upc / gcd64(pl.upc, pl.n_sc) * pl.n_sc;
  const int u = pl.units - 1;
  pl.runs = (int)(u / pl.upc + u / pl.n_sc - u / lcm) + 1;
  int64_t off = 0;
  pl.vtt_off = off;
  off = align_up64(off + (int64_t)w.blocks * w.in_features * 32, 256);
  pl.x_off = off;
  off = align_up64(off + (int64_t)pl.tpad * w.in_features * 2, 256);
  pl.part_off = off;
  off = align_up64(off + (int64_t)pl.runs * pl.tpad * kTile * 4, 256);
  pl.bytes = off;
}

unsigned long long g_sg_wait_ns = kDefaultWaitNs;

}  // namespace

void signgemm_set_wait_limit_ns(unsigned long long ns) { g_sg_wait_ns = ns; }

bool signgemm_supported(const bsb_weight& w, int64_t rows) {
  return rows >= 1 && rows <= kMaxRows && w.k == 16 && w.blocks >= 1 && w.in_features >= 128 && w.in_features % 128 == 0 &&
         w.out_features >= 1 && ((uintptr_t)w.qweight % 16 == 0) && (w.blocks == 1 || w.q_block_stride % 16 == 0) &&
         ((uintptr_t)w.u % 16 == 0) && (w.blocks == 1 || w.u_block_stride % 8 == 0) && ((uintptr_t)w.vt % 2 == 0);
}

int64_t signgemm_workspace_bytes(const bsb_weight& w, int64_t rows) {
  SgPlan pl;
  make_plan(w, rows, pl);
  return pl.bytes;
}

// exactly one of y (fp16) and y32 (fp32 partial sums of a tensor-parallel shard) is non-null
int launch_signgemm(const bsb_weight& w, const __half* x, int64_t rows, int64_t x_stride, __half* y, float* y32, int64_t y_stride,
                    void* workspace, int64_t workspace_bytes, cudaStream_t s) {
  BSB_CHECK_ARG(signgemm_supported(w, rows), "fused sign-GEMM: unsupported shape/alignment (out=%d in=%d k=%d rows=%lld)",
                w.out_features, w.in_features, w.k, (long long)rows);
  BSB_CHECK_ARG((y != nullptr) != (y32 != nullptr), "fused sign-GEMM: exactly one of the fp16 and the fp32 output");
  SgPlan pl;
  make_plan(w, rows, pl);
  if (workspace == nullptr || workspace_bytes < pl.bytes) {
    set_error("fused sign-GEMM: workspace of %lld bytes needed, %lld given", (long long)pl.bytes, (long long)workspace_bytes);
    return BSB_EWORKSPACE;
  }
  BSB_CHECK_ARG((uintptr_t)workspace % 256 == 0, "fused sign-GEMM: workspace must be 256-byte aligned");
  uint8_t* base = (uint8_t*)workspace;
  __half* vtt = (__half*)(base + pl.vtt_off);
  __half* xp = (__half*)(base + pl.x_off);
  SgParams P;
  memset(&P, 0, sizeof(P));
  P.M = w.out_features;
  P.N = w.in_features;
  P.nb = w.blocks;
  P.n_sc = pl.n_sc;
  P.tpad = pl.tpad;
  P.units_total = pl.units;
  P.units_per_cta = pl.upc;
  P.lcm_units = (int)((int64_t)pl.upc / gcd64(pl.upc, pl.n_sc) * pl.n_sc);
  P.partials = (float*)(base + pl.part_off);
  P.status = device_status_word();
  if (P.status == nullptr) return BSB_ECUDA;
  P.wait_ns = g_sg_wait_ns;
  const int N = w.in_features, M = w.out_features;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)(N / 8), (cuuint64_t)M, (cuuint64_t)w.blocks};
    const cuuint64_t strides[2] = {(cuuint64_t)(N / 8), (cuuint64_t)(w.blocks > 1 ? w.q_block_stride : (int64_t)M * (N / 8))};
    const cuuint32_t box[3] = {64, (cuuint32_t)kTile, 1};
    if (int rc = encode(&P.map_sign, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w.qweight, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B, "signs")) return rc;
  }
  {
    const cuuint64_t dims[3] = {16, (cuuint64_t)M, (cuuint64_t)w.blocks};
    const cuuint64_t strides[2] = {32, (cuuint64_t)(w.blocks > 1 ? w.u_block_stride * 2 : (int64_t)M * 32)};
    const cuuint32_t box[3] = {16, (cuuint32_t)kTile, 1};
    if (int rc = encode(&P.map_u, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, w.u, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B, "u")) return rc;
  }
  {
    const cuuint64_t dims[3] = {16, (cuuint64_t)N, (cuuint64_t)w.blocks};
    const cuuint64_t strides[2] = {32, (cuuint64_t)N * 32};
    const cuuint32_t box[3] = {16, 256, 1};
    if (int rc = encode(&P.map_vtt, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, vtt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_32B, "vt transposed")) return rc;
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)pl.tpad};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kChunk, (cuuint32_t)pl.tpad};
    if (int rc = encode(&P.map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xp, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "x")) return rc;
  }
  {
    const int64_t work = (int64_t)w.blocks * N + (int64_t)pl.tpad * (N / 2);
    const int blocks = (int)min((int64_t)sm_count() * 8, ceil_div64(work, 256));
    sg_prep_kernel<<<blocks, 256, 0, s>>>(w, x, x_stride, (int)rows, pl.tpad, vtt, xp);
    if (int rc = check_launch("sg_prep_kernel")) return rc;
  }
  const int smem = kStages * kStageBytes + kGroups * kABytes + kSubs * pl.tpad * 128 + 512 + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  BSB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    BSB_CUDA(cudaFuncSetAttribute(signgemm_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set[dev] = true;
  }
  signgemm_tc5_kernel<<<pl.grid, kThreads, smem, s>>>(P);
  if (int rc = check_launch("signgemm_tc5_kernel")) return rc;
  {
    const int64_t total = rows * M;
    const int blocks = (int)min((int64_t)sm_count() * 8, ceil_div64(total, 256));
    sg_reduce_kernel<<<blocks, 256, 0, s>>>(P, reinterpret_cast<const __half*>(w.bias), (int)rows, y, y32, y_stride);
  }
  return check_launch("sg_reduce_kernel");
}

}  // namespace bsb
