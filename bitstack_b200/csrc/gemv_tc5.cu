// Decode path, tcgen05 generation: packed sign bits -> e4m3 operand in TENSOR MEMORY
// -> tcgen05.mma (kind::f8f6f4, M=128, N=32, K=32) with the x-scaled factors Z' as the
// shared-memory operand, staged by bulk TMA copies.
//
// Replaces, for single-row inputs, every fused level of the reference forward
// (bitstack/modules/BitStackLinear.py:116-157).
//
// Math.  For block j, Z_j[n,r] = Vt_j[r,n] x[n] and
//     y[m] = sum_j sum_r U_j[m,r] D_j[m,r],   D_j[m,r] = sum_n S_j[m,n] Z_j[n,r].
// A 32-bit word of packed signs (32 columns of one row) is expanded by eight logic
// instructions into eight registers of four e4m3 numbers: register i holds, in byte
// c, the number v0_i + b d_i where b is the sign bit of column 8c+7-i (class table
// below).  The eight registers are one row of a 128 x 32 A operand and go to tensor
// memory with tcgen05.st.  The B operand (32 x 32) holds Z'[n,r] = 2 s_r Z / d_class(n)
// as two e4m3 pieces (rows 0-15 "hi", 16-31 "lo") in the same K order, so
//     T[m,r] = D_hi + D_lo = C_r + 2 s_r sum_n b Z,    D_j[m,r] = (T - C_r)/s_r - sum_n Z.
//
// CTA = 512 threads, two per multiprocessor: a loader thread streams sign tiles (tiled TMA) and
// Z' slabs (bulk copies) into shared-memory rings; two groups of four producer warps expand
// sign bytes into tensor memory, each feeding its own MMA-issuing thread and accumulators;
// four epilogue warps apply U and accumulate y over blocks.  All hand-offs are mbarriers
// with time-bounded waits: on a timeout the kernel raises a status word and leaves, it never
// spins forever.  Roles with slack (loader, epilogue) poll with one lane and a growing sleep:
// the polling of idle roles otherwise saturates the special-function issue path and slows the
// warps on the critical path (measured 130 -> 114 us on a 14336 x 4096, 16-block weight).
#include <cuda.h>
#include <cuda_fp8.h>

#if defined(BSB_TRACE) && !defined(BSB_TUNING)
#define BSB_TUNING
#endif

#include <vector>

#include "common.cuh"

namespace bsb {

namespace {

constexpr int kChunkCols = 512;                 // columns per Z' slab / per 64 B of a sign row
constexpr int kChunkBytes = kChunkCols * 32;    // 16 words x 1 KB operand tile
constexpr int kTileRows = 128;
constexpr int kThreads = 512;                    // 8 producer warps, 2 MMA issuers, loader, (idle), 4 epilogue warps
#ifndef BSB_NZ
#define BSB_NZ 3
#endif
constexpr int kNZ = BSB_NZ;                          // Z' slabs resident in shared memory
constexpr int kSignTileBytes = kTileRows * 64;
constexpr int kTmemCols = 256;                  // 4 x 32 (D: 2 issuers x 2 buffers) + 4 x 32 (A: 2 issuers x 2 stages)
constexpr int kMaxGroup = 4;
constexpr float kTargetMax = 320.f;
constexpr float kMinD = 0.75f;
constexpr unsigned long long kDefaultWaitNs = 200ull * 1000 * 1000;   // default limit of every wait (bsb_set_wait_limit_ms)

__constant__ float kV0[8] = {8.f, 4.f, 2.f, 0.75f, 0.375f, 0.09375f, 0.f, 1.f};
// class steps d_i (set bit minus clear bit): 1, 1, 1, 0.75, 1.125, 1.40625, 2, -2 (kTwoOverD below holds 2 / d_i)
__host__ __device__ constexpr uint32_t class_byte(int i) {
  return i == 0 ? 0x50u : i == 1 ? 0x48u : i == 2 ? 0x40u : i == 3 ? 0x34u
       : i == 4 ? 0x2Cu : i == 5 ? 0x1Cu : i == 6 ? 0x00u : 0x38u;
}

struct alignas(64) TcParams {
  CUtensorMap sign_map[kMaxGroup];   // u8 [blocks][out][in/8], box 1 x 128 x 64, 64-byte swizzle
  bsb_weight w[kMaxGroup];
  const float* vt_absmax[kMaxGroup];
  const float* x_absmax;           // optional max |x| per input row of this pass (from the kernel that produced x), or nullptr
  int absmax_const;                // every vt_absmax came from the caller (a constant of the weight), none is computed in front of this call
  __half* y[kMaxGroup];            // fp16 rows, or fp32 rows when out_f32 is set
  int out_f32;                     // outputs are fp32 partial sums of a tensor-parallel shard (no rounding)
  int n_weights;
  int rows;                        // input rows of this pass (1 or 2): the B operand holds 32 columns per row
  int64_t x_stride;                // elements between input rows
  int64_t y_stride[kMaxGroup];     // elements between output rows
  int n_chunks;                    // ceil(in / 512)
  int step_base[kMaxGroup + 1];    // first work step of each weight; a step = (row group, block, chunk)
  int seg_base[kMaxGroup + 1];     // first row group of each weight (index of its counter)
  int blk_base[kMaxGroup + 1];
  // CTAs 0 .. n_first-1 take steps_first consecutive steps each, the others steps_per_cta (the last one fewer).
  // n_first > 0 only when unequal shares are selected (tuning knob): the first CTA to become resident on a
  // multiprocessor runs ~1.3x faster than the second one while both are there (its older warps win the issue
  // arbitration).
  int n_first, steps_first;
  int steps_per_cta;
  uint8_t* zops;     // [(weight,block)][chunk][16 words][rows][1 KB]
  float* kconst;     // [(weight,block)][chunk][rows][16]
  float* inv_scale;  // [(weight,block)][rows][16]
  int* counters;     // [row group]: CTAs that have delivered their partial sums
  int* status;       // the library's sticky status word of this device: 0 = fine, else the code of the first wait that gave up
  unsigned long long wait_ns;   // time limit of every wait
#ifdef BSB_TUNING
  unsigned long long* timeline;   // optional [8] wall-clock marks of this call (see TL_MIN / TL_MAX), or nullptr
  unsigned long long* trace;  // optional [CTA][16] cycle counters, or nullptr
  int dbg;           // 0 = normal; 1 = MMA side only, 2 = producer side only (timing experiments, wrong results); 3 = the Z' loader
                     // never loads (the waits behind it run out: exercises the give-up path)
#endif
  float* partials;   // [CTA][2][rows][RT * 128]: sums of a row group that the CTA shares with other CTAs
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
// wall-clock marks of one call in the tuning build: slot 0 / 1 / 2 = first Z' CTA entered / first passed its wait / last
// left; 3 = first decode CTA entered, 4 = first Z' slab consumed, 5 = last epilogue done, 6 = last decode CTA left,
// 7 = last Z' CTA has the row maximum, 8 / 9 = last decode / Z' CTA entered, 10 = first decode CTA done,
// 11 = last decode CTA consumed its first Z' slab
#ifdef BSB_TUNING
#define TL_MIN(slot) do { if (P.timeline) atomicMin(P.timeline + (slot), (unsigned long long)global_ns()); } while (0)
#define TL_MAX(slot) do { if (P.timeline) atomicMax(P.timeline + (slot), (unsigned long long)global_ns()); } while (0)
#else
#define TL_MIN(slot) do { } while (0)
#define TL_MAX(slot) do { } while (0)
#endif
// mbarrier.try_wait suspends the thread in hardware until the phase completes or a short, implementation-defined
// time has passed: a waiting role costs almost no issue slots.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// time-bounded wait; false = gave up after `limit_ns`
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
// Wait of a whole warp in which one lane does the waiting (roles with slack: epilogue); the other lanes then
// observe the completed phase once (their own acquire).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, limit_ns) ? 1 : 0;
  ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
  if (ok) ok = mbar_test(bar, parity) ? 1 : 0;
  return __all_sync(0xFFFFFFFFu, ok) != 0;
}
// producer-group wait: every lane waits for itself (electing one waiting lane per warp adds a shuffle and a
// second test to the hand-off, which measured slower on the whole kernel)
__device__ __forceinline__ bool mbar_wait_group(uint64_t* bar, uint32_t parity, unsigned long long limit_ns) {
  return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, limit_ns) ? 1 : 0) != 0;
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, int cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, int cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
}
// D[tmem] += A[tmem] . B[smem]^T, e4m3 x e4m3 -> f32, always accumulating, without an output-lane
// mask: the shortest operand list (every operand of the instruction has to be moved to a uniform
// register first)
__device__ __forceinline__ void mma_ts_f8_acc(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.eq.b32 p, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void mma_ts_f8_first(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xFFFFFFFF;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok));
  return ok != 0;
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// K-major operand without swizzle: 8-row x 16-byte core matrices; the two 16-byte K
// halves of a core-matrix row group are `lbo` bytes apart, row groups `sbo` bytes apart
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
__host__ __device__ constexpr uint32_t make_idesc_f8(int M, int N) {
  return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void bulk_g2s(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// 3-D tiled TMA load (no multicast): box lands in shared memory, bytes are counted on `bar`
__device__ __forceinline__ void tma_load_3d(void* smem, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem)), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}
// (word & mask_I) | c  in one LOP3: the mask is an immediate, the OR-constant a register
template <int I>
__device__ __forceinline__ uint32_t expand_c(uint32_t word, uint32_t c) {
  uint32_t out;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(out) : "r"(word), "n"(0x01010101u << I), "r"(c));
  return out;
}
__device__ __forceinline__ void expand_word_c(uint32_t word, const uint32_t (&c)[8], uint32_t* r) {
  r[0] = expand_c<0>(word, c[0]); r[1] = expand_c<1>(word, c[1]); r[2] = expand_c<2>(word, c[2]); r[3] = expand_c<3>(word, c[3]);
  r[4] = expand_c<4>(word, c[4]); r[5] = expand_c<5>(word, c[5]); r[6] = expand_c<6>(word, c[6]); r[7] = expand_c<7>(word, c[7]);
}

// ------------------------------------------------------------------ max |vt| per (block, rank)
// grid = (16 ranks, blocks).  Sets the scale of the e4m3 operand; a pure function of the stored factors.
__global__ void __launch_bounds__(256) vt_absmax_kernel(bsb_weight w, float* __restrict__ out) {
  const int r = blockIdx.x, j = blockIdx.y;
  const __half* vt = reinterpret_cast<const __half*>(w.vt) + (int64_t)j * w.vt_block_stride + (int64_t)r * w.in_features;
  float m = 0.f;
  for (int n = threadIdx.x; n < w.in_features; n += blockDim.x) m = fmaxf(m, fabsf(__half2float(vt[n])));
  __shared__ float red[8];
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    out[j * 16 + r] = m;
  }
}

// ------------------------------------------------------------------ Z' preparation
// grid = (n_chunks, total blocks, input rows), 512 threads: thread = (32-column word, half of the eight bit classes,
// rank).  Operand tile of word w (32 columns): byte offset (n%8)*16 + (n/8)*256 + (k%16) + (k/16)*128 with
// n = 16*piece + rank and k = 4*i + c for the column 8c+7-i of the word (i = bit class, c = byte of the packed word).
// Everything that does not depend on x (the factors, their maximum, the per-class multipliers) is fetched and
// computed BEFORE the wait for the kernels in front; after it the chain is: load x, row maximum, one reciprocal,
// two multiplies and the fp8 split per element, store.
__constant__ float kTwoOverD[8] = {2.f / 1.f, 2.f / 1.f, 2.f / 1.f, 2.f / 0.75f, 2.f / 1.125f, 2.f / 1.40625f, 2.f / 2.f, 2.f / -2.f};
constexpr int kZprepThreads = 512;

__global__ void __launch_bounds__(kZprepThreads) zprep_tc5_kernel(const __grid_constant__ TcParams P, const __half* __restrict__ x) {
  __shared__ float red[16];
  __shared__ float kred[16][2][16];

  const int chunk = blockIdx.x;
  int wi = 0;
  while (wi + 1 < P.n_weights && (int)blockIdx.y >= P.blk_base[wi + 1]) ++wi;
  const bsb_weight& w = P.w[wi];
  const int j = blockIdx.y - P.blk_base[wi];
  const int N = w.in_features;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = tid & 15, kh = (tid >> 4) & 1, word = tid >> 5;   // a warp = one word
  const int col0 = chunk * kChunkCols + word * 32;
  const int R = P.rows, row = blockIdx.z;
  const bool in_range = col0 < N;   // in_features is a multiple of 128, so a word is inside or outside as a whole
  // this thread's columns: 8c + base + e (c = 0..3, e = 0..3), whose bit class is 7 - base - e = 4 kh + (3 - e)
  const int base = kh ? 0 : 4;

  if (tid == 0) { TL_MIN(0); TL_MAX(9); }
  uint2 vq[4];
  const __half* vt = reinterpret_cast<const __half*>(w.vt) + (int64_t)j * w.vt_block_stride + (int64_t)r * N + col0 + base;
#pragma unroll
  for (int c = 0; c < 4; ++c) vq[c] = in_range ? __ldg(reinterpret_cast<const uint2*>(vt + 8 * c)) : make_uint2(0, 0);
  // the maximum of |vt| is a constant of the weight when the caller passed it in; when it was computed into the
  // scratch by a kernel in front of this one it may only be read after the wait
  float vmax = P.absmax_const ? P.vt_absmax[wi][j * 16 + r] : 0.f;
  float vtd[4][4];   // vt * 2 / d_class
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const __half2* h = reinterpret_cast<const __half2*>(&vq[c]);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    vtd[c][0] = a.x; vtd[c][1] = a.y; vtd[c][2] = b.x; vtd[c][3] = b.y;
  }
  // x and the scratch of the previous call are safe to touch once the kernels before this one are done; then the
  // decode kernel of this call may be scheduled (it waits for this grid before it touches anything written here)
#ifdef BSB_ZPREP_EARLY   // measurement variant: the decode kernel's CTAs are dispatched while this kernel still waits
  pdl_trigger();
  pdl_wait();
#else
  pdl_enter();
#endif
  if (tid == 0) TL_MIN(1);
  if (!P.absmax_const) vmax = P.vt_absmax[wi][j * 16 + r];

  x += (int64_t)row * P.x_stride;
  if (blockIdx.x == 0 && blockIdx.y == 0 && row == 0)
    for (int i = tid; i < P.seg_base[P.n_weights]; i += blockDim.x) P.counters[i] = 0;
  uint2 xq[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) xq[c] = in_range ? __ldg(reinterpret_cast<const uint2*>(x + col0 + base + 8 * c)) : make_uint2(0, 0);
  // max |x| over the whole row sets the scale of the e4m3 operand: taken from the producer of x when it delivered
  // it, else computed here (every CTA reads the whole row; CTAs start at different places so that they do not all
  // ask the same L2 lines at the same moment)
  float xm = 0.f;
  if (P.x_absmax != nullptr) {
    xm = P.x_absmax[row];
  } else {
    const int nvec = N / 8;
    const int rot = (int)((blockIdx.x * 37u + blockIdx.y * 101u) * 64u % (unsigned)nvec);
    for (int i = tid; i < nvec; i += kZprepThreads) {
      int n8 = i + rot;
      if (n8 >= nvec) n8 -= nvec;
      const uint4 q = __ldg(reinterpret_cast<const uint4*>(x) + n8);
      const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(__habs2(h[k]));
        xm = fmaxf(xm, fmaxf(f.x, f.y));
      }
    }
    for (int o = 16; o > 0; o >>= 1) xm = fmaxf(xm, __shfl_xor_sync(0xFFFFFFFFu, xm, o));
    if (lane == 0) red[warp] = xm;
    __syncthreads();
    xm = red[0];
#pragma unroll
    for (int i = 1; i < kZprepThreads / 32; ++i) xm = fmaxf(xm, red[i]);
  }
  if (tid == 0) TL_MAX(7);

  const float bound = vmax * xm;
  const float scale = (bound > 0.f) ? __fdividef(kTargetMax * kMinD * 0.5f, bound) : 1.f;
  const float inv_scale = 1.f / scale;
  if (chunk == 0 && tid < 16) P.inv_scale[((int64_t)blockIdx.y * R + row) * 16 + r] = inv_scale;

  // the operand tile of a word holds the rows one after the other (row i = B columns 32i .. 32i+31)
  uint8_t* tile = P.zops + (((int64_t)blockIdx.y * P.n_chunks + chunk) * 16 + word) * (1024 * R) + row * 1024;
  float c_sum = 0.f, z_sum = 0.f;
  uint32_t hi[4], lo[4];
  float xf[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const __half2* h = reinterpret_cast<const __half2*>(&xq[c]);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    xf[c][0] = a.x; xf[c][1] = a.y; xf[c][2] = b.x; xf[c][3] = b.y;
  }
#pragma unroll
  for (int il = 0; il < 4; ++il) {
    const int e = 3 - il;
    const float mul = scale * (kh ? kTwoOverD[4 + il] : kTwoOverD[il]);
    const float v0 = kh ? kV0[4 + il] : kV0[il];
    uint32_t h32 = 0, l32 = 0;
#pragma unroll
    for (int cp = 0; cp < 2; ++cp) {   // two columns per conversion instruction
      const float za = vtd[2 * cp][e] * xf[2 * cp][e], zb = vtd[2 * cp + 1][e] * xf[2 * cp + 1][e];
      const float2 zp = make_float2(za * mul, zb * mul);
      const __nv_fp8x2_storage_t qh = __nv_cvt_float2_to_fp8x2(zp, __NV_SATFINITE, __NV_E4M3);
      const float2 fh = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(qh, __NV_E4M3)));
      const __nv_fp8x2_storage_t ql = __nv_cvt_float2_to_fp8x2(make_float2(zp.x - fh.x, zp.y - fh.y), __NV_SATFINITE, __NV_E4M3);
      const float2 fl = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(ql, __NV_E4M3)));
      c_sum = fmaf(v0, (fh.x + fl.x) + (fh.y + fl.y), c_sum);
      z_sum += za + zb;
      h32 |= (uint32_t)qh << (16 * cp);
      l32 |= (uint32_t)ql << (16 * cp);
    }
    hi[il] = h32;
    lo[il] = l32;
  }
  // n = r (hi) and n = 16 + r (lo); 16 consecutive k bytes starting at 16*kh
  const int off_hi = (r % 8) * 16 + (r / 8) * 256 + kh * 128;
  const int off_lo = (r % 8) * 16 + ((16 + r) / 8) * 256 + kh * 128;
  *reinterpret_cast<uint4*>(tile + off_hi) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<uint4*>(tile + off_lo) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  // constant of this (block, chunk, rank): C_r / s_r + sum Z over the chunk's columns
  kred[word][kh][r] = c_sum * inv_scale + z_sum;
  __syncthreads();
  if (tid < 16) {
    float v = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) v += kred[i][0][tid] + kred[i][1][tid];
    P.kconst[(((int64_t)blockIdx.y * P.n_chunks + chunk) * R + row) * 16 + tid] = v;
  }
  if (tid == 0) TL_MAX(2);
}

// cycle accounting for the optional trace (one elected lane per role writes)
#ifdef BSB_TRACE
#define TR_BEGIN(var) const long long var = tr ? clock64() : 0
#define TR_ADD(slot, var) do { if (tr) S.trace[slot] += (unsigned long long)(clock64() - var); } while (0)
#else
#define TR_BEGIN(var) do { } while (0)
#define TR_ADD(slot, var) do { } while (0)
#endif
// wall-clock mark of one thread into the CTA's trace record (slots 16-31)
#ifdef BSB_TRACE
#define TR_NS(slot) do { if (P.trace) P.trace[(int64_t)blockIdx.x * 32 + (slot)] = global_ns(); } while (0)
#else
#define TR_NS(slot) do { } while (0)
#endif
// timing experiments of the tuning build select a mode at run time; the product build has none of it
#ifdef BSB_TUNING
#define DBG_IS(n) (P.dbg == (n))
#else
#define DBG_IS(n) false
#endif
// a wait gave up: record the first such event of the device (sticky until the host reads it) and mark the CTA
#define GIVE_UP(code) do { atomicCAS(P.status, 0, (code)); S.failed = 1; } while (0)

// ------------------------------------------------------------------ main kernel
// Work is the sequence of STEPS (weight, row group, block, chunk) in that order, a step being one
// 512-column chunk of one block for the RT 128-row tiles of a row group.  Every CTA takes the same
// number of consecutive steps (stream-K): the grid fills both CTA slots of every multiprocessor
// whatever the shape, at the price that a row group may be shared by several CTAs.  Within its
// range a CTA meets BLOCK SEGMENTS (consecutive chunks of one block: one accumulate / epilogue
// cycle) and ROW SEGMENTS (consecutive block segments of one row group: one output flush).  A row
// group that lies wholly inside one CTA is written directly; otherwise each CTA delivers fp32
// partial sums and the last CTA to arrive adds them in CTA order (deterministic, no float atomics).
//
// A single thread can only issue a tcgen05.mma every ~28 ns (and a commit costs it ~60 ns)
// while the tensor pipe itself accepts several such streams side by side, so the CTA runs TWO
// independent operand pipelines, each a group of four producer warps feeding one MMA issuer
// with its own accumulators:
//   RT == 1: pipeline e takes the e-th 32 bytes of every 64-byte sign row (K halves of one row
//            tile); the epilogue adds the two accumulators.
//   RT == 2: pipeline e takes row tile e (all 64 bytes of a row); both pipelines read the SAME
//            Z' slab, which halves the Z' traffic from L2 per sign byte.
// Every D is double buffered across block segments.  Tensor-memory columns:
//   D(e, b) = e*64 + b*32           (4 x 32)
//   A(e, s) = 128 + e*64 + s*32     (2 issuers x 2 stages x 4 MMAs)
// R = input rows per pass (1 or 2).  With two rows the B operand is 64 columns wide (one MMA serves both
// rows: the sign expansion, the tensor-memory stores and the MMA issue are paid once), the Z' slab of a
// step is 32 KB, and the accumulators (64 columns each) are single-buffered to stay inside 256 columns.
template <int R>
struct __align__(1024) SmemLayout {
  static constexpr int kSlabs = (R == 1) ? kNZ : 2;          // Z' slabs resident
  static constexpr int kSignTiles = (R == 1) ? 6 : 4;        // sign tiles resident
  uint8_t zs[kSlabs][kChunkBytes * R];  // Z' operand slabs (bulk-copied)
  uint8_t sg[kSignTiles * kSignTileBytes];   // sign tiles: row r at r*64, 16-byte piece p at ((p ^ ((r>>1)&3)) * 16)
  uint64_t afull[2][2], aempty[2][2], zfull[kSlabs], zempty[kSlabs], sfull[6], sempty[6], dfull[2][2], dempty[2];
#ifdef BSB_TRACE
  unsigned long long trace[16];
#endif
  uint32_t tmem_base;
  int failed;                           // a wait of this CTA gave up: its outputs are marked NaN
  int n_pending;
  int pending[2][2];                    // row groups shared with other CTAs (at most the first and the last): weight, row group
  int last[2];                          // this CTA was the last to deliver row group pending[q]
};

constexpr int kWarpMma = 8;     // warps 8, 9: MMA issuers 0, 1
constexpr int kWarpLoad = 10;   // warp 10: tensor-memory allocation, sign tiles (TMA); warp 11: Z' slabs (bulk copies)
constexpr int kWarpEpi = 12;    // warps 12-15: epilogue (tensor-memory lane quarters 0-3)

// one output element: fp16 (rounded once), or fp32 when the call delivers partial sums
__device__ __forceinline__ void store_y(const TcParams& P, int wi, int r, int m, float v) {
  const int64_t i = (int64_t)r * P.y_stride[wi] + m;
  if (P.out_f32) reinterpret_cast<float*>(P.y[wi])[i] = v;
  else P.y[wi][i] = __float2half_rn(v);
}
__device__ __forceinline__ int first_step_of_cta(const TcParams& P, int c) {
  return c < P.n_first ? c * P.steps_first : P.n_first * P.steps_first + (c - P.n_first) * P.steps_per_cta;
}
__device__ __forceinline__ int cta_of_step(const TcParams& P, int step) {
  const int b = P.n_first * P.steps_first;
  return step < b ? step / P.steps_first : P.n_first + (step - b) / P.steps_per_cta;
}

// position of a step in (weight, row group, block, chunk) order
struct Walk {
  int wi, rg, js, ci, NB, n_rg;
  __device__ __forceinline__ void init(const TcParams& P, int step, int rows_per_group) {
    wi = 0;
    while (wi + 1 < P.n_weights && step >= P.step_base[wi + 1]) ++wi;
    load(P, rows_per_group);
    const int local = step - P.step_base[wi];
    const int per_rg = NB * P.n_chunks;
    rg = local / per_rg;
    const int rem = local - rg * per_rg;
    js = rem / P.n_chunks;
    ci = rem - js * P.n_chunks;
  }
  __device__ __forceinline__ void load(const TcParams& P, int rows_per_group) {
    NB = P.w[wi].blocks;
    n_rg = (P.w[wi].out_features + rows_per_group - 1) / rows_per_group;
  }
  // advance by n chunks that stay inside the current block
  __device__ __forceinline__ void advance(const TcParams& P, int rows_per_group, int n = 1) {
    ci += n;
    if (ci >= P.n_chunks) {
      ci = 0;
      if (++js == NB) {
        js = 0;
        if (++rg == n_rg) {
          rg = 0;
          if (wi + 1 < P.n_weights) { ++wi; load(P, rows_per_group); }
        }
      }
    }
  }
};

template <int RT, int R>
__global__ void __launch_bounds__(kThreads, 2) gemv_tc5_kernel(const __grid_constant__ TcParams P) {
  using Smem = SmemLayout<R>;
  constexpr int kSlotBytes = RT * kSignTileBytes;   // one ring slot = the RT sign tiles of a step
  constexpr int kNS = Smem::kSignTiles / RT;        // ring slots
  constexpr int kNZr = Smem::kSlabs;                // Z' ring slots
  constexpr int kSlabBytes = kChunkBytes * R;       // Z' slab of one step
  constexpr int kND = (R == 1) ? 2 : 1;             // accumulator buffers per pipeline
  constexpr int kDCols = 32 * R;                    // columns of one accumulator
  constexpr int kPP = 2 * RT;                       // operand stages (4 MMAs each) per step and pipeline
  constexpr int kRows = RT * kTileRows;             // rows of a row group
  extern __shared__ uint8_t smem_raw[];
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  pdl_trigger();   // the kernel after this one may be launched; it waits for this grid before it reads y
  if (threadIdx.x == 0) { TL_MIN(3); TL_MAX(8); }
  const int NCH = P.n_chunks;
  const int step0 = first_step_of_cta(P, blockIdx.x);
  const int total = min((int)blockIdx.x < P.n_first ? P.steps_first : P.steps_per_cta, P.step_base[P.n_weights] - step0);   // steps of this CTA

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // trace slots: 0-3 producer group 0 (total, tile wait, ring wait, expand+store), 4-8 issuer 0 (total,
  // Z' wait, operand wait, accumulator wait, issue), 9-10 epilogue (accumulator wait, total), 11 loader
  // wait, 12 CTA total, 13 set-up
#ifdef BSB_TRACE
  unsigned long long* tr = (P.trace && lane == 0 && (warp == 0 || warp == kWarpMma || warp == kWarpLoad || warp == kWarpEpi))
                               ? P.trace + (int64_t)blockIdx.x * 32 : nullptr;
#endif
  TR_BEGIN(t_cta);
  const unsigned long long wait_ns = P.wait_ns;

  // ---- set-up ---------------------------------------------------------------------
  if (warp == kWarpLoad) {
    tmem_alloc(&S.tmem_base, kTmemCols);
    tmem_relinquish();
  }
#ifdef BSB_TRACE
  if (tid < 14) S.trace[tid] = 0;
#endif
  if (tid == 0) {
    S.n_pending = 0;
    S.failed = 0;
#ifdef BSB_TRACE
    S.trace[14] = global_ns();   // wall-clock start / end of the CTA body (slots 14, 15)
#endif
    for (int e = 0; e < 2; ++e)
      for (int i = 0; i < 2; ++i) {
        mbar_init(&S.afull[e][i], kTileRows);
        mbar_init(&S.aempty[e][i], 1);
        mbar_init(&S.dfull[e][i], 1);
      }
    for (int i = 0; i < kNZr; ++i) { mbar_init(&S.zfull[i], 1); mbar_init(&S.zempty[i], 2); }
    for (int i = 0; i < kNS; ++i) { mbar_init(&S.sfull[i], 1); mbar_init(&S.sempty[i], 2 * kTileRows); }
    for (int i = 0; i < 2; ++i) mbar_init(&S.dempty[i], kTileRows);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = S.tmem_base;
  const uint32_t colA = 2 * kND * kDCols;   // = 128: accumulators D(e, b) at (e*kND + b)*kDCols, operand stages behind them
#ifdef BSB_TRACE
  if (tid == 0) { unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid)); S.trace[13] = smid; }   // slot 13: the multiprocessor
#endif

  if (warp == kWarpLoad) {
    // ---- sign loader: tiled TMA into the tile ring (the packed signs do not depend on the Z'
    //      kernel, so this role never waits for it) -------------------------------------------
    if (lane == 0) {
      Walk wk;
      wk.init(P, step0, kRows);
      for (int g = 0; g < total; ++g) {
        const int slot = g % kNS, n = g / kNS;
        TR_BEGIN(t0);
        if (n >= 1 && !mbar_wait(&S.sempty[slot], (n - 1) & 1, wait_ns)) { GIVE_UP(7); break; }
        TR_ADD(11, t0);
        mbar_expect_tx(&S.sfull[slot], kSlotBytes);
#pragma unroll
        for (int t = 0; t < RT; ++t)   // rows past the end of the weight read as zeros
          tma_load_3d(S.sg + slot * kSlotBytes + t * kSignTileBytes, &P.sign_map[wk.wi], wk.ci * (kChunkCols / 8),
                      wk.rg * kRows + t * kTileRows, wk.js, &S.sfull[slot]);
        wk.advance(P, kRows);
      }
      TR_NS(19);
    }
  } else if (warp == kWarpLoad + 1) {
    // ---- Z' loader: one 16 KB bulk copy per step ---------------------------------------------
    if (lane == 0 && !DBG_IS(2) && !DBG_IS(3)) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      Walk wk;
      wk.init(P, step0, kRows);
      for (int g = 0; g < total; ++g) {
        const int slot = g % kNZr, n = g / kNZr;
        if (n >= 1 && !mbar_wait(&S.zempty[slot], (n - 1) & 1, wait_ns)) { GIVE_UP(1); break; }
        const uint8_t* zsrc = P.zops + ((int64_t)(P.blk_base[wk.wi] + wk.js) * NCH + wk.ci) * kSlabBytes;
        mbar_expect_tx(&S.zfull[slot], kSlabBytes);
        bulk_g2s(S.zs[slot], zsrc, kSlabBytes, &S.zfull[slot]);
        if (g == 0) TR_NS(24);
        wk.advance(P, kRows);
      }
      TR_NS(20);
    }
  } else if (warp == kWarpMma || warp == kWarpMma + 1) {
    // ---- MMA issuer e: RT == 1: words 8e .. 8e+7 of every chunk; RT == 2: all 16 words for row
    //      tile e; accumulator D(e, parity of the block segment) -----------------------------
    // The whole warp runs the loop and the waits (a warp-wide poll costs the same issue slots as a
    // one-lane poll) so that addresses and descriptors stay warp-uniform values; one elected lane
    // issues the MMAs and commits.
    if (!DBG_IS(2)) {
      const int e = warp - kWarpMma;
#ifdef BSB_TRACE
      if (e != 0) tr = nullptr;
#endif
      const bool leader = elect_one();
      const uint32_t idesc = make_idesc_f8(128, kDCols);
      Walk wk;
      wk.init(P, step0, kRows);
      int it = 0, bs = 0;       // operand stages and block segments so far
      bool first = true;        // first step of a block segment
      bool ok = true;
      TR_BEGIN(t_mma);
      for (int g = 0; g < total && ok; ++g) {
        const int b = bs % kND;
        if (first && bs >= kND) {
          TR_BEGIN(t0);
          if (!mbar_wait(&S.dempty[b], ((bs / kND) - 1) & 1, wait_ns)) { if (leader) GIVE_UP(6); ok = false; break; }
          TR_ADD(7, t0);
          tc_fence_after();
        }
        const int zslot = g % kNZr;
        TR_BEGIN(t1);
        if (!mbar_wait(&S.zfull[zslot], (g / kNZr) & 1, wait_ns)) { if (leader) GIVE_UP(2); ok = false; break; }
        TR_ADD(5, t1);
        if (g == 0 && leader) { TL_MIN(4); TL_MAX(11); if (e == 0) TR_NS(21); }
        const uint32_t zaddr = smem_u32(S.zs[zslot]) + (RT == 1 ? (uint32_t)e * 8u * 1024u * R : 0u);
        const uint32_t dcol = tbase + (e * kND + b) * kDCols;
#pragma unroll 1
        for (int pp = 0; pp < kPP; ++pp, ++it) {
          const int slot = it & 1;
          TR_BEGIN(t2);
          if (!DBG_IS(1) && !mbar_wait(&S.afull[e][slot], (it >> 1) & 1, wait_ns)) { if (leader) GIVE_UP(3); ok = false; break; }
          TR_ADD(6, t2);
          TR_BEGIN(t3);
          tc_fence_after();
          const uint64_t bdesc = make_smem_desc(zaddr + (uint32_t)(pp * 4) * 1024u * R, 128, 256);
          const uint32_t acol = tbase + colA + e * 64 + slot * 32;
          if (leader) {
            // R KB operand tiles follow each other: the descriptor's address field counts 16-byte units
            mma_ts_f8_first(dcol, acol, bdesc, idesc, (!first || pp > 0) ? 1u : 0u);
            mma_ts_f8_acc(dcol, acol + 8, bdesc + 64 * R, idesc);
            mma_ts_f8_acc(dcol, acol + 16, bdesc + 128 * R, idesc);
            mma_ts_f8_acc(dcol, acol + 24, bdesc + 192 * R, idesc);
            mma_commit(&S.aempty[e][slot]);
          }
          TR_ADD(8, t3);
        }
        if (!ok) break;
        const bool seg_end = (wk.ci == NCH - 1) || (g == total - 1);
        if (leader) {
          mma_commit(&S.zempty[zslot]);
          if (seg_end) mma_commit(&S.dfull[e][b]);
        }
        if (seg_end) ++bs;
        first = seg_end;
        wk.advance(P, kRows);
      }
      TR_ADD(4, t_mma);
      if (leader && e == 0) TR_NS(17);
    }
  } else if (warp < kWarpMma) {
    // ---- producer group e: one sign row per thread.  RT == 1: bytes 32e .. 32e+31 of the row
    //      of the only tile; RT == 2: all 64 bytes of the row of tile e ----------------------
    if (!DBG_IS(1)) {
      const int e = warp >> 2;
#ifdef BSB_TRACE
      if (e != 0) tr = nullptr;
#endif
      const int rtid = tid & (kTileRows - 1);
      const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16) + colA + e * 64;
      const int sw = (rtid >> 1) & 3;   // 64-byte swizzle of the TMA tile
      const int tile_off = (RT == 1 ? 0 : e * kSignTileBytes) + rtid * 64;
      const int piece0 = (RT == 1 ? e * 2 : 0);
      // OR-constants of the eight bit classes, held in registers so that one LOP3 expands four signs
      uint32_t cc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) asm volatile("mov.u32 %0, %1;" : "=r"(cc[i]) : "r"(class_byte(i) * 0x01010101u));
      bool ok = true;
      TR_BEGIN(t_prod);
#pragma unroll 1
      for (int g = 0; g < total && ok; ++g) {
        const int slot_s = g % kNS;
        TR_BEGIN(t0);
        const bool landed = mbar_wait_group(&S.sfull[slot_s], (g / kNS) & 1, wait_ns);
        TR_ADD(1, t0);
        if (!landed) { GIVE_UP(8); ok = false; break; }
        const uint8_t* srow = S.sg + slot_s * kSlotBytes + tile_off;
        // two 16-byte pieces are in registers at a time; the slot may be refilled once all 256
        // readers have taken their last piece
        uint4 v[2];
#pragma unroll
        for (int pp = 0; pp < kPP; ++pp) {
          if ((pp & 1) == 0) {
            v[0] = *reinterpret_cast<const uint4*>(srow + (((piece0 + pp) ^ sw) << 4));
            v[1] = *reinterpret_cast<const uint4*>(srow + (((piece0 + pp + 1) ^ sw) << 4));
            if (pp == kPP - 2) mbar_arrive(&S.sempty[slot_s]);
          }
          const int it = g * kPP + pp, slot = it & 1;
          TR_BEGIN(t2);
          uint32_t r[32];
          const uint32_t wd[4] = {v[pp & 1].x, v[pp & 1].y, v[pp & 1].z, v[pp & 1].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) expand_word_c(wd[q], cc, r + q * 8);
          TR_ADD(3, t2);
          if (it >= 2 && !DBG_IS(2)) {
            TR_BEGIN(t1);
            const bool got = mbar_wait_group(&S.aempty[e][slot], ((it >> 1) - 1) & 1, wait_ns);
            TR_ADD(2, t1);
            if (!got) { GIVE_UP(4); ok = false; break; }
            tc_fence_after();
          }
          // store and hand over at once: with only two stages per issuer every nanosecond of
          // hand-off latency is on the critical path
          tmem_st32(lane_base + slot * 32, r);
          tmem_wait_st();
          tc_fence_before();
          if (!DBG_IS(2)) mbar_arrive(&S.afull[e][slot]);
        }
      }
      TR_ADD(0, t_prod);
      if (tid == 0) TR_NS(16);
    }
  } else if (warp >= kWarpEpi) {
    // ---- epilogue warps: y[m] += sum_r U_j[m,r] (T[m,r] / s_r - K_r) per block segment; T = sum
    //      of the hi and lo pieces (RT == 1: of both issuers' accumulators) ------------------
    if (!DBG_IS(1) && !DBG_IS(2)) {
    asm volatile("griddepcontrol.wait;" ::: "memory");   // constants below come from the Z' kernel
    const int quarter = warp & 3;                     // tensor-memory lanes this warp may read
    const int rtid = quarter * 32 + lane;
    const uint32_t lane_base = tbase + ((uint32_t)(quarter * 32) << 16);
    float yacc[RT][R];
#pragma unroll
    for (int t = 0; t < RT; ++t)
#pragma unroll
      for (int r = 0; r < R; ++r) yacc[t][r] = 0.f;
    bool ok = true;
    Walk wk;
    wk.init(P, step0, kRows);
    bool whole = (wk.js == 0 && wk.ci == 0);   // the current row group began inside this CTA
    bool first_seg = true;                    // partial-sum slot 0 belongs to the CTA's first row segment, slot 1 to any later one
    int n_pend = 0;
    TR_BEGIN(t_epi);
#pragma unroll 1
    for (int g = 0, bs = 0; g < total; ++bs) {
      const int len = min(NCH - wk.ci, total - g);    // chunks of this block segment
      const bsb_weight& w = P.w[wk.wi];
      const int M = w.out_features;
      const int j = wk.js, b = bs % kND;
      const int row0 = wk.rg * kRows;
      const int jb = P.blk_base[wk.wi] + j;
      // operands of this block segment's epilogue, fetched while its MMAs run
      uint4 uq[RT][2];
#pragma unroll
      for (int t = 0; t < RT; ++t) {
        const int row = min(row0 + t * kTileRows + rtid, M - 1);
        const __half* u = reinterpret_cast<const __half*>(w.u) + (int64_t)j * w.u_block_stride + (int64_t)row * 16;
        uq[t][0] = __ldg(reinterpret_cast<const uint4*>(u));
        uq[t][1] = __ldg(reinterpret_cast<const uint4*>(u) + 1);
      }
      float inv_mine[R], k_mine[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        inv_mine[r] = 0.f;
        k_mine[r] = 0.f;
        if (lane < 16) {
          inv_mine[r] = P.inv_scale[((int64_t)jb * R + r) * 16 + lane];
          const float* kc = P.kconst + (((int64_t)jb * NCH + wk.ci) * R + r) * 16 + lane;
          for (int c = 0; c < len; ++c) k_mine[r] += kc[c * R * 16];
        }
      }
      TR_BEGIN(t0);
      if (RT == 1) {
        const bool both = mbar_wait_warp(&S.dfull[0][b], (bs / kND) & 1, wait_ns) && mbar_wait_warp(&S.dfull[1][b], (bs / kND) & 1, wait_ns);
        if (!both) { if (lane == 0) GIVE_UP(5); ok = false; break; }
      }
      TR_ADD(9, t0);
#pragma unroll
      for (int t = 0; t < RT; ++t) {
        if (RT == 2) {
          if (!mbar_wait_warp(&S.dfull[t][b], (bs / kND) & 1, wait_ns)) { if (lane == 0) GIVE_UP(5); ok = false; break; }
        }
        tc_fence_after();
        const uint32_t* uw = reinterpret_cast<const uint32_t*>(&uq[t][0]);
#pragma unroll
        for (int r = 0; r < R; ++r) {     // input row r = accumulator columns 32r .. 32r+31
#pragma unroll
        for (int h = 0; h < 2; ++h) {   // ranks 8h .. 8h+7
          float T[8];
          uint32_t d0[8], d1[8];
          const uint32_t c0 = lane_base + ((RT == 1 ? 0 : t * kND) + b) * kDCols + r * 32 + h * 8;
          tmem_ld8(c0, d0);        // hi piece
          tmem_ld8(c0 + 16, d1);   // lo piece
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) T[i] = __uint_as_float(d0[i]) + __uint_as_float(d1[i]);
          if (RT == 1) {           // second issuer's accumulator (other K half)
            tmem_ld8(c0 + kND * kDCols, d0);
            tmem_ld8(c0 + kND * kDCols + 16, d1);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i) T[i] += __uint_as_float(d0[i]) + __uint_as_float(d1[i]);
          }
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int r0 = 8 * h + 2 * rr;
            const __half2 h2 = *reinterpret_cast<const __half2*>(&uw[4 * h + rr]);
            const float i0 = __shfl_sync(0xFFFFFFFFu, inv_mine[r], r0), i1 = __shfl_sync(0xFFFFFFFFu, inv_mine[r], r0 + 1);
            const float k0 = __shfl_sync(0xFFFFFFFFu, k_mine[r], r0), k1 = __shfl_sync(0xFFFFFFFFu, k_mine[r], r0 + 1);
            yacc[t][r] = fmaf(__low2float(h2), T[2 * rr] * i0 - k0, yacc[t][r]);
            yacc[t][r] = fmaf(__high2float(h2), T[2 * rr + 1] * i1 - k1, yacc[t][r]);
          }
        }
        }
      }
      if (!ok) break;
      tc_fence_before();
      mbar_arrive(&S.dempty[b]);
      g += len;
      // end of the row segment: the row group ends here, or the CTA does
      const bool group_end = (wk.js == wk.NB - 1) && (wk.ci + len == NCH);
      if (group_end || g == total) {
        const bool direct = whole && group_end;
        float* part = P.partials + ((int64_t)blockIdx.x * 2 + (first_seg ? 0 : 1)) * (R * kRows);
#pragma unroll
        for (int t = 0; t < RT; ++t) {
          const int m = row0 + t * kTileRows + rtid;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            if (direct) {
              if (m < M) {
                float v = yacc[t][r];
                if (w.bias) v += __half2float(reinterpret_cast<const __half*>(w.bias)[m]);
                store_y(P, wk.wi, r, m, v);
              }
            } else {
              part[r * kRows + t * kTileRows + rtid] = yacc[t][r];
            }
            yacc[t][r] = 0.f;
          }
        }
        if (!direct) {   // (made visible to the other CTAs by the counting thread's fence at the end of the kernel)
          if (rtid == 0) {
            S.pending[n_pend][0] = wk.wi;
            S.pending[n_pend][1] = wk.rg;
            S.n_pending = n_pend + 1;
          }
          ++n_pend;
        }
        whole = true;
        first_seg = false;
      }
      wk.advance(P, kRows, len);
    }
    TR_ADD(10, t_epi);
    if (warp == kWarpEpi && lane == 0) { TL_MAX(5); TR_NS(18); }
    }
  }

  // ---- tear-down: tensor memory is released only after every role is done ---------------
  tc_fence_before();
  __syncthreads();
#ifdef BSB_TRACE
  if (warp == 0) TR_ADD(12, t_cta);
  if (P.trace) {
    if (tid == 0) S.trace[15] = global_ns();
    __syncthreads();
    if (tid < 16) P.trace[(int64_t)blockIdx.x * 32 + tid] = S.trace[tid];
  }
#endif
  if (warp == kWarpLoad) {
    __syncwarp();
    tmem_dealloc(tbase, kTmemCols);
  }
  // ---- a wait of this CTA gave up: everything the CTA was to produce becomes NaN (outputs it owns alone directly,
  //      shared row groups through its partial sums), so a timed-out call can never pass for a result ----
  if (S.failed) {
    const float nan = __int_as_float(0x7FC00000);
    int g = 0, n_pend = 0;
    bool first_seg = true;
    while (g < total) {
      Walk wk;
      wk.init(P, step0 + g, kRows);
      const int rem = (wk.NB - wk.js) * NCH - wk.ci;   // steps left in this row group
      const int len = min(rem, total - g);
      const bool direct = (wk.js == 0 && wk.ci == 0) && len == rem;
      const bsb_weight& w = P.w[wk.wi];
      float* part = P.partials + ((int64_t)blockIdx.x * 2 + (first_seg ? 0 : 1)) * (R * kRows);
      if (tid < kRows) {
        const int m = wk.rg * kRows + tid;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (!direct) part[r * kRows + tid] = nan;
          else if (m < w.out_features) store_y(P, wk.wi, r, m, nan);
        }
      }
      if (!direct) {
        if (tid == 0) {
          S.pending[n_pend][0] = wk.wi;
          S.pending[n_pend][1] = wk.rg;
        }
        ++n_pend;
      }
      first_seg = false;
      g += len;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) S.n_pending = n_pend;
    __syncthreads();
  }
  // ---- shared row groups: the last CTA to deliver adds the partial sums in CTA order ------
  // Both row groups of the CTA are handled side by side: thread 0 counts the first one in, thread 256 the second, and
  // threads 0-255 / 256-511 add up whichever of the two this CTA completed.  The block barrier above ordered every
  // thread's partial sums before the counting thread's release, which orders them before the count; on the reading
  // side the acquiring count and the barrier below order the other CTAs' sums before the loads (strong loads, from L2).
  const int n_pending = S.n_pending;
  if (tid == 0) { TL_MAX(6); TL_MIN(10); TR_NS(22); }
  if (n_pending == 0) return;
  asm volatile("griddepcontrol.wait;" ::: "memory");     // the counters were zeroed by the Z' kernel
  const int q = tid >> 8, rl = tid & 255;
  int wi = 0, rg = 0, gs = 0, c_first = 0, c_last = -1;
  if (q < n_pending) {
    wi = S.pending[q][0];
    rg = S.pending[q][1];
    const int per_rg = P.w[wi].blocks * NCH;
    gs = P.step_base[wi] + rg * per_rg;                                   // steps gs .. gs + per_rg - 1 are the row group's
    c_first = cta_of_step(P, gs);
    c_last = cta_of_step(P, gs + per_rg - 1);
    if (rl == 0) {
      int old;   // release of this CTA's sums and acquire of the others' in one operation
      asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(P.counters + P.seg_base[wi] + rg) : "memory");
      S.last[q] = (old == c_last - c_first);
    }
  }
  __syncthreads();
  if (q < n_pending && S.last[q]) {
    const bsb_weight& w = P.w[wi];
    const int m = rg * kRows + rl;
    if (rl < kRows && m < w.out_features) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float sum = 0.f;
        // kFix loads in flight at a time; the additions stay in CTA order (bit-identical run to run)
        constexpr int kFix = (R == 1) ? 16 : 8;
        for (int c0 = c_first; c0 <= c_last; c0 += kFix) {
          float v[kFix];
#pragma unroll
          for (int i = 0; i < kFix; ++i) {
            const int c = min(c0 + i, c_last);
            // the row group is CTA c's first row segment unless it starts after c's first step
            const int slot = (gs <= first_step_of_cta(P, c)) ? 0 : 1;
            asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v[i]) : "l"(P.partials + (((int64_t)c * 2 + slot) * R + r) * kRows + rl));
            if (c0 + i > c_last) v[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < kFix; ++i) sum += v[i];
        }
        if (w.bias) sum += __half2float(reinterpret_cast<const __half*>(w.bias)[m]);
        store_y(P, wi, r, m, sum);
      }
    }
  }
  if (tid == 0) { TL_MAX(6); TR_NS(23); }
}

struct TcPlan {
  TcParams P;
  int64_t bytes;
  int total_blocks, total_items;
  int row_tiles;                    // RT: 128-row tiles per CTA (1 or 2)
  int64_t absmax_off[kMaxGroup];
};

constexpr int kMinStepsPair = 1;   // measured: two row tiles per CTA are as fast or faster as soon as every CTA still gets a step
#ifdef BSB_TUNING
static int g_force_rt = 0;      // 0 = choose, 1 / 2 = forced
static int g_target_ctas = 0;   // 0 = two per multiprocessor, else this many
constexpr int kMinStepsUneven = 4;      // steps per CTA from which the two waves get different shares
// steps of a first-wave CTA per 100 of a second-wave one.  140 makes an isolated launch 5-8 % faster (the two CTAs of a
// multiprocessor then finish together) but a decode step 6 % SLOWER: with kernels queued back to back the first 148 CTAs
// are not placed one per multiprocessor, and two long CTAs can share one.  Equal shares (100) are the product's choice.
static int g_older_share_pct = 100;
#endif

// R = input rows per pass (1 or 2).
void make_tc_plan(const bsb_weight* ws, int n, int R, TcPlan& pl) {
  TcParams& P = pl.P;
  memset(&P, 0, sizeof(P));
  P.n_weights = n;
  P.rows = R;
  const int N = ws[0].in_features;
  P.n_chunks = (int)ceil_div64(N, kChunkCols);
  // CTAs wanted: two per multiprocessor (both stay resident and share its tensor pipe)
#ifdef BSB_TUNING
  const int target = g_target_ctas > 0 ? g_target_ctas : sm_count() * 2;
#else
  const int target = sm_count() * 2;
#endif
  int64_t steps1 = 0, steps2 = 0;
  for (int i = 0; i < n; ++i) {
    steps1 += ceil_div64(ws[i].out_features, kTileRows) * ws[i].blocks * P.n_chunks;
    steps2 += ceil_div64(ws[i].out_features, 2 * kTileRows) * ws[i].blocks * P.n_chunks;
  }
  // two row tiles per CTA halve the Z' traffic; taken when every CTA still gets a step
  int RT = (steps2 >= (int64_t)target * kMinStepsPair) ? 2 : 1;
#ifdef BSB_TUNING
  if (g_force_rt) RT = g_force_rt;
#endif
  pl.row_tiles = RT;
  const int64_t steps = RT == 2 ? steps2 : steps1;
  int L = (int)ceil_div64(steps, target);
  if (L < 1) L = 1;
  P.steps_per_cta = L;
  P.n_first = 0;
  P.steps_first = L;
  int grid = (int)ceil_div64(steps, L);
#ifdef BSB_TUNING
  const int sms = sm_count();
  if (g_older_share_pct > 100 && target == 2 * sms && steps >= (int64_t)target * kMinStepsUneven) {
    // two waves of one CTA per multiprocessor: the second wave's share is 1 / (1 + older share)
    const int64_t den = (int64_t)sms * (100 + g_older_share_pct);
    const int L2 = (int)((steps * 100 + den / 2) / den);   // nearest
    const int L1 = (int)ceil_div64(steps - (int64_t)sms * L2, sms);
    if (L2 >= 1 && L1 >= L2) {
      P.n_first = sms;
      P.steps_first = L1;
      P.steps_per_cta = L2;
      const int64_t rest = steps - (int64_t)sms * L1;
      grid = sms + (rest > 0 ? (int)ceil_div64(rest, L2) : 0);
    }
  }
#endif
  int segs = 0, blks = 0;
  int64_t st = 0;
  for (int i = 0; i < n; ++i) {
    P.w[i] = ws[i];
    const int n_rg = (int)ceil_div64(ws[i].out_features, RT * kTileRows);
    P.step_base[i] = (int)st;
    P.seg_base[i] = segs;
    P.blk_base[i] = blks;
    st += (int64_t)n_rg * ws[i].blocks * P.n_chunks;
    segs += n_rg;
    blks += ws[i].blocks;
  }
  P.step_base[n] = (int)st;
  P.seg_base[n] = segs;
  P.blk_base[n] = blks;
  const int tiles = segs;
  const int items = grid;
  const int64_t part_floats = (int64_t)grid * 2 * R * RT * kTileRows;
  pl.total_blocks = blks;
  pl.total_items = items;
  int64_t off = 0;
  const int64_t z_off = off;
  off = align_up64(off + (int64_t)blks * P.n_chunks * kChunkBytes * R, 256);
  const int64_t k_off = off;
  off = align_up64(off + (int64_t)blks * P.n_chunks * R * 16 * 4, 256);
  const int64_t s_off = off;
  off = align_up64(off + (int64_t)blks * R * 16 * 4, 256);
  const int64_t c_off = off;
  off = align_up64(off + (int64_t)tiles * 4, 256);
  const int64_t p_off = off;
  off = align_up64(off + part_floats * 4, 256);
  for (int i = 0; i < n; ++i) {
    pl.absmax_off[i] = off;
    off = align_up64(off + (int64_t)ws[i].blocks * 16 * 4, 256);
  }
  pl.bytes = off;
  P.zops = (uint8_t*)z_off;
  P.kconst = (float*)k_off;
  P.inv_scale = (float*)s_off;
  P.counters = (int*)c_off;
  P.partials = (float*)p_off;
}

}  // namespace

// cuTensorMapEncodeTiled is a driver-API symbol; it is looked up through the runtime so that
// the library links against cudart only
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode_fn() {
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

// packed signs of one weight as a 3-D byte tensor [blocks][out][in/8]; one box = 128 rows x 64 bytes
static int make_sign_map(const bsb_weight& w, CUtensorMap* map) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return BSB_ECUDA;
  }
  const cuuint64_t dims[3] = {(cuuint64_t)(w.in_features / 8), (cuuint64_t)w.out_features, (cuuint64_t)w.blocks};
  const cuuint64_t strides[2] = {(cuuint64_t)(w.in_features / 8), (cuuint64_t)(w.blocks > 1 ? w.q_block_stride : (int64_t)w.out_features * (w.in_features / 8))};
  const cuuint32_t box[3] = {64, (cuuint32_t)kTileRows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)w.qweight, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (out=%d in=%d blocks=%d stride=%lld)", (int)r, w.out_features,
              w.in_features, w.blocks, (long long)w.q_block_stride);
    return BSB_ECUDA;
  }
  return BSB_OK;
}

int launch_vt_absmax(const bsb_weight& w, float* out, cudaStream_t s) {
  BSB_CHECK_ARG(w.k == 16, "vt_absmax: only k == 16");
  if (w.blocks == 0) return BSB_OK;
  vt_absmax_kernel<<<dim3(16, w.blocks), 256, 0, s>>>(w, out);
  return check_launch("vt_absmax_kernel");
}

static unsigned long long g_wait_ns = kDefaultWaitNs;
void gemv_tc5_set_wait_limit_ns(unsigned long long ns) { g_wait_ns = ns; }
#ifdef BSB_TUNING
static unsigned long long* g_trace = nullptr;
static int g_dbg = 0;
// wall-clock timeline: every decode call takes the next 12-slot record of a device buffer the caller provides
// (slots 0, 1, 3, 4 preset to ~0ull, the others to 0); -1 capacity = off
static unsigned long long* g_timeline = nullptr;
static int g_timeline_cap = 0, g_timeline_n = 0;
void gemv_tc5_set_timeline(unsigned long long* p, int records) { g_timeline = p; g_timeline_cap = records; g_timeline_n = 0; }
void gemv_tc5_set_dbg(int m) {
  if (m >= 200 && m <= 202) g_force_rt = m - 200;   // row tiles per CTA: 200 = choose, 201 / 202 = forced
  else if (m >= 1000 && m < 2000) g_target_ctas = m - 1000;   // grid size wanted (1000 = default)
  else if (m >= 2100 && m <= 2300) g_older_share_pct = m - 2000;   // first-wave share in percent (2100 = equal)
  else g_dbg = m;
}
void gemv_tc5_set_trace(unsigned long long* p) { g_trace = p; }
#endif

bool gemv_tc5_supported(const bsb_weight& w) {
  return w.k == 16 && w.blocks >= 1 && w.in_features >= 128 && w.in_features % 128 == 0 && w.out_features >= 1 &&
         ((uintptr_t)w.qweight % 16 == 0) && (w.q_block_stride % 16 == 0) &&
         ((uintptr_t)w.vt % 16 == 0) && (w.vt_block_stride % 8 == 0) &&
         ((uintptr_t)w.u % 16 == 0) && (w.u_block_stride % 8 == 0);
}

int64_t gemv_tc5_workspace_bytes(const bsb_weight* ws, int n_weights, int rows_per_pass) {
  if (n_weights < 1 || n_weights > kMaxGroup || rows_per_pass < 1 || rows_per_pass > 2) return -1;
  TcPlan pl;
  make_tc_plan(ws, n_weights, rows_per_pass, pl);
  return pl.bytes;
}

// rows = 1 or 2 input rows in one pass: x rows x_stride apart, row r of weight i goes to ys[i] + r * y_strides[i]
// (y_strides may be nullptr when rows == 1)
int launch_gemv_tc5(const bsb_weight* ws, int n_weights, const __half* x, int64_t x_stride, int rows, __half* const* ys,
                    const int64_t* y_strides, void* workspace, int64_t workspace_bytes, cudaStream_t s, bool out_f32,
                    const float* x_absmax) {
  BSB_CHECK_ARG(n_weights >= 1 && n_weights <= kMaxGroup, "gemv: 1..%d weights per group", kMaxGroup);
  BSB_CHECK_ARG(rows == 1 || (rows == 2 && y_strides != nullptr && x_stride % 8 == 0), "gemv: 1 or 2 rows per pass (16-byte aligned rows)");
  for (int i = 0; i < n_weights; ++i) {
    BSB_CHECK_ARG(gemv_tc5_supported(ws[i]), "gemv: weight %d has an unsupported shape/alignment", i);
    BSB_CHECK_ARG(ws[i].in_features == ws[0].in_features, "gemv: grouped weights must share in_features");
  }
  TcPlan pl;
  make_tc_plan(ws, n_weights, rows, pl);
  if (workspace == nullptr || workspace_bytes < pl.bytes) {
    set_error("gemv: workspace of %lld bytes needed, %lld given", (long long)pl.bytes, (long long)workspace_bytes);
    return BSB_EWORKSPACE;
  }
  BSB_CHECK_ARG((uintptr_t)workspace % 256 == 0, "gemv: workspace must be 256-byte aligned");
  static bool attr_set[64] = {false};
  int dev = 0;
  BSB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    BSB_CUDA(cudaFuncSetAttribute(gemv_tc5_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemLayout<1>) + 1024));
    BSB_CUDA(cudaFuncSetAttribute(gemv_tc5_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemLayout<1>) + 1024));
    BSB_CUDA(cudaFuncSetAttribute(gemv_tc5_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemLayout<2>) + 1024));
    BSB_CUDA(cudaFuncSetAttribute(gemv_tc5_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SmemLayout<2>) + 1024));
    attr_set[dev] = true;
  }
  TcParams& P = pl.P;
  uint8_t* base = (uint8_t*)workspace;
  P.zops = base + (int64_t)(uintptr_t)P.zops;
  P.kconst = (float*)(base + (int64_t)(uintptr_t)P.kconst);
  P.inv_scale = (float*)(base + (int64_t)(uintptr_t)P.inv_scale);
  P.counters = (int*)(base + (int64_t)(uintptr_t)P.counters);
  P.partials = (float*)(base + (int64_t)(uintptr_t)P.partials);
  P.status = device_status_word();
  if (P.status == nullptr) return BSB_ECUDA;
  P.wait_ns = g_wait_ns;
#ifdef BSB_TUNING
  P.trace = g_trace;
  P.dbg = g_dbg;
  P.timeline = (g_timeline && g_timeline_n < g_timeline_cap) ? g_timeline + 12 * (g_timeline_n++) : nullptr;
#endif
  P.x_stride = x_stride;
  P.out_f32 = out_f32 ? 1 : 0;
  P.absmax_const = 1;
  P.x_absmax = x_absmax;
  for (int i = 0; i < n_weights; ++i) {
    P.y[i] = ys[i];
    P.y_stride[i] = y_strides ? y_strides[i] : 0;
    if (int rc = make_sign_map(ws[i], &P.sign_map[i])) return rc;
    if (ws[i].vt_absmax) {
      P.vt_absmax[i] = ws[i].vt_absmax;
    } else {
      P.absmax_const = 0;
      float* am = (float*)(base + pl.absmax_off[i]);
      if (int rc = launch_vt_absmax(ws[i], am, s)) return rc;
      P.vt_absmax[i] = am;
    }
  }
  {
    const dim3 zgrid(P.n_chunks, pl.total_blocks, rows);
    cudaError_t le = launch_pdl(zprep_tc5_kernel, zgrid, dim3(kZprepThreads), 0, s, P, x);
    if (le != cudaSuccess) {
      set_error("launch of zprep_tc5_kernel failed: %s", cudaGetErrorString(le));
      return BSB_ECUDA;
    }
  }
  if (int rc = check_launch("zprep_tc5_kernel")) return rc;
  profile_mark(s, false);
  {
    // programmatic dependent launch: the decode kernel may start while the Z' kernel still runs
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.total_items);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = (rows == 2 ? sizeof(SmemLayout<2>) : sizeof(SmemLayout<1>)) + 1024;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = rows == 2 ? (pl.row_tiles == 2 ? cudaLaunchKernelEx(&cfg, gemv_tc5_kernel<2, 2>, P)
                                                    : cudaLaunchKernelEx(&cfg, gemv_tc5_kernel<1, 2>, P))
                               : (pl.row_tiles == 2 ? cudaLaunchKernelEx(&cfg, gemv_tc5_kernel<2, 1>, P)
                                                    : cudaLaunchKernelEx(&cfg, gemv_tc5_kernel<1, 1>, P));
    if (le != cudaSuccess) {
      set_error("launch of gemv_tc5_kernel failed: %s", cudaGetErrorString(le));
      return BSB_ECUDA;
    }
  }
  profile_mark(s, true);
  return check_launch("gemv_tc5_kernel");
}

#ifdef BSB_TUNING
// ------------------------------------------------------------------ issue-rate probe (tuning build only)
// What one multiprocessor can do with the decode kernel's MMA: every CTA has `issuers` warps (1 or 2), each with its
// own accumulator of n_cols columns and its own barrier; the elected lane of a warp issues `per_commit` M128 x n_cols
// x K32 e4m3 MMAs (A from tensor memory, B from shared memory), commits, waits for the commit -- `iters` times -- and
// reports the wall-clock time of its loop.  alloc_cols (256 or 512 tensor-memory columns per CTA) decides whether two
// CTAs or one fit on a multiprocessor.
namespace {
__global__ void __launch_bounds__(128) mma_rate_kernel(int n_cols, int per_commit, int iters, int issuers, int alloc_cols,
                                                       unsigned long long wait_ns, unsigned long long* ns_out, int* status) {
  __shared__ __align__(1024) uint8_t b_tile[256 * 32];   // up to 256 columns x 32 bytes of K, K-major, no swizzle
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 256 * 32 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(b_tile)[i] = 0x38383838u;   // 1.0
  if (warp == 0) {
    tmem_alloc(&tmem_slot, alloc_cols);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the generic-proxy writes of b_tile before the MMAs read it
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_slot;
  const uint32_t a_col = tbase + issuers * n_cols;   // the A operand: 32 columns behind the accumulators, zeroed
  {
    uint32_t z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) z[i] = 0u;
    tmem_st32(a_col + ((uint32_t)(warp * 32) << 16), z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp < issuers) {
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_f8(128, n_cols);
    const uint64_t bdesc = make_smem_desc(smem_u32(b_tile), 128, 256);
    const uint32_t d = tbase + warp * n_cols;
    const uint64_t t0 = global_ns();
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      if (leader) {
        mma_ts_f8_first(d, a_col, bdesc, idesc, it > 0 ? 1u : 0u);
        for (int k = 1; k < per_commit; ++k) mma_ts_f8_acc(d, a_col, bdesc, idesc);
        mma_commit(&bar[warp]);
      }
      __syncwarp();
      if (!mbar_wait(&bar[warp], it & 1, wait_ns)) {
        if (leader) atomicCAS(status, 0, 90);
        ok = false;
      }
    }
    if (leader) ns_out[blockIdx.x * 2 + warp] = global_ns() - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tmem_dealloc(tbase, alloc_cols);
  }
}
}  // namespace

// ns per MMA per multiprocessor (all issuers of all its CTAs together), from the slowest issuer of the grid
int gemv_tc5_mma_rate(int n_cols, int per_commit, int iters, int issuers, int ctas_per_sm, float* ns_per_mma_per_sm) {
  BSB_CHECK_ARG(n_cols >= 16 && n_cols <= 256 && n_cols % 16 == 0 && per_commit >= 1 && iters >= 1 && (issuers == 1 || issuers == 2) &&
                (ctas_per_sm == 1 || ctas_per_sm == 2) && ns_per_mma_per_sm != nullptr, "mma rate probe: bad arguments");
  const int alloc_cols = ctas_per_sm == 2 ? 256 : 512;
  BSB_CHECK_ARG(issuers * n_cols + 32 <= alloc_cols, "mma rate probe: %d accumulators of %d columns do not fit %d columns", issuers, n_cols, alloc_cols);
  const int grid = sm_count() * ctas_per_sm;
  unsigned long long* d_ns = nullptr;
  BSB_CUDA(cudaMalloc(&d_ns, (size_t)grid * 2 * sizeof(unsigned long long)));
  BSB_CUDA(cudaMemset(d_ns, 0, (size_t)grid * 2 * sizeof(unsigned long long)));
  int* status = device_status_word();
  if (status == nullptr) return BSB_ECUDA;
  // unused dynamic shared memory pins the number of CTAs a multiprocessor can host to ctas_per_sm
  const int dyn_smem = (ctas_per_sm == 2 ? 100 : 200) * 1024;
  BSB_CUDA(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dyn_smem));
  mma_rate_kernel<<<grid, 128, dyn_smem>>>(n_cols, per_commit, iters, issuers, alloc_cols, g_wait_ns, d_ns, status);
  cudaError_t e = cudaDeviceSynchronize();
  std::vector<unsigned long long> h((size_t)grid * 2);
  if (e == cudaSuccess) e = cudaMemcpy(h.data(), d_ns, h.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaFree(d_ns);
  if (e != cudaSuccess) {
    set_error("mma rate probe: %s", cudaGetErrorString(e));
    return BSB_ECUDA;
  }
  unsigned long long worst = 0;
  for (unsigned long long v : h) worst = v > worst ? v : worst;
  *ns_per_mma_per_sm = (float)((double)worst / ((double)iters * per_commit * issuers * ctas_per_sm));
  return BSB_OK;
}
#endif

}  // namespace bsb

// ------------------------------------------------------------------ allocation-free entry point
// Scratch for bsb_linear_forward_noalloc: lives in the library image, so every GPU that loads
// the library holds these bytes until the process exits.
static constexpr int64_t kNoAllocScratchBytes = 16ll << 20;
static __device__ __align__(256) uint8_t g_noalloc_scratch[kNoAllocScratchBytes];

extern "C" int64_t bsb_noalloc_scratch_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int bsb_linear_forward_noalloc(const bsb_weight* w, const uint16_t* x, int64_t rows, int64_t x_stride,
                                          uint16_t* y, int64_t y_stride, void* stream) {
  using namespace bsb;
  BSB_CHECK_ARG(w != nullptr && x != nullptr && y != nullptr, "NULL argument");
  if (int rc = check_weight(w)) return rc;   // same dimension / block-stride checks as every other forward entry
  BSB_CHECK_ARG(rows >= 1, "at least one input row is needed");
  BSB_CHECK_ARG(w->blocks >= 1 && gemv_tc5_supported(*w),
                "noalloc forward: needs k == 16, in_features %% 128 == 0, 16-byte aligned tensors, >= 1 active block");
  BSB_CHECK_ARG(x_stride >= w->in_features && y_stride >= w->out_features, "row stride smaller than the row");
  const int64_t need = gemv_tc5_workspace_bytes(w, 1, 1);
  if (need > kNoAllocScratchBytes) {
    set_error("noalloc forward: this weight needs %lld bytes of scratch, the built-in area holds %lld "
              "(use bsb_linear_forward with a caller-provided workspace)", (long long)need, (long long)kNoAllocScratchBytes);
    return BSB_ELIMIT;
  }
  // device address of the built-in scratch: looked up once per device, with that device current
  static void* scratch_ptr[64] = {nullptr};
  int dev = 0;
  BSB_CUDA(cudaGetDevice(&dev));
  BSB_CHECK_ARG(dev >= 0 && dev < 64, "device index %d out of range", dev);
  if (scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    BSB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    scratch_ptr[dev] = p;
  }
  for (int64_t r = 0; r < rows; ++r) {
    __half* yr = reinterpret_cast<__half*>(y) + r * y_stride;
    if (int rc = launch_gemv_tc5(w, 1, reinterpret_cast<const __half*>(x) + r * x_stride, x_stride, 1, &yr, nullptr,
                                 scratch_ptr[dev], kNoAllocScratchBytes, (cudaStream_t)stream))
      return rc;
  }
  return BSB_OK;
}

