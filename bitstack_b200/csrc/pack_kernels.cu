// Sign bit packing / unpacking on the device.
//
// Convention (bitstack/utils/pack_utils.py:5-26 of the reference): element e of the
// row-major flattened sign matrix lives in byte e>>3, bit 7-(e&7); +1 is a set
// bit, -1 a clear bit; the last byte is padded with clear bits.
#include "common.cuh"

namespace bsb {

namespace {

// 4 packed bytes -> 32 int8 signs.  `quad` holds the 4 bytes in memory order
// (byte 0 in the low bits).
__device__ __forceinline__ void expand_byte(uint32_t b, uint32_t& lo, uint32_t& hi) {
  const uint32_t rep = b * 0x01010101u;
  const uint32_t zlo = __vcmpeq4(rep & 0x10204080u, 0u);  // 0xFF where the bit is clear
  const uint32_t zhi = __vcmpeq4(rep & 0x01020408u, 0u);
  lo = zlo | (~zlo & 0x01010101u);  // clear -> 0xFF (-1), set -> 0x01 (+1)
  hi = zhi | (~zhi & 0x01010101u);
}

__global__ void __launch_bounds__(256) unpack_vec_kernel(const uint32_t* __restrict__ packed,
                                                         int64_t n_quads, uint4* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_quads; i += stride) {
    const uint32_t q = __ldg(packed + i);
    uint4 a, b;
    expand_byte(q & 0xFFu, a.x, a.y);
    expand_byte((q >> 8) & 0xFFu, a.z, a.w);
    expand_byte((q >> 16) & 0xFFu, b.x, b.y);
    expand_byte(q >> 24, b.z, b.w);
    out[2 * i] = a;
    out[2 * i + 1] = b;
  }
}

// element-wise tail / unaligned path: one thread per output element
__global__ void __launch_bounds__(256) unpack_scalar_kernel(const uint8_t* __restrict__ packed,
                                                            int64_t first, int64_t n,
                                                            int8_t* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t e = first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const uint32_t b = packed[e >> 3];
    out[e] = ((b >> (7 - (int)(e & 7))) & 1u) ? (int8_t)1 : (int8_t)-1;
  }
}

__global__ void __launch_bounds__(256) pack_kernel(const int8_t* __restrict__ sign, int64_t n,
                                                   uint8_t* __restrict__ packed,
                                                   int32_t* __restrict__ bad) {
  const int64_t n_bytes = (n + 7) >> 3;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int my_bad = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_bytes; i += stride) {
    uint32_t b = 0;
    const int64_t base = i << 3;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (base + q < n) {
        const int v = sign[base + q];
        my_bad += (v != 1 && v != -1);
        b |= (uint32_t)(v == 1) << (7 - q);
      }
    }
    packed[i] = (uint8_t)b;
  }
  if (bad != nullptr) {
    // one atomic per warp that saw a bad value; no trap, the host reads the count
    const unsigned total = __reduce_add_sync(0xFFFFFFFFu, (unsigned)my_bad);
    if ((threadIdx.x & 31) == 0 && total) atomicAdd(bad, (int)total);
  }
}

int grid_for(int64_t items, int threads) {
  int64_t g = ceil_div64(items, threads);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

int launch_unpack_sign(const uint8_t* packed, int64_t n, int8_t* out, cudaStream_t s) {
  if (n == 0) return BSB_OK;
  int64_t done = 0;
  const bool aligned = ((uintptr_t)packed % 4 == 0) && ((uintptr_t)out % 16 == 0);
  if (aligned && n >= 32) {
    const int64_t n_quads = n / 32;
    unpack_vec_kernel<<<grid_for(n_quads, 256), 256, 0, s>>>((const uint32_t*)packed, n_quads,
                                                             (uint4*)out);
    if (int rc = check_launch("unpack_vec_kernel")) return rc;
    done = n_quads * 32;
  }
  if (done < n) {
    unpack_scalar_kernel<<<grid_for(n - done, 256), 256, 0, s>>>(packed, done, n, out);
    if (int rc = check_launch("unpack_scalar_kernel")) return rc;
  }
  return BSB_OK;
}

int launch_pack_sign(const int8_t* sign, int64_t n, uint8_t* packed, int32_t* bad, cudaStream_t s) {
  if (n == 0) return BSB_OK;
  const int64_t n_bytes = (n + 7) >> 3;
  pack_kernel<<<grid_for(n_bytes, 256), 256, 0, s>>>(sign, n, packed, bad);
  return check_launch("pack_kernel");
}

}  // namespace bsb
