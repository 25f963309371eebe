// Dropout mask of the attention matrix, from a counter-based generator so that the forward
// and both backward kernels regenerate the same bits from (seed, offset) without storing a
// mask: Philox4x32-10 (Salmon, Moraes, Dror, Shaw, "Parallel random numbers: as easy as 1, 2, 3",
// SC'11), the generator behind the (philox seed, philox offset) pair the aten flash-attention
// ops return (reference: torch_mojo_backend/eager_kernels/aten_fast.py:7726-7734 and
// torch_mojo_backend/mojo_device/torch_mojo_device_module.py:84-99, which reserves the counter
// interval).
//
// Layout of the stream.  One Philox call yields 16 bytes, one per element of a run of 16
// consecutive key columns of one query row:
//     key     = (seed low 32 bits, seed high 32 bits)
//     counter = (key column / 16,  query row,  low 32 bits of (offset + b*Hq + h),  high 32 bits of it)
//     byte 4*w + q of the call (word w of the output, byte q counted from the low end)
//             belongs to key column 16*(column / 16) + 4*w + q
// An element is KEPT when its byte >= threshold, threshold = round(256 * p) clamped to 255, so
// the drop probability is threshold / 256 and kept probabilities are scaled by
// 256 / (256 - threshold).  One forward call consumes B*Hq consecutive values of `offset`.
#pragma once
#include <stdint.h>

#include "common.cuh"

namespace b200fa {

__host__ __device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
  const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
  const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n1 = static_cast<uint32_t>(p1);
  const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
  const uint32_t n3 = static_cast<uint32_t>(p0);
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

// Philox4x32-10: four 32-bit outputs for a 128-bit counter and a 64-bit key.
__host__ __device__ __forceinline__ void philox4x32_10(uint64_t seed, uint32_t c0, uint32_t c1, uint32_t c2,
                                                       uint32_t c3, uint32_t (&out)[4]) {
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  uint32_t c[4] = {c0, c1, c2, c3};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}

// The 16 bytes for key columns [16*col_block, 16*col_block + 16) of query row `row` of head `bh`.
__host__ __device__ __forceinline__ void dropout_bytes16(const DropoutParams& d, int bh, int row, int col_block,
                                                         uint32_t (&out)[4]) {
  const uint64_t hi = d.offset + static_cast<uint64_t>(bh);
  philox4x32_10(d.seed, static_cast<uint32_t>(col_block), static_cast<uint32_t>(row), static_cast<uint32_t>(hi),
                static_cast<uint32_t>(hi >> 32), out);
}

// One element (slow: a whole Philox call; the exact-fp32 SIMT kernels use it).
__host__ __device__ __forceinline__ bool dropout_keep(const DropoutParams& d, int bh, int row, int col) {
  uint32_t r[4];
  dropout_bytes16(d, bh, row, col >> 4, r);
  const uint32_t byte = (r[(col >> 2) & 3] >> ((col & 3) * 8)) & 0xffu;
  return byte >= d.threshold;
}

#ifdef __CUDACC__
// keep-bits of 16 consecutive columns (bit i <-> column 16*col_block + i)
__device__ __forceinline__ uint32_t dropout_bits16(const DropoutParams& d, int bh, int row, int col_block) {
  uint32_t r[4];
  dropout_bytes16(d, bh, row, col_block, r);
  const uint32_t thr4 = d.threshold * 0x01010101u;
  uint32_t bits = 0;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t ge = __vcmpgeu4(r[w], thr4) & 0x01010101u;    // 1 per byte that is kept
    bits |= ((ge * 0x01020408u) >> 24 & 0xfu) << (4 * w);        // the four flags gathered into a nibble
  }
  return bits;
}

// keep-bits of the 128 key columns [col0, col0 + 128) of one query row (col0 a multiple of 128):
// bits[w] bit i <-> column col0 + 32*w + i
__device__ __forceinline__ void dropout_row_bits(const DropoutParams& d, int bh, int row, int col0,
                                                 uint32_t (&bits)[4]) {
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const int blk = (col0 >> 4) + 2 * w;
    bits[w] = dropout_bits16(d, bh, row, blk) | (dropout_bits16(d, bh, row, blk + 1) << 16);
  }
}
#endif

}  // namespace b200fa
