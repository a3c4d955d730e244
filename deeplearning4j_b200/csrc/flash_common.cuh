// Shared pieces of the fused attention kernels (head size 64, bf16).
#pragma once
#include "common.cuh"

namespace dl4j {

constexpr int FA_D = 64;
constexpr float FA_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// n (multiple of 8) fp32 values of row r, starting at column col0 (multiple of 8), into a K-major bf16 tile of 128 rows
// made of 64-column blocks (16 KB each, 128-byte swizzle): the layout a tcgen05 K-major A operand (or, read
// transposed, an MN-major operand) expects.
__device__ __forceinline__ void fa_store_row(uint8_t* tile, int r, int col0, int n, const float* e) {
#pragma unroll
  for (int j = 0; j < n / 8; ++j) {
    const int col = col0 + 8 * j;
    uint4 u;
    __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) hh[i] = __floats2bfloat162_rn(e[j * 8 + 2 * i], e[j * 8 + 2 * i + 1]);
    const int chunk = ((col & 63) >> 3) ^ (r & 7);
    *reinterpret_cast<uint4*>(tile + (col >> 6) * (128 * 128) + r * 128 + chunk * 16) = u;
  }
}

// Dropout on the attention weights (AttentionHelper.cpp applies it to the softmax output): the keep decision of element
// (batch*head, query row, key column) is a pure function of a 64-bit seed and those three indices, so the backward pass
// regenerates the forward's mask instead of storing it.  One Philox4x32-7 block yields 8 x 16 bits = the decisions of 8
// consecutive key columns; an element is dropped when its 16-bit value is below `thr` = round(p * 65536).
__device__ __forceinline__ uint32_t fa_keep8(uint32_t seed_lo, uint32_t seed_hi, uint32_t bh, uint32_t row, uint32_t col8, uint32_t thr) {
  uint32_t c0 = col8, c1 = row, c2 = bh, c3 = 0x5eed5eedu, k0 = seed_lo, k1 = seed_hi;
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0; c1 = lo1; c2 = hi0 ^ c3 ^ k1; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  const uint32_t w[4] = {c0, c1, c2, c3};
  uint32_t keep = 0;
#pragma unroll
  for (int e = 0; e < 8; ++e) keep |= (((w[e >> 1] >> (16 * (e & 1))) & 0xffffu) >= thr ? 1u : 0u) << e;
  return keep;
}

// keep bits of 32 consecutive key columns starting at col0 (a multiple of 8)
__device__ __forceinline__ uint32_t fa_keep32(uint32_t seed_lo, uint32_t seed_hi, uint32_t bh, uint32_t row, uint32_t col0, uint32_t thr) {
  uint32_t k = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) k |= fa_keep8(seed_lo, seed_hi, bh, row, (col0 >> 3) + g, thr) << (8 * g);
  return k;
}

}  // namespace dl4j

// Tensor map over a [B, H, T, 64] bf16 view given by its element strides (unit stride along the head dimension)
static inline int fa_encode(CUtensorMap* map, const void* base, int B, int H, int T, long sb, long sh, long st, uint32_t box_rows) {
  dl4j_PFN_encodeTiled enc = dl4j_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)dl4j::FA_D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {(cuuint32_t)dl4j::FA_D, box_rows, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
