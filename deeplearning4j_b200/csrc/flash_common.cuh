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
