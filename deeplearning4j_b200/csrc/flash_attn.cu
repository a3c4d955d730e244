// Fused scaled-dot-product attention forward for head size 64 and 256 or 512 keys (bf16), one CTA per
// (batch, head, 128-query block):
//     S = Q K^T (tcgen05, fp32 in TMEM)  ->  masked, scaled softmax in registers  ->  P (bf16) staged in shared memory
//     ->  O = P V (tcgen05)  ->  normalise, store O [B, Tq, H, 64] and the row log-sum-exp [B, H, Tq].
// The score matrix never reaches HBM (AttentionHelper.cpp computes matmul, scale, mask add, softmax over the full
// score matrix and a second matmul as separate ops).  Keys are processed in halves of 256: each half has its own
// running maximum / sum and its own O accumulator, and the two are merged in the epilogue, so nothing in TMEM has to
// be rescaled.  Warp 0 issues the TMA loads, warp 1 the MMAs, warps 2-5 own one query row per thread.
#include "common.cuh"

namespace dl4j {

constexpr int FA_D = 64;
constexpr int FA_BM = 128;        // queries per CTA
constexpr int FA_BN = 256;        // keys per half
constexpr int FA_THREADS = 192;
constexpr int FA_Q_BYTES = FA_BM * FA_D * 2;      // 16 KB
constexpr int FA_KV_BYTES = FA_BN * FA_D * 2;     // 32 KB per half
constexpr int FA_P_BYTES = FA_BM * FA_BN * 2;     // 64 KB
constexpr int FA_TMEM_COLS = 512;                 // S: 0..255, O(half 0): 256..319, O(half 1): 320..383
constexpr float FA_LOG2E = 1.4426950408889634f;

struct FlashFwdParams {
  __nv_bfloat16* out;        // [B, Tq, H, 64]
  float* lse;                // [B, H, Tq]
  const float* key_mask;     // [B, Tk] (non-zero = keep) or null
  int B, H, Tq, Tk;
  float scale;
  int* status;
};

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const FlashFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + FA_Q_BYTES;                 // two halves
  uint8_t* v_s = k_s + 2 * FA_KV_BYTES;            // two halves
  uint8_t* p_s = v_s + 2 * FA_KV_BYTES;
  float* mask_s = reinterpret_cast<float*>(p_s + FA_P_BYTES);          // [512]
  uint64_t* bars = reinterpret_cast<uint64_t*>(mask_s + 2 * FA_BN);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* v_full = bars + 3;      // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blocks = (p.Tq + FA_BM - 1) / FA_BM;
  const int qb = blockIdx.x % q_blocks;
  const int h = (blockIdx.x / q_blocks) % p.H;
  const int b = blockIdx.x / (q_blocks * p.H);
  const int halves = p.Tk / FA_BN;
  const int q0 = qb * FA_BM;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    mbar_init(q_full, 1);
    mbar_init(&k_full[0], 1); mbar_init(&k_full[1], 1);
    mbar_init(&v_full[0], 1); mbar_init(&v_full[1], 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, FA_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, FA_Q_BYTES);
      tma_load_4d(q_s, &tmap_q, q_full, 0, q0, h, b);
      for (int hf = 0; hf < halves; ++hf) {
        mbar_expect_tx(&k_full[hf], FA_KV_BYTES);
        tma_load_4d(k_s + hf * FA_KV_BYTES, &tmap_k, &k_full[hf], 0, hf * FA_BN, h, b);
      }
      for (int hf = 0; hf < halves; ++hf) {
        mbar_expect_tx(&v_full[hf], FA_KV_BYTES);
        tma_load_4d(v_s + hf * FA_KV_BYTES, &tmap_v, &v_full[hf], 0, hf * FA_BN, h, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(1, 0, 0, FA_BM, FA_BN);      // S = Q K^T: both operands K-major (K = head dim)
      const uint32_t idesc_o = make_idesc(1, 0, 1, FA_BM, FA_D);       // O = P V: V [keys, 64] is MN-major for the B operand
      const uint64_t dq = make_smem_desc_sw128(smem_u32(q_s), 16, 1024);
      bool ok = mbar_wait_bounded(q_full, 0, p.status, DL4J_ERR_TIMEOUT_MMA);
      for (int hf = 0; hf < halves && ok; ++hf) {
        if (!mbar_wait_bounded(&k_full[hf], 0, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint64_t dk = make_smem_desc_sw128(smem_u32(k_s + hf * FA_KV_BYTES), 16, 1024);
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k)
          umma_f16(tmem_base, dq + ((uint64_t)(k * 32) >> 4), dk + ((uint64_t)(k * 32) >> 4), idesc_s, k > 0 ? 1u : 0u);
        umma_commit(s_full);         // also covers the P V MMAs of the previous half: P may be overwritten after this
        if (!mbar_wait_bounded(p_full, (uint32_t)(hf & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        if (!mbar_wait_bounded(&v_full[hf], 0, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pv = smem_u32(v_s + hf * FA_KV_BYTES);
        const uint32_t pp = smem_u32(p_s);
#pragma unroll
        for (int k = 0; k < FA_BN / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(pp + (k >> 2) * (FA_BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(pv + k * (16 * 128), 64 * 128, 1024);
          umma_f16(tmem_base + FA_BN + hf * FA_D, da, db, idesc_o, k > 0 ? 1u : 0u);
        }
      }
      if (ok) umma_commit(o_full);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;                    // query row of this thread within the block
    const int t = threadIdx.x - 64;                 // 0..127
    // key mask of this batch element -> shared memory (1 = keep)
    for (int i = t; i < p.Tk; i += 128) mask_s[i] = p.key_mask ? p.key_mask[(long)b * p.Tk + i] : 1.f;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float k2 = p.scale * FA_LOG2E;
    float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.f, 0.f};
    bool ok = true;
    for (int hf = 0; hf < halves && ok; ++hf) {
      if (!mbar_wait_bounded(s_full, (uint32_t)(hf & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const float* mk = mask_s + hf * FA_BN;
      float m = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (mk[c * 32 + j] != 0.f) m = fmaxf(m, __uint_as_float(v[j]));
      }
      const float mref = (m == -INFINITY) ? 0.f : m;
      float l = 0.f;
#pragma unroll 1
      for (int c = 0; c < FA_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + c * 32, v);
        tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          e[j] = mk[c * 32 + j] != 0.f ? fa_exp2((__uint_as_float(v[j]) - mref) * k2) : 0.f;
          l += e[j];
        }
        // 32 columns = four 16-byte chunks of this row inside key block c / 2 of the K-major, 128-byte-swizzled P tile
        uint8_t* row = p_s + (c >> 1) * (FA_BM * 128) + r * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 u;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
          for (int i = 0; i < 4; ++i) hh[i] = __floats2bfloat162_rn(e[j * 8 + 2 * i], e[j * 8 + 2 * i + 1]);
          const int chunk = ((c & 1) * 4 + j) ^ (r & 7);
          *reinterpret_cast<uint4*>(row + chunk * 16) = u;
        }
      }
      mx[hf] = m;
      sum[hf] = l;
      tc_fence_before();
      fence_proxy_async_smem();       // P was written through the generic proxy; the MMA reads it through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait_bounded(o_full, 0, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      const float m = fmaxf(mx[0], mx[1]);
      const float mref = (m == -INFINITY) ? 0.f : m;
      const float a0 = (mx[0] == -INFINITY) ? 0.f : fa_exp2((mx[0] - mref) * k2);
      const float a1 = (halves < 2 || mx[1] == -INFINITY) ? 0.f : fa_exp2((mx[1] - mref) * k2);
      const float l = sum[0] * a0 + sum[1] * a1;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      float o[FA_D];
      {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr + FA_BN, v0);
        tmem_ld_32x32(taddr + FA_BN + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { o[j] = __uint_as_float(v0[j]) * a0; o[32 + j] = __uint_as_float(v1[j]) * a0; }
      }
      if (halves > 1) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr + FA_BN + FA_D, v0);
        tmem_ld_32x32(taddr + FA_BN + FA_D + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) { o[j] = fmaf(__uint_as_float(v0[j]), a1, o[j]); o[32 + j] = fmaf(__uint_as_float(v1[j]), a1, o[32 + j]); }
      }
      const int tq = q0 + r;
      if (tq < p.Tq) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + (((long)b * p.Tq + tq) * p.H + h) * FA_D);
#pragma unroll
        for (int j = 0; j < FA_D / 8; ++j) {
          uint4 u;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
          for (int i = 0; i < 4; ++i) hh[i] = __floats2bfloat162_rn(o[j * 8 + 2 * i] * inv, o[j * 8 + 2 * i + 1] * inv);
          dst[j] = u;
        }
        if (p.lse) p.lse[((long)b * p.H + h) * p.Tq + tq] = l > 0.f ? mref * p.scale + __logf(l) : -INFINITY;
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FA_TMEM_COLS);
  }
}

}  // namespace dl4j

using namespace dl4j;

// Tensor map over a [B, H, T, 64] bf16 view given by its element strides (unit stride along the head dimension)
static int fa_encode(CUtensorMap* map, const void* base, int B, int H, int T, long sb, long sh, long st, uint32_t box_rows) {
  dl4j_PFN_encodeTiled enc = dl4j_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)FA_D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)st * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {FA_D, box_rows, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// q / k / v: [B, H, T, 64] bf16 views with element strides {sb, sh, st} (head dimension contiguous, strides multiples of 8,
// base 16-byte aligned).  out [B, Tq, H, 64] bf16 contiguous, lse [B, H, Tq] fp32, key_mask [B, Tk] fp32 or null.
// Limits: Tk in {256, 512}.
DL4J_API int dl4j_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const float* key_mask, int B, int H,
                                 int Tq, int Tk, const long* q_strides, const long* k_strides, const long* v_strides, float scale,
                                 void* stream_) {
  if (B < 1 || H < 1 || Tq < 1 || (Tk != FA_BN && Tk != 2 * FA_BN)) return -DL4J_ERR_BAD_ARG;
  CUtensorMap tq, tk, tv;
  int r = fa_encode(&tq, q, B, H, Tq, q_strides[0], q_strides[1], q_strides[2], FA_BM);
  if (r) return -1000 - r;
  r = fa_encode(&tk, k, B, H, Tk, k_strides[0], k_strides[1], k_strides[2], FA_BN);
  if (r) return -1000 - r;
  r = fa_encode(&tv, v, B, H, Tk, v_strides[0], v_strides[1], v_strides[2], FA_BN);
  if (r) return -1000 - r;
  int dev = 0;
  cudaGetDevice(&dev);
  FlashFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.key_mask = key_mask;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk;
  p.scale = scale;
  p.status = dl4j_status_word(dev);
  const size_t smem = FA_Q_BYTES + 4 * FA_KV_BYTES + FA_P_BYTES + 2 * FA_BN * sizeof(float) + 256 + 1024;
  cudaError_t e = cudaFuncSetAttribute(flash_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int q_blocks = (Tq + FA_BM - 1) / FA_BM;
  flash_attn_fwd_kernel<<<B * H * q_blocks, FA_THREADS, smem, (cudaStream_t)stream_>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}
