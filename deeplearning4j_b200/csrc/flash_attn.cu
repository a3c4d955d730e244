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

// ------------------------------------------------------------------------------------------------ backward
// One CTA per (batch, head, block of 128 keys); it walks the query blocks.  Per query block i:
//     S = Q_i K_j^T and dP = dO_i V_j^T (TMEM)  ->  threads: P = exp(S * scale - lse), dS = scale * P * (dP - D)
//     ->  P, dS staged in shared memory (bf16)  ->  dV += P^T dO_i, dK += dS^T Q_i (accumulated in TMEM over i),
//     dQ_i = dS K_j (TMEM, added to the fp32 dQ buffer with vector atomics: four key blocks contribute to it).
// P^T and dS^T are the same shared-memory tiles read through MN-major descriptors, so nothing is transposed.
// D = rowsum(dO * O) and the forward's log-sum-exp come from the caller.
namespace dl4j {

constexpr int FB_BLK = 128;                       // queries per step and keys per CTA
constexpr int FB_TILE = FB_BLK * FA_D * 2;        // 16 KB: one [128, 64] bf16 tile
constexpr int FB_PS = FB_BLK * FB_BLK * 2;        // 32 KB: P or dS
constexpr int FB_TMEM_COLS = 512;                 // S 0..127, dP 128..255, dQ 256..319, dV 320..383, dK 384..447

struct FlashBwdParams {
  const float* lse;          // [B, H, Tq]
  const float* dvec;         // [B, H, Tq]  rowsum(dO * O)
  const float* key_mask;     // [B, Tk] or null
  float* dq;                 // [B, H, Tq, 64] fp32, zero on entry
  __nv_bfloat16* dk;         // [B, Tk, H, 64]
  __nv_bfloat16* dv;         // [B, Tk, H, 64]
  long o_bs, o_ts;           // element strides of dk / dv between batch entries and between keys (heads are 64 apart)
  int B, H, Tq, Tk;
  float scale;
  int* status;
};

__device__ __forceinline__ void fb_store_row(uint8_t* tile, int r, int c, const float* e) {
  // 32 values of row r starting at column 32 * c of a [128, 128] bf16 K-major tile (two 64-column blocks, 128-byte swizzle)
  uint8_t* row = tile + (c >> 1) * (FB_BLK * 128) + r * 128;
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

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                      const FlashBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;
  uint8_t* v_s = k_s + FB_TILE;
  uint8_t* q_s = v_s + FB_TILE;                   // two stages
  uint8_t* do_s = q_s + 2 * FB_TILE;              // two stages
  uint8_t* p_s = do_s + 2 * FB_TILE;
  uint8_t* ds_s = p_s + FB_PS;
  float* mask_s = reinterpret_cast<float*>(ds_s + FB_PS);      // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(mask_s + FB_BLK);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;     // [2]
  uint64_t* qdo_empty = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* dq_full = bars + 7;
  uint64_t* dq_empty = bars + 8;
  uint64_t* fin_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = p.Tk / FB_BLK;
  const int kb = blockIdx.x % k_blocks;
  const int h = (blockIdx.x / k_blocks) % p.H;
  const int b = blockIdx.x / (k_blocks * p.H);
  const int k0 = kb * FB_BLK;
  const int nq = (p.Tq + FB_BLK - 1) / FB_BLK;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 4);
    mbar_init(fin_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, FB_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t T_S = 0, T_DP = 128, T_DQ = 256, T_DV = 320, T_DK = 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * FB_TILE);
      tma_load_4d(k_s, &tmap_k, kv_full, 0, k0, h, b);
      tma_load_4d(v_s, &tmap_v, kv_full, 0, k0, h, b);
      for (int i = 0; i < nq; ++i) {
        const int st = i & 1;
        if (!mbar_wait_bounded(&qdo_empty[st], (uint32_t)(((i >> 1) & 1) ^ 1), p.status, DL4J_ERR_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&qdo_full[st], 2 * FB_TILE);
        tma_load_4d(q_s + st * FB_TILE, &tmap_q, &qdo_full[st], 0, i * FB_BLK, h, b);
        tma_load_4d(do_s + st * FB_TILE, &tmap_do, &qdo_full[st], 0, i * FB_BLK, h, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id_s = make_idesc(1, 0, 0, FB_BLK, FB_BLK);      // [q, keys] = A[q, d] K-major x B[keys, d] K-major
      const uint32_t id_kv = make_idesc(1, 1, 1, FB_BLK, FA_D);       // [keys, d] = A^T (P / dS tile, MN-major) x B[q, d] MN-major
      const uint32_t id_dq = make_idesc(1, 0, 1, FB_BLK, FA_D);       // [q, d] = dS K-major x K_j[keys, d] MN-major
      bool ok = mbar_wait_bounded(kv_full, 0, p.status, DL4J_ERR_TIMEOUT_MMA);
      const uint32_t ak = smem_u32(k_s), av = smem_u32(v_s), ap = smem_u32(p_s), ads = smem_u32(ds_s);
      const uint64_t dk_k = make_smem_desc_sw128(ak, 16, 1024), dv_k = make_smem_desc_sw128(av, 16, 1024);
      for (int i = 0; i < nq && ok; ++i) {
        const int st = i & 1;
        if (!mbar_wait_bounded(&qdo_full[st], (uint32_t)((i >> 1) & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aq = smem_u32(q_s + st * FB_TILE), ado = smem_u32(do_s + st * FB_TILE);
        const uint64_t dq_k = make_smem_desc_sw128(aq, 16, 1024), ddo_k = make_smem_desc_sw128(ado, 16, 1024);
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) {
          umma_f16(tmem_base + T_S, dq_k + ((uint64_t)(k * 32) >> 4), dk_k + ((uint64_t)(k * 32) >> 4), id_s, k > 0 ? 1u : 0u);
          umma_f16(tmem_base + T_DP, ddo_k + ((uint64_t)(k * 32) >> 4), dv_k + ((uint64_t)(k * 32) >> 4), id_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait_bounded(p_full, (uint32_t)(i & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        if (!mbar_wait_bounded(dq_empty, (uint32_t)((i & 1) ^ 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < FB_BLK / 16; ++k) {
          // reduction over the 128 query rows: 16 rows (2048 bytes) per step in the MN-major tiles
          const uint64_t a_pt = make_smem_desc_sw128(ap + k * 2048, FB_BLK * 128, 1024);
          const uint64_t a_dst = make_smem_desc_sw128(ads + k * 2048, FB_BLK * 128, 1024);
          const uint64_t b_do = make_smem_desc_sw128(ado + k * 2048, FB_BLK * 128, 1024);
          const uint64_t b_q = make_smem_desc_sw128(aq + k * 2048, FB_BLK * 128, 1024);
          umma_f16(tmem_base + T_DV, a_pt, b_do, id_kv, (i > 0 || k > 0) ? 1u : 0u);
          umma_f16(tmem_base + T_DK, a_dst, b_q, id_kv, (i > 0 || k > 0) ? 1u : 0u);
          // reduction over the 128 keys: dS K-major (two 64-key blocks of 16 KB, 32 bytes per step), K_j MN-major
          const uint64_t a_ds = make_smem_desc_sw128(ads + (k >> 2) * (FB_BLK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t b_k = make_smem_desc_sw128(ak + k * 2048, FB_BLK * 128, 1024);
          umma_f16(tmem_base + T_DQ, a_ds, b_k, id_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);
        umma_commit(dq_full);
      }
      if (ok) umma_commit(fin_full);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int t = threadIdx.x - 64;
    mask_s[t] = p.key_mask ? p.key_mask[(long)b * p.Tk + k0 + t] : 1.f;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float k2 = p.scale * FA_LOG2E;
    bool ok = true;
    for (int i = 0; i < nq && ok; ++i) {
      const int tq = i * FB_BLK + r;
      const bool row_ok = tq < p.Tq;
      const long ridx = ((long)b * p.H + h) * p.Tq + tq;
      const float lse = row_ok ? p.lse[ridx] : INFINITY;          // +inf: exp2(-inf) = 0 for rows past the end
      const float dv_r = row_ok ? p.dvec[ridx] : 0.f;
      const float lse2 = lse * FA_LOG2E;
      if (!mbar_wait_bounded(s_full, (uint32_t)(i & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < FB_BLK / 32; ++c) {
        uint32_t sv[32], dpv[32];
        tmem_ld_32x32(taddr + T_S + c * 32, sv);
        tmem_ld_32x32(taddr + T_DP + c * 32, dpv);
        tmem_ld_wait();
        float pe[32], de[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const bool keep = mask_s[c * 32 + j] != 0.f && lse != -INFINITY;
          const float pv = keep ? fa_exp2(fmaf(__uint_as_float(sv[j]), k2, -lse2)) : 0.f;
          pe[j] = pv;
          de[j] = pv * (__uint_as_float(dpv[j]) - dv_r) * p.scale;
        }
        fb_store_row(p_s, r, c, pe);
        fb_store_row(ds_s, r, c, de);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      if (!mbar_wait_bounded(dq_full, (uint32_t)(i & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr + T_DQ, v0);
        tmem_ld_32x32(taddr + T_DQ + 32, v1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_empty);
        if (row_ok) {
          float4* dst = reinterpret_cast<float4*>(p.dq + ridx * FA_D);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            atomicAdd(dst + j, make_float4(__uint_as_float(v0[4 * j]), __uint_as_float(v0[4 * j + 1]), __uint_as_float(v0[4 * j + 2]),
                                           __uint_as_float(v0[4 * j + 3])));
            atomicAdd(dst + 8 + j, make_float4(__uint_as_float(v1[4 * j]), __uint_as_float(v1[4 * j + 1]), __uint_as_float(v1[4 * j + 2]),
                                               __uint_as_float(v1[4 * j + 3])));
          }
        }
      }
    }
    if (ok && mbar_wait_bounded(fin_full, 0, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      // accumulator rows are keys here: thread r owns key k0 + r
      const long orow = (long)b * p.o_bs + (long)(k0 + r) * p.o_ts + (long)h * FA_D;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        uint32_t v0[32], v1[32];
        const uint32_t base = taddr + (which == 0 ? T_DV : T_DK);
        tmem_ld_32x32(base, v0);
        tmem_ld_32x32(base + 32, v1);
        tmem_ld_wait();
        uint4* dst = reinterpret_cast<uint4*>((which == 0 ? p.dv : p.dk) + orow);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 u;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
          const uint32_t* src = j < 4 ? v0 + 8 * j : v1 + 8 * (j - 4);
#pragma unroll
          for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(__uint_as_float(src[2 * e]), __uint_as_float(src[2 * e + 1]));
          dst[j] = u;
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FB_TMEM_COLS);
  }
}

}  // namespace dl4j

// q / k / v / dout: [B, H, T, 64] bf16 views (element strides {sb, sh, st}); lse, dvec [B, H, Tq] fp32; dq [B, H, Tq, 64] fp32
// zeroed by the caller; dk, dv bf16 addressed as base + b * o_bs + key * o_ts + head * 64.  Limits: Tk a multiple of 128.
DL4J_API int dl4j_flash_attn_bwd(const void* q, const void* k, const void* v, const void* dout, const float* lse, const float* dvec,
                                 const float* key_mask, float* dq, void* dk, void* dv, int B, int H, int Tq, int Tk, const long* q_strides,
                                 const long* k_strides, const long* v_strides, const long* do_strides, long o_bs, long o_ts, float scale, void* stream_) {
  if (B < 1 || H < 1 || Tq < 1 || Tk < FB_BLK || Tk % FB_BLK) return -DL4J_ERR_BAD_ARG;
  CUtensorMap tq, tk, tv, tdo;
  int r = fa_encode(&tq, q, B, H, Tq, q_strides[0], q_strides[1], q_strides[2], FB_BLK);
  if (r) return -1000 - r;
  r = fa_encode(&tk, k, B, H, Tk, k_strides[0], k_strides[1], k_strides[2], FB_BLK);
  if (r) return -1000 - r;
  r = fa_encode(&tv, v, B, H, Tk, v_strides[0], v_strides[1], v_strides[2], FB_BLK);
  if (r) return -1000 - r;
  r = fa_encode(&tdo, dout, B, H, Tq, do_strides[0], do_strides[1], do_strides[2], FB_BLK);
  if (r) return -1000 - r;
  int dev = 0;
  cudaGetDevice(&dev);
  FlashBwdParams p;
  p.lse = lse; p.dvec = dvec; p.key_mask = key_mask;
  p.dq = dq;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.o_bs = o_bs; p.o_ts = o_ts;
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk;
  p.scale = scale;
  p.status = dl4j_status_word(dev);
  const size_t smem = 6 * FB_TILE + 2 * FB_PS + FB_BLK * sizeof(float) + 256 + 1024;
  cudaError_t e = cudaFuncSetAttribute(flash_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  flash_attn_bwd_kernel<<<B * H * (Tk / FB_BLK), FA_THREADS, smem, (cudaStream_t)stream_>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}
