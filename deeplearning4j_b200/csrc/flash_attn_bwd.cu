// Fused scaled-dot-product attention, backward pass (head size 64, bf16).
#include "flash_common.cuh"

using namespace dl4j;

// ------------------------------------------------------------------------------------------------ backward
// One CTA per (batch, head, block of 128 keys); it walks the query blocks.  Per query block i:
//     S = Q_i K_j^T and dP = dO_i V_j^T (TMEM)  ->  threads: P = exp(S * scale - lse), dS = scale * P * (dP - D)
//     ->  P, dS staged in shared memory (bf16)  ->  dV += P^T dO_i, dK += dS^T Q_i (accumulated in TMEM over i),
//     dQ_i = dS K_j (TMEM, added to the fp32 dQ buffer with vector atomics: four key blocks contribute to it).
// P^T and dS^T are the same shared-memory tiles read through MN-major descriptors, so nothing is transposed.
// D = rowsum(dO * O) and the forward's log-sum-exp come from the caller.
namespace dl4j {

constexpr int FB_THREADS = 64 + 512;              // warp 0 TMA, warp 1 MMA, 16 compute warps (four threads per row)
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
  const unsigned long long* seed;   // dropout seed of the forward pass (device memory), read when drop_thr != 0
  uint32_t drop_thr;
  float inv_keep;
};

template <bool DROP>
__global__ void __launch_bounds__(FB_THREADS, 1)
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
    mbar_init(p_full, 16);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 16);
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
      const uint64_t d_q_k0 = make_smem_desc_sw128(smem_u32(q_s), 16, 1024), d_do_k0 = make_smem_desc_sw128(smem_u32(do_s), 16, 1024);
      constexpr uint64_t STAGE_STEP_K = (uint64_t)(FB_TILE >> 4);
      // S_i = Q_i K_j^T and dP_i = dO_i V_j^T; issued one block ahead so that they overlap the threads' work on block i - 1
      auto issue_s = [&](int i) -> bool {
        const int st = i & 1;
        if (!mbar_wait_bounded(&qdo_full[st], (uint32_t)((i >> 1) & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint64_t dq_k = d_q_k0 + (st ? STAGE_STEP_K : 0), ddo_k = d_do_k0 + (st ? STAGE_STEP_K : 0);
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k) {
          umma_f16(tmem_base + T_S, dq_k + ((uint64_t)(k * 32) >> 4), dk_k + ((uint64_t)(k * 32) >> 4), id_s, k > 0 ? 1u : 0u);
          umma_f16(tmem_base + T_DP, ddo_k + ((uint64_t)(k * 32) >> 4), dv_k + ((uint64_t)(k * 32) >> 4), id_s, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        return true;
      };
      // descriptors are built once; inside the loops they only advance by a constant (one 64-bit add per operand), which keeps
      // the single issuing thread at a few instructions per MMA
      const uint64_t d_pt = make_smem_desc_sw128(ap, FB_BLK * 128, 1024), d_dst = make_smem_desc_sw128(ads, FB_BLK * 128, 1024);
      const uint64_t d_dsk = make_smem_desc_sw128(ads, 16, 1024), d_kmn = make_smem_desc_sw128(ak, FB_BLK * 128, 1024);
      const uint64_t d_do_mn0 = make_smem_desc_sw128(smem_u32(do_s), FB_BLK * 128, 1024), d_q_mn0 = make_smem_desc_sw128(smem_u32(q_s), FB_BLK * 128, 1024);
      constexpr uint64_t STAGE_STEP = (uint64_t)(FB_TILE >> 4);     // second Q / dO stage: same descriptor, start address + one tile
      if (ok) ok = issue_s(0);
      for (int i = 0; i < nq && ok; ++i) {
        const int st = i & 1;
        const uint64_t d_do_st = d_do_mn0 + (st ? STAGE_STEP : 0), d_q_st = d_q_mn0 + (st ? STAGE_STEP : 0);
        if (!mbar_wait_bounded(p_full, (uint32_t)(i & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < FB_BLK / 16; ++k) {
          // reduction over the 128 query rows: 16 rows (2048 bytes) per step in the MN-major tiles
          const uint64_t a_pt = d_pt + (uint64_t)(k * (2048 >> 4)), a_dst = d_dst + (uint64_t)(k * (2048 >> 4));
          const uint64_t b_do = d_do_st + (uint64_t)(k * (2048 >> 4)), b_q = d_q_st + (uint64_t)(k * (2048 >> 4));
          umma_f16(tmem_base + T_DV, a_pt, b_do, id_kv, (i > 0 || k > 0) ? 1u : 0u);
          umma_f16(tmem_base + T_DK, a_dst, b_q, id_kv, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);      // Q_i / dO_i are not read again: their stage can be refilled
        // dQ_{i-1} must have left tensor memory before dQ_i overwrites it; the threads read it out while dV / dK were issued
        if (!mbar_wait_bounded(dq_empty, (uint32_t)((i & 1) ^ 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < FB_BLK / 16; ++k) {
          // reduction over the 128 keys: dS K-major (two 64-key blocks of 16 KB, 32 bytes per step), K_j MN-major
          const uint64_t a_ds = d_dsk + (uint64_t)(((k >> 2) * (FB_BLK * 128) + (k & 3) * 32) >> 4);
          const uint64_t b_k = d_kmn + (uint64_t)(k * (2048 >> 4));
          umma_f16(tmem_base + T_DQ, a_ds, b_k, id_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        // S / dP of block i were read out of tensor memory before p_full(i) completed, so block i + 1 may overwrite them now
        if (i + 1 < nq) ok = issue_s(i + 1);
      }
      if (ok) umma_commit(fin_full);
    }
  } else {
    const int cw = warp - 2;                        // 0..15
    const int q = warp & 3;                         // TMEM lane quadrant this warp may access (warp index modulo 4)
    const int cq = cw >> 2;                         // column quarter (32 columns) owned by this thread
    const int r = q * 32 + lane;
    const int t = threadIdx.x - 64;                 // 0..511
    if (t < FB_BLK) mask_s[t] = p.key_mask ? p.key_mask[(long)b * p.Tk + k0 + t] : 1.f;
    asm volatile("bar.sync 1, 512;" ::: "memory");
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float k2 = p.scale * FA_LOG2E;
    // key mask of this thread's 32 columns as a bit word; without masked keys the inner loop has no select at all
    uint32_t mbits = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) mbits |= (mask_s[cq * 32 + j] != 0.f ? 1u : 0u) << j;
    const bool all_keys = mbits == 0xffffffffu;
    const float sc = p.scale;
    constexpr bool drop = DROP;
    uint32_t seed_lo = 0u, seed_hi = 0u;
    if (drop) { const unsigned long long sd = *p.seed; seed_lo = (uint32_t)sd; seed_hi = (uint32_t)(sd >> 32); }
    const uint32_t bh = (uint32_t)(b * p.H + h);
    bool ok = true;
    const long rbase = ((long)b * p.H + h) * p.Tq;
    // per-row log-sum-exp and D of the next query block are fetched one block ahead (+inf: exp2(-inf) = 0 past the end)
    float lse_n = r < p.Tq ? p.lse[rbase + r] : INFINITY, dv_n = r < p.Tq ? p.dvec[rbase + r] : 0.f;
    auto dq_flush = [&](int blk) -> bool {
      // dQ_blk: 64 columns per row, 16 per thread (all four column groups take part)
      if (!mbar_wait_bounded(dq_full, (uint32_t)(blk & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) return false;
      tc_fence_after();
      uint32_t v0[16];
      tmem_ld_32x16(taddr + T_DQ + cq * 16, v0);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
      const int tqb = blk * FB_BLK + r;
      if (tqb < p.Tq) {
        float4* dst = reinterpret_cast<float4*>(p.dq + (rbase + tqb) * FA_D + cq * 16);
#pragma unroll
        for (int j = 0; j < 4; ++j)      // fire-and-forget 16-byte reductions at L2
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "r"(v0[4 * j]), "r"(v0[4 * j + 1]),
                       "r"(v0[4 * j + 2]), "r"(v0[4 * j + 3])
                       : "memory");
      }
      return true;
    };
    for (int i = 0; i < nq && ok; ++i) {
      const int tq = i * FB_BLK + r;
      const float lse = lse_n, dv_r = dv_n;
      if (i + 1 < nq) {
        const int tn = tq + FB_BLK;
        lse_n = tn < p.Tq ? p.lse[rbase + tn] : INFINITY;
        dv_n = tn < p.Tq ? p.dvec[rbase + tn] : 0.f;
      }
      // a fully masked row (lse = -inf) and rows past the end (+inf) both give exp2(-inf) = 0 for every key
      const float lse2 = (lse == -INFINITY) ? INFINITY : lse * FA_LOG2E;
      const float dvs = dv_r * sc;
      if (!mbar_wait_bounded(s_full, (uint32_t)(i & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t sv[32], dpv[32];
        tmem_ld_32x32(taddr + T_S + cq * 32, sv);
        tmem_ld_32x32(taddr + T_DP + cq * 32, dpv);
        tmem_ld_wait();
        float pe[32], de[32];
        if constexpr (DROP) {
          // the forward's mask, regenerated: dV takes the dropped weights, dS = P * (mask / keep * dP - D) * scale
          const uint32_t kw = fa_keep32(seed_lo, seed_hi, bh, (uint32_t)tq, (uint32_t)(k0 + cq * 32), p.drop_thr);
          const float ik = p.inv_keep;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float pv = ((mbits >> j) & 1u) ? fa_exp2(fmaf(__uint_as_float(sv[j]), k2, -lse2)) : 0.f;
            const float mk = ((kw >> j) & 1u) ? ik : 0.f;
            pe[j] = pv * mk;
            de[j] = pv * fmaf(__uint_as_float(dpv[j]) * mk, sc, -dvs);
          }
        } else if (all_keys) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float pv = fa_exp2(fmaf(__uint_as_float(sv[j]), k2, -lse2));
            pe[j] = pv;
            de[j] = pv * fmaf(__uint_as_float(dpv[j]), sc, -dvs);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float pv = ((mbits >> j) & 1u) ? fa_exp2(fmaf(__uint_as_float(sv[j]), k2, -lse2)) : 0.f;
            pe[j] = pv;
            de[j] = pv * fmaf(__uint_as_float(dpv[j]), sc, -dvs);
          }
        }
        fa_store_row(p_s, r, cq * 32, 32, pe);
        fa_store_row(ds_s, r, cq * 32, 32, de);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // dQ of the previous block: read out of tensor memory and reduced into global memory now, while the MMA thread issues
      // the dV / dK products of this block (the reductions stall their warp on the L2 atomics queue for about a microsecond)
      if (i > 0 && !dq_flush(i - 1)) { ok = false; break; }
    }
    if (ok && nq > 0) ok = dq_flush(nq - 1);
    if (ok && mbar_wait_bounded(fin_full, 0, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) {
      tc_fence_after();
      // accumulator rows are keys here: thread r owns key k0 + r; column groups 0, 1 -> dV, 2, 3 -> dK
      const long orow = (long)b * p.o_bs + (long)(k0 + r) * p.o_ts + (long)h * FA_D + (cq & 1) * 32;
      uint32_t v0[32];
      tmem_ld_32x32(taddr + (cq < 2 ? T_DV : T_DK) + (cq & 1) * 32, v0);
      tmem_ld_wait();
      uint4* dst = reinterpret_cast<uint4*>((cq < 2 ? p.dv : p.dk) + orow);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u;
        __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(__uint_as_float(v0[8 * j + 2 * e]), __uint_as_float(v0[8 * j + 2 * e + 1]));
        dst[j] = u;
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
                                 const long* k_strides, const long* v_strides, const long* do_strides, long o_bs, long o_ts, float scale,
                                 float dropout_p, const void* seed, void* stream_) {
  if (B < 1 || H < 1 || Tq < 1 || Tk < FB_BLK || Tk % FB_BLK) return -DL4J_ERR_BAD_ARG;
  if (dropout_p < 0.f || dropout_p >= 1.f || (dropout_p > 0.f && !seed)) return -DL4J_ERR_BAD_ARG;
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
  p.seed = reinterpret_cast<const unsigned long long*>(seed);
  p.drop_thr = dropout_p > 0.f ? (uint32_t)(dropout_p * 65536.f + 0.5f) : 0u;
  p.inv_keep = p.drop_thr ? 65536.f / (65536.f - (float)p.drop_thr) : 1.f;
  const size_t smem = 6 * FB_TILE + 2 * FB_PS + FB_BLK * sizeof(float) + 256 + 1024;
  auto kern = p.drop_thr ? flash_attn_bwd_kernel<true> : flash_attn_bwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  kern<<<B * H * (Tk / FB_BLK), FB_THREADS, smem, (cudaStream_t)stream_>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ small helpers of the backward pass
namespace dl4j {

// dvec[b, h, t] = sum_d dO[b, h, t, d] * O[b, t, h, d]; eight threads per row, 8 elements each
__global__ void __launch_bounds__(256)
attn_dvec_kernel(const __nv_bfloat16* __restrict__ dO, long sb, long sh, long st, const __nv_bfloat16* __restrict__ O, float* __restrict__ dvec,
                 int B, int H, int T) {
  const long rows = (long)B * H * T;
  const long g = blockIdx.x * 256L + threadIdx.x;
  const long row = g >> 3;
  const int part = (int)(g & 7);
  float acc = 0.f;
  if (row < rows) {
    const int t = (int)(row % T);
    const int h = (int)((row / T) % H);
    const int b = (int)(row / ((long)T * H));
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(dO + b * sb + h * sh + t * st) + part);
    const uint4 c = __ldg(reinterpret_cast<const uint4*>(O + (((long)b * T + t) * H + h) * FA_D) + part);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* ch = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(ah[i]), y = __bfloat1622float2(ch[i]);
      acc = fmaf(x.x, y.x, fmaf(x.y, y.y, acc));
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (row < rows && part == 0) dvec[row] = acc;
}

// dq (bf16, addressed base + b * o_bs + t * o_ts + h * 64) = acc [B, H, T, 64] fp32; the accumulator is cleared for its next use
__global__ void __launch_bounds__(256)
attn_dq_finish_kernel(float* __restrict__ acc, __nv_bfloat16* __restrict__ out, long o_bs, long o_ts, int B, int H, int T) {
  const long n8 = (long)B * H * T * (FA_D / 8);
  for (long g = blockIdx.x * 256L + threadIdx.x; g < n8; g += (long)gridDim.x * 256) {
    const int part = (int)(g & 7);
    const long row = g >> 3;
    const int t = (int)(row % T);
    const int h = (int)((row / T) % H);
    const int b = (int)(row / ((long)T * H));
    float4* src = reinterpret_cast<float4*>(acc) + 2 * g;
    const float4 x = src[0], y = src[1];
    uint4 u;
    __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
    hh[0] = __floats2bfloat162_rn(x.x, x.y); hh[1] = __floats2bfloat162_rn(x.z, x.w);
    hh[2] = __floats2bfloat162_rn(y.x, y.y); hh[3] = __floats2bfloat162_rn(y.z, y.w);
    reinterpret_cast<uint4*>(out + b * o_bs + t * o_ts + (long)h * FA_D)[part] = u;
    src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

}  // namespace dl4j

DL4J_API int dl4j_attn_dvec(const void* dout, const long* do_strides, const void* out, float* dvec, int B, int H, int T, void* stream) {
  const long threads = (long)B * H * T * 8;
  attn_dvec_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), do_strides[0], do_strides[1], do_strides[2], reinterpret_cast<const __nv_bfloat16*>(out),
      dvec, B, H, T);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_attn_dq_finish(float* acc, void* out, long o_bs, long o_ts, int B, int H, int T, void* stream) {
  const long n8 = (long)B * H * T * 8;
  long blocks = (n8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  attn_dq_finish_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(acc, reinterpret_cast<__nv_bfloat16*>(out), o_bs, o_ts, B, H, T);
  return (int)cudaGetLastError();
}
