// Fused scaled-dot-product attention forward for head size 64 (bf16), one CTA per (batch, head, 128-query block), two
// CTAs resident per SM so that one CTA's softmax overlaps the other's loads and MMAs:
//     for each block of 128 keys:  S = Q K_j^T (tcgen05, fp32 in TMEM)  ->  online softmax in registers  ->
//     P_j (bf16) staged in shared memory  ->  P_j V_j (tcgen05, TMEM)  ->  O = O * alpha + P_j V_j in registers
//     finally: normalise, store O [B, Tq, H, 64] and the row log-sum-exp [B, H, Tq].
// The score matrix never reaches HBM (AttentionHelper.cpp computes matmul, scale, mask add, softmax over the full
// score matrix and a second matmul as separate ops).  Warp 0 issues the TMA loads (K / V blocks through a 3-slot
// ring), warp 1 the MMAs, warps 2-9 do the softmax: two threads per query row, each owning half of the columns.
#include "flash_common.cuh"

namespace dl4j {

constexpr int FF_BM = 128;                    // queries per CTA
constexpr int FF_BN = 128;                    // keys per block
constexpr int FF_THREADS = 64 + 256;
constexpr int FF_TILE = 128 * FA_D * 2;       // 16 KB: Q tile, one K block or one V block
constexpr int FF_P_BYTES = FF_BM * FF_BN * 2; // 32 KB
constexpr int FF_SLOTS = 3;
constexpr int FF_TMEM_COLS = 256;             // S: 0..127, P V: 128..191
constexpr uint32_t FF_T_PV = 128;

struct FlashFwdParams {
  __nv_bfloat16* out;        // [B, Tq, H, 64]
  float* lse;                // [B, H, Tq]
  const float* key_mask;     // [B, Tk] (non-zero = keep) or null
  int B, H, Tq, Tk;
  float scale;
  int* status;
  const unsigned long long* seed;   // device-resident dropout seed (read when drop_thr != 0)
  uint32_t drop_thr;                // round(p * 65536); 0 = no dropout
  float inv_keep;                   // 1 / (1 - p)
};

template <bool DROP>
__global__ void __launch_bounds__(FF_THREADS, 2)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const FlashFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = q_s + FF_TILE;                    // FF_SLOTS tiles, filled in the order K_0, V_0, K_1, V_1, ...
  uint8_t* p_s = kv_s + FF_SLOTS * FF_TILE;
  float* mask_s = reinterpret_cast<float*>(p_s + FF_P_BYTES);         // [2][128] key mask of the current and the next key block
  float* xch = mask_s + 2 * FF_BN;                                    // [2][2][128] per-row exchange between the two column halves, by block parity
  uint64_t* bars = reinterpret_cast<uint64_t*>(xch + 4 * FF_BM + 4);     // 4 floats: failure flag + padding
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;          // [FF_SLOTS]
  uint64_t* kv_empty = kv_full + FF_SLOTS;
  uint64_t* s_full = kv_empty + FF_SLOTS;
  uint64_t* p_full = s_full + 1;
  uint64_t* pv_full = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blocks = (p.Tq + FF_BM - 1) / FF_BM;
  const int qb = blockIdx.x % q_blocks;
  const int h = (blockIdx.x / q_blocks) % p.H;
  const int b = blockIdx.x / (q_blocks * p.H);
  const int nb = p.Tk / FF_BN;
  const int q0 = qb * FF_BM;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < FF_SLOTS; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);
    mbar_init(pv_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, FF_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, FF_TILE);
      tma_load_4d(q_s, &tmap_q, q_full, 0, q0, h, b);
      for (int t = 0; t < 2 * nb; ++t) {              // tile t: K block t/2 (even) or V block t/2 (odd)
        const int slot = t % FF_SLOTS;
        const uint32_t ph = (uint32_t)((t / FF_SLOTS) & 1);
        if (!mbar_wait_bounded(&kv_empty[slot], ph ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&kv_full[slot], FF_TILE);
        tma_load_4d(kv_s + slot * FF_TILE, (t & 1) ? &tmap_v : &tmap_k, &kv_full[slot], 0, (t >> 1) * FF_BN, h, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(1, 0, 0, FF_BM, FF_BN);      // S = Q K^T: both operands K-major (K = head dim)
      const uint32_t idesc_o = make_idesc(1, 0, 1, FF_BM, FA_D);       // P V: V [keys, 64] is MN-major for the B operand
      const uint64_t dq = make_smem_desc_sw128(smem_u32(q_s), 16, 1024);
      const uint32_t pp = smem_u32(p_s);
      bool ok = mbar_wait_bounded(q_full, 0, p.status, DL4J_ERR_TIMEOUT_MMA);
      auto issue_s = [&](int j) -> bool {
        const int t = 2 * j, slot = t % FF_SLOTS;
        if (!mbar_wait_bounded(&kv_full[slot], (uint32_t)((t / FF_SLOTS) & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint64_t dk = make_smem_desc_sw128(smem_u32(kv_s + slot * FF_TILE), 16, 1024);
#pragma unroll
        for (int k = 0; k < FA_D / 16; ++k)
          umma_f16(tmem_base, dq + ((uint64_t)(k * 32) >> 4), dk + ((uint64_t)(k * 32) >> 4), idesc_s, k > 0 ? 1u : 0u);
        umma_commit(&kv_empty[slot]);
        umma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nb && ok; ++j) {
        // P_j is in shared memory (and S_j has been read out of TMEM) once p_full completes
        if (!mbar_wait_bounded(p_full, (uint32_t)(j & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        // S_{j+1} first: the threads take its row maxima while P_j V_j runs (S_j has been read out, K_{j+1} sits in the ring)
        if (j + 1 < nb && !(ok = issue_s(j + 1))) break;
        const int t = 2 * j + 1, slot = t % FF_SLOTS;
        if (!mbar_wait_bounded(&kv_full[slot], (uint32_t)((t / FF_SLOTS) & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pv = smem_u32(kv_s + slot * FF_TILE);
#pragma unroll
        for (int k = 0; k < FF_BN / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(pp + (k >> 2) * (FF_BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(pv + k * (16 * 128), 64 * 128, 1024);
          umma_f16(tmem_base + FF_T_PV, da, db, idesc_o, k > 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[slot]);
        umma_commit(pv_full);
      }
    }
  } else {
    const int cw = warp - 2;                        // 0..7
    const int q = warp & 3;                         // TMEM lane quadrant this warp may access (warp index modulo 4)
    const int ch = cw >> 2;                         // column half owned by this thread
    const int r = q * 32 + lane;                    // query row within the block
    const int t = threadIdx.x - 64;                 // 0..255
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    const float k2 = p.scale * FA_LOG2E;
    constexpr bool drop = DROP;
    uint32_t seed_lo = 0u, seed_hi = 0u;
    if (drop) { const unsigned long long sd = *p.seed; seed_lo = (uint32_t)sd; seed_hi = (uint32_t)(sd >> 32); }
    const uint32_t bh = (uint32_t)(b * p.H + h);
    float run_m = -INFINITY, run_l = 0.f;           // running row maximum (raw scores) and this thread's partial row sum
    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = 0.f;
    float alpha_prev = 0.f;                         // rescale factor that goes with the pending P V product
    bool broke = false;
    // O = O * alpha + P_blk V_blk (this thread: 32 of the 64 head-dimension columns); deferred by one block so that the product
    // runs on the tensor core while the threads take the next block's row maxima
    auto o_update = [&](int blk, float a) {
      if (!mbar_wait_bounded(pv_full, (uint32_t)(blk & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) {
        *reinterpret_cast<volatile int*>(xch + 4 * FF_BM) = 1;      // seen by everybody after the next barrier
      } else {
        tc_fence_after();
        uint32_t pv[32];
        tmem_ld_32x32(taddr + FF_T_PV + ch * 32, pv);
        tmem_ld_wait();
        tc_fence_before();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = fmaf(o[i], a, __uint_as_float(pv[i]));
      }
    };
    volatile int* fail_s = reinterpret_cast<volatile int*>(xch + 4 * FF_BM);    // set by any thread whose bounded wait expired
    if (t == 0) *fail_s = 0;
    // Key mask: block 0 is staged here, block j + 1 is fetched into a register at the top of block j and stored at its end, so
    // no global-memory latency sits between the barriers.  Without a mask the loops below have no select at all.
    const bool has_mask = p.key_mask != nullptr;
    if (has_mask && t < FF_BN) mask_s[t] = p.key_mask[(long)b * p.Tk + t];
    asm volatile("bar.sync 1, 256;" ::: "memory");
    for (int j = 0; j < nb; ++j) {
      float mask_next = 1.f;
      if (has_mask && j + 1 < nb && t < FF_BN) mask_next = p.key_mask[(long)b * p.Tk + (j + 1) * FF_BN + t];
      float* xj = xch + (j & 1) * (2 * FF_BM);       // exchange buffer of this block (the other parity may still be read)
      if (!mbar_wait_bounded(s_full, (uint32_t)(j & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) *fail_s = 1;
      tc_fence_after();
      // this thread's 64 keys as two bit words
      uint32_t mb0 = 0xffffffffu, mb1 = 0xffffffffu;
      if (has_mask) {
        const float* mk = mask_s + (j & 1) * FF_BN + ch * 64;
        mb0 = 0u; mb1 = 0u;
#pragma unroll
        for (int i = 0; i < 32; ++i) { mb0 |= (mk[i] != 0.f ? 1u : 0u) << i; mb1 |= (mk[32 + i] != 0.f ? 1u : 0u) << i; }
      }
      const bool all_keys = (mb0 & mb1) == 0xffffffffu;
      float m = -INFINITY;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32];
        tmem_ld_32x32(taddr + ch * 64 + half * 32, sv);
        tmem_ld_wait();
        const uint32_t mb = half ? mb1 : mb0;
        if (all_keys) {
#pragma unroll
          for (int i = 0; i < 32; ++i) m = fmaxf(m, __uint_as_float(sv[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if ((mb >> i) & 1u) m = fmaxf(m, __uint_as_float(sv[i]));
        }
      }
      // the next block's mask is published before this block's barrier and read after it (its buffer was last read before
      // the previous block's barrier)
      if (has_mask && j + 1 < nb && t < FF_BN) mask_s[((j + 1) & 1) * FF_BN + t] = mask_next;
      xj[ch * FF_BM + r] = m;
      asm volatile("bar.sync 1, 256;" ::: "memory");      // the only barrier of the block
      if (*fail_s) { broke = true; break; }          // uniform: every thread reads the flag after the same barrier
      m = fmaxf(m, xj[(ch ^ 1) * FF_BM + r]);
      const float new_m = fmaxf(run_m, m);
      const float mref = (new_m == -INFINITY) ? 0.f : new_m;
      const float alpha = (run_m == -INFINITY) ? 0.f : fa_exp2((run_m - mref) * k2);
      run_m = new_m;
      const float mk2 = mref * k2;
      if (j > 0) o_update(j - 1, alpha_prev);         // also: P_{j-1} V_{j-1} has finished reading P before P_j is written below
      alpha_prev = alpha;
      float l = 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t sv[32];
        tmem_ld_32x32(taddr + ch * 64 + half * 32, sv);
        tmem_ld_wait();
        float e[32];
        const uint32_t mb = half ? mb1 : mb0;
        if (all_keys) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { e[i] = fa_exp2(fmaf(__uint_as_float(sv[i]), k2, -mk2)); l += e[i]; }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            e[i] = ((mb >> i) & 1u) ? fa_exp2(fmaf(__uint_as_float(sv[i]), k2, -mk2)) : 0.f;
            l += e[i];
          }
        }
        if constexpr (DROP) {       // the row sum above is the undropped one: O = (P o mask / keep) V / l
          const uint32_t kw = fa_keep32(seed_lo, seed_hi, bh, (uint32_t)(q0 + r), (uint32_t)(j * FF_BN + ch * 64 + half * 32), p.drop_thr);
#pragma unroll
          for (int i = 0; i < 32; ++i) e[i] = ((kw >> i) & 1u) ? e[i] * p.inv_keep : 0.f;
        }
        fa_store_row(p_s, r, ch * 64 + half * 32, 32, e);
      }
      run_l = fmaf(run_l, alpha, l);
      tc_fence_before();
      fence_proxy_async_smem();       // P was written through the generic proxy; the MMA reads it through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (!broke && nb > 0) o_update(nb - 1, alpha_prev);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!*fail_s) {
      float* xl = xch + (nb & 1) * (2 * FF_BM);
      xl[ch * FF_BM + r] = run_l;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const float l = run_l + xl[(ch ^ 1) * FF_BM + r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int tq = q0 + r;
      if (tq < p.Tq) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + (((long)b * p.Tq + tq) * p.H + h) * FA_D + ch * 32);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          uint4 u;
          __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
          for (int i = 0; i < 4; ++i) hh[i] = __floats2bfloat162_rn(o[jj * 8 + 2 * i] * inv, o[jj * 8 + 2 * i + 1] * inv);
          dst[jj] = u;
        }
        if (p.lse && ch == 0) {
          const float mref = (run_m == -INFINITY) ? 0.f : run_m;
          p.lse[((long)b * p.H + h) * p.Tq + tq] = l > 0.f ? mref * p.scale + __logf(l) : -INFINITY;
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, FF_TMEM_COLS);
  }
}

}  // namespace dl4j

using namespace dl4j;

// q / k / v: [B, H, T, 64] bf16 views with element strides {sb, sh, st} (head dimension contiguous, strides multiples of 8,
// base 16-byte aligned).  out [B, Tq, H, 64] bf16 contiguous, lse [B, H, Tq] fp32, key_mask [B, Tk] fp32 or null.
// Limits: Tk a multiple of 128.  dropout_p > 0: `seed` points to a 64-bit seed in device memory; pass the same seed and
// probability to the backward pass.
DL4J_API int dl4j_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const float* key_mask, int B, int H,
                                 int Tq, int Tk, const long* q_strides, const long* k_strides, const long* v_strides, float scale,
                                 float dropout_p, const void* seed, void* stream_) {
  if (B < 1 || H < 1 || Tq < 1 || Tk < FF_BN || Tk % FF_BN) return -DL4J_ERR_BAD_ARG;
  if (dropout_p < 0.f || dropout_p >= 1.f || (dropout_p > 0.f && !seed)) return -DL4J_ERR_BAD_ARG;
  CUtensorMap tq, tk, tv;
  int r = fa_encode(&tq, q, B, H, Tq, q_strides[0], q_strides[1], q_strides[2], FF_BM);
  if (r) return -1000 - r;
  r = fa_encode(&tk, k, B, H, Tk, k_strides[0], k_strides[1], k_strides[2], FF_BN);
  if (r) return -1000 - r;
  r = fa_encode(&tv, v, B, H, Tk, v_strides[0], v_strides[1], v_strides[2], FF_BN);
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
  p.seed = reinterpret_cast<const unsigned long long*>(seed);
  p.drop_thr = dropout_p > 0.f ? (uint32_t)(dropout_p * 65536.f + 0.5f) : 0u;
  p.inv_keep = p.drop_thr ? 65536.f / (65536.f - (float)p.drop_thr) : 1.f;
  const size_t smem = FF_TILE * (1 + FF_SLOTS) + FF_P_BYTES + (2 * FF_BN + 4 * FF_BM + 4) * sizeof(float) + 256 + 1024;
  auto kern = p.drop_thr ? flash_attn_fwd_kernel<true> : flash_attn_fwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int q_blocks = (Tq + FF_BM - 1) / FF_BM;
  kern<<<B * H * q_blocks, FF_THREADS, smem, (cudaStream_t)stream_>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}
