// bf16/fp16 GEMM on the 5th-generation tensor cores: D = act(A·B + bias) (+ residual).
//
// Replaces the reference's cuBLAS call sites and naive SIMT fallbacks
// (libnd4j/include/helpers/cuda/MmulHelper.cu:41-129 usualCudaGemm, :501-517 cublas*gemm) and the
// matmul+addBias+activation sequences of xw_plus_b / relu_layer / DenseLayer.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      : TMA producer  - cp.async.bulk.tensor tiles of A and B into a multi-stage smem ring
//   warp 1      : MMA issuer    - one elected lane issues tcgen05.mma (128 x BLOCK_N x 16), accumulators
//                                 live in TMEM, double-buffered (2 x BLOCK_N columns) so the epilogue of
//                                 tile i overlaps the main loop of tile i+1
//   warps 2..5  : epilogue      - tcgen05.ld 32 lanes x 32 columns, bias / activation / residual,
//                                 16-byte global stores (or fp32 vector reductions for split-K)
// Operands may be K-major (reduction dimension contiguous) or MN-major (output dimension contiguous),
// which covers forward (X·Wᵀ), data-gradient (dY·W) and weight-gradient (dYᵀ·X) without transposes.
#include "common.cuh"

namespace dl4j {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;         // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  long ldc;               // elements
  long ld_aux, ld_res;
  void* C;
  void* aux;              // optional pre-activation output (same dtype as inputs)
  const void* bias;       // optional [N], dtype bias_fp32 ? float : input dtype
  const void* residual;   // optional [M, N] input dtype
  int bias_fp32;
  int out_fp32;           // C is float
  int act;                // 0 none, 1 relu, 2 gelu(erf), 3 gelu(tanh), 4 sigmoid, 5 tanh
  int atomic_out;         // accumulate into fp32 C with vector reductions (split-K / grad accumulation)
  int splits;             // split-K factor (>1 requires atomic_out)
  int fmt;                // 0 fp16, 1 bf16
  float alpha;
  int* status;
  int batch1, batch2;     // two batch dimensions (1 when unused); batch index = b2 * batch1 + b1
  long c_stride_b1, c_stride_b2;   // output batch strides in elements
  int tma_store;          // epilogue stages tiles in shared memory and writes them with TMA (needs 16-byte aligned C rows)
  int tma_aux;            // same for the auxiliary pre-activation output
  int bias_mma;           // the bias is added on the tensor core: one extra K=16 step ones[128 x 1] x bias[1 x N] per tile
  int raster_gn;          // tile raster: column-tile groups of this width, column index fastest inside a group
  int res_act;            // != 0: `residual` holds pre-activations z and the result is multiplied by act'(z) instead of added to
                          // (the data-gradient GEMM of a layer that feeds an activation writes dz directly)
};

// Tile order.  CTAs that run at the same time take consecutive tile numbers, so the order decides what they share in L2:
// within a group of `gn` column tiles the column index runs fastest, i.e. the CTAs of one wave cover few row panels of A
// (each read from DRAM once and hit in L2 by the other column tiles) and at most gn column panels of B.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int gn, int& mt, int& nt) {
  const int per_group = tiles_m * gn;
  const int g = tile / per_group;
  const int n_base = g * gn;
  const int gw = min(gn, tiles_n - n_base);
  const int r = tile - g * per_group;
  mt = r / gw;
  nt = n_base + (r - mt * gw);
}

template <int BLOCK_N, bool A_MN, bool B_MN>
struct GemmSmem {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int EPI_SLAB = 32 * 128;                 // one warp's 32 rows x 128 bytes
  static constexpr int EPI_BYTES = 4 * 2 * EPI_SLAB;        // 4 epilogue warps x 2 ring buffers
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case 1: return fmaxf(v, 0.0f);
    case 2: return gelu_erf(v);
    case 3: return gelu_tanh(v);
    case 4: return sigmoidf_(v);
    case 5: return tanhf(v);
    case 6: return gelu_sigmoid(v);
    default: return v;
  }
}

// v *= act'(z): the activation-gradient factor applied in the epilogue of a data-gradient GEMM.  The GELU forms use one
// tanh.approx per value (sigmoid(y) = 0.5 + 0.5 tanh(y / 2)).
__device__ __forceinline__ float tanh_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
__device__ __forceinline__ float mul_act_grad(float v, float z, int act) {
  switch (act) {
    case 1: return z > 0.f ? v : 0.f;
    case 2: return v * (0.5f * (1.f + erff(z * 0.70710678118654752f)) + z * 0.3989422804014327f * __expf(-0.5f * z * z));
    case 3: {
      const float z2 = z * z;
      const float t = tanh_fast(0.7978845608028654f * z * fmaf(0.044715f, z2, 1.f));
      return v * (fmaf(0.5f, t, 0.5f) + 0.5f * z * (1.f - t * t) * 0.7978845608028654f * fmaf(0.134145f, z2, 1.f));
    }
    case 4: { const float sg = fmaf(0.5f, tanh_fast(0.5f * z), 0.5f); return v * sg * (1.f - sg); }
    case 5: { const float t = tanh_fast(z); return v * (1.f - t * t); }
    case 6: { const float sg = fmaf(0.5f, tanh_fast(0.851f * z), 0.5f); return v * fmaf(1.702f * z * sg, 1.f - sg, sg); }
    default: return v;
  }
}

// Warp-uniform dispatch hoisted out of the element loop.
__device__ __forceinline__ void apply_act32(float (&v)[32], int act) {
  if (act == 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
  } else if (act == 2) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
  } else if (act == 3) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
  } else if (act == 6) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_sigmoid(v[j]);
  } else if (act == 4) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = sigmoidf_(v[j]);
  } else if (act == 5) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = tanhf(v[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], act);
  }
}

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ uint32_t pack2(float a, float b, int fmt) {
  if (fmt == 1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float unpack_lo(uint32_t u, int fmt) {
  if (fmt == 1) return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&u));
  return __half2float(*reinterpret_cast<__half*>(&u));
}

// bias[col] as float (0 beyond N); the bias vector is fp32 or the operand type
__device__ __forceinline__ float load_bias(const GemmParams& p, int col) {
  if (col >= p.N) return 0.f;
  return p.bias_fp32 ? __ldg(reinterpret_cast<const float*>(p.bias) + col)
                     : unpack_lo((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.bias) + col), p.fmt);
}
__device__ __forceinline__ float unpack_hi(uint32_t u, int fmt) {
  uint32_t h = u >> 16;
  if (fmt == 1) return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&h));
  return __half2float(*reinterpret_cast<__half*>(&h));
}

template <int BLOCK_N, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux,
                    const __grid_constant__ CUtensorMap tmap_ones, const __grid_constant__ CUtensorMap tmap_bias,
                    const GemmParams p) {
  using S = GemmSmem<BLOCK_N, A_MN, B_MN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * S::STAGE_BYTES;       // 1024-byte aligned (stage sizes are multiples of 1024)
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + S::EPI_BYTES);
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + STAGES;          // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;      // [2]
  uint64_t* tmem_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int kb_total = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int kb_per_split = (kb_total + p.splits - 1) / p.splits;
  const int per_batch = tiles_m * tiles_n * p.splits;
  const int num_work = per_batch * p.batch1 * p.batch2;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);   // one arrive per epilogue warp
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BLOCK_N);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int batch = w / per_batch, wr = w % per_batch;
        const int b1 = batch % p.batch1, b2 = batch / p.batch1;
        const int tile = wr / p.splits, split = wr % p.splits;
        int mt, nt;
        tile_coords(tile, tiles_m, tiles_n, p.raster_gn, mt, nt);
        const int m0 = mt * BLOCK_M, n0 = nt * BLOCK_N;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kb_total);
        if (p.bias_mma) {
          // bias stage: both operands MN-major with a single valid K row (row 0 = ones / bias, rows 1..15 zero-filled by
          // TMA because the maps' K extent is 1); only the 16 K rows of the one MMA step are written (2 KB per 64-column box
          // at the usual box addresses), so the usual stage layout and descriptors apply
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], (BLOCK_M / 64 + BLOCK_N / 64) * (64 * UMMA_K * 2));
#pragma unroll
          for (int i = 0; i < BLOCK_M / 64; ++i)
            tma_load_4d(sa + i * (64 * BLOCK_K * 2), &tmap_ones, &full_bar[stage], i * 64, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < BLOCK_N / 64; ++i)
            tma_load_4d(sb + i * (64 * BLOCK_K * 2), &tmap_bias, &full_bar[stage], n0 + i * 64, 0, 0, 0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          const int k0 = kb * BLOCK_K;
          if (!A_MN) {
            tma_load_4d(sa, &tmap_a, &full_bar[stage], k0, m0, b1, b2);
          } else {
#pragma unroll
            for (int i = 0; i < BLOCK_M / 64; ++i)
              tma_load_4d(sa + i * (64 * BLOCK_K * 2), &tmap_a, &full_bar[stage], m0 + i * 64, k0, b1, b2);
          }
          if (!B_MN) {
            tma_load_4d(sb, &tmap_b, &full_bar[stage], k0, n0, b1, b2);
          } else {
#pragma unroll
            for (int i = 0; i < BLOCK_N / 64; ++i)
              tma_load_4d(sb + i * (64 * BLOCK_K * 2), &tmap_b, &full_bar[stage], n0 + i * 64, k0, b1, b2);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.fmt, A_MN ? 1 : 0, B_MN ? 1 : 0, BLOCK_M, BLOCK_N);
      // K-major: 8-row groups are 1024 B apart (SBO); MN-major: 64-element column blocks are one
      // TMA box apart (LBO = 64 rows x 128 B) and 8-row K groups 1024 B apart (SBO).
      constexpr uint32_t LBO_A = A_MN ? 64 * BLOCK_K * 2 : 16, LBO_B = B_MN ? 64 * BLOCK_K * 2 : 16;
      constexpr uint32_t KSTEP_A = A_MN ? UMMA_K * 128 : UMMA_K * 2, KSTEP_B = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
        const int split = (w % per_batch) % p.splits;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kb_total);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        if (p.bias_mma) {
          // accumulator := ones[128 x 16] * bias[16 x BLOCK_N] (only K row 0 is non-zero): every row starts at the bias
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          umma_f16(tmem_d, make_smem_desc_sw128(sa, 64 * BLOCK_K * 2, 1024), make_smem_desc_sw128(sb, 64 * BLOCK_K * 2, 1024),
                   make_idesc(p.fmt, 1, 1, BLOCK_M, BLOCK_N), 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, LBO_A, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, LBO_B, 1024);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            umma_f16(tmem_d, da + ((uint64_t)(k * KSTEP_A) >> 4), db + ((uint64_t)(k * KSTEP_B) >> 4), idesc,
                     (kb > kb0 || k > 0 || p.bias_mma) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);   // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[buf]);       // accumulator ready for the epilogue
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quadrant this warp may access
    int it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
      const int batch = w / per_batch, wr = w % per_batch;
      const long c_off = (long)(batch % p.batch1) * p.c_stride_b1 + (long)(batch / p.batch1) * p.c_stride_b2;
      const int tile = wr / p.splits, split = wr % p.splits;
      int mt, nt;
      tile_coords(tile, tiles_m, tiles_n, p.raster_gn, mt, nt);
      const int m0 = mt * BLOCK_M, n0 = nt * BLOCK_N;
      const int kb0 = split * kb_per_split;
      const bool has_k = kb0 < min(kb0 + kb_per_split, kb_total);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const bool lead_split = split == 0;
      // lane L of the warp fetches bias[col0 + L] one 32-column group ahead of its use (first group here, before the
      // wait for the accumulator), and the group is broadcast with shuffles: no load latency inside the tile loop
      const bool use_bias = p.bias != nullptr && lead_split && !p.bias_mma;
      float bias_cur = use_bias ? load_bias(p, n0 + lane) : 0.f;
      if (!mbar_wait_bounded(&tmem_full[buf], acc_phase, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr_row = tmem_base + buf * BLOCK_N + ((uint32_t)(q * 32) << 16);
      if (p.tma_store) {
        // -------- staged epilogue: registers -> swizzled smem slab (32 rows x 128 B per warp) -> TMA store / reduce
        const int b1 = batch % p.batch1, b2 = batch / p.batch1;
        uint8_t* ring = epi_smem + q * (2 * S::EPI_SLAB);
        const int sw = lane & 7;
        uint8_t* my_row0 = ring + lane * 128;
        const int cols_per_store = p.out_fp32 ? 32 : 64;
        int ring_idx = 0;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N; c += cols_per_store) {
          if (n0 + c >= p.N) break;                                   // warp-uniform
          const bool want_aux = p.aux != nullptr && p.tma_aux;
          // buffers: without aux alternate the ring (one store may still be reading the other slab);
          // with aux both slabs are filled in this iteration, so every earlier store must have been read.
          if (lane == 0) { if (want_aux) bulk_wait_read<0>(); else bulk_wait_read<1>(); }
          __syncwarp();
          uint8_t* slab_out = my_row0 + (want_aux ? S::EPI_SLAB : ring_idx * S::EPI_SLAB);
          uint8_t* slab_aux = my_row0;
          const int halves = p.out_fp32 ? 1 : 2;
#pragma unroll 1
          for (int hf = 0; hf < halves; ++hf) {
            const int col0 = n0 + c + hf * 32;
            if (col0 >= p.N) break;                                   // warp-uniform; TMA clips the unwritten half
            uint32_t r[32];
            tmem_ld_32x32(taddr_row + c + hf * 32, r);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = has_k ? __uint_as_float(r[j]) * p.alpha : 0.0f;
            if (use_bias) {
              const int next_col0 = hf + 1 < halves ? col0 + 32 : n0 + c + cols_per_store;
              const float bias_next = load_bias(p, next_col0 + lane);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, bias_cur, j);
              bias_cur = bias_next;
            }
            if (want_aux) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 u = make_uint4(pack2(v[8 * j], v[8 * j + 1], p.fmt), pack2(v[8 * j + 2], v[8 * j + 3], p.fmt),
                                           pack2(v[8 * j + 4], v[8 * j + 5], p.fmt), pack2(v[8 * j + 6], v[8 * j + 7], p.fmt));
                *reinterpret_cast<uint4*>(slab_aux + (((hf * 4 + j) ^ sw) << 4)) = u;
              }
            }
            if (p.act != 0) apply_act32(v, p.act);
            if (p.residual != nullptr && lead_split && row_ok) {
              const uint16_t* rs = reinterpret_cast<const uint16_t*>(p.residual) + (long)row * p.ld_res + col0;
              if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(rs) & 15) == 0)) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  const uint4 u = *reinterpret_cast<const uint4*>(rs + j);
                  const float z8[8] = {unpack_lo(u.x, p.fmt), unpack_hi(u.x, p.fmt), unpack_lo(u.y, p.fmt), unpack_hi(u.y, p.fmt),
                                       unpack_lo(u.z, p.fmt), unpack_hi(u.z, p.fmt), unpack_lo(u.w, p.fmt), unpack_hi(u.w, p.fmt)};
                  if (p.res_act) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[j + e] = mul_act_grad(v[j + e], z8[e], p.res_act);
                  } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[j + e] += z8[e];
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) {
                    const float z = unpack_lo((uint32_t)rs[j], p.fmt);
                    v[j] = p.res_act ? mul_act_grad(v[j], z, p.res_act) : v[j] + z;
                  }
              }
            }
            if (p.out_fp32) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(slab_out + ((j ^ sw) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 u = make_uint4(pack2(v[8 * j], v[8 * j + 1], p.fmt), pack2(v[8 * j + 2], v[8 * j + 3], p.fmt),
                                           pack2(v[8 * j + 4], v[8 * j + 5], p.fmt), pack2(v[8 * j + 6], v[8 * j + 7], p.fmt));
                *reinterpret_cast<uint4*>(slab_out + (((hf * 4 + j) ^ sw) << 4)) = u;
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int r0 = m0 + q * 32;
            if (r0 < p.M) {
              if (want_aux) tma_store_4d(&tmap_aux, ring, n0 + c, r0, b1, b2);
              uint8_t* src = ring + (want_aux ? S::EPI_SLAB : ring_idx * S::EPI_SLAB);
              if (p.atomic_out) tma_reduce_add_4d(&tmap_c, src, n0 + c, r0, b1, b2);
              else tma_store_4d(&tmap_c, src, n0 + c, r0, b1, b2);
            }
            bulk_commit();
          }
          ring_idx ^= 1;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BLOCK_N; c += 32) {
        const int col0 = n0 + c;
        if (col0 >= p.N) break;             // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = has_k ? __uint_as_float(r[j]) * p.alpha : 0.0f;
        const bool full_chunk = col0 + 32 <= p.N;
        if (p.bias != nullptr && lead_split && !p.bias_mma) {
          if (p.bias_fp32) {
            const float* b = reinterpret_cast<const float*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (full_chunk || col0 + j < p.N) v[j] += __ldg(b + j);
          } else if (p.fmt == 1) {
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (full_chunk || col0 + j < p.N) v[j] += __bfloat162float(b[j]);
          } else {
            const __half* b = reinterpret_cast<const __half*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (full_chunk || col0 + j < p.N) v[j] += __half2float(b[j]);
          }
        }
        if (row_ok) {
          if (p.aux != nullptr) {
            uint16_t* a = reinterpret_cast<uint16_t*>(p.aux) + (long)row * p.ld_aux + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(a) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 u = make_uint4(pack2(v[j], v[j + 1], p.fmt), pack2(v[j + 2], v[j + 3], p.fmt),
                                     pack2(v[j + 4], v[j + 5], p.fmt), pack2(v[j + 6], v[j + 7], p.fmt));
                *reinterpret_cast<uint4*>(a + j) = u;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) a[j] = (uint16_t)(pack2(v[j], 0.f, p.fmt) & 0xffff);
            }
          }
          if (p.act != 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
          }
          if (p.residual != nullptr && lead_split) {
            const uint16_t* rs = reinterpret_cast<const uint16_t*>(p.residual) + (long)row * p.ld_res + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(rs) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                const uint4 u = *reinterpret_cast<const uint4*>(rs + j);
                const float z8[8] = {unpack_lo(u.x, p.fmt), unpack_hi(u.x, p.fmt), unpack_lo(u.y, p.fmt), unpack_hi(u.y, p.fmt),
                                     unpack_lo(u.z, p.fmt), unpack_hi(u.z, p.fmt), unpack_lo(u.w, p.fmt), unpack_hi(u.w, p.fmt)};
#pragma unroll
                for (int e = 0; e < 8; ++e) v[j + e] = p.res_act ? mul_act_grad(v[j + e], z8[e], p.res_act) : v[j + e] + z8[e];
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                const float z = unpack_lo((uint32_t)rs[j], p.fmt);
                v[j] = p.res_act ? mul_act_grad(v[j], z, p.res_act) : v[j] + z;
              }
            }
          }
          if (p.out_fp32) {
            float* o = reinterpret_cast<float*>(p.C) + c_off + (long)row * p.ldc + col0;
            const bool al = full_chunk && ((reinterpret_cast<uintptr_t>(o) & 15) == 0);
            if (p.atomic_out) {
              if (al) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + j), "f"(v[j]), "f"(v[j + 1]),
                               "f"(v[j + 2]), "f"(v[j + 3]) : "memory");
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) atomicAdd(o + j, v[j]);
              }
            } else if (al) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) o[j] = v[j];
            }
          } else {
            uint16_t* o = reinterpret_cast<uint16_t*>(p.C) + c_off + (long)row * p.ldc + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 u = make_uint4(pack2(v[j], v[j + 1], p.fmt), pack2(v[j + 2], v[j + 3], p.fmt),
                                     pack2(v[j + 4], v[j + 5], p.fmt), pack2(v[j + 6], v[j + 7], p.fmt));
                *reinterpret_cast<uint4*>(o + j) = u;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) o[j] = (uint16_t)(pack2(v[j], 0.f, p.fmt) & 0xffff);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) bulk_wait<0>();          // staged tiles must have left shared memory before the CTA exits
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BLOCK_N);
  }
}

}  // namespace dl4j

// =============================================================================== host side
using namespace dl4j;

static int encode_2d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                     uint32_t box_inner, uint32_t box_outer, uint64_t nb1 = 1, uint64_t nb2 = 1, uint64_t sb1_bytes = 0,
                     uint64_t sb2_bytes = 0, CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
  dl4j_PFN_encodeTiled enc = dl4j_get_encode_tiled();
  if (!enc) return -1;
  // rank-4 map {inner, outer, batch1, batch2}; unit batch dims get a harmless 16-byte-multiple stride
  if (sb1_bytes == 0) sb1_bytes = row_stride_bytes * outer;
  if (sb2_bytes == 0) sb2_bytes = sb1_bytes * nb1;
  cuuint64_t dims[4] = {inner, outer, nb1, nb2};
  cuuint64_t strides[3] = {row_stride_bytes, sb1_bytes, sb2_bytes};
  cuuint32_t box[4] = {box_inner, box_outer, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// 128 ones in each operand format: the A operand of the bias step
#define DL4J_REP8(x) x, x, x, x, x, x, x, x
#define DL4J_REP128(x) DL4J_REP8(DL4J_REP8(x)), DL4J_REP8(DL4J_REP8(x))
static __device__ __align__(128) uint16_t g_ones_bf16[128] = {DL4J_REP128(0x3F80)};
static __device__ __align__(128) uint16_t g_ones_f16[128] = {DL4J_REP128(0x3C00)};

template <int BLOCK_N, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
                       const CUtensorMap& tones, const CUtensorMap& tbias, const GemmParams& p, int grid, cudaStream_t stream) {
  using S = GemmSmem<BLOCK_N, A_MN, B_MN>;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, A_MN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(ta, tb, tc, tx, tones, tbias, p);
  return (int)cudaGetLastError();
}

// C[M,N] = act(alpha * A·B + bias) (+ residual)
//   a_mn = 0: A stored [M, K] (row stride lda);  a_mn = 1: A stored [K, M] (row stride lda)
//   b_mn = 0: B stored [N, K] (row stride ldb);  b_mn = 1: B stored [K, N] (row stride ldb)
// Alignment contract (checked): base pointers 16-byte aligned, lda/ldb multiples of 8 elements.
static int gemm_impl(const void* A, const void* B, void* C, void* aux, const void* bias, const void* residual, int M,
                     int N, int K, long lda, long ldb, long ldc, long ld_aux, long ld_res, int a_mn, int b_mn, int fmt,
                     int bias_fp32, int out_fp32, int act, int atomic_out, int splits, float alpha, int block_n,
                     int num_sms, void* stream_, int batch1, int batch2, const long* a_bs, const long* b_bs,
                     const long* c_bs) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -DL4J_ERR_BAD_ARG;
  if (splits < 1) splits = 1;
  if (splits > 1 && !(atomic_out && out_fp32)) return -DL4J_ERR_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ld_aux = ld_aux; p.ld_res = ld_res; p.C = C; p.aux = aux; p.bias = bias;
  // `act` carries two ids: bits 0-7 the forward activation applied to the result, bits 8-15 an activation whose derivative at
  // `residual` multiplies the result (then `residual` is not added)
  p.residual = residual; p.bias_fp32 = bias_fp32; p.out_fp32 = out_fp32; p.act = act & 0xff; p.res_act = (act >> 8) & 0xff;
  if (p.res_act && (!residual || p.act)) return -DL4J_ERR_BAD_ARG;
  p.atomic_out = atomic_out;
  p.splits = splits; p.fmt = fmt; p.alpha = alpha; p.status = dl4j_status_word(dev);
  p.batch1 = batch1; p.batch2 = batch2; p.c_stride_b1 = c_bs[0]; p.c_stride_b2 = c_bs[1];
  if ((a_bs[0] & 7) || (a_bs[1] & 7) || (b_bs[0] & 7) || (b_bs[1] & 7)) return -DL4J_ERR_BAD_ARG;
  const uint64_t nb1 = batch1, nb2 = batch2;
  if (block_n != 128 && block_n != 256) block_n = 256;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = encode_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BLOCK_K, BLOCK_M, nb1, nb2, a_bs[0] * 2, a_bs[1] * 2);
  else       r = encode_2d(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BLOCK_K, nb1, nb2, a_bs[0] * 2, a_bs[1] * 2);
  if (r) return r > 0 ? -1000 - r : r;
  if (!b_mn) r = encode_2d(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BLOCK_K, (uint32_t)block_n, nb1, nb2, b_bs[0] * 2, b_bs[1] * 2);
  else       r = encode_2d(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BLOCK_K, nb1, nb2, b_bs[0] * 2, b_bs[1] * 2);
  if (r) return r > 0 ? -1000 - r : r;
  // output maps: a 32-row x 128-byte box per epilogue warp (64 16-bit or 32 fp32 columns)
  CUtensorMap tc, tx;
  memset(&tc, 0, sizeof(tc));
  memset(&tx, 0, sizeof(tx));
  const int esz = out_fp32 ? 4 : 2;
  p.tma_store = 0; p.tma_aux = 0;
  if (!(reinterpret_cast<uintptr_t>(C) & 15) && ((ldc * esz) % 16 == 0) && ((c_bs[0] * esz) % 16 == 0) && ((c_bs[1] * esz) % 16 == 0) &&
      (!aux || (!(reinterpret_cast<uintptr_t>(aux) & 15) && (ld_aux * 2) % 16 == 0))) {
    r = encode_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * esz, out_fp32 ? 32 : 64, 32, nb1, nb2, c_bs[0] * esz,
                  c_bs[1] * esz, out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    if (r == 0) p.tma_store = 1;
    if (r == 0 && aux) {
      r = encode_2d(&tx, aux, (uint64_t)N, (uint64_t)M, (uint64_t)ld_aux * 2, 64, 32, 1, 1, 0, 0);
      if (r == 0) p.tma_aux = 1; else p.tma_store = 0;
    }
  }
  // bias on the tensor core: needs the bias in the operand format, 16-byte aligned, and alpha = 1 (the accumulator then
  // already holds A.B + bias); the epilogue's per-element broadcast of the bias competes with the MMA operand fetch for
  // the shared-memory path and costs a quarter of a short-K tile
  CUtensorMap tones, tbias;
  memset(&tones, 0, sizeof(tones));
  memset(&tbias, 0, sizeof(tbias));
  p.bias_mma = 0;
  if (bias && !bias_fp32 && alpha == 1.0f && splits == 1 && batch1 == 1 && batch2 == 1 && !(reinterpret_cast<uintptr_t>(bias) & 15)) {
    void* ones = nullptr;
    cudaError_t ce = fmt == 1 ? cudaGetSymbolAddress(&ones, g_ones_bf16) : cudaGetSymbolAddress(&ones, g_ones_f16);
    if (ce == cudaSuccess && encode_2d(&tones, ones, 128, 1, 256, 64, UMMA_K) == 0 &&
        encode_2d(&tbias, bias, (uint64_t)N, 1, (uint64_t)((N + 7) / 8 * 8) * 2, 64, UMMA_K) == 0)
      p.bias_mma = 1;
  }
  {
    const int tn = (N + block_n - 1) / block_n;
    p.raster_gn = tn < 16 ? tn : 16;
  }
  const long tiles_l = (long)((M + BLOCK_M - 1) / BLOCK_M) * ((N + block_n - 1) / block_n) * splits * batch1 * batch2;
  if (tiles_l > 0x7fffffffL) return -DL4J_ERR_BAD_ARG;
  const int tiles = (int)tiles_l;
  if (num_sms <= 0) num_sms = 148;
  const int grid = tiles < num_sms ? tiles : num_sms;
#define DL4J_GEMM_CASE(BN, AM, BM) \
  if (block_n == BN && a_mn == AM && b_mn == BM) return launch_gemm<BN, AM != 0, BM != 0>(ta, tb, tc, tx, tones, tbias, p, grid, stream);
  DL4J_GEMM_CASE(256, 0, 0) DL4J_GEMM_CASE(256, 0, 1) DL4J_GEMM_CASE(256, 1, 0) DL4J_GEMM_CASE(256, 1, 1)
  DL4J_GEMM_CASE(128, 0, 0) DL4J_GEMM_CASE(128, 0, 1) DL4J_GEMM_CASE(128, 1, 0) DL4J_GEMM_CASE(128, 1, 1)
#undef DL4J_GEMM_CASE
  return -DL4J_ERR_BAD_ARG;
}

// C[M,N] = act(alpha * A·B + bias) (+ residual)
//   a_mn = 0: A stored [M, K] (row stride lda);  a_mn = 1: A stored [K, M] (row stride lda)
//   b_mn = 0: B stored [N, K] (row stride ldb);  b_mn = 1: B stored [K, N] (row stride ldb)
// Alignment contract (checked): base pointers 16-byte aligned, lda/ldb multiples of 8 elements.
DL4J_API int dl4j_gemm(const void* A, const void* B, void* C, void* aux, const void* bias, const void* residual, int M,
                       int N, int K, long lda, long ldb, long ldc, long ld_aux, long ld_res, int a_mn, int b_mn, int fmt,
                       int bias_fp32, int out_fp32, int act, int atomic_out, int splits, float alpha, int block_n,
                       int num_sms, void* stream_) {
  const long z[2] = {0, 0};
  return gemm_impl(A, B, C, aux, bias, residual, M, N, K, lda, ldb, ldc, ld_aux, ld_res, a_mn, b_mn, fmt, bias_fp32, out_fp32,
                   act, atomic_out, splits, alpha, block_n, num_sms, stream_, 1, 1, z, z, z);
}

// Batched form: batch index (b1, b2) with per-operand element strides {stride_b1, stride_b2} (multiples of 8 for A and B).
// Used for attention (batch = [heads, examples] over strided views of the fused QKV buffer) and batched_gemm.
DL4J_API int dl4j_gemm_batched(const void* A, const void* B, void* C, int M, int N, int K, long lda, long ldb, long ldc,
                               int a_mn, int b_mn, int fmt, int out_fp32, float alpha, int block_n, int num_sms,
                               int batch1, int batch2, const long* a_bs, const long* b_bs, const long* c_bs, void* stream_) {
  if (batch1 < 1 || batch2 < 1) return 0;
  return gemm_impl(A, B, C, nullptr, nullptr, nullptr, M, N, K, lda, ldb, ldc, 0, 0, a_mn, b_mn, fmt, 0, out_fp32, 0, 0, 1,
                   alpha, block_n, num_sms, stream_, batch1, batch2, a_bs, b_bs, c_bs);
}
