// 2-D convolution (stride 1, any kernel size / padding / dilation) as an implicit GEMM on the 5th-generation
// tensor cores: forward, data gradient and weight gradient.  No im2col buffer is ever written.
//
// Replaces the reference's im2col + GEMM convolution (libnd4j/include/ops/declarable/helpers/cuda/
// convolutions_conv2d.cu:35-121, helpers/cuda/im2col.cu:35-90, convolutions_conv2dBP.cu) and its cuDNN helper
// (ops/declarable/platform/cudnn/conv2d.cu).  Activations are NHWC (channels-last), weights [Cout, kH, kW, Cin].
//
// The gather that im2col materialises is done by the TMA unit instead: an output tile is a box of
// BW x BH x BI output pixels (columns x rows x images, at most 128), and for filter tap (r, s) the A operand of that
// tile is the same box of the input shifted by (r * dilation - pad, s * dilation - pad) -- one
// cp.async.bulk.tensor.4d load per tap and 64-channel slice, whose out-of-range pixels (the zero padding) are
// filled with zeros by the hardware.  The main loop is the GEMM's: TMA producer warp -> smem ring -> one thread
// issuing tcgen05.mma into double-buffered TMEM accumulators -> four epilogue warps.
//
//   forward   y[p, co]  = sum_{r,s,ci} x[p + (r,s) - pad, ci] * w[co, r, s, ci]        A K-major,  B K-major
//   dgrad     dx[p, ci] = sum_{r,s,co} dy[p - (r,s) + pad, co] * w[co, r, s, ci]       A K-major,  B MN-major
//   wgrad     dw[co, r, s, ci] = sum_p dy[p, co] * x[p + (r,s) - pad, ci]              A MN-major, B MN-major
//
// The weight tensor map {Cin, kH*kW, Cout} serves forward and dgrad (different box positions, no transposed copy);
// wgrad reduces over pixel boxes of exactly 64 pixels, split across CTAs, and adds its fp32 tiles into a
// [Cout, kH*kW, Cin] buffer with TMA reduce-add.  No load uses cluster multicast.
#include "common.cuh"

#include <algorithm>
#include <cstdlib>

namespace dl4j {

constexpr int CV_THREADS = 192;
constexpr int CV_HALO_THREADS = 192 + 96;    // conv_halo_kernel: three more MMA-issuing warps behind the four epilogue warps
constexpr int CV_BLOCK_K = 64;
constexpr int CV_UMMA_K = 16;
constexpr int CV_MAX_TAPS = 64;
constexpr int CV_MAX_ACC = 8;        // TMEM accumulator buffers: 512 columns / BLOCK_N      // kH * kW handled by these kernels (7 x 7 = 49)

struct ConvParams {
  int mode;                 // 0 forward, 1 data gradient
  int BW, BH, BI;           // output-pixel box of one tile (BW * BH * BI <= 128)
  int tiles_w, tiles_h, tiles_i, tiles_n;
  int n_out;                // output channels of this GEMM (Cout forward, Cin dgrad)
  int k_ch;                 // reduction channels per tap (Cin forward, Cout dgrad)
  int taps_h, taps_w, dil_h, dil_w, pad_h, pad_w;
  int act;                  // 0 none, 1 relu
  const void* bias;         // optional [n_out]
  int bias_fp32;
  int fmt;                  // 0 fp16, 1 bf16
  int* status;
};

template <int BLOCK_N>
struct ConvSmem {
  static constexpr int A_BYTES = 128 * CV_BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * CV_BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BLOCK_N == 256) ? 4 : 6;
  static constexpr int EPI_BYTES = 2 * 128 * 128;           // two staging tiles of 128 rows x 128 bytes
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
};

__device__ __forceinline__ uint32_t cv_pack2(float a, float b, int fmt) {
  if (fmt == 1) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               :
               : "l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}

// ------------------------------------------------------------------------------------------------ forward / dgrad
template <int BLOCK_N>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap tmap_a,     // activation {C, W, H, N}, box {64, BW, BH, BI}
                  const __grid_constant__ CUtensorMap tmap_b,     // weights {Cin, taps, Cout}, box {64, 1, 64}
                  const __grid_constant__ CUtensorMap tmap_c,     // output {C, W, H, N}, box {64, BW, BH, BI}
                  const ConvParams p) {
  using S = ConvSmem<BLOCK_N>;
  constexpr int STAGES = S::STAGES;
  constexpr int NACC = 512 / BLOCK_N;      // accumulator buffers in flight: small tiles are bound by the MMA -> epilogue round trip
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + S::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + CV_MAX_ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * CV_MAX_ACC);
  volatile int* epi_fail = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 2 * CV_MAX_ACC + 1);
  // per-tap input shifts, tabulated once: the single producer thread must spend as few instructions per load as it can
  // (its issue rate, not the memory system, bounded the first version of this kernel)
  __shared__ short2 tap_shift[CV_MAX_TAPS];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_i;
  const int num_work = m_tiles * p.tiles_n;
  const int taps = p.taps_h * p.taps_w;
  const int kc = (p.k_ch + CV_BLOCK_K - 1) / CV_BLOCK_K;
  const int k_iters = taps * kc;
  const uint32_t a_box_bytes = (uint32_t)(p.BW * p.BH * p.BI) * 128u;
  for (int t = threadIdx.x; t < taps; t += CV_THREADS) {
    const int r = t / p.taps_w, s = t - r * p.taps_w;
    tap_shift[t] = make_short2((short)(p.mode == 0 ? s * p.dil_w - p.pad_w : p.pad_w - s * p.dil_w),
                               (short)(p.mode == 0 ? r * p.dil_h - p.pad_h : p.pad_h - r * p.dil_h));
  }

  if (threadIdx.x == 0) {
    *epi_fail = 0;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < NACC; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 4); }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int nt = w % p.tiles_n, mt = w / p.tiles_n;
        const int w0 = (mt % p.tiles_w) * p.BW, h0 = ((mt / p.tiles_w) % p.tiles_h) * p.BH;
        const int i0 = (mt / (p.tiles_w * p.tiles_h)) * p.BI;
        const int n0 = nt * BLOCK_N;
        for (int t = 0; t < taps && ok; ++t) {
          const short2 sh = tap_shift[t];
          const int dw = sh.x, dh = sh.y;
          for (int c = 0; c < kc; ++c) {
            if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
            uint8_t* sa = smem + stage * S::STAGE_BYTES;
            uint8_t* sb = sa + S::A_BYTES;
            mbar_expect_tx(&full_bar[stage], a_box_bytes + S::B_BYTES);
            tma_load_4d(sa, &tmap_a, &full_bar[stage], c * CV_BLOCK_K, w0 + dw, h0 + dh, i0);
#pragma unroll
            for (int i = 0; i < BLOCK_N / 64; ++i) {
              if (p.mode == 0) tma_load_3d(sb + i * 8192, &tmap_b, &full_bar[stage], c * CV_BLOCK_K, t, n0 + i * 64);
              else             tma_load_3d(sb + i * 8192, &tmap_b, &full_bar[stage], n0 + i * 64, t, c * CV_BLOCK_K);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const int b_mn = p.mode == 0 ? 0 : 1;
      const uint32_t idesc = make_idesc(p.fmt, 0, b_mn, 128, BLOCK_N);
      const uint32_t lbo_b = b_mn ? 8192u : 16u;
      const uint32_t kstep_b = b_mn ? CV_UMMA_K * 128 : CV_UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
        const int buf = it % NACC;
        const uint32_t acc_phase = (it / NACC) & 1;
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        for (int ki = 0; ki < k_iters; ++ki) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, lbo_b, 1024);
#pragma unroll
          for (int k = 0; k < CV_BLOCK_K / CV_UMMA_K; ++k)
            umma_f16(tmem_d, da + ((uint64_t)(k * CV_UMMA_K * 2) >> 4), db + ((uint64_t)(k * kstep_b) >> 4), idesc,
                     (ki > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;
    const int row = q * 32 + lane;                 // accumulator row = pixel index inside the box
    const int sw = row & 7;
    const bool issuer = (warp == 2 && lane == 0);
    int it = 0, chunk = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
      const int nt = w % p.tiles_n, mt = w / p.tiles_n;
      const int w0 = (mt % p.tiles_w) * p.BW, h0 = ((mt / p.tiles_w) % p.tiles_h) * p.BH;
      const int i0 = (mt / (p.tiles_w * p.tiles_h)) * p.BI;
      const int n0 = nt * BLOCK_N;
      const int buf = it % NACC;
      const uint32_t acc_phase = (it / NACC) & 1;
      if (!mbar_wait_bounded(&tmem_full[buf], acc_phase, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) *epi_fail = 1;
      // the four epilogue warps meet at named barriers below, so they must leave together: share the verdict
      named_bar_sync(1, 128);
      if (*epi_fail != 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr_row = tmem_base + buf * BLOCK_N + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BLOCK_N; c += 64, ++chunk) {
        if (n0 + c >= p.n_out) break;              // uniform over the four warps
        uint8_t* tile = epi_smem + (chunk & 1) * (128 * 128);
        uint8_t* my_row = tile + row * 128;
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          const int col0 = n0 + c + hf * 32;
          uint32_t r[32];
          tmem_ld_32x32(taddr_row + c + hf * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (p.bias != nullptr) {
            if (p.bias_fp32) {
              const float* b = reinterpret_cast<const float*>(p.bias);
#pragma unroll
              for (int j = 0; j < 32; ++j) if (col0 + j < p.n_out) v[j] += __ldg(b + col0 + j);
            } else {
              const uint16_t* b = reinterpret_cast<const uint16_t*>(p.bias);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.n_out) {
                  const uint32_t u = __ldg(b + col0 + j);
                  v[j] += p.fmt == 1 ? __uint_as_float(u << 16) : __half2float(__ushort_as_half((unsigned short)u));
                }
            }
          }
          if (p.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 u = make_uint4(cv_pack2(v[8 * j], v[8 * j + 1], p.fmt), cv_pack2(v[8 * j + 2], v[8 * j + 3], p.fmt),
                                       cv_pack2(v[8 * j + 4], v[8 * j + 5], p.fmt), cv_pack2(v[8 * j + 6], v[8 * j + 7], p.fmt));
            *reinterpret_cast<uint4*>(my_row + (((hf * 4 + j) ^ sw) << 4)) = u;
          }
        }
        fence_proxy_async_smem();
        // the store of the previous chunk (other staging tile) must have been read before the next chunk overwrites it
        if (issuer) bulk_wait_read<0>();
        named_bar_sync(1, 128);
        if (issuer) {
          tma_store_4d(&tmap_c, tile, n0 + c, w0, h0, i0);
          bulk_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (issuer) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}


// ------------------------------------------------------------------------------------------------ forward / dgrad, halo form
// Same contraction as conv_igemm_kernel, but the input is fetched once per 64-channel slice instead of once per filter tap:
// an output tile is 8 columns x 16 rows of one image, and the slice of the input that all taps of that tile touch (the tile
// plus its halo, HR rows x PW columns with PW a multiple of 8) is one TMA box in shared memory.  The A operand of tap (r, s)
// is that box read through a descriptor whose start address is moved by (r * PW + s) pixels: accumulator row 8 h + w is
// the pixel at box row h + r, box column w + s, i.e. the 8-row swizzle atoms follow the box rows (stride PW * 128 bytes) and
// the column shift s only moves the start address by s rows of 128 bytes: the tensor core applies the 128-byte swizzle to
// the absolute shared-memory address (as the TMA did when it wrote the box), so the descriptor's base-offset field stays 0
// (measured: a non-zero base offset here gives wrong sums, zero gives the right ones).
// Weights: one box per tap and slice through a second ring; when the whole [taps x slices] set of one column tile fits
// (3x3 with 64 channels), it is loaded once per CTA and stays resident.
struct HaloParams {
  int mode;
  int PW, HR;               // halo box: columns (multiple of 8) and rows
  int tiles_w, tiles_h, tiles_i, tiles_n;
  int n_out, k_ch;
  int taps_h, taps_w, dil_h, dil_w;
  int org_h, org_w;         // halo origin relative to the tile origin
  int act;
  const void* bias;
  int bias_fp32, fmt;
  int sa_stages, sb_stages, b_resident;
  int issuers, nacc;        // MMA-issuing warps (1 .. 4) and accumulator buffers in use (a multiple of issuers, <= 512 / BLOCK_N)
  int* status;
};

template <int BLOCK_N>
__global__ void __launch_bounds__(CV_HALO_THREADS, 1)
conv_halo_kernel(const __grid_constant__ CUtensorMap tmap_a,     // activation {C, W, H, N}, box {64, PW, HR, 1}
                 const __grid_constant__ CUtensorMap tmap_b,     // weights {Cin, taps, Cout}, box {64, 1, 64}
                 const __grid_constant__ CUtensorMap tmap_c,     // output {C, W, H, N}, box {64, 8, 16, 1}
                 const HaloParams p) {
  constexpr int B_BYTES = BLOCK_N * 128;
  const int NACC = p.nacc;                  // accumulator buffers in use (a multiple of the number of issuing warps)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int a_bytes = p.HR * p.PW * 128;
  uint8_t* smem_b = smem + p.sa_stages * a_bytes;
  uint8_t* epi_smem = smem_b + p.sb_stages * B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + 2 * 128 * 128);
  const int SA = p.sa_stages, SB = p.sb_stages;
  uint64_t* full_a = bars;
  uint64_t* empty_a = full_a + SA;
  uint64_t* full_b = empty_a + SA;
  uint64_t* empty_b = full_b + SB;
  uint64_t* tmem_full = empty_b + SB;
  uint64_t* tmem_empty = tmem_full + CV_MAX_ACC;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + CV_MAX_ACC);
  volatile int* epi_fail = reinterpret_cast<volatile int*>(tmem_empty + CV_MAX_ACC + 1);
  // byte offset of tap t inside the halo box, tabulated once: the MMA thread's per-tap work is a table read, two ORs and
  // four tcgen05.mma (with index arithmetic in that loop the issuing thread, not the tensor core, set the kernel's speed)
  __shared__ uint32_t tap_off[CV_MAX_TAPS];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = p.tiles_w * p.tiles_h * p.tiles_i;
  const int num_work = m_tiles * p.tiles_n;
  const int taps = p.taps_h * p.taps_w;
  const int kc = (p.k_ch + CV_BLOCK_K - 1) / CV_BLOCK_K;
  for (int t = threadIdx.x; t < taps; t += CV_HALO_THREADS) {
    const int r = t / p.taps_w, s = t - r * p.taps_w;
    const int oh = p.mode == 0 ? r * p.dil_h : (p.taps_h - 1 - r) * p.dil_h;
    const int ow = p.mode == 0 ? s * p.dil_w : (p.taps_w - 1 - s) * p.dil_w;
    tap_off[t] = (uint32_t)(oh * p.PW + ow) * 128u;
  }

  if (threadIdx.x == 0) {
    *epi_fail = 0;
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    prefetch_tmap(&tmap_c);
    for (int i = 0; i < SA; ++i) { mbar_init(&full_a[i], 1); mbar_init(&empty_a[i], 1); }
    for (int i = 0; i < SB; ++i) { mbar_init(&full_b[i], 1); mbar_init(&empty_b[i], 1); }
    for (int i = 0; i < CV_MAX_ACC; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 4); }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // with resident weights every CTA keeps one column tile for its whole life: work items are strided so that nt is fixed
  // (the host launches a grid that is a multiple of tiles_n in that case)

  if (warp == 0) {
    if (lane == 0) {
      int sa = 0, sb = 0;
      uint32_t pa = 0, pb = 0;
      bool ok = true, first = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int nt = w % p.tiles_n, mt = w / p.tiles_n;
        const int w0 = (mt % p.tiles_w) * 8, h0 = ((mt / p.tiles_w) % p.tiles_h) * 16;
        const int i0 = mt / (p.tiles_w * p.tiles_h);
        const int n0 = nt * BLOCK_N;
        for (int c = 0; c < kc && ok; ++c) {
          if (!mbar_wait_bounded(&empty_a[sa], pa ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(&full_a[sa], (uint32_t)a_bytes);
          tma_load_4d(smem + sa * a_bytes, &tmap_a, &full_a[sa], c * CV_BLOCK_K, w0 + p.org_w, h0 + p.org_h, i0);
          if (++sa == SA) { sa = 0; pa ^= 1; }
          if (p.b_resident && !first) continue;
          for (int t = 0; t < taps; ++t) {
            if (!p.b_resident && !mbar_wait_bounded(&empty_b[sb], pb ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
            uint8_t* dst = smem_b + sb * B_BYTES;
            mbar_expect_tx(&full_b[sb], B_BYTES);
#pragma unroll
            for (int i = 0; i < BLOCK_N / 64; ++i) {
              if (p.mode == 0) tma_load_3d(dst + i * 8192, &tmap_b, &full_b[sb], c * CV_BLOCK_K, t, n0 + i * 64);
              else             tma_load_3d(dst + i * 8192, &tmap_b, &full_b[sb], n0 + i * 64, t, c * CV_BLOCK_K);
            }
            if (++sb == SB) { sb = 0; pb ^= 1; }
          }
        }
        first = false;
      }
    }
  } else if ((warp == 1 || warp >= 6) && p.issuers > 1) {
    // Several issuing warps (resident weights only): one thread gets at most one tcgen05.mma into the pipe per ~147 clocks
    // whatever its shape, an N = 64 instruction occupies the tensor core for ~48.  Warp j takes the tiles j, j + NI, ... of this
    // CTA, each into an accumulator buffer of its own.  NACC and the number of A stages are multiples of NI (x slices per tile),
    // so a buffer or a stage always falls to the same warp and that warp sees every phase of its barriers in order.
    const int me = warp == 1 ? 0 : warp - 5;
    const int NI = p.issuers;
    if (lane == 0 && me < NI) {
      const int b_mn = p.mode == 0 ? 0 : 1;
      const uint32_t idesc = make_idesc(p.fmt, 0, b_mn, 128, BLOCK_N);
      const uint32_t lbo_b = b_mn ? 8192u : 16u;
      const uint32_t kstep_b = b_mn ? CV_UMMA_K * 128 : CV_UMMA_K * 2;
      const uint64_t desc_a_hi = make_smem_desc_sw128(0, 16, (uint32_t)p.PW * 128u);
      const uint64_t desc_b_hi = make_smem_desc_sw128(0, lbo_b, 1024);
      const uint32_t kb16 = kstep_b >> 4;
      const uint32_t a_base0 = smem_u32(smem), b_base0 = smem_u32(smem_b);
      bool ok = true, first = true;
      int it = me;
      for (long w = (long)blockIdx.x + (long)me * gridDim.x; w < num_work && ok; w += (long)NI * gridDim.x, it += NI) {
        const int buf = it % NACC;
        const uint32_t acc_phase = (uint32_t)((it / NACC) & 1);
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        uint32_t acc = 0;
        for (int c = 0; c < kc && ok; ++c) {
          const long ga = (long)it * kc + c;             // position of this slice in the producer's sequence of A loads
          const int sa = (int)(ga % SA);
          if (!mbar_wait_bounded(&full_a[sa], (uint32_t)((ga / SA) & 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = a_base0 + (uint32_t)(sa * a_bytes);
#pragma unroll 1
          for (int t = 0; t < taps; ++t) {
            const int sb = c * taps + t;                 // resident weights: one slot per (slice, tap), filled once
            if (first) {
              if (!mbar_wait_bounded(&full_b[sb], 0, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
              tc_fence_after();
            }
            const uint64_t da = desc_a_hi | (uint64_t)((a_base + tap_off[t]) >> 4);
            const uint64_t db = desc_b_hi | (uint64_t)((b_base0 + (uint32_t)(sb * B_BYTES)) >> 4);
            umma_f16(tmem_d, da, db, idesc, acc);
            umma_f16(tmem_d, da + 2, db + kb16, idesc, 1u);
            umma_f16(tmem_d, da + 4, db + 2 * kb16, idesc, 1u);
            umma_f16(tmem_d, da + 6, db + 3 * kb16, idesc, 1u);
            acc = 1u;
          }
          umma_commit(&empty_a[sa]);
        }
        if (ok) umma_commit(&tmem_full[buf]);
        first = false;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const int b_mn = p.mode == 0 ? 0 : 1;
      const uint32_t idesc = make_idesc(p.fmt, 0, b_mn, 128, BLOCK_N);
      const uint32_t lbo_b = b_mn ? 8192u : 16u;
      const uint32_t kstep_b = b_mn ? CV_UMMA_K * 128 : CV_UMMA_K * 2;
      const uint64_t desc_a_hi = make_smem_desc_sw128(0, 16, (uint32_t)p.PW * 128u);
      const uint64_t desc_b_hi = make_smem_desc_sw128(0, lbo_b, 1024);
      const uint32_t kb16 = kstep_b >> 4;
      const uint32_t a_base0 = smem_u32(smem), b_base0 = smem_u32(smem_b);
      const bool resident = p.b_resident != 0;
      int sa = 0, sb = 0;
      uint32_t pa = 0, pb = 0;
      uint32_t a_base = a_base0, b_addr = b_base0;
      int it = 0;
      bool ok = true, first = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
        const int buf = it % NACC;
        const uint32_t acc_phase = (it / NACC) & 1;
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        uint32_t acc = 0;
        const bool wait_b = !(resident && !first);
        for (int c = 0; c < kc && ok; ++c) {
          if (!mbar_wait_bounded(&full_a[sa], pa, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
#pragma unroll 1
          for (int t = 0; t < taps; ++t) {
            if (wait_b) {
              if (!mbar_wait_bounded(&full_b[sb], pb, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
              tc_fence_after();
            }
            const uint64_t da = desc_a_hi | (uint64_t)((a_base + tap_off[t]) >> 4);
            const uint64_t db = desc_b_hi | (uint64_t)(b_addr >> 4);
            umma_f16(tmem_d, da, db, idesc, acc);
            umma_f16(tmem_d, da + 2, db + kb16, idesc, 1u);
            umma_f16(tmem_d, da + 4, db + 2 * kb16, idesc, 1u);
            umma_f16(tmem_d, da + 6, db + 3 * kb16, idesc, 1u);
            acc = 1u;
            if (!resident) umma_commit(&empty_b[sb]);
            b_addr += B_BYTES;
            if (++sb == SB) { sb = 0; pb ^= 1; b_addr = b_base0; }
          }
          umma_commit(&empty_a[sa]);
          a_base += (uint32_t)a_bytes;
          if (++sa == SA) { sa = 0; pa ^= 1; a_base = a_base0; }
        }
        umma_commit(&tmem_full[buf]);
        first = false;
      }
    }
  } else if (warp >= 2 && warp < 6) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int sw = row & 7;
    const bool issuer = (warp == 2 && lane == 0);
    int it = 0, chunk = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
      const int nt = w % p.tiles_n, mt = w / p.tiles_n;
      const int w0 = (mt % p.tiles_w) * 8, h0 = ((mt / p.tiles_w) % p.tiles_h) * 16;
      const int i0 = mt / (p.tiles_w * p.tiles_h);
      const int n0 = nt * BLOCK_N;
      const int buf = it % NACC;
      const uint32_t acc_phase = (it / NACC) & 1;
      if (!mbar_wait_bounded(&tmem_full[buf], acc_phase, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) *epi_fail = 1;
      named_bar_sync(1, 128);
      if (*epi_fail != 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr_row = tmem_base + buf * BLOCK_N + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BLOCK_N; c += 64, ++chunk) {
        if (n0 + c >= p.n_out) break;
        uint8_t* tile = epi_smem + (chunk & 1) * (128 * 128);
        uint8_t* my_row = tile + row * 128;
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          const int col0 = n0 + c + hf * 32;
          uint32_t r[32];
          tmem_ld_32x32(taddr_row + c + hf * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (p.bias != nullptr) {
            if (p.bias_fp32) {
              const float* b = reinterpret_cast<const float*>(p.bias);
#pragma unroll
              for (int j = 0; j < 32; ++j) if (col0 + j < p.n_out) v[j] += __ldg(b + col0 + j);
            } else {
              const uint16_t* b = reinterpret_cast<const uint16_t*>(p.bias);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.n_out) {
                  const uint32_t u = __ldg(b + col0 + j);
                  v[j] += p.fmt == 1 ? __uint_as_float(u << 16) : __half2float(__ushort_as_half((unsigned short)u));
                }
            }
          }
          if (p.act == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 u = make_uint4(cv_pack2(v[8 * j], v[8 * j + 1], p.fmt), cv_pack2(v[8 * j + 2], v[8 * j + 3], p.fmt),
                                       cv_pack2(v[8 * j + 4], v[8 * j + 5], p.fmt), cv_pack2(v[8 * j + 6], v[8 * j + 7], p.fmt));
            *reinterpret_cast<uint4*>(my_row + (((hf * 4 + j) ^ sw) << 4)) = u;
          }
        }
        fence_proxy_async_smem();
        if (issuer) bulk_wait_read<0>();
        named_bar_sync(1, 128);
        if (issuer) {
          tma_store_4d(&tmap_c, tile, n0 + c, w0, h0, i0);
          bulk_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (issuer) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------------ weight gradient
struct WgradParams {
  int BW, BH, BI;           // pixel box of one reduction step (BW * BH * BI == 64)
  int tiles_w, tiles_h, tiles_i;
  int tiles_m, tiles_n;     // Cout / 128, Cin / BLOCK_N
  int c_out, c_in;
  int taps_h, taps_w, dil_h, dil_w, pad_h, pad_w;
  int splits;
  int fmt;
  int* status;
};

template <int BLOCK_N>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_dy,    // {Cout, OW, OH, N}, box {64, BW, BH, BI}
                  const __grid_constant__ CUtensorMap tmap_x,     // {Cin, W, H, N}, box {64, BW, BH, BI}
                  const __grid_constant__ CUtensorMap tmap_dw,    // fp32 {Cin, taps, Cout}, box {32, 1, 32}
                  const WgradParams p) {
  using S = ConvSmem<BLOCK_N>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * S::STAGE_BYTES;       // 4 warps x 2 slabs of 32 rows x 128 bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + S::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int taps = p.taps_h * p.taps_w;
  const int k_total = p.tiles_w * p.tiles_h * p.tiles_i;            // pixel boxes
  const int k_per_split = (k_total + p.splits - 1) / p.splits;
  const int num_work = taps * p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_dy);
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_dw);
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tmem_full[i], 1); mbar_init(&tmem_empty[i], 4); }
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

  // work item -> (split, tap, m tile, n tile); splits of one output tile are neighbours so they run at the same time
  auto decode = [&](int w, int& split, int& t, int& m0, int& n0) {
    split = w % p.splits;
    int r = w / p.splits;
    t = r % taps;
    r /= taps;
    n0 = (r % p.tiles_n) * BLOCK_N;
    m0 = (r / p.tiles_n) * 128;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        int split, t, m0, n0;
        decode(w, split, t, m0, n0);
        const int r = t / p.taps_w, s = t - r * p.taps_w;
        const int dh = r * p.dil_h - p.pad_h, dw = s * p.dil_w - p.pad_w;
        const int k0 = split * k_per_split, k1 = min(k0 + k_per_split, k_total);
        // walk the pixel boxes with counters (a division per load made this thread the bottleneck)
        int w0 = (k0 % p.tiles_w) * p.BW, h0 = ((k0 / p.tiles_w) % p.tiles_h) * p.BH;
        int i0 = (k0 / (p.tiles_w * p.tiles_h)) * p.BI;
        const int w_end = p.tiles_w * p.BW, h_end = p.tiles_h * p.BH;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
#pragma unroll
          for (int i = 0; i < 2; ++i) tma_load_4d(sa + i * 8192, &tmap_dy, &full_bar[stage], m0 + i * 64, w0, h0, i0);
#pragma unroll
          for (int i = 0; i < BLOCK_N / 64; ++i)
            tma_load_4d(sb + i * 8192, &tmap_x, &full_bar[stage], n0 + i * 64, w0 + dw, h0 + dh, i0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          w0 += p.BW;
          if (w0 >= w_end) { w0 = 0; h0 += p.BH; if (h0 >= h_end) { h0 = 0; i0 += p.BI; } }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.fmt, 1, 1, 128, BLOCK_N);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
        int split, t, m0, n0;
        decode(w, split, t, m0, n0);
        const int k0 = split * k_per_split, k1 = min(k0 + k_per_split, k_total);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, 8192, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, 8192, 1024);
#pragma unroll
          for (int k = 0; k < CV_BLOCK_K / CV_UMMA_K; ++k)
            umma_f16(tmem_d, da + ((uint64_t)(k * CV_UMMA_K * 128) >> 4), db + ((uint64_t)(k * CV_UMMA_K * 128) >> 4), idesc,
                     (kb > k0 || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;
    uint8_t* ring = epi_smem + q * (2 * 32 * 128);
    const int sw = lane & 7;
    int it = 0, ring_idx = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++it) {
      int split, t, m0, n0;
      decode(w, split, t, m0, n0);
      const int k0 = split * k_per_split;
      const bool has_k = k0 < min(k0 + k_per_split, k_total);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait_bounded(&tmem_full[buf], acc_phase, p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr_row = tmem_base + buf * BLOCK_N + ((uint32_t)(q * 32) << 16);
      const int r0 = m0 + q * 32;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N; c += 32) {
        if (n0 + c >= p.c_in || r0 >= p.c_out || !has_k) break;      // warp-uniform
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        uint8_t* slab = ring + ring_idx * (32 * 128) + lane * 128;
        uint32_t r[32];
        tmem_ld_32x32(taddr_row + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(slab + ((j ^ sw) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_3d(&tmap_dw, ring + ring_idx * (32 * 128), n0 + c, t, r0);
          bulk_commit();
        }
        ring_idx ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BLOCK_N);
  }
}

// grad[o][i][s] += g_cl[o][s][i] for the fp32 channels-last gradient the kernel above produces
__global__ void __launch_bounds__(256)
conv_wgrad_f32_from_cl_kernel(const float* __restrict__ g_cl, float* __restrict__ grad, int O, int I, int S) {
  const long total = (long)O * I * S;
  for (long g = blockIdx.x * 256L + threadIdx.x; g < total; g += (long)gridDim.x * 256) {
    const int s = (int)(g % S);
    const int i = (int)((g / S) % I);
    const long o = g / ((long)I * S);
    grad[g] += g_cl[(o * S + s) * I + i];
  }
}

}  // namespace dl4j

// =============================================================================== host side
using namespace dl4j;

static int encode_nd(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                     const uint64_t* strides_bytes /* rank-1 */, const uint32_t* box) {
  dl4j_PFN_encodeTiled enc = dl4j_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t d[5];
  cuuint64_t st[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
  CUresult r = enc(map, dt, (cuuint32_t)rank, const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -1000 - (int)r;
}

// Chooses the output-pixel box {bw, bh, bi} with bw * bh * bi <= max_rows (== max_rows when `exact`, with power-of-two
// sides) that wastes the fewest tensor-core rows over an ow x oh x n output.
static void pick_box(int ow, int oh, int n, int max_rows, bool exact, int& bw, int& bh, int& bi) {
  double best = -1.0;
  bw = bh = bi = 1;
  for (int w = 1; w <= max_rows && w <= 256; ++w) {
    if (exact ? (max_rows % w != 0) : (w > ow)) continue;
    for (int h = 1; w * h <= max_rows; ++h) {
      if (exact ? ((max_rows / w) % h != 0) : (h > oh)) continue;
      const int i = exact ? max_rows / (w * h) : std::min(n, max_rows / (w * h));
      if (i < 1 || i > 256 || h > 256) continue;
      if (exact && (w > 2 * ow || h > 2 * oh || i > 2 * n)) continue;
      const double tw = (ow + w - 1) / w, th = (oh + h - 1) / h, ti = (n + i - 1) / i;
      const double eff = ((double)ow * oh * n) / (tw * th * ti * max_rows);
      // prefer wide boxes at equal efficiency (longer contiguous runs per TMA row)
      if (eff > best + 1e-9 || (eff > best - 1e-9 && w > bw)) { best = eff; bw = w; bh = h; bi = i; }
    }
  }
}

static int cv_num_sms() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n > 0 ? n : 148;
}

template <int BN>
static int launch_conv(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const ConvParams& p, int grid,
                       cudaStream_t stream) {
  auto kern = conv_igemm_kernel<BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ConvSmem<BN>::TOTAL);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, CV_THREADS, ConvSmem<BN>::TOTAL, stream>>>(ta, tb, tc, p);
  return (int)cudaGetLastError();
}

template <int BN>
static int launch_wgrad(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const WgradParams& p, int grid,
                        cudaStream_t stream) {
  auto kern = conv_wgrad_kernel<BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ConvSmem<BN>::TOTAL);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, CV_THREADS, ConvSmem<BN>::TOTAL, stream>>>(ta, tb, tc, p);
  return (int)cudaGetLastError();
}


template <int BN>
static int launch_halo(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const HaloParams& p, int grid,
                       int smem_bytes, cudaStream_t stream) {
  auto kern = conv_halo_kernel<BN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  kern<<<grid, CV_HALO_THREADS, smem_bytes, stream>>>(ta, tb, tc, p);
  return (int)cudaGetLastError();
}

static bool conv_halo_auto() {
  static const bool on = [] { const char* e = getenv("DL4J_CONV_HALO_AUTO"); return !(e && e[0] == '0'); }();
  return on;
}

// Halo form of forward / dgrad; returns 1 when the case is left to the per-tap kernel (small images, no room in shared memory).
static int try_conv_halo(int mode, const void* in, const void* w_cl, void* out, const void* bias, int N, int in_c, int in_w, int in_h,
                         int out_c, int out_w, int out_h, int Cin, int Cout, int kH, int kW, int pad_h, int pad_w, int dil_h,
                         int dil_w, int fmt, int bias_fp32, int act, bool force, bool multi_only, cudaStream_t stream) {
  const int PW = (8 + (kW - 1) * dil_w + 7) / 8 * 8, HR = 16 + (kH - 1) * dil_h;
  if (PW > 256 || HR > 256) return 1;
  const int tiles_w = (out_w + 7) / 8, tiles_h = (out_h + 15) / 16;
  const double eff = (double)out_w * out_h / ((double)tiles_w * 8 * tiles_h * 16);
  if (!force && eff < 0.6) return 1;
  const int bn = out_c <= 64 ? 64 : (out_c <= 128 ? 128 : 256);
  const int a_bytes = HR * PW * 128, b_bytes = bn * 128;
  const int taps = kH * kW, kc = (in_c + 63) / 64;
  const int budget = 227 * 1024 - 1024 - 1536 - 2 * 128 * 128;
  HaloParams p;
  memset(&p, 0, sizeof(p));
  const int tiles_n = (out_c + bn - 1) / bn;
  const int sms = cv_num_sms();
  if (taps * kc <= 24 && taps * kc * b_bytes + 2 * a_bytes <= budget && tiles_n <= sms) {
    p.b_resident = 1;
    p.sb_stages = taps * kc;
    p.sa_stages = std::min(4, (budget - p.sb_stages * b_bytes) / a_bytes);
  } else {
    p.b_resident = 0;
    p.sa_stages = 2;
    p.sb_stages = std::min(6, (budget - 2 * a_bytes) / b_bytes);
    if (p.sb_stages < 2) return 1;
    if (p.sb_stages >= 4 && budget - p.sb_stages * b_bytes >= 3 * a_bytes) p.sa_stages = 3;
  }
  p.issuers = 1;
  p.nacc = 512 / bn;
  if (p.b_resident) {
    // several issuing warps: accumulator buffers and A stages in multiples of the warp count (x slices per tile)
    const int sa_max = (budget - p.sb_stages * b_bytes) / a_bytes;
    for (int ni = 4; ni >= 2; --ni) {
      const int unit = ni * kc;
      const int nacc = (512 / bn) / ni * ni;
      const int sa = std::min(sa_max, 2 * unit) / unit * unit;
      if (nacc >= ni && sa >= unit) { p.issuers = ni; p.nacc = nacc; p.sa_stages = sa; break; }
    }
  }
  if (multi_only && p.issuers < 2) return 1;
  const int smem_bytes = p.sa_stages * a_bytes + p.sb_stages * b_bytes + 2 * 128 * 128 + 1024 + 1536;
  if (smem_bytes > 227 * 1024 || (2 * (p.sa_stages + p.sb_stages) + 2 * CV_MAX_ACC + 2) * 8 > 1536) return 1;
  int dev = 0;
  cudaGetDevice(&dev);
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  p.mode = mode; p.PW = PW; p.HR = HR;
  p.tiles_w = tiles_w; p.tiles_h = tiles_h; p.tiles_i = N; p.tiles_n = tiles_n;
  p.n_out = out_c; p.k_ch = in_c;
  p.taps_h = kH; p.taps_w = kW; p.dil_h = dil_h; p.dil_w = dil_w;
  p.org_h = mode == 0 ? -pad_h : pad_h - (kH - 1) * dil_h;
  p.org_w = mode == 0 ? -pad_w : pad_w - (kW - 1) * dil_w;
  p.act = act; p.bias = bias; p.bias_fp32 = bias_fp32; p.fmt = fmt;
  p.status = dl4j_status_word(dev);
  CUtensorMap ta, tb, tc;
  int r;
  {
    uint64_t dims[4] = {(uint64_t)in_c, (uint64_t)in_w, (uint64_t)in_h, (uint64_t)N};
    uint64_t st[3] = {(uint64_t)in_c * 2, (uint64_t)in_c * in_w * 2, (uint64_t)in_c * in_w * in_h * 2};
    uint32_t box[4] = {64, (uint32_t)PW, (uint32_t)HR, 1};
    if ((r = encode_nd(&ta, in, dt, 4, dims, st, box)) != 0) return r;
  }
  {
    uint64_t dims[3] = {(uint64_t)Cin, (uint64_t)kH * kW, (uint64_t)Cout};
    uint64_t st[2] = {(uint64_t)Cin * 2, (uint64_t)Cin * kH * kW * 2};
    uint32_t box[3] = {64, 1, 64};
    if ((r = encode_nd(&tb, w_cl, dt, 3, dims, st, box)) != 0) return r;
  }
  {
    uint64_t dims[4] = {(uint64_t)out_c, (uint64_t)out_w, (uint64_t)out_h, (uint64_t)N};
    uint64_t st[3] = {(uint64_t)out_c * 2, (uint64_t)out_c * out_w * 2, (uint64_t)out_c * out_w * out_h * 2};
    uint32_t box[4] = {64, 8, 16, 1};
    if ((r = encode_nd(&tc, out, dt, 4, dims, st, box)) != 0) return r;
  }
  const long work = (long)tiles_w * tiles_h * N * tiles_n;
  if (work > 0x7fffffffL) return 1;
  int grid = work < sms ? (int)work : sms;
  if (p.b_resident) grid = std::max(tiles_n, grid / tiles_n * tiles_n);   // a CTA keeps its column tile: stride % tiles_n == 0
  if (bn == 64) return launch_halo<64>(ta, tb, tc, p, grid, smem_bytes, stream);
  if (bn == 128) return launch_halo<128>(ta, tb, tc, p, grid, smem_bytes, stream);
  return launch_halo<256>(ta, tb, tc, p, grid, smem_bytes, stream);
}

// Forward (mode 0) and data gradient (mode 1) of a stride-1 convolution.
//   mode 0: in = x [N, H, W, Cin], out = y [N, OH, OW, Cout];  mode 1: in = dy [N, OH, OW, Cout], out = dx [N, H, W, Cin].
//   w_cl: [Cout, kH, kW, Cin] in the activation type.  All tensors dense, 16-byte aligned, channel counts multiples of 8.
//   fuse_w (forward only, pad_w == 0): the kW taps of a filter row and the Cin channels are one contiguous run of
//   kW * Cin <= 64 input elements per output pixel and are loaded as one K slice (used for few-channel stems).
DL4J_API int dl4j_conv2d(int mode, const void* in, const void* w_cl, void* out, const void* bias, int N, int H, int W, int Cin,
                         int OH, int OW, int Cout, int kH, int kW, int pad_h, int pad_w, int dil_h, int dil_w, int fmt,
                         int bias_fp32, int act, int fuse_w, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (N <= 0 || H <= 0 || W <= 0 || OH <= 0 || OW <= 0 || Cin <= 0 || Cout <= 0) return 0;
  if ((Cin & 7) || (Cout & 7) || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(w_cl) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (fmt != 0 && fmt != 1) || kH * kW > CV_MAX_TAPS)
    return -DL4J_ERR_BAD_ARG;
  if ((fuse_w & 1) && (mode != 0 || pad_w != 0 || dil_w != 1 || kW * Cin > 64 || OW + kW - 1 > W)) return -DL4J_ERR_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // geometry of the GEMM: output pixels x n_out, reduction over taps x k_ch
  const int in_c = mode == 0 ? Cin : Cout, in_w = mode == 0 ? W : OW, in_h = mode == 0 ? H : OH;
  const int out_c = mode == 0 ? Cout : Cin, out_w = mode == 0 ? OW : W, out_h = mode == 0 ? OH : H;
  if (!(fuse_w & 1) && (fuse_w & 4)) {
    // halo form on request (flag 4): one input fetch per channel slice instead of one per tap.  It moves a quarter of the
    // bytes of the per-tap kernel but measured 20-40 % slower on the ResNet-50 shapes, so the per-tap kernel is the default.
    const int hr = try_conv_halo(mode, in, w_cl, out, bias, N, in_c, in_w, in_h, out_c, out_w, out_h, Cin, Cout, kH, kW, pad_h,
                                 pad_w, dil_h, dil_w, fmt, bias_fp32, act, true, false, stream);
    if (hr != 1) return hr;
  } else if (!(fuse_w & 1) && conv_halo_auto()) {
    // automatic: only where the halo kernel can keep its weights resident and issue from several warps (few input channels);
    // there it is tensor-bound while the per-tap kernel is bound by its nine-fold input traffic
    const int hr = try_conv_halo(mode, in, w_cl, out, bias, N, in_c, in_w, in_h, out_c, out_w, out_h, Cin, Cout, kH, kW, pad_h,
                                 pad_w, dil_h, dil_w, fmt, bias_fp32, act, false, true, stream);
    if (hr != 1) return hr;
  }
  fuse_w &= 1;
  ConvParams p;
  memset(&p, 0, sizeof(p));
  p.mode = mode;
  pick_box(out_w, out_h, N, 128, false, p.BW, p.BH, p.BI);
  p.tiles_w = (out_w + p.BW - 1) / p.BW; p.tiles_h = (out_h + p.BH - 1) / p.BH; p.tiles_i = (N + p.BI - 1) / p.BI;
  p.n_out = out_c;
  p.k_ch = fuse_w ? kW * Cin : in_c;
  p.taps_h = kH; p.taps_w = fuse_w ? 1 : kW;
  p.dil_h = dil_h; p.dil_w = dil_w; p.pad_h = pad_h; p.pad_w = pad_w;
  p.act = act; p.bias = bias; p.bias_fp32 = bias_fp32; p.fmt = fmt;
  p.status = dl4j_status_word(dev);
  const int bn = out_c <= 64 ? 64 : (out_c <= 128 ? 128 : 256);
  p.tiles_n = (out_c + bn - 1) / bn;
  CUtensorMap ta, tb, tc;
  int r;
  {
    uint64_t dims[4] = {(uint64_t)in_c, (uint64_t)in_w, (uint64_t)in_h, (uint64_t)N};
    uint64_t st[3] = {(uint64_t)in_c * 2, (uint64_t)in_c * in_w * 2, (uint64_t)in_c * in_w * in_h * 2};
    if (fuse_w) { dims[0] = (uint64_t)kW * Cin; dims[1] = (uint64_t)OW; }
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
    if ((r = encode_nd(&ta, in, dt, 4, dims, st, box)) != 0) return r;
  }
  {
    uint64_t dims[3] = {(uint64_t)Cin, (uint64_t)kH * kW, (uint64_t)Cout};
    uint64_t st[2] = {(uint64_t)Cin * 2, (uint64_t)Cin * kH * kW * 2};
    if (fuse_w) { dims[0] = (uint64_t)kW * Cin; dims[1] = (uint64_t)kH; st[0] = (uint64_t)kW * Cin * 2; }
    uint32_t box[3] = {64, 1, 64};
    if ((r = encode_nd(&tb, w_cl, dt, 3, dims, st, box)) != 0) return r;
  }
  {
    uint64_t dims[4] = {(uint64_t)out_c, (uint64_t)out_w, (uint64_t)out_h, (uint64_t)N};
    uint64_t st[3] = {(uint64_t)out_c * 2, (uint64_t)out_c * out_w * 2, (uint64_t)out_c * out_w * out_h * 2};
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
    if ((r = encode_nd(&tc, out, dt, 4, dims, st, box)) != 0) return r;
  }
  const long work = (long)p.tiles_w * p.tiles_h * p.tiles_i * p.tiles_n;
  if (work > 0x7fffffffL) return -DL4J_ERR_BAD_ARG;
  const int sms = cv_num_sms();
  const int grid = work < sms ? (int)work : sms;
  if (bn == 64) return launch_conv<64>(ta, tb, tc, p, grid, stream);
  if (bn == 128) return launch_conv<128>(ta, tb, tc, p, grid, stream);
  return launch_conv<256>(ta, tb, tc, p, grid, stream);
}

// Weight gradient of a stride-1 convolution, added into dw_cl (fp32 [Cout, kH, kW, Cin], the caller zeroes or reuses it).
// fuse_w: as in dl4j_conv2d (pad_w == 0, kW * Cin <= 64): one reduction per filter row over the kW * Cin contiguous inputs.
DL4J_API int dl4j_conv2d_wgrad(const void* dy, const void* x, float* dw_cl, int N, int H, int W, int Cin, int OH, int OW,
                               int Cout, int kH, int kW, int pad_h, int pad_w, int dil_h, int dil_w, int fmt, int fuse_w,
                               void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (N <= 0 || H <= 0 || W <= 0 || OH <= 0 || OW <= 0 || Cin <= 0 || Cout <= 0) return 0;
  if ((Cin & 7) || (Cout & 7) || (reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) ||
      (reinterpret_cast<uintptr_t>(dw_cl) & 15) || (fmt != 0 && fmt != 1) || kH * kW > CV_MAX_TAPS)
    return -DL4J_ERR_BAD_ARG;
  if (fuse_w && (pad_w != 0 || dil_w != 1 || kW * Cin > 64 || OW + kW - 1 > W)) return -DL4J_ERR_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const CUtensorMapDataType dt = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const int n_ch = fuse_w ? kW * Cin : Cin;          // channels of the B operand / columns of one gradient row
  const int taps_w = fuse_w ? 1 : kW;
  WgradParams p;
  memset(&p, 0, sizeof(p));
  pick_box(OW, OH, N, 64, true, p.BW, p.BH, p.BI);
  p.tiles_w = (OW + p.BW - 1) / p.BW; p.tiles_h = (OH + p.BH - 1) / p.BH; p.tiles_i = (N + p.BI - 1) / p.BI;
  p.c_out = Cout; p.c_in = n_ch;
  p.taps_h = kH; p.taps_w = taps_w; p.dil_h = dil_h; p.dil_w = dil_w; p.pad_h = pad_h; p.pad_w = pad_w;
  p.fmt = fmt;
  p.status = dl4j_status_word(dev);
  const int bn = n_ch <= 64 ? 64 : (n_ch <= 128 ? 128 : 256);
  p.tiles_m = (Cout + 127) / 128;
  p.tiles_n = (n_ch + bn - 1) / bn;
  const int sms = cv_num_sms();
  const long k_total = (long)p.tiles_w * p.tiles_h * p.tiles_i;
  const long tiles = (long)kH * taps_w * p.tiles_m * p.tiles_n;
  long splits = tiles >= 2L * sms ? 1 : (2L * sms + tiles - 1) / tiles;
  if (splits > k_total) splits = k_total;
  if (splits > 256) splits = 256;
  if (splits < 1) splits = 1;
  {  // no empty splits: the last split must own at least one box
    const long per = (k_total + splits - 1) / splits;
    splits = (k_total + per - 1) / per;
  }
  p.splits = (int)splits;
  CUtensorMap ta, tb, tc;
  int r;
  {
    uint64_t dims[4] = {(uint64_t)Cout, (uint64_t)OW, (uint64_t)OH, (uint64_t)N};
    uint64_t st[3] = {(uint64_t)Cout * 2, (uint64_t)Cout * OW * 2, (uint64_t)Cout * OW * OH * 2};
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
    if ((r = encode_nd(&ta, dy, dt, 4, dims, st, box)) != 0) return r;
  }
  {
    uint64_t dims[4] = {(uint64_t)n_ch, (uint64_t)(fuse_w ? OW : W), (uint64_t)H, (uint64_t)N};
    uint64_t st[3] = {(uint64_t)Cin * 2, (uint64_t)Cin * W * 2, (uint64_t)Cin * W * H * 2};
    uint32_t box[4] = {64, (uint32_t)p.BW, (uint32_t)p.BH, (uint32_t)p.BI};
    if ((r = encode_nd(&tb, x, dt, 4, dims, st, box)) != 0) return r;
  }
  {
    uint64_t dims[3] = {(uint64_t)n_ch, (uint64_t)kH * taps_w, (uint64_t)Cout};
    uint64_t st[2] = {(uint64_t)n_ch * 4, (uint64_t)Cin * kH * kW * 4};
    uint32_t box[3] = {32, 1, 32};
    if ((r = encode_nd(&tc, dw_cl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, dims, st, box)) != 0) return r;
  }
  const long work = tiles * splits;
  if (work > 0x7fffffffL) return -DL4J_ERR_BAD_ARG;
  const int grid = work < sms ? (int)work : sms;
  if (bn == 64) return launch_wgrad<64>(ta, tb, tc, p, grid, stream);
  if (bn == 128) return launch_wgrad<128>(ta, tb, tc, p, grid, stream);
  return launch_wgrad<256>(ta, tb, tc, p, grid, stream);
}

// grad[O, I, kH*kW] += dw_cl[O, kH*kW, I] (both fp32): folds the channels-last gradient into the parameter's own layout.
DL4J_API int dl4j_conv_wgrad_f32_from_cl(const float* g_cl, float* grad, int O, int I, int S, void* stream) {
  const long total = (long)O * I * S;
  if (total <= 0) return -DL4J_ERR_BAD_ARG;
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  conv_wgrad_f32_from_cl_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(g_cl, grad, O, I, S);
  return (int)cudaGetLastError();
}
