// Memory-bound fused NN kernels: layer norm (fwd/bwd), softmax + cross-entropy (fwd with gradient
// emission), LSTM cell (fwd/bwd), bias/activation backward with bias-gradient reduction.
//
// Reference counterparts: layer_norm = standardize + broadcast mul + addBias
// (libnd4j/include/ops/declarable/generic/nn/layer_norm.cpp:35-78); softMaxCuda / softmax_cross_entropy
// (helpers/cuda/activations.cu:303-353, generic/loss/softmaxCrossEntropy*.cpp); lstmCell as NDArray
// algebra (helpers/cuda/lstm.cu:45-110) and DL4J's LSTMHelpers.java:180-330 gate order [a, f, o, g].
// Each op reads its operands once from HBM and writes once.
#include "common.cuh"

namespace dl4j {

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};

// Eight elements as raw 16-byte words (one for 16-bit types, two for float): lets a kernel issue the loads of several rows
// before converting any of them.
template <typename T> struct Raw8 { uint4 q[sizeof(T) / 2]; };
template <typename T> __device__ __forceinline__ Raw8<T> ld_raw8(const T* p) {
  Raw8<T> r;
#pragma unroll
  for (int i = 0; i < (int)(sizeof(T) / 2); ++i) r.q[i] = __ldcs(reinterpret_cast<const uint4*>(p) + i);
  return r;
}
template <typename T> __device__ __forceinline__ void unpack8(const Raw8<T>& r, float (&v)[8]) {
  Vec8<T>::load(reinterpret_cast<const T*>(&r), v);
}

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ldf<__half>(const __half* p) { return __half2float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }
template <> __device__ __forceinline__ void stf<__half>(__half* p, float v) { *p = __float2half(v); }

// ----------------------------------------------------------------------------- layer norm
// One warp per row; C % 8 == 0 and C <= 32 * 8 * LN_MAXV.  Optional residual input: x = x + res is
// normalised and (when sum_out != null) the sum is also written out for the next residual branch.
constexpr int LN_MAXV = 4;
constexpr int LN_WARPS = 8;

template <typename T, int NV>
__global__ void __launch_bounds__(LN_WARPS * 32)
layer_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ gain,
                      const float* __restrict__ bias, T* __restrict__ y, T* __restrict__ sum_out,
                      float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int C, float eps) {
  // One warp per row, rows strided over a fixed grid; the raw 16-byte loads of the next row are issued before the current row's
  // reductions so that every warp always has a row in flight.
  const int lane = threadIdx.x & 31;
  const int nvec = C / 8;
  const int stride = gridDim.x * LN_WARPS;
  int row = blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  Raw8<T> qx[NV], qr[NV];
  auto fetch = [&](int r) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec && DL4J_IN_BOUNDS((long long)r * C + vi * 8 + 7, (long long)rows * C)) {
        qx[i] = ld_raw8(x + (long long)r * C + vi * 8);
        if (res) qr[i] = ld_raw8(res + (long long)r * C + vi * 8);
      }
    }
  };
  if (row < rows) fetch(row);
  for (; row < rows; row += stride) {
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        unpack8(qx[i], v[i]);
        if (res) {
          float r[8];
          unpack8(qr[i], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
          if (sum_out) Vec8<T>::store(sum_out + (long long)row * C + vi * 8, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      }
    }
    if (row + stride < rows) fetch(row + stride);
    const float mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + i * 32 < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; q += d * d; }
      }
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float g[8], bb[8], o[8];
        Vec8<float>::load(gain + vi * 8, g);
        if (bias) Vec8<float>::load(bias + vi * 8, bb);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[j] + (bias ? bb[j] : 0.f);
        Vec8<T>::store(y + (long long)row * C + vi * 8, o);
      }
    }
  }
}

// The same forward pass with the rows brought in by the copy engine: each warp owns a ring of LN_STAGES row buffers in shared
// memory and one lane keeps LN_STAGES untiled bulk copies (cp.async.bulk, one whole row each, completion counted on an mbarrier
// per buffer) in flight, so the bytes outstanding per SM are set by the ring depth instead of by registers and occupancy.  The
// register-prefetch kernel above holds one row per warp in flight at two blocks per SM (98 registers) and reads at about a
// quarter of the copy bandwidth; here every warp has LN_STAGES rows on the way whatever the occupancy (two blocks per SM).
// Needs 16-byte aligned x / res and C * sizeof(T) a multiple of 16 (C % 8 == 0 gives that).  A wait that runs out (about 2 s)
// stores DL4J_ERR_TIMEOUT_PRODUCER in *status and the warp returns.
constexpr int LN_STAGES = 4;

__device__ __forceinline__ void ln_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <typename T, int NV, bool RES>
__global__ void __launch_bounds__(LN_WARPS * 32, 2)
layer_norm_fwd_bulk_kernel(const T* __restrict__ x, const T* __restrict__ res, const float* __restrict__ gain,
                           const float* __restrict__ bias, T* __restrict__ y, T* __restrict__ sum_out,
                           float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int C, float eps,
                           int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char ln_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = C / 8;
  const uint32_t row_bytes = (uint32_t)C * sizeof(T);
  const int nring = RES ? 2 : 1;
  unsigned char* ring = ln_smem + (size_t)warp * LN_STAGES * nring * row_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ln_smem + (size_t)LN_WARPS * LN_STAGES * nring * row_bytes) + warp * LN_STAGES;
  const long long stride = (long long)gridDim.x * LN_WARPS;
  const long long first = (long long)blockIdx.x * LN_WARPS + warp;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < LN_STAGES; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  auto issue = [&](int s, long long r) {                   // lane 0 only
    mbar_expect_tx(&bars[s], row_bytes * nring);
    ln_bulk_load(ring + (size_t)s * nring * row_bytes, x + r * C, row_bytes, &bars[s]);
    if (RES) ln_bulk_load(ring + ((size_t)s * nring + 1) * row_bytes, res + r * C, row_bytes, &bars[s]);
  };
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < LN_STAGES; ++s)
      if (first + s * stride < rows) issue(s, first + s * stride);
  }
  // This lane's gain / bias columns stay in registers for all its rows: read per row they were four times the bytes of the row
  // itself through the L1 pipe, which then ran at 82 % while DRAM sat at 36 %.
  float g[NV][8], bb[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      Vec8<float>::load(gain + vi * 8, g[i]);
      if (bias) Vec8<float>::load(bias + vi * 8, bb[i]);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) bb[i][j] = 0.f;
      }
    }
  }
  int k = 0;
  for (long long row = first; row < rows; row += stride, ++k) {
    const int s = k % LN_STAGES;
    if (!mbar_wait_bounded(&bars[s], (uint32_t)(k / LN_STAGES) & 1u, status, DL4J_ERR_TIMEOUT_PRODUCER)) return;
    const T* bx = reinterpret_cast<const T*>(ring + (size_t)s * nring * row_bytes);
    float v[NV][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        Vec8<T>::load(bx + vi * 8, v[i]);
        if (RES) {
          float r[8];
          Vec8<T>::load(bx + C + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += v[i][j];
      }
    }
    __syncwarp();                                          // every lane has read the buffer: it can be refilled
    if (lane == 0 && row + LN_STAGES * stride < rows) issue(s, row + LN_STAGES * stride);
    if (RES && sum_out) {
#pragma unroll
      for (int i = 0; i < NV; ++i)
        if (lane + i * 32 < nvec) Vec8<T>::store(sum_out + row * C + (lane + i * 32) * 8, v[i]);
    }
    const float mean = warp_sum(sum) / C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
      if (lane + i * 32 < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; q += d * d; }
      }
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[i][j] - mean) * rstd * g[i][j] + bb[i][j];
        Vec8<T>::store(y + row * C + vi * 8, o);
      }
    }
  }
}

// dx = rstd * (dy*g - mean(dy*g) - xhat * mean(dy*g*xhat));  dgain += dy*xhat;  dbias += dy.
// Each warp walks rows with a grid stride.  The per-column sums for dgain / dbias are kept in shared memory
// (one float per column and sum, lanes hit distinct banks) instead of registers: that keeps the kernel near
// 64 registers, so four blocks fit per SM and enough loads are in flight to follow HBM.  NV = C / 256 rounded up.
template <typename T, int NV>
__global__ void __launch_bounds__(LN_WARPS * 32, 2)
layer_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gain,
                      const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                      float* __restrict__ dgain, float* __restrict__ dbias, int rows, int C) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nvec = C / 8;
  // per-lane column partial sums live in registers for the whole kernel; they meet in shared memory once at the end
  float ag[NV][8], ab[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { ag[i][j] = 0.f; ab[i][j] = 0.f; }
  for (int row = blockIdx.x * LN_WARPS + wid; row < rows; row += gridDim.x * LN_WARPS) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NV][8], dg[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        Vec8<T>::load(dy + (long long)row * C + vi * 8, dg[i]);
        Vec8<T>::load(x + (long long)row * C + vi * 8, xh[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float gn[8];
        Vec8<float>::load(gain + vi * 8, gn);      // L1 resident after the first row
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          const float d = dg[i][j];
          ag[i][j] = fmaf(d, xh[i][j], ag[i][j]);
          ab[i][j] += d;
          dg[i][j] = d * gn[j];
          s1 += dg[i][j];
          s2 = fmaf(dg[i][j], xh[i][j], s2);
        }
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (dg[i][j] - s1 - xh[i][j] * s2);
        Vec8<T>::store(dx + (long long)row * C + vi * 8, o);
      }
    }
  }
  // column c = (vi * 8 + j) lives at acc[..][j * (NV * 32) + vi]: the 32 lanes of a warp (consecutive vi) hit 32 banks
  __shared__ float acc[2][NV * 256];
  for (int w = 0; w < LN_WARPS; ++w) {
    if (wid == w) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + i * 32;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int idx = j * (NV * 32) + vi;
          if (w == 0) { acc[0][idx] = ag[i][j]; acc[1][idx] = ab[i][j]; }
          else { acc[0][idx] += ag[i][j]; acc[1][idx] += ab[i][j]; }
        }
      }
    }
    __syncthreads();
  }
  for (int idx = threadIdx.x; idx < NV * 256; idx += LN_WARPS * 32) {
    const int j = idx / (NV * 32), vi = idx - j * (NV * 32);
    const int col = vi * 8 + j;
    if (col < C) {
      if (dgain) atomicAdd(dgain + col, acc[0][idx]);
      if (dbias) atomicAdd(dbias + col, acc[1][idx]);
    }
  }
}

// Split form of the backward for large row counts: a lean per-row dx kernel (no column accumulators, so many warps stay resident)
// and a column kernel for dgain / dbias that re-reads dy and x (they are L2 resident right after the first kernel when they fit).
template <typename T, int NV>
__global__ void __launch_bounds__(LN_WARPS * 32)
layer_norm_bwd_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gain,
                         const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx, int rows, int C) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nvec = C / 8;
  const int stride = gridDim.x * LN_WARPS;
  int row = blockIdx.x * LN_WARPS + wid;
  Raw8<T> qd[NV], qx[NV];
  float mean_n = 0.f, rstd_n = 0.f;
  auto fetch = [&](int r) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        qd[i] = ld_raw8(dy + (long long)r * C + vi * 8);
        qx[i] = ld_raw8(x + (long long)r * C + vi * 8);
      }
    }
    mean_n = mean_in[r];
    rstd_n = rstd_in[r];
  };
  if (row < rows) fetch(row);
  for (; row < rows; row += stride) {
    const float mean = mean_n, rstd = rstd_n;
    float xh[NV][8], dg[NV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float gn[8];
        unpack8(qd[i], dg[i]);
        unpack8(qx[i], xh[i]);
        Vec8<float>::load(gain + vi * 8, gn);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          dg[i][j] *= gn[j];
          s1 += dg[i][j];
          s2 = fmaf(dg[i][j], xh[i][j], s2);
        }
      }
    }
    if (row + stride < rows) fetch(row + stride);       // next row in flight during the reductions and the stores
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (dg[i][j] - s1 - xh[i][j] * s2);
        Vec8<T>::store(dx + (long long)row * C + vi * 8, o);
      }
    }
  }
}

// dgain[c] += sum_r dy[r, c] * xhat[r, c], dbias[c] += sum_r dy[r, c]; block = 8 column threads (64 columns) x 32 row lanes
template <typename T>
__global__ void __launch_bounds__(256, 3)
layer_norm_bwd_cols_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean_in,
                           const float* __restrict__ rstd_in, float* __restrict__ dgain, float* __restrict__ dbias, int rows, int C,
                           int rows_per_block) {
  // Same shape as the bias-gradient kernel: a warp reads 512 contiguous bytes of one row, 8 warps x 4 rows in flight per thread.
  __shared__ float red[2][8][256 + 8];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + tx * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(r0 + rows_per_block, rows);
  float sg[8], sb[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { sg[j] = 0.f; sb[j] = 0.f; }
  if (col < C) {
    for (int r = r0 + ty; r < r1; r += 32) {
      Raw8<T> qd[4], qx[4];
      float mu[4], rs[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + u * 8;
        if (rr < r1) {
          const long long o = (long long)rr * C + col;
          qd[u] = ld_raw8(dy + o);
          qx[u] = ld_raw8(x + o);
          mu[u] = mean_in[rr];
          rs[u] = rstd_in[rr];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (r + u * 8 < r1) {
          float d[8], xv[8];
          unpack8(qd[u], d);
          unpack8(qx[u], xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            sb[j] += d[j];
            sg[j] = fmaf(d[j], (xv[j] - mu[u]) * rs[u], sg[j]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { red[0][ty][tx * 8 + j] = sg[j]; red[1][ty][tx * 8 + j] = sb[j]; }
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < C) {
    float tg = 0.f, tb = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { tg += red[0][w][threadIdx.x]; tb += red[1][w][threadIdx.x]; }
    if (dgain) atomicAdd(dgain + c, tg);
    if (dbias) atomicAdd(dbias + c, tb);
  }
}

// ----------------------------------------------------------------------------- embedding / row-gather gradient
// grad[idx[r], :] += dy[r, :] accumulated in fp32 with 16-byte vector reductions (the table's master gradient is fp32 while dy
// is the compute type); an index outside [0, V) is skipped and recorded in the status word.
template <typename T>
__global__ void __launch_bounds__(256)
scatter_add_rows_kernel(const T* __restrict__ dy, const long long* __restrict__ idx, float* __restrict__ grad, long long n,
                        int C, long long ld_dy, long long V, int* status) {
  const int c8 = C / 8;
  const long long total = n * c8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / c8;
    const int c = (int)(i % c8) * 8;
    const long long t = idx[r];
    if (t < 0 || t >= V) { if (status) atomicCAS(status, 0, DL4J_ERR_BOUNDS); continue; }
    float v[8];
    Vec8<T>::load(dy + r * ld_dy + c, v);
    float* o = grad + t * (long long)C + c;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]) : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + 4), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
  }
}

// ----------------------------------------------------------------------------- softmax cross entropy
// One block per row.  labels: dense probabilities (same dtype as logits) or int64 class indices.
// loss[r] = -sum_j labels_j * log softmax_j ; grad_out (optional) = softmax * sum(labels) - labels.
constexpr int SX_THREADS = 256;

__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[wid] = v;
  __syncthreads();
  if (wid == 0) {
    float t = lane < SX_THREADS / 32 ? sh[lane] : (is_max ? -INFINITY : 0.f);
    t = is_max ? warp_max(t) : warp_sum(t);
    if (lane == 0) sh[0] = t;
  }
  __syncthreads();
  return sh[0];
}

template <typename T>
__global__ void __launch_bounds__(SX_THREADS)
softmax_xent_kernel(const T* __restrict__ logits, const T* __restrict__ dense_labels, const long long* __restrict__ idx_labels,
                    float* __restrict__ loss, T* __restrict__ grad_out, int C, long long ld, int ignore_index) {
  __shared__ float sh[SX_THREADS / 32];
  const long long row = blockIdx.x;
  const T* z = logits + row * ld;
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < C; j += SX_THREADS) mx = fmaxf(mx, ldf(z + j));
  mx = block_reduce(mx, sh, true);
  float se = 0.f, sl = 0.f, slz = 0.f;
  for (int j = threadIdx.x; j < C; j += SX_THREADS) {
    const float v = ldf(z + j);
    se += __expf(v - mx);
    if (dense_labels) {
      const float l = ldf(dense_labels + row * (long long)C + j);
      sl += l;
      slz += l * v;
    }
  }
  se = block_reduce(se, sh, false);
  const float lse = mx + __logf(se);
  long long tgt = -1;
  if (dense_labels) {
    sl = block_reduce(sl, sh, false);
    slz = block_reduce(slz, sh, false);
  } else {
    tgt = idx_labels[row];
    if (tgt != ignore_index) (void)DL4J_IN_BOUNDS(tgt, C);          // debug build: a label outside [0, C) is recorded, then ignored
    if (tgt == ignore_index || tgt < 0 || tgt >= C) { tgt = -1; sl = 0.f; slz = 0.f; }
    else { sl = 1.f; slz = ldf(z + tgt); }
  }
  if (threadIdx.x == 0) loss[row] = sl * lse - slz;
  if (grad_out) {
    T* g = grad_out + row * ld;
    const float inv = 1.f / se;
    for (int j = threadIdx.x; j < C; j += SX_THREADS) {
      const float pj = __expf(ldf(z + j) - mx) * inv;
      const float l = dense_labels ? ldf(dense_labels + row * (long long)C + j) : (j == tgt ? 1.f : 0.f);
      stf(g + j, pj * sl - l);
    }
  }
}

// Split form used for training: the forward pass makes one online (max, sum) sweep over the row and stores only the loss, the
// log-sum-exp and the label mass; the backward pass writes grad = (softmax * label_mass - labels) * dloss[row] in one sweep, so
// the upstream scale needs no pass of its own.  Rows are read in 16-byte vectors when VEC (row pitch and base allow it).
template <typename T, bool VEC>
__global__ void __launch_bounds__(SX_THREADS)
softmax_xent_fwd_kernel(const T* __restrict__ logits, const T* __restrict__ dense_labels, const long long* __restrict__ idx_labels,
                        float* __restrict__ loss, float* __restrict__ lse_out, float* __restrict__ mass_out, int C, long long ld,
                        int ignore_index) {
  __shared__ float sh[SX_THREADS / 32];
  const long long row = blockIdx.x;
  const T* z = logits + row * ld;
  const T* lab = dense_labels ? dense_labels + row * (long long)C : nullptr;
  float mx = -INFINITY, se = 0.f, sl = 0.f, slz = 0.f;
  auto take = [&](float v, float l) {
    if (v > mx) { se = se * __expf(mx - v) + 1.f; mx = v; } else if (v != -INFINITY) { se += __expf(v - mx); }
    sl += l; slz += l * v;
  };
  if (VEC) {
    const int C8 = C & ~7;
    for (int j = threadIdx.x * 8; j < C8; j += SX_THREADS * 8) {
      float v[8], l[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      Vec8<T>::load(z + j, v);
      if (lab) Vec8<T>::load(lab + j, l);
      float m8 = v[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) m8 = fmaxf(m8, v[i]);
      if (m8 > mx) { se *= __expf(mx - m8); mx = m8; }
#pragma unroll
      for (int i = 0; i < 8; ++i) { se += mx == -INFINITY ? 0.f : __expf(v[i] - mx); sl += l[i]; slz += l[i] * v[i]; }
    }
    for (int j = C8 + threadIdx.x; j < C; j += SX_THREADS) take(ldf(z + j), lab ? ldf(lab + j) : 0.f);
  } else {
    for (int j = threadIdx.x; j < C; j += SX_THREADS) take(ldf(z + j), lab ? ldf(lab + j) : 0.f);
  }
  const float gmx = block_reduce(mx, sh, true);
  se = block_reduce(mx == -INFINITY ? 0.f : se * __expf(mx - gmx), sh, false);
  const float lse = gmx + __logf(se);
  if (lab) {
    sl = block_reduce(sl, sh, false);
    slz = block_reduce(slz, sh, false);
  } else {
    const long long tgt = idx_labels[row];
    if (tgt != ignore_index) (void)DL4J_IN_BOUNDS(tgt, C);
    if (tgt == ignore_index || tgt < 0 || tgt >= C) { sl = 0.f; slz = 0.f; }
    else { sl = 1.f; slz = ldf(z + tgt); }
  }
  if (threadIdx.x == 0) { loss[row] = sl * lse - slz; lse_out[row] = lse; mass_out[row] = sl; }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(SX_THREADS)
softmax_xent_bwd_kernel(const T* __restrict__ logits, const T* __restrict__ dense_labels, const long long* __restrict__ idx_labels,
                        const float* __restrict__ lse, const float* __restrict__ mass, const float* __restrict__ dloss,
                        T* __restrict__ grad, int C, long long ld, long long ld_grad, int ignore_index) {
  const long long row = blockIdx.x;
  const T* z = logits + row * ld;
  const T* lab = dense_labels ? dense_labels + row * (long long)C : nullptr;
  T* g = grad + row * ld_grad;
  const float l0 = lse[row], sl = mass[row], d = dloss[row];
  long long tgt = -1;
  if (!lab) { tgt = idx_labels[row]; if (tgt == ignore_index || tgt < 0 || tgt >= C) tgt = -1; }
  const float a = sl * d;
  if (VEC) {
    const int C8 = C & ~7;
    for (int j = threadIdx.x * 8; j < C8; j += SX_THREADS * 8) {
      float v[8], l[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      Vec8<T>::load(z + j, v);
      if (lab) Vec8<T>::load(lab + j, l);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float li = lab ? l[i] : ((long long)(j + i) == tgt ? 1.f : 0.f);
        v[i] = __expf(v[i] - l0) * a - li * d;
      }
      Vec8<T>::store(g + j, v);
    }
    for (int j = C8 + threadIdx.x; j < C; j += SX_THREADS)
      stf(g + j, __expf(ldf(z + j) - l0) * a - (lab ? ldf(lab + j) : ((long long)j == tgt ? 1.f : 0.f)) * d);
  } else {
    for (int j = threadIdx.x; j < C; j += SX_THREADS)
      stf(g + j, __expf(ldf(z + j) - l0) * a - (lab ? ldf(lab + j) : ((long long)j == tgt ? 1.f : 0.f)) * d);
  }
}

// ----------------------------------------------------------------------------- LSTM cell
// z [mb, 4n] pre-activations in DL4J gate order [a(block input), f, o, g]; c_prev fp32 [mb, n].
// Writes h (T), c (fp32) and the activated gates (T, [mb,4n]) for the backward pass.
template <typename T>
__global__ void lstm_cell_fwd_kernel(const T* __restrict__ z, const float* __restrict__ c_prev, T* __restrict__ h,
                                     float* __restrict__ c, T* __restrict__ gates, int mb, int n) {
  const long long total = (long long)mb * n;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n), j = (int)(i % n);
    const T* zr = z + (long long)r * 4 * n;
    const float a = tanhf(ldf(zr + j));
    const float f = sigmoidf_(ldf(zr + n + j));
    const float o = sigmoidf_(ldf(zr + 2 * n + j));
    const float g = sigmoidf_(ldf(zr + 3 * n + j));
    const float cn = f * c_prev[i] + g * a;
    c[i] = cn;
    stf(h + i, o * tanhf(cn));
    if (gates) {
      T* gr = gates + (long long)r * 4 * n;
      stf(gr + j, a); stf(gr + n + j, f); stf(gr + 2 * n + j, o); stf(gr + 3 * n + j, g);
    }
  }
}

// dh (T), dc_in (fp32, gradient flowing into c from the next step, may be null) -> dz (T), dc_prev (fp32)
template <typename T>
__global__ void lstm_cell_bwd_kernel(const T* __restrict__ dh, const float* __restrict__ dc_in, const T* __restrict__ gates,
                                     const float* __restrict__ c, const float* __restrict__ c_prev, T* __restrict__ dz,
                                     float* __restrict__ dc_prev, int mb, int n) {
  const long long total = (long long)mb * n;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n), j = (int)(i % n);
    const T* gr = gates + (long long)r * 4 * n;
    const float a = ldf(gr + j), f = ldf(gr + n + j), o = ldf(gr + 2 * n + j), g = ldf(gr + 3 * n + j);
    const float tc = tanhf(c[i]);
    const float dhv = dh ? ldf(dh + i) : 0.f;
    const float dc = (dc_in ? dc_in[i] : 0.f) + dhv * o * (1.f - tc * tc);
    T* dr = dz + (long long)r * 4 * n;
    stf(dr + j, dc * g * (1.f - a * a));
    stf(dr + n + j, dc * c_prev[i] * f * (1.f - f));
    stf(dr + 2 * n + j, dhv * tc * o * (1.f - o));
    stf(dr + 3 * n + j, dc * a * g * (1.f - g));
    dc_prev[i] = dc * f;
  }
}

// ----------------------------------------------------------------------------- bias / activation backward
// dz = dy * act'(z) (written only when dz != null) and dbias[c] += sum_r dz[r, c].
// Block = 32 column-pairs x 8 row lanes; grid.x over column tiles of 64, grid.y over row slabs.
__device__ __forceinline__ float act_grad(float z, int act) {
  switch (act) {
    case 1: return z > 0.f ? 1.f : 0.f;
    case 2: {
      const float cdf = 0.5f * (1.f + erff(z * 0.70710678118654752f));
      return cdf + z * 0.3989422804014327f * __expf(-0.5f * z * z);
    }
    case 3: {
      const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * z * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * z * z);
    }
    case 4: { const float s = sigmoidf_(z); return s * (1.f - s); }
    case 5: { const float t = tanhf(z); return 1.f - t * t; }
    case 6: { const float s = sigmoidf_(1.702f * z); return s + 1.702f * z * s * (1.f - s); }
    default: return 1.f;
  }
}
__device__ __forceinline__ float tanh_approx(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
// d[j] *= act'(z[j]) for eight values with the activation dispatched once; the GELU forms use one tanh.approx per value
// (sigmoid(y) = 0.5 + 0.5 tanh(y / 2)), which keeps the kernel bound by memory rather than by the special-function unit.
__device__ __forceinline__ void act_grad8(float (&d)[8], const float (&z)[8], int act) {
  if (act == 6) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = fmaf(0.5f, tanh_approx(0.851f * z[j]), 0.5f);
      d[j] *= fmaf(1.702f * z[j] * s, 1.f - s, s);
    }
  } else if (act == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] = z[j] > 0.f ? d[j] : 0.f;
  } else if (act == 3) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float z2 = z[j] * z[j];
      const float t = tanh_approx(0.7978845608028654f * z[j] * fmaf(0.044715f, z2, 1.f));
      d[j] *= fmaf(0.5f, t, 0.5f) + 0.5f * z[j] * (1.f - t * t) * 0.7978845608028654f * fmaf(0.134145f, z2, 1.f);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] *= act_grad(z[j], act);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
bias_act_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ z, T* __restrict__ dz, float* __restrict__ dbias,
                    int rows, int C, int act, int rows_per_block) {
  __shared__ float red[8][65];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + tx * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(r0 + rows_per_block, rows);
  float s0 = 0.f, s1 = 0.f;
  if (col < C) {
    const bool pair = col + 1 < C;
    for (int r = r0 + ty; r < r1; r += 8) {
      const long long o = (long long)r * C + col;
      float d0 = ldf(dy + o), d1 = pair ? ldf(dy + o + 1) : 0.f;
      if (act != 0) {
        d0 *= act_grad(ldf(z + o), act);
        if (pair) d1 *= act_grad(ldf(z + o + 1), act);
      }
      if (dz) { stf(dz + o, d0); if (pair) stf(dz + o + 1, d1); }
      s0 += d0; s1 += d1;
    }
  }
  red[ty][tx * 2] = s0; red[ty][tx * 2 + 1] = s1;
  __syncthreads();
  if (dbias && threadIdx.x < 64) {
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < C) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
      atomicAdd(dbias + c, t);
    }
  }
}

// Vector form for C % 8 == 0: a thread owns 8 adjacent columns (one 16-byte load per row), eight threads span a 64-column
// tile (128 contiguous bytes per row) and the block's 32 row lanes walk a row slab with two independent row loads in
// flight per thread; many small blocks keep enough warps resident to hide the load latency; one atomicAdd per column and block.
template <typename T>
__global__ void __launch_bounds__(256, 3)
bias_act_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ z, T* __restrict__ dz, float* __restrict__ dbias,
                        int rows, int C, int act, int rows_per_block) {
  // A warp reads 512 contiguous bytes of one row (32 lanes x 8 elements); the block's 8 warps take 8 rows at a time and every
  // thread keeps 4 rows in flight (raw 16-byte loads, converted after all of them are issued).
  __shared__ float red[8][256 + 8];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + tx * 8;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(r0 + rows_per_block, rows);
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  if (col < C) {
    for (int r = r0 + ty; r < r1; r += 32) {
      Raw8<T> qd[4], qz[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + u * 8;
        if (rr < r1) {
          const long long o = (long long)rr * C + col;
          qd[u] = ld_raw8(dy + o);
          if (act != 0) qz[u] = ld_raw8(z + o);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + u * 8;
        if (rr < r1) {
          float d[8];
          unpack8(qd[u], d);
          if (act != 0) {
            float zz[8];
            unpack8(qz[u], zz);
            act_grad8(d, zz, act);
          }
          if (dz) Vec8<T>::store(dz + (long long)rr * C + col, d);
#pragma unroll
          for (int j = 0; j < 8; ++j) s[j] += d[j];
        }
      }
    }
  }
  if (!dbias) return;
#pragma unroll
  for (int j = 0; j < 8; ++j) red[ty][tx * 8 + j] = s[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < C) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    atomicAdd(dbias + c, t);
  }
}

// ----------------------------------------------------------------------------- attention softmax
// In-place row softmax over scores S [rows, Tk] (already scaled by the GEMM epilogue) with an optional
// key mask [B, Tk] (non-zero = keep); row r belongs to example r / rows_per_example.  One warp per row.
template <typename T>
__global__ void __launch_bounds__(LN_WARPS * 32)
attn_softmax_fwd_kernel(T* __restrict__ S, const float* __restrict__ key_mask, long long rows, int Tk, int rows_per_example) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = Tk / 8;
  T* sr = S + row * Tk;
  const float* mk = key_mask ? key_mask + (row / rows_per_example) * Tk : nullptr;
  float v[LN_MAXV][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      Vec8<T>::load(sr + vi * 8, v[i]);
      if (mk) {
        float m[8];
        Vec8<float>::load(mk + vi * 8, m);
#pragma unroll
        for (int j = 0; j < 8; ++j) if (m[j] == 0.f) v[i][j] = -INFINITY;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[i][j]);
    }
  }
  mx = warp_max(mx);
  if (mx == -INFINITY) mx = 0.f;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i)
    if (lane + i * 32 < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { v[i][j] = __expf(v[i][j] - mx); s += v[i][j]; }
    }
  s = warp_sum(s);
  const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= inv;
      Vec8<T>::store(sr + vi * 8, v[i]);
    }
  }
}

// dS = scale * P * (dP - sum_j dP_j P_j), written over dP.
template <typename T>
__global__ void __launch_bounds__(LN_WARPS * 32)
attn_softmax_bwd_kernel(const T* __restrict__ P, T* __restrict__ dP, long long rows, int Tk, float scale) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nvec = Tk / 8;
  float p[LN_MAXV][8], d[LN_MAXV][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
      Vec8<T>::load(P + row * Tk + vi * 8, p[i]);
      Vec8<T>::load(dP + row * Tk + vi * 8, d[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += p[i][j] * d[i][j];
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < LN_MAXV; ++i) {
    const int vi = lane + i * 32;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) d[i][j] = scale * p[i][j] * (d[i][j] - dot);
      Vec8<T>::store(dP + row * Tk + vi * 8, d[i]);
    }
  }
}

}  // namespace dl4j

using namespace dl4j;

// DL4J_LN_BULK=0 keeps the register-prefetch forward kernel.
static bool ln_bulk_enabled() {
  static const bool on = [] { const char* e = getenv("DL4J_LN_BULK"); return !(e && e[0] == '0'); }();
  return on;
}

// dtype: 0 = fp16, 1 = bf16, 2 = fp32
#define DL4J_DISPATCH_T(dtype, ...)                                     \
  if (dtype == 1) { using T = __nv_bfloat16; __VA_ARGS__; }            \
  else if (dtype == 0) { using T = __half; __VA_ARGS__; }              \
  else { using T = float; __VA_ARGS__; }

DL4J_API int dl4j_layer_norm_fwd(const void* x, const void* res, const float* gain, const float* bias, void* y,
                                 void* sum_out, float* mean, float* rstd, int rows, int C, float eps, int dtype, void* stream) {
  if (C % 8 != 0 || C > 32 * 8 * LN_MAXV) return -DL4J_ERR_BAD_ARG;
  int grid = (rows + LN_WARPS - 1) / LN_WARPS;
  const int cap_f = 148 * dl4j_launch_grid("LAYER_NORM_FWD", 4);
  if (grid > cap_f) grid = cap_f;
  const int nvf = (C + 255) / 256;
  const size_t esz = dtype == 2 ? 4 : 2;
  const bool aligned = (((uintptr_t)x | (uintptr_t)(res ? res : x)) & 15) == 0 && ((size_t)C * esz) % 16 == 0;
  if (aligned && ln_bulk_enabled() && rows >= 1024) {
    const int nring = res ? 2 : 1;
    const size_t smem = (size_t)LN_WARPS * LN_STAGES * nring * C * esz + (size_t)LN_WARPS * LN_STAGES * sizeof(uint64_t);
    if (smem <= 100 * 1024) {
      int gb = (rows + LN_WARPS - 1) / LN_WARPS;
      const int cap_b = 148 * dl4j_launch_grid("LAYER_NORM_FWD_BULK", 2);
      if (gb > cap_b) gb = cap_b;
      int dev = 0;
      cudaGetDevice(&dev);
      int* status = dl4j_status_word(dev);
#define DL4J_LN_BULK(NVV, RESV)                                                                                        \
  DL4J_DISPATCH_T(dtype, {                                                                                            \
    auto kern = layer_norm_fwd_bulk_kernel<T, NVV, RESV>;                                                             \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                               \
    kern<<<gb, LN_WARPS * 32, smem, (cudaStream_t)stream>>>((const T*)x, (const T*)res, gain, bias, (T*)y,            \
                                                           (T*)sum_out, mean, rstd, rows, C, eps, status);            \
  })
#define DL4J_LN_BULK_NV(RESV)                    \
  if (nvf == 1) { DL4J_LN_BULK(1, RESV); }       \
  else if (nvf == 2) { DL4J_LN_BULK(2, RESV); }  \
  else if (nvf == 3) { DL4J_LN_BULK(3, RESV); }  \
  else { DL4J_LN_BULK(4, RESV); }
      if (res) { DL4J_LN_BULK_NV(true); } else { DL4J_LN_BULK_NV(false); }
#undef DL4J_LN_BULK_NV
#undef DL4J_LN_BULK
      return (int)cudaGetLastError();
    }
  }
#define DL4J_LN_FWD(NVV)                                                                                     \
  DL4J_DISPATCH_T(dtype, (layer_norm_fwd_kernel<T, NVV><<<grid, LN_WARPS * 32, 0, (cudaStream_t)stream>>>(   \
      (const T*)x, (const T*)res, gain, bias, (T*)y, (T*)sum_out, mean, rstd, rows, C, eps)))
  if (nvf == 1) { DL4J_LN_FWD(1); }
  else if (nvf == 2) { DL4J_LN_FWD(2); }
  else if (nvf == 3) { DL4J_LN_FWD(3); }
  else { DL4J_LN_FWD(4); }
#undef DL4J_LN_FWD
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_layer_norm_bwd(const void* dy, const void* x, const float* gain, const float* mean, const float* rstd,
                                 void* dx, float* dgain, float* dbias, int rows, int C, int dtype, void* stream) {
  if (C % 8 != 0 || C > 32 * 8 * LN_MAXV) return -DL4J_ERR_BAD_ARG;
  const int nv = (C + 255) / 256;
  if (rows >= 2048) {
    int g1 = (rows + LN_WARPS - 1) / LN_WARPS;
    const int cap_dx = 148 * dl4j_launch_grid("LAYER_NORM_BWD_DX", 4);
    if (g1 > cap_dx) g1 = cap_dx;
#define DL4J_LN_DX(NVV)                                                                                           \
  DL4J_DISPATCH_T(dtype, (layer_norm_bwd_dx_kernel<T, NVV><<<g1, LN_WARPS * 32, 0, (cudaStream_t)stream>>>(       \
      (const T*)dy, (const T*)x, gain, mean, rstd, (T*)dx, rows, C)))
    if (nv == 1) { DL4J_LN_DX(1); }
    else if (nv == 2) { DL4J_LN_DX(2); }
    else if (nv == 3) { DL4J_LN_DX(3); }
    else { DL4J_LN_DX(4); }
#undef DL4J_LN_DX
    if (dgain || dbias) {
      const int ct = (C + 255) / 256;
      int slabs = (148 * dl4j_launch_grid("LAYER_NORM_BWD_COLS", 6) + ct - 1) / ct;
      if (slabs < 1) slabs = 1;
      int rpb = (rows + slabs - 1) / slabs;
      rpb = (rpb + 31) / 32 * 32;
      slabs = (rows + rpb - 1) / rpb;
      dim3 g2(ct, slabs);
      DL4J_DISPATCH_T(dtype, (layer_norm_bwd_cols_kernel<T><<<g2, 256, 0, (cudaStream_t)stream>>>(
          (const T*)dy, (const T*)x, mean, rstd, dgain, dbias, rows, C, rpb)));
    }
    return (int)cudaGetLastError();
  }
  int grid = (rows + LN_WARPS - 1) / LN_WARPS;
  if (grid > 148 * 2) grid = 148 * 2;
#define DL4J_LN_BWD(NVV)                                                                                       \
  DL4J_DISPATCH_T(dtype, (layer_norm_bwd_kernel<T, NVV><<<grid, LN_WARPS * 32, 0, (cudaStream_t)stream>>>(     \
      (const T*)dy, (const T*)x, gain, mean, rstd, (T*)dx, dgain, dbias, rows, C)))
  if (nv == 1) { DL4J_LN_BWD(1); }
  else if (nv == 2) { DL4J_LN_BWD(2); }
  else if (nv == 3) { DL4J_LN_BWD(3); }
  else { DL4J_LN_BWD(4); }
#undef DL4J_LN_BWD
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_softmax_xent(const void* logits, const void* dense_labels, const long long* idx_labels, float* loss,
                               void* grad_out, int rows, int C, long long ld, int ignore_index, int dtype, void* stream) {
  if (rows <= 0) return 0;
  DL4J_DISPATCH_T(dtype, (softmax_xent_kernel<T><<<rows, SX_THREADS, 0, (cudaStream_t)stream>>>(
      (const T*)logits, (const T*)dense_labels, idx_labels, loss, (T*)grad_out, C, ld, ignore_index)));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_scatter_add_rows(const void* dy, const long long* idx, float* grad, long long n, int C, long long ld_dy,
                                   long long V, int dtype, void* stream) {
  if (n <= 0 || C <= 0) return 0;
  if (!dy || !idx || !grad || C % 8 != 0 || ((uintptr_t)dy % 16) || ((uintptr_t)grad % 16) || (ld_dy % 8)) return -DL4J_ERR_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  const long long total = n * (C / 8);
  long long blocks = (total + 255) / 256;
  const long long cap_s = 148LL * dl4j_launch_grid("SCATTER_ADD_ROWS", 16);
  if (blocks > cap_s) blocks = cap_s;
  DL4J_DISPATCH_T(dtype, (scatter_add_rows_kernel<T><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const T*)dy, idx, grad, n, C, ld_dy, V, dl4j_status_word(dev))));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_softmax_xent_fwd(const void* logits, const void* dense_labels, const long long* idx_labels, float* loss,
                                   float* lse, float* mass, int rows, int C, long long ld, int ignore_index, int dtype,
                                   void* stream) {
  if (rows <= 0) return 0;
  if (!logits || !loss || !lse || !mass || (!dense_labels && !idx_labels)) return -DL4J_ERR_BAD_ARG;
  const int esz = dtype == 2 ? 4 : 2;
  const bool vec = ((uintptr_t)logits % 16 == 0) && ((ld * esz) % 16 == 0) &&
                   (!dense_labels || (((uintptr_t)dense_labels % 16 == 0) && (((long long)C * esz) % 16 == 0)));
  if (vec) {
    DL4J_DISPATCH_T(dtype, (softmax_xent_fwd_kernel<T, true><<<rows, SX_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)logits, (const T*)dense_labels, idx_labels, loss, lse, mass, C, ld, ignore_index)));
  } else {
    DL4J_DISPATCH_T(dtype, (softmax_xent_fwd_kernel<T, false><<<rows, SX_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)logits, (const T*)dense_labels, idx_labels, loss, lse, mass, C, ld, ignore_index)));
  }
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_softmax_xent_bwd(const void* logits, const void* dense_labels, const long long* idx_labels, const float* lse,
                                   const float* mass, const float* dloss, void* grad, int rows, int C, long long ld,
                                   long long ld_grad, int ignore_index, int dtype, void* stream) {
  if (rows <= 0) return 0;
  if (!logits || !lse || !mass || !dloss || !grad || (!dense_labels && !idx_labels)) return -DL4J_ERR_BAD_ARG;
  const int esz = dtype == 2 ? 4 : 2;
  const bool vec = ((uintptr_t)logits % 16 == 0) && ((ld * esz) % 16 == 0) && ((uintptr_t)grad % 16 == 0) &&
                   ((ld_grad * esz) % 16 == 0) &&
                   (!dense_labels || (((uintptr_t)dense_labels % 16 == 0) && (((long long)C * esz) % 16 == 0)));
  if (vec) {
    DL4J_DISPATCH_T(dtype, (softmax_xent_bwd_kernel<T, true><<<rows, SX_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)logits, (const T*)dense_labels, idx_labels, lse, mass, dloss, (T*)grad, C, ld, ld_grad, ignore_index)));
  } else {
    DL4J_DISPATCH_T(dtype, (softmax_xent_bwd_kernel<T, false><<<rows, SX_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)logits, (const T*)dense_labels, idx_labels, lse, mass, dloss, (T*)grad, C, ld, ld_grad, ignore_index)));
  }
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_lstm_cell_fwd(const void* z, const float* c_prev, void* h, float* c, void* gates, int mb, int n,
                                int dtype, void* stream) {
  long long total = (long long)mb * n;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  DL4J_DISPATCH_T(dtype, (lstm_cell_fwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const T*)z, c_prev, (T*)h, c, (T*)gates, mb, n)));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_lstm_cell_bwd(const void* dh, const float* dc_in, const void* gates, const float* c, const float* c_prev,
                                void* dz, float* dc_prev, int mb, int n, int dtype, void* stream) {
  long long total = (long long)mb * n;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 8) grid = 148 * 8;
  DL4J_DISPATCH_T(dtype, (lstm_cell_bwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const T*)dh, dc_in, (const T*)gates, c, c_prev, (T*)dz, dc_prev, mb, n)));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_bias_act_bwd(const void* dy, const void* z, void* dz, float* dbias, int rows, int C, int act, int dtype,
                               void* stream) {
  if (rows <= 0 || C <= 0) return 0;
  if (dy == nullptr || (act != 0 && z == nullptr)) return -DL4J_ERR_BAD_ARG;
  if (C % 8 == 0) {
    const int ct = (C + 255) / 256;
    int slabs = (148 * dl4j_launch_grid("BIAS_ACT_BWD", 6) + ct - 1) / ct;      // default: about two rounds of resident blocks (3 per SM)
    if (slabs < 1) slabs = 1;
    int rpb = (rows + slabs - 1) / slabs;
    rpb = (rpb + 31) / 32 * 32;
    slabs = (rows + rpb - 1) / rpb;
    dim3 grid(ct, slabs);
    DL4J_DISPATCH_T(dtype, (bias_act_bwd_vec_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const T*)dy, (const T*)z, (T*)dz, dbias, rows, C, act, rpb)));
    return (int)cudaGetLastError();
  }
  const int col_tiles = (C + 63) / 64;
  int row_slabs = (148 * 4 + col_tiles - 1) / col_tiles;
  if (row_slabs < 1) row_slabs = 1;
  int rpb = (rows + row_slabs - 1) / row_slabs;
  rpb = (rpb + 7) / 8 * 8;
  row_slabs = (rows + rpb - 1) / rpb;
  dim3 grid(col_tiles, row_slabs);
  DL4J_DISPATCH_T(dtype, (bias_act_bwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const T*)dy, (const T*)z, (T*)dz, dbias, rows, C, act, rpb)));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_attn_softmax_fwd(void* S, const float* key_mask, long long rows, int Tk, int rows_per_example, int dtype,
                                   void* stream) {
  if (rows <= 0) return 0;
  if (Tk % 8 != 0 || Tk > 32 * 8 * LN_MAXV) return -DL4J_ERR_BAD_ARG;
  const long long grid = (rows + LN_WARPS - 1) / LN_WARPS;
  DL4J_DISPATCH_T(dtype, (attn_softmax_fwd_kernel<T><<<(unsigned)grid, LN_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (T*)S, key_mask, rows, Tk, rows_per_example)));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_attn_softmax_bwd(const void* P, void* dP, long long rows, int Tk, float scale, int dtype, void* stream) {
  if (rows <= 0) return 0;
  if (Tk % 8 != 0 || Tk > 32 * 8 * LN_MAXV) return -DL4J_ERR_BAD_ARG;
  const long long grid = (rows + LN_WARPS - 1) / LN_WARPS;
  DL4J_DISPATCH_T(dtype, (attn_softmax_bwd_kernel<T><<<(unsigned)grid, LN_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (const T*)P, (T*)dP, rows, Tk, scale)));
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ 16-bit matrix transpose
// out[c, r] = in[r, c] for a row-major [rows, cols] matrix of 2-byte elements (both even).  64 x 64 tiles through shared memory:
// the loads read 128 contiguous bytes per row, the stores write 128 contiguous bytes per output row (the generic strided copy of
// the tensor library reaches about 0.8 TB/s on this shape of problem; the recurrent weights are transposed once per tBPTT segment).
namespace dl4j {

__global__ void __launch_bounds__(256) transpose16_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int rows, int cols) {
  __shared__ uint16_t tile[64][64 + 2];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;        // 32 x 8 threads, two adjacent elements per thread
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + ty + 8 * i, c = c0 + 2 * tx;
    uint32_t v = 0;
    if (r < rows && c < cols) v = *reinterpret_cast<const uint32_t*>(in + (size_t)r * cols + c);
    tile[ty + 8 * i][2 * tx] = (uint16_t)(v & 0xffffu);
    tile[ty + 8 * i][2 * tx + 1] = (uint16_t)(v >> 16);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = c0 + ty + 8 * i, r = r0 + 2 * tx;             // output row c, output columns r, r + 1
    if (c < cols && r < rows) {
      const uint32_t v = (uint32_t)tile[2 * tx][ty + 8 * i] | ((uint32_t)tile[2 * tx + 1][ty + 8 * i] << 16);
      *reinterpret_cast<uint32_t*>(out + (size_t)c * rows + r) = v;
    }
  }
}

}  // namespace dl4j

// in [rows, cols] -> out [cols, rows], both dense row-major 16-bit matrices with even extents and 4-byte aligned bases.
DL4J_API int dl4j_transpose16(const void* in, void* out, int rows, int cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((rows & 1) || (cols & 1) || (reinterpret_cast<uintptr_t>(in) & 3) || (reinterpret_cast<uintptr_t>(out) & 3)) return -DL4J_ERR_BAD_ARG;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  dl4j::transpose16_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const uint16_t*>(in), reinterpret_cast<uint16_t*>(out),
                                                                    rows, cols);
  return (int)cudaGetLastError();
}
