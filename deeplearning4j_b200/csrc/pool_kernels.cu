// Max pooling over channels-last bf16 activations [N, H, W, C] (C % 8 == 0), 8 channels per thread.
// Forward also records, per output element, which window position (kh * kW + kw, first maximum in scan order like
// the reference's argmax) won; backward is then a gather: every input element sums the output gradients of the (few)
// windows that selected it, so no atomics and no 8-byte indices are needed
// (libnd4j pooling2d / ConvolutionUtils::pooling2dBP semantics for MAX pooling).
#include "common.cuh"

namespace dl4j {

constexpr int PL_THREADS = 256;

struct PoolShape {
  int N, H, W, C, OH, OW, kH, kW, sH, sW, pH, pW;
};

__device__ __forceinline__ void pl_unpack8(const uint4& u, float* o) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
__device__ __forceinline__ uint4 pl_pack8(const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

__global__ void __launch_bounds__(PL_THREADS)
maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, unsigned char* __restrict__ idx, const PoolShape s) {
  const int cv_n = s.C >> 3;
  const long long total = (long long)s.N * s.OH * s.OW * cv_n;
  for (long long g = blockIdx.x * (long long)PL_THREADS + threadIdx.x; g < total; g += (long long)gridDim.x * PL_THREADS) {
    const int cv = (int)(g % cv_n);
    long long t = g / cv_n;
    const int ow = (int)(t % s.OW); t /= s.OW;
    const int oh = (int)(t % s.OH);
    const int n = (int)(t / s.OH);
    float best[8];
    unsigned char bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; bi[j] = 0; }
    const int ih0 = oh * s.sH - s.pH, iw0 = ow * s.sW - s.pW;
    for (int kh = 0; kh < s.kH; ++kh) {
      const int ih = ih0 + kh;
      if (ih < 0 || ih >= s.H) continue;
      for (int kw = 0; kw < s.kW; ++kw) {
        const int iw = iw0 + kw;
        if (iw < 0 || iw >= s.W) continue;
        float v[8];
        const long long xo = (((long long)n * s.H + ih) * s.W + iw) * cv_n + cv;      // in 16-byte groups
        if (!DL4J_IN_BOUNDS(xo, (long long)s.N * s.H * s.W * cv_n)) continue;
        pl_unpack8(__ldg(reinterpret_cast<const uint4*>(x) + xo), v);
        const unsigned char pos = (unsigned char)(kh * s.kW + kw);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v[j] > best[j]) { best[j] = v[j]; bi[j] = pos; }
      }
    }
    reinterpret_cast<uint4*>(y)[g] = pl_pack8(best);
    if (idx) {
      uint2 p;
      p.x = bi[0] | (bi[1] << 8) | (bi[2] << 16) | ((unsigned)bi[3] << 24);
      p.y = bi[4] | (bi[5] << 8) | (bi[6] << 16) | ((unsigned)bi[7] << 24);
      reinterpret_cast<uint2*>(idx)[g] = p;
    }
  }
}

__global__ void __launch_bounds__(PL_THREADS)
maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const unsigned char* __restrict__ idx, __nv_bfloat16* __restrict__ dx, const PoolShape s) {
  const int cv_n = s.C >> 3;
  const long long total = (long long)s.N * s.H * s.W * cv_n;
  for (long long g = blockIdx.x * (long long)PL_THREADS + threadIdx.x; g < total; g += (long long)gridDim.x * PL_THREADS) {
    const int cv = (int)(g % cv_n);
    long long t = g / cv_n;
    const int iw = (int)(t % s.W); t /= s.W;
    const int ih = (int)(t % s.H);
    const int n = (int)(t / s.H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // windows (oh, ow) that contain (ih, iw): oh * sH - pH <= ih < oh * sH - pH + kH
    const int hp = ih + s.pH, wp = iw + s.pW;
    const int oh_hi = min(hp / s.sH, s.OH - 1);
    const int oh_lo = max(hp - s.kH + s.sH, 0) / s.sH;        // ceil((hp - kH + 1) / sH) clamped at 0
    const int ow_hi = min(wp / s.sW, s.OW - 1);
    const int ow_lo = max(wp - s.kW + s.sW, 0) / s.sW;
    for (int oh = oh_lo; oh <= oh_hi; ++oh) {
      const int kh = hp - oh * s.sH;
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const int kw = wp - ow * s.sW;
        const unsigned pos = (unsigned)(kh * s.kW + kw);
        const long long o = (((long long)n * s.OH + oh) * s.OW + ow) * cv_n + cv;
        if (!DL4J_IN_BOUNDS(o, (long long)s.N * s.OH * s.OW * cv_n)) continue;
        const uint2 p = __ldg(reinterpret_cast<const uint2*>(idx) + o);
        float d[8];
        pl_unpack8(__ldg(reinterpret_cast<const uint4*>(dy) + o), d);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (((p.x >> (8 * j)) & 0xffu) == pos) acc[j] += d[j];
          if (((p.y >> (8 * j)) & 0xffu) == pos) acc[4 + j] += d[4 + j];
        }
      }
    }
    reinterpret_cast<uint4*>(dx)[g] = pl_pack8(acc);
  }
}

// Strided spatial subsampling x[:, ::sH, ::sW, :] (the input side of a strided 1x1 convolution) and its adjoint, which
// writes the zeros and the scattered gradient in one pass.
__global__ void __launch_bounds__(PL_THREADS)
subsample_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, const PoolShape s) {
  const int cv_n = s.C >> 3;
  const long long total = (long long)s.N * s.OH * s.OW * cv_n;
  for (long long g = blockIdx.x * (long long)PL_THREADS + threadIdx.x; g < total; g += (long long)gridDim.x * PL_THREADS) {
    const int cv = (int)(g % cv_n);
    long long t = g / cv_n;
    const int ow = (int)(t % s.OW); t /= s.OW;
    const int oh = (int)(t % s.OH);
    const int n = (int)(t / s.OH);
    const long long xo = (((long long)n * s.H + (long long)oh * s.sH) * s.W + (long long)ow * s.sW) * cv_n + cv;
    if (!DL4J_IN_BOUNDS(xo, (long long)s.N * s.H * s.W * cv_n)) continue;
    reinterpret_cast<uint4*>(y)[g] = __ldg(reinterpret_cast<const uint4*>(x) + xo);
  }
}

__global__ void __launch_bounds__(PL_THREADS)
subsample_bwd_kernel(const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, const PoolShape s) {
  const int cv_n = s.C >> 3;
  const long long total = (long long)s.N * s.H * s.W * cv_n;
  for (long long g = blockIdx.x * (long long)PL_THREADS + threadIdx.x; g < total; g += (long long)gridDim.x * PL_THREADS) {
    const int cv = (int)(g % cv_n);
    long long t = g / cv_n;
    const int iw = (int)(t % s.W); t /= s.W;
    const int ih = (int)(t % s.H);
    const int n = (int)(t / s.H);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ih % s.sH == 0 && iw % s.sW == 0) {
      const int oh = ih / s.sH, ow = iw / s.sW;
      const long long yo = (((long long)n * s.OH + oh) * s.OW + ow) * cv_n + cv;
      if (oh < s.OH && ow < s.OW && DL4J_IN_BOUNDS(yo, (long long)s.N * s.OH * s.OW * cv_n)) v = __ldg(reinterpret_cast<const uint4*>(dy) + yo);
    }
    reinterpret_cast<uint4*>(dx)[g] = v;
  }
}

static inline int pl_grid(long long total) {
  long long b = (total + PL_THREADS - 1) / PL_THREADS;
  if (b > 148 * 16) b = 148 * 16;
  return (int)(b < 1 ? 1 : b);
}

static inline bool pl_ok(const PoolShape& s) {
  return s.N > 0 && s.H > 0 && s.W > 0 && s.C >= 8 && s.C % 8 == 0 && s.OH > 0 && s.OW > 0 && s.kH > 0 && s.kW > 0 && s.kH * s.kW <= 255 &&
         s.sH > 0 && s.sW > 0 && s.pH >= 0 && s.pW >= 0 && s.pH < s.kH && s.pW < s.kW;
}

}  // namespace dl4j

using namespace dl4j;

// shape: 12 ints {N, H, W, C, OH, OW, kH, kW, sH, sW, pH, pW}; idx (N*OH*OW*C bytes) may be null for inference
DL4J_API int dl4j_maxpool_fwd(const void* x, void* y, void* idx, const int* shape, void* stream) {
  PoolShape s;
  memcpy(&s, shape, sizeof(s));
  if (!pl_ok(s)) return -DL4J_ERR_BAD_ARG;
  const long long total = (long long)s.N * s.OH * s.OW * (s.C >> 3);
  maxpool_fwd_kernel<<<pl_grid(total), PL_THREADS, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y), reinterpret_cast<unsigned char*>(idx), s);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_maxpool_bwd(const void* dy, const void* idx, void* dx, const int* shape, void* stream) {
  PoolShape s;
  memcpy(&s, shape, sizeof(s));
  if (!pl_ok(s) || !idx) return -DL4J_ERR_BAD_ARG;
  const long long total = (long long)s.N * s.H * s.W * (s.C >> 3);
  maxpool_bwd_kernel<<<pl_grid(total), PL_THREADS, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const unsigned char*>(idx), reinterpret_cast<__nv_bfloat16*>(dx), s);
  return (int)cudaGetLastError();
}

// shape as above with kH = kW = 1, pH = pW = 0: OH = ceil(H / sH), OW = ceil(W / sW)
DL4J_API int dl4j_subsample(const void* in, void* out, const int* shape, int backward, void* stream) {
  PoolShape s;
  memcpy(&s, shape, sizeof(s));
  if (s.N <= 0 || s.H <= 0 || s.W <= 0 || s.C < 8 || s.C % 8 || s.sH < 1 || s.sW < 1 || s.OH != (s.H + s.sH - 1) / s.sH ||
      s.OW != (s.W + s.sW - 1) / s.sW)
    return -DL4J_ERR_BAD_ARG;
  if (backward) {
    const long long total = (long long)s.N * s.H * s.W * (s.C >> 3);
    subsample_bwd_kernel<<<pl_grid(total), PL_THREADS, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                                                 reinterpret_cast<__nv_bfloat16*>(out), s);
  } else {
    const long long total = (long long)s.N * s.OH * s.OW * (s.C >> 3);
    subsample_fwd_kernel<<<pl_grid(total), PL_THREADS, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                                                 reinterpret_cast<__nv_bfloat16*>(out), s);
  }
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ convolution weight layouts
// DL4J keeps convolution kernels as fp32 [O, I, kH, kW] ('c' order); the tensor-core convolution kernels want bf16 [O, kH, kW, I]
// (channels-last).  Forward: one cast + relayout pass.  Backward: the channels-last bf16 weight gradient is added into the fp32
// [O, I, kH, kW] gradient buffer in one pass.
namespace dl4j {

__global__ void __launch_bounds__(256)
conv_weight_to_cl_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int O, int I, int S) {
  // out[o][s][i] = w[o][i][s], S = kH * kW
  const long total = (long)O * I * S;
  for (long g = blockIdx.x * 256L + threadIdx.x; g < total; g += (long)gridDim.x * 256) {
    const int i = (int)(g % I);
    const int s = (int)((g / I) % S);
    const long o = g / ((long)I * S);
    out[g] = __float2bfloat16(w[(o * I + i) * S + s]);
  }
}

__global__ void __launch_bounds__(256)
conv_wgrad_from_cl_kernel(const __nv_bfloat16* __restrict__ g_cl, float* __restrict__ grad, int O, int I, int S) {
  // grad[o][i][s] += g_cl[o][s][i]; threads walk the destination so that the read-modify-write is coalesced
  const long total = (long)O * I * S;
  for (long g = blockIdx.x * 256L + threadIdx.x; g < total; g += (long)gridDim.x * 256) {
    const int s = (int)(g % S);
    const int i = (int)((g / S) % I);
    const long o = g / ((long)I * S);
    grad[g] += __bfloat162float(g_cl[(o * S + s) * I + i]);
  }
}

}  // namespace dl4j

DL4J_API int dl4j_conv_weight_to_cl(const float* w, void* out, int O, int I, int S, void* stream) {
  const long total = (long)O * I * S;
  if (total <= 0) return -DL4J_ERR_BAD_ARG;
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  conv_weight_to_cl_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(w, reinterpret_cast<__nv_bfloat16*>(out), O, I, S);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_conv_wgrad_from_cl(const void* g_cl, float* grad, int O, int I, int S, void* stream) {
  const long total = (long)O * I * S;
  if (total <= 0) return -DL4J_ERR_BAD_ARG;
  long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  conv_wgrad_from_cl_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(g_cl), grad, O, I, S);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ stem space-to-depth
// A stride-2 convolution over a few input channels (an RGB stem) runs as a stride-1 convolution over a 2x2 space-to-depth view of the
// zero-padded input.  This kernel builds that view in one pass: out[n, hs, ws, (bh * 2 + bw) * C + c] = x[n, c, 2 hs + bh - pH,
// 2 ws + bw - pW] (0 outside the image, 0 in the channels 4 C .. CP - 1), channels-last bf16 / fp16 with CP a multiple of 8, from
// an input of the same element type with arbitrary strides.  One thread writes one output pixel (CP elements, 16-byte stores).
namespace dl4j {
template <int CP>
__global__ void __launch_bounds__(256)
stem_s2d_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ out, int N, int C, int H, int W, long long sn, long long sc,
                long long sh, long long sw, int pH, int pW, int Hs, int Ws) {
  const long long total = (long long)N * Hs * Ws;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ws = (int)(i % Ws);
    const int hs = (int)((i / Ws) % Hs);
    const long long n = i / ((long long)Ws * Hs);
    __align__(16) uint16_t v[CP];
#pragma unroll
    for (int j = 0; j < CP; ++j) v[j] = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int ih = 2 * hs + (b >> 1) - pH, iw = 2 * ws + (b & 1) - pW;
      if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
        const uint16_t* src = x + n * sn + ih * sh + iw * sw;
        for (int c = 0; c < C; ++c)
          if (b * C + c < CP) v[b * C + c] = __ldg(src + c * sc);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + i * CP);
#pragma unroll
    for (int j = 0; j < CP / 8; ++j) dst[j] = reinterpret_cast<const uint4*>(v)[j];
  }
}
}  // namespace dl4j

// x: 16-bit elements (bf16 or fp16) [N, C, H, W] addressed with element strides {sn, sc, sh, sw}; out [N, Hs, Ws, CP] contiguous,
// CP in {8, 16, 32} and 4 C <= CP.
DL4J_API int dl4j_stem_space_to_depth(const void* x, void* out, int N, int C, int H, int W, const long long* strides, int pH, int pW,
                                      int Hs, int Ws, int CP, void* stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || Hs <= 0 || Ws <= 0) return 0;
  if (!x || !out || !strides || 4 * C > CP || ((uintptr_t)out & 15)) return -DL4J_ERR_BAD_ARG;
  const long long total = (long long)N * Hs * Ws;
  const int grid = pl_grid(total);
  const uint16_t* xi = reinterpret_cast<const uint16_t*>(x);
  uint16_t* o = reinterpret_cast<uint16_t*>(out);
  cudaStream_t st = (cudaStream_t)stream;
  if (CP == 8) stem_s2d_kernel<8><<<grid, 256, 0, st>>>(xi, o, N, C, H, W, strides[0], strides[1], strides[2], strides[3], pH, pW, Hs, Ws);
  else if (CP == 16) stem_s2d_kernel<16><<<grid, 256, 0, st>>>(xi, o, N, C, H, W, strides[0], strides[1], strides[2], strides[3], pH, pW, Hs, Ws);
  else if (CP == 32) stem_s2d_kernel<32><<<grid, 256, 0, st>>>(xi, o, N, C, H, W, strides[0], strides[1], strides[2], strides[3], pH, pW, Hs, Ws);
  else return -DL4J_ERR_BAD_ARG;
  return (int)cudaGetLastError();
}
