// Layer-norm backward that allocates nothing: its working memory is a fixed device array that ships
// inside the library image.  Contract, limits and the reasons for this entry point: dl4j_noalloc.h.
#include "common.cuh"
#include "dl4j_noalloc.h"

#include <cstdio>
#include <mutex>

namespace {

constexpr int NA_WARPS = 8;                          // one row per warp, eight rows per block pass
constexpr int NA_MAXV = DL4J_NOALLOC_LN_MAX_C / 256; // 8-element vectors per lane
constexpr int NA_COUNTER_BYTES = 256;
constexpr size_t NA_PARTIAL_FLOATS = (size_t)DL4J_NOALLOC_LN_MAX_BLOCKS * 2 * DL4J_NOALLOC_LN_MAX_C;
constexpr size_t NA_SCRATCH_BYTES = NA_COUNTER_BYTES + NA_PARTIAL_FLOATS * sizeof(float);

// [0, 256): counters (word 0 = blocks that have parked their partials); then float partial[block][2][MAX_C].
// Device code never names this array: the kernel gets its address as an argument.
static __device__ __align__(256) unsigned char g_ln_scratch[NA_SCRATCH_BYTES];

template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&o)[8]);
template <> __device__ __forceinline__ void ld8<float>(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void ld8<__half>(const __half* p, float (&o)[8]) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void st8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}
template <> __device__ __forceinline__ void st8<__half>(__half* p, const float (&v)[8]) {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}

template <typename T>
__global__ void __launch_bounds__(NA_WARPS * 32)
ln_bwd_scratch_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gain,
                      const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                      float* __restrict__ dgain, float* __restrict__ dbias, long long rows, int C, int accumulate,
                      unsigned char* scratch) {
  unsigned int* counters = reinterpret_cast<unsigned int*>(scratch);
  float* partial = reinterpret_cast<float*>(scratch + NA_COUNTER_BYTES);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nvec = C / 8;
  float ag[NA_MAXV][8], ab[NA_MAXV][8], g[NA_MAXV][8];
#pragma unroll
  for (int i = 0; i < NA_MAXV; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { ag[i][j] = 0.f; ab[i][j] = 0.f; g[i][j] = 0.f; }
    if (lane + i * 32 < nvec) ld8<float>(gain + (lane + i * 32) * 8, g[i]);
  }
  for (long long row = (long long)blockIdx.x * NA_WARPS + wid; row < rows; row += (long long)gridDim.x * NA_WARPS) {
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[NA_MAXV][8], dg[NA_MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float d[8];
        ld8<T>(dy + row * C + vi * 8, d);
        ld8<T>(x + row * C + vi * 8, xh[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          ag[i][j] += d[j] * xh[i][j];
          ab[i][j] += d[j];
          dg[i][j] = d[j] * g[i][j];
          s1 += dg[i][j];
          s2 += dg[i][j] * xh[i][j];
        }
      }
    }
    s1 = dl4j::warp_sum(s1) / C;
    s2 = dl4j::warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < NA_MAXV; ++i) {
      const int vi = lane + i * 32;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (dg[i][j] - s1 - xh[i][j] * s2);
        st8<T>(dx + row * C + vi * 8, o);
      }
    }
  }

  // Stage 1: fold the eight warps of this block in shared memory and park one partial per column in scratch.
  __shared__ float red[NA_WARPS][32 * 8 + 1];
  __shared__ bool is_last;
  float* mine = partial + (size_t)blockIdx.x * 2 * DL4J_NOALLOC_LN_MAX_C;
#pragma unroll
  for (int i = 0; i < NA_MAXV; ++i) {            // unrolled: ag / ab are indexed by constants and stay in registers
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 8; ++j) red[wid][lane * 8 + j] = pass == 0 ? ag[i][j] : ab[i][j];
      __syncthreads();
      for (int c = threadIdx.x; c < 256; c += NA_WARPS * 32) {
        const int col = i * 256 + c;
        if (col < C) {
          float t = 0.f;
#pragma unroll
          for (int w = 0; w < NA_WARPS; ++w) t += red[w][c];
          mine[pass * DL4J_NOALLOC_LN_MAX_C + col] = t;
        }
      }
    }
  }
  // Stage 2: the block that draws the last ticket adds the parked partials in block order.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&counters[0], 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < 2 * C; idx += NA_WARPS * 32) {
    const int pass = idx / C, col = idx - pass * C;
    float* dst = pass == 0 ? dgain : dbias;
    if (dst == nullptr) continue;
    float t = 0.f;
    for (unsigned int b = 0; b < gridDim.x; ++b)
      t += __ldcg(partial + (size_t)b * 2 * DL4J_NOALLOC_LN_MAX_C + pass * DL4J_NOALLOC_LN_MAX_C + col);
    dst[col] = accumulate ? dst[col] + t : t;
  }
  if (threadIdx.x == 0) counters[0] = 0u;            // leave the counter block zero for the next call
}

std::mutex g_setup_mu;
unsigned char* g_scratch_ptr[64] = {nullptr};

// One-time, per-device: device address of the scratch array (no allocation; may load the module).
int scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_ln_scratch);
    if (e != cudaSuccess) return (int)e;
    if (p == nullptr) return (int)cudaErrorInvalidSymbol;
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

int reject(const char* why, long long rows, int C) {
  std::fprintf(stderr,
               "dl4j_layer_norm_bwd_noalloc: %s (rows=%lld, C=%d; limits: C %% 8 == 0, C <= %d, 1 <= rows <= %lld)\n", why,
               rows, C, DL4J_NOALLOC_LN_MAX_C, (long long)DL4J_NOALLOC_LN_MAX_ROWS);
  return -DL4J_ERR_BAD_ARG;
}

}  // namespace

DL4J_API int dl4j_layer_norm_bwd_noalloc(const void* dy, const void* x, const float* gain, const float* mean,
                                         const float* rstd, void* dx, float* dgain, float* dbias, long long rows, int C,
                                         int dtype, int accumulate, void* stream) {
  if (C < 8 || C % 8 != 0) return reject("C must be a positive multiple of 8", rows, C);
  if (C > DL4J_NOALLOC_LN_MAX_C) return reject("C exceeds the scratch array's width", rows, C);
  if (rows < 1 || rows > DL4J_NOALLOC_LN_MAX_ROWS) return reject("rows out of range", rows, C);
  if (dtype < 0 || dtype > 2) return reject("dtype must be 0 (f16), 1 (bf16) or 2 (f32)", rows, C);
  if (!dy || !x || !gain || !mean || !rstd || !dx) return reject("null input or dx pointer", rows, C);
  // the kernel moves dy / x / dx / gain with 16-byte vector accesses; rows keep the base's alignment because C % 8 == 0
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) |
       reinterpret_cast<uintptr_t>(gain)) & 15)
    return reject("dy, x, dx and gain must be 16-byte aligned", rows, C);
  if ((reinterpret_cast<uintptr_t>(mean) | reinterpret_cast<uintptr_t>(rstd) | reinterpret_cast<uintptr_t>(dgain) |
       reinterpret_cast<uintptr_t>(dbias)) & 3)
    return reject("mean, rstd, dgain and dbias must be 4-byte aligned", rows, C);
  unsigned char* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  long long blocks = (rows + NA_WARPS - 1) / NA_WARPS;
  const int grid = (int)(blocks < DL4J_NOALLOC_LN_MAX_BLOCKS ? blocks : DL4J_NOALLOC_LN_MAX_BLOCKS);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(scratch, 0, NA_COUNTER_BYTES, s);   // counters must start at zero
  if (e != cudaSuccess) return (int)e;
  if (dtype == 2)
    ln_bwd_scratch_kernel<float><<<grid, NA_WARPS * 32, 0, s>>>((const float*)dy, (const float*)x, gain, mean, rstd,
                                                               (float*)dx, dgain, dbias, rows, C, accumulate, scratch);
  else if (dtype == 1)
    ln_bwd_scratch_kernel<__nv_bfloat16><<<grid, NA_WARPS * 32, 0, s>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, gain, mean, rstd, (__nv_bfloat16*)dx, dgain, dbias, rows, C,
        accumulate, scratch);
  else
    ln_bwd_scratch_kernel<__half><<<grid, NA_WARPS * 32, 0, s>>>((const __half*)dy, (const __half*)x, gain, mean, rstd,
                                                                (__half*)dx, dgain, dbias, rows, C, accumulate, scratch);
  return (int)cudaGetLastError();
}
