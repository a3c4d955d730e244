// Batch normalisation over channels-last activations (x viewed as [rows, C], rows = N*H*W), bf16 in / out with fp32
// statistics, fused with the ReLU that follows it and with the residual add of a bottleneck block:
//     y = act(gamma * (x - mean) * invstd + beta [+ residual])
// Training forward is three launches (per-channel sums, finalise, apply) instead of the stats / transform / relu /
// add / running-stat-update chain; the finalise step also updates the running mean and DL4J's log10(stdev)
// (or variance) parameter in place (BatchNormalization.java, BatchNormalizationParamInitializer.java).
// Backward is two launches: per-channel reductions of dy and dy*xhat behind the ReLU mask, then dx (and the
// residual gradient) with dgamma / dbeta accumulated into the flat gradient buffer.
#include "common.cuh"

namespace dl4j {

constexpr int BN_THREADS = 256;

__device__ __forceinline__ void bn_unpack8(const uint4& u, float* o) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
__device__ __forceinline__ uint4 bn_pack8(const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}
__device__ __forceinline__ void ld8f(const float* p, float* o) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

// Block-level finish of the per-thread partials: threads that share a channel vector are folded in shared memory, then
// one atomicAdd per channel and block.  acc0 -> out[c], acc1 -> out[C + c].
__device__ __forceinline__ void bn_block_reduce(const float* s, const float* q, float* __restrict__ out, int C, int cv_n) {
  __shared__ float red[BN_THREADS][17];
#pragma unroll
  for (int j = 0; j < 8; ++j) { red[threadIdx.x][j] = s[j]; red[threadIdx.x][8 + j] = q[j]; }
  __syncthreads();
  const int lanes = BN_THREADS / cv_n;
  for (int c = threadIdx.x; c < C; c += BN_THREADS) {
    const int cv = c >> 3, j = c & 7;
    float a = 0.f, b = 0.f;
    for (int l = 0; l < lanes; ++l) { a += red[l * cv_n + cv][j]; b += red[l * cv_n + cv][8 + j]; }
    atomicAdd(out + c, a);
    atomicAdd(out + C + c, b);
  }
}

struct BnFinalize {
  const float* gamma; const float* beta; float* run_mean; float* run_stat; int use_log_std; float decay, eps, inv_rows;
  float* save_mean; float* save_invstd; float* scale; float* shift; const float* pre_bias;
};

__device__ __forceinline__ void bn_finalize_channel(const float* sums, const BnFinalize& f, int c, int C) {
  const float* gamma = f.gamma; const float* beta = f.beta; float* run_mean = f.run_mean; float* run_stat = f.run_stat;
  const int use_log_std = f.use_log_std; const float decay = f.decay, eps = f.eps, inv_rows = f.inv_rows;
  float* save_mean = f.save_mean; float* save_invstd = f.save_invstd; float* scale = f.scale; float* shift = f.shift;
  const float* pre_bias = f.pre_bias;
  const float mean = __ldcg(sums + c) * inv_rows;
  const float var = fmaxf(__ldcg(sums + C + c) * inv_rows - mean * mean, 0.f);
  const float invstd = rsqrtf(var + eps);
  const float g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
  save_mean[c] = mean;
  save_invstd[c] = invstd;
  scale[c] = g * invstd;
  shift[c] = b - mean * g * invstd;
  // pre_bias: bias of the producing convolution, left out of x because the batch mean cancels it; the running mean
  // (used at inference, where it does not cancel) still has to see it
  if (run_mean) run_mean[c] = decay * run_mean[c] + (1.f - decay) * (mean + (pre_bias ? pre_bias[c] : 0.f));
  if (run_stat) {
    const float old_var = use_log_std ? exp10f(2.f * run_stat[c]) : run_stat[c];
    const float nv = decay * old_var + (1.f - decay) * var;
    run_stat[c] = use_log_std ? 0.5f * log10f(fmaxf(nv, 1e-30f)) : nv;
  }
}

// sums[c] = sum_r x[r, c], sums[C + c] = sum_r x[r, c]^2.  C / 8 is a power of two <= 256, so a thread keeps one channel
// vector for its whole row range and accumulates in registers.
// With `ticket` the block that finishes last also turns the sums into mean / invstd / scale / shift and updates the running
// statistics (one launch less per batch-norm layer than a separate per-channel kernel).
__global__ void __launch_bounds__(BN_THREADS)
bn_stats_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ sums, long long rows, int C, long long rows_per_block,
                unsigned int* ticket, const BnFinalize fin) {
  const int cv_n = C >> 3;
  const int cv = threadIdx.x & (cv_n - 1), rl = threadIdx.x / cv_n;
  const int step = BN_THREADS / cv_n;
  const long long r0 = blockIdx.x * rows_per_block;
  const long long r1 = min(r0 + rows_per_block, rows);
  float s[8], q[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; q[j] = 0.f; }
  const __nv_bfloat16* base = x + cv * 8;
  for (long long r = r0 + rl; r < r1; r += 4LL * step) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long rr = r + (long long)u * step;
      v[u] = rr < r1 && DL4J_IN_BOUNDS(rr * C + cv * 8 + 7, rows * (long long)C)
                 ? __ldg(reinterpret_cast<const uint4*>(base + rr * C)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float f[8];
      bn_unpack8(v[u], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[j] += f[j]; q[j] = fmaf(f[j], f[j], q[j]); }
    }
  }
  bn_block_reduce(s, q, sums, C, cv_n);
  if (ticket == nullptr) return;
  __shared__ unsigned int my_ticket;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) my_ticket = atomicAdd(ticket, 1u);
  __syncthreads();
  if (my_ticket != gridDim.x - 1) return;
  __threadfence();
  for (int c = threadIdx.x; c < C; c += BN_THREADS) bn_finalize_channel(sums, fin, c, C);
}

// Per channel: batch mean / biased variance -> invstd, scale, shift; running statistics updated in place with
// DL4J's rule  global = decay * global + (1 - decay) * batch  (the variance kept as log10 of the standard deviation
// when use_log_std is set).
// y = act(x * scale + shift [+ res])
__global__ void __launch_bounds__(BN_THREADS)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res, const float* __restrict__ scale,
                const float* __restrict__ shift, __nv_bfloat16* __restrict__ y, long long n_vec, int C, int relu) {
  const int cv_n = C >> 3;
  for (long long g = blockIdx.x * (long long)BN_THREADS + threadIdx.x; g < n_vec; g += (long long)gridDim.x * BN_THREADS) {
    const int c0 = (int)(g & (cv_n - 1)) * 8;
    float f[8], sc[8], sh[8];
    bn_unpack8(__ldg(reinterpret_cast<const uint4*>(x) + g), f);
    ld8f(scale + c0, sc);
    ld8f(shift + c0, sh);
    if (res) {
      float r[8];
      bn_unpack8(__ldg(reinterpret_cast<const uint4*>(res) + g), r);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], sc[j], sh[j]) + r[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = fmaf(f[j], sc[j], sh[j]);
    }
    if (relu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
    }
    reinterpret_cast<uint4*>(y)[g] = bn_pack8(f);
  }
}

// sums[c] = sum_r dyr, sums[C + c] = sum_r dyr * xhat, with dyr = dy masked by the ReLU (mask from y when given: needed
// when a residual was added; else recomputed from x).
__global__ void __launch_bounds__(BN_THREADS)
bn_bwd_reduce_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                     const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ scale,
                     const float* __restrict__ shift, float* __restrict__ sums, long long rows, int C, long long rows_per_block, int relu) {
  const int cv_n = C >> 3;
  const int cv = threadIdx.x & (cv_n - 1), rl = threadIdx.x / cv_n;
  const int step = BN_THREADS / cv_n;
  const long long r0 = blockIdx.x * rows_per_block;
  const long long r1 = min(r0 + rows_per_block, rows);
  float s[8], q[8], mu[8], is[8], sc[8], sh[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { s[j] = 0.f; q[j] = 0.f; }
  ld8f(mean + cv * 8, mu);
  ld8f(invstd + cv * 8, is);
  ld8f(scale + cv * 8, sc);
  ld8f(shift + cv * 8, sh);
  const long long off = cv * 8;
  for (long long r = r0 + rl; r < r1; r += 2LL * step) {
    uint4 vd[2], vx[2], vy[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const long long rr = r + (long long)u * step;
      const bool in = rr < r1;
      vd[u] = in ? __ldg(reinterpret_cast<const uint4*>(dy + rr * C + off)) : make_uint4(0u, 0u, 0u, 0u);
      vx[u] = in ? __ldg(reinterpret_cast<const uint4*>(x + rr * C + off)) : make_uint4(0u, 0u, 0u, 0u);
      vy[u] = (in && y && relu) ? __ldg(reinterpret_cast<const uint4*>(y + rr * C + off)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float d[8], xv[8], yv[8];
      bn_unpack8(vd[u], d);
      bn_unpack8(vx[u], xv);
      bn_unpack8(vy[u], yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        bool keep = true;
        if (relu) keep = y ? (yv[j] > 0.f) : (fmaf(xv[j], sc[j], sh[j]) > 0.f);
        const float dv = keep ? d[j] : 0.f;
        s[j] += dv;
        q[j] = fmaf(dv, (xv[j] - mu[j]) * is[j], q[j]);
      }
    }
  }
  bn_block_reduce(s, q, sums, C, cv_n);
}

// dx = scale * (dyr - (sum_dy + xhat * sum_dy_xhat) / rows); dres = dyr; dgamma += sum_dy_xhat, dbeta += sum_dy.
__global__ void __launch_bounds__(BN_THREADS)
bn_bwd_apply_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                    const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ scale,
                    const float* __restrict__ shift, const float* __restrict__ sums, __nv_bfloat16* __restrict__ dx,
                    __nv_bfloat16* __restrict__ dres, float* __restrict__ dgamma, float* __restrict__ dbeta, long long n_vec, int C,
                    float inv_rows, int relu) {
  const int cv_n = C >> 3;
  const long long gid = blockIdx.x * (long long)BN_THREADS + threadIdx.x;
  if (gid < C) {
    if (dgamma) dgamma[gid] += sums[C + gid];
    if (dbeta) dbeta[gid] += sums[gid];
  }
  for (long long g = gid; g < n_vec; g += (long long)gridDim.x * BN_THREADS) {
    const int c0 = (int)(g & (cv_n - 1)) * 8;
    float d[8], xv[8], mu[8], is[8], sc[8], sh[8], sd[8], sq[8], o[8];
    bn_unpack8(__ldg(reinterpret_cast<const uint4*>(dy) + g), d);
    bn_unpack8(__ldg(reinterpret_cast<const uint4*>(x) + g), xv);
    ld8f(mean + c0, mu);
    ld8f(invstd + c0, is);
    ld8f(scale + c0, sc);
    ld8f(sums + c0, sd);
    ld8f(sums + C + c0, sq);
    if (relu) {
      if (y) {
        float yv[8];
        bn_unpack8(__ldg(reinterpret_cast<const uint4*>(y) + g), yv);
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = yv[j] > 0.f ? d[j] : 0.f;
      } else {
        ld8f(shift + c0, sh);
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = fmaf(xv[j], sc[j], sh[j]) > 0.f ? d[j] : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xhat = (xv[j] - mu[j]) * is[j];
      o[j] = sc[j] * (d[j] - (sd[j] + xhat * sq[j]) * inv_rows);
    }
    reinterpret_cast<uint4*>(dx)[g] = bn_pack8(o);
    if (dres) reinterpret_cast<uint4*>(dres)[g] = bn_pack8(d);
  }
}

// y = relu(a + b): the block-ending add of an identity shortcut when no batch norm precedes it
__global__ void __launch_bounds__(BN_THREADS)
add_relu_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, long long n_vec) {
  for (long long g = blockIdx.x * (long long)BN_THREADS + threadIdx.x; g < n_vec; g += (long long)gridDim.x * BN_THREADS) {
    float fa[8], fb[8];
    bn_unpack8(__ldg(reinterpret_cast<const uint4*>(a) + g), fa);
    bn_unpack8(__ldg(reinterpret_cast<const uint4*>(b) + g), fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) fa[j] = fmaxf(fa[j] + fb[j], 0.f);
    reinterpret_cast<uint4*>(y)[g] = bn_pack8(fa);
  }
}

static inline bool bn_shape_ok(long long rows, int C) { return rows > 0 && C >= 8 && C <= 2048 && (C & (C - 1)) == 0; }

static inline int bn_grid_rows(long long rows, int C, long long* rows_per_block) {
  const int step = BN_THREADS / (C >> 3);
  long long blocks = 148 * 4;
  long long rpb = (rows + blocks - 1) / blocks;
  const long long quantum = 4LL * step;
  rpb = (rpb + quantum - 1) / quantum * quantum;
  *rows_per_block = rpb;
  return (int)((rows + rpb - 1) / rpb);
}

static inline int bn_grid_elems(long long n_vec) {
  long long b = (n_vec + BN_THREADS - 1) / BN_THREADS;
  if (b > 148 * 8) b = 148 * 8;
  return (int)(b < 1 ? 1 : b);
}

}  // namespace dl4j

using namespace dl4j;

// Training forward.  work: 4 * C + 8 floats of scratch laid out as [sums(2C) | ticket(8) | scale(C) | shift(C)]; scale / shift and
// save_mean / save_invstd are kept by the caller for the backward pass.  run_mean / run_stat may be null.
DL4J_API int dl4j_bn_fwd_train(const void* x, const void* res, const float* gamma, const float* beta, float* run_mean, float* run_stat,
                               int use_log_std, float decay, float eps, int relu, void* y, float* save_mean, float* save_invstd,
                               float* work, const float* pre_bias, long long rows, int C, void* stream_) {
  if (!bn_shape_ok(rows, C)) return -DL4J_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  float* sums = work;
  float* scale = work + 2 * C + 8;
  float* shift = work + 3 * C + 8;
  cudaMemsetAsync(sums, 0, sizeof(float) * (2 * C + 8), st);          // the sums and the ticket of the statistics kernel
  long long rpb;
  const int g1 = bn_grid_rows(rows, C, &rpb);
  BnFinalize fin;
  fin.gamma = gamma; fin.beta = beta; fin.run_mean = run_mean; fin.run_stat = run_stat; fin.use_log_std = use_log_std;
  fin.decay = decay; fin.eps = eps; fin.inv_rows = 1.0f / (float)rows; fin.save_mean = save_mean; fin.save_invstd = save_invstd;
  fin.scale = scale; fin.shift = shift; fin.pre_bias = pre_bias;
  bn_stats_kernel<<<g1, BN_THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), sums, rows, C, rpb,
                                             reinterpret_cast<unsigned int*>(work + 2 * C), fin);
  const long long n_vec = rows * (C >> 3);
  bn_apply_kernel<<<bn_grid_elems(n_vec), BN_THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                reinterpret_cast<const __nv_bfloat16*>(res), scale, shift,
                                                                reinterpret_cast<__nv_bfloat16*>(y), n_vec, C, relu);
  return (int)cudaGetLastError();
}

// Inference / fixed statistics: y = act(x * scale + shift [+ res]) with caller-provided per-channel scale and shift.
DL4J_API int dl4j_bn_apply(const void* x, const void* res, const float* scale, const float* shift, int relu, void* y, long long rows, int C,
                           void* stream_) {
  if (!bn_shape_ok(rows, C)) return -DL4J_ERR_BAD_ARG;
  const long long n_vec = rows * (C >> 3);
  bn_apply_kernel<<<bn_grid_elems(n_vec), BN_THREADS, 0, (cudaStream_t)stream_>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(res), scale, shift,
      reinterpret_cast<__nv_bfloat16*>(y), n_vec, C, relu);
  return (int)cudaGetLastError();
}

// Backward of dl4j_bn_fwd_train.  y is needed only when a residual was added before the ReLU (else the mask is recomputed
// from x); work is the same [sums | scale | shift] scratch with scale / shift still holding the forward values.
DL4J_API int dl4j_bn_bwd(const void* dy, const void* x, const void* y, const float* save_mean, const float* save_invstd, float* work,
                         void* dx, void* dres, float* dgamma, float* dbeta, long long rows, int C, int relu, void* stream_) {
  if (!bn_shape_ok(rows, C)) return -DL4J_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream_;
  float* sums = work;
  const float* scale = work + 2 * C + 8;
  const float* shift = work + 3 * C + 8;
  cudaMemsetAsync(sums, 0, sizeof(float) * 2 * C, st);
  long long rpb;
  int g1 = bn_grid_rows(rows, C, &rpb);
  bn_bwd_reduce_kernel<<<g1, BN_THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
                                                  reinterpret_cast<const __nv_bfloat16*>(y), save_mean, save_invstd, scale, shift, sums,
                                                  rows, C, rpb, relu);
  const long long n_vec = rows * (C >> 3);
  int g2 = bn_grid_elems(n_vec);
  if ((long long)g2 * BN_THREADS < C) g2 = (C + BN_THREADS - 1) / BN_THREADS;
  bn_bwd_apply_kernel<<<g2, BN_THREADS, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy), reinterpret_cast<const __nv_bfloat16*>(x),
                                                 reinterpret_cast<const __nv_bfloat16*>(y), save_mean, save_invstd, scale, shift, sums,
                                                 reinterpret_cast<__nv_bfloat16*>(dx), reinterpret_cast<__nv_bfloat16*>(dres), dgamma,
                                                 dbeta, n_vec, C, 1.0f / (float)rows, relu);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_add_relu(const void* a, const void* b, void* y, long long n, void* stream_) {
  if (n <= 0 || (n & 7)) return -DL4J_ERR_BAD_ARG;
  const long long n_vec = n >> 3;
  add_relu_kernel<<<bn_grid_elems(n_vec), BN_THREADS, 0, (cudaStream_t)stream_>>>(
      reinterpret_cast<const __nv_bfloat16*>(a), reinterpret_cast<const __nv_bfloat16*>(b), reinterpret_cast<__nv_bfloat16*>(y), n_vec);
  return (int)cudaGetLastError();
}
