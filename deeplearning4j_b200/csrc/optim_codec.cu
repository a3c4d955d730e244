// Multi-segment fused updater over the flattened DL4J parameter / gradient / state buffers, and the
// threshold ("flexible") and bitmap gradient codecs.
//
// Updater math: libnd4j/include/ops/declarable/helpers/cuda/updater{Adam,Nesterovs,AdaGrad,AdaDelta,
// AdaMax,AdaBelief,AmsGrad,Nadam,RmsProp}.cu; block/regularisation order:
// deeplearning4j-nn/.../nn/updater/UpdaterBlock.java:118-165 (L1/L2 before the updater, weight decay
// after, then params -= update).  One launch covers every parameter of the network: a chunk table maps
// CUDA blocks to (offset, count, segment) and a segment table carries per-parameter coefficients.
//
// Codec semantics: libnd4j/include/loops/cuda/type_conversions.cu:215-500 (message layout
// [k, N, bits(tau), flag, payload...], residual kept in the source buffer, bitmap half-threshold rule).
#include "common.cuh"
#include "updater_math.cuh"

namespace dl4j {

constexpr int UPD_THREADS = 256;

// mode 0: params -= update (and refresh the bf16 shadow); mode 1: residual += update, params untouched
// (threshold gradient sharing accumulates the post-updater update before encoding it).
__global__ void __launch_bounds__(UPD_THREADS)
fused_update_kernel(float* __restrict__ params, float* __restrict__ grads, float* __restrict__ state,
                    __nv_bfloat16* __restrict__ shadow, float* __restrict__ residual, const UpdChunk* __restrict__ chunks,
                    const UpdSegment* __restrict__ segs, const UpdHyperTable ht, float grad_scale, int zero_grads) {
  const UpdChunk ch = chunks[blockIdx.x];
  const UpdSegment sg = segs[ch.seg];
  const UpdHyper h = ht.h[sg.hyper];
  const long long rel0 = ch.offset - sg.block_start;
  float* st0 = state + sg.state_off + rel0;
  float* st1 = st0 + sg.block_numel;
  float* st2 = st1 + sg.block_numel;
  float* p = params + ch.offset;
  float* g = grads + ch.offset;
  if (sg.kernel_id == 9) {              // NoOp / state parameters: leave untouched
    if (zero_grads)
      for (int i = threadIdx.x; i < ch.count; i += UPD_THREADS) g[i] = 0.f;
    return;
  }
  float* res = residual ? residual + ch.offset : nullptr;
  __nv_bfloat16* sh = shadow ? shadow + sg.shadow_off + (ch.offset - sg.offset) : nullptr;
  // Scalar head up to a 16-byte boundary of the parameter pointer, then 4 elements per thread.  Parameters and gradients share
  // their offsets; the state slots sit block_numel elements apart (DL4J's [m | v] layout), the shadow and the residual have
  // offsets of their own, so any of those streams may be off the 16-byte grid at that point: each stream is moved with one
  // 16-byte access when it is aligned and with four 4-byte accesses otherwise (the warp still covers a contiguous 512 bytes).
  int head = (int)((4 - ((reinterpret_cast<uintptr_t>(p) >> 2) & 3)) & 3);
  if (head > ch.count) head = ch.count;
  const int ns = upd_n_state(sg.kernel_id);
  const bool pg_ok = ((reinterpret_cast<uintptr_t>(p + head) | reinterpret_cast<uintptr_t>(g + head)) & 15) == 0;
  const bool a_al = (reinterpret_cast<uintptr_t>(st0 + head) & 15) == 0, b_al = (reinterpret_cast<uintptr_t>(st1 + head) & 15) == 0;
  const bool c_al = (reinterpret_cast<uintptr_t>(st2 + head) & 15) == 0;
  const bool r_al = res && (reinterpret_cast<uintptr_t>(res + head) & 15) == 0;
  const bool s_al = sh && (reinterpret_cast<uintptr_t>(sh + head) & 7) == 0;
  const int nvec = pg_ok ? (ch.count - head) / 4 : 0;
  // vectors per thread and iteration, every load issued before the first use.  Measured on 105 M parameters (Adam, fp32): one
  // vector 0.469 ms (0.96 of the copy bandwidth), two vectors 0.575 ms (124 registers: fewer resident warps outweigh the extra
  // bytes in flight per thread)
  constexpr int U = 1;
  for (int q0 = threadIdx.x; q0 < nvec; q0 += U * UPD_THREADS) {
    float4 w4[U], g4[U], a4[U], b4[U], c4[U], r4[U];
#pragma unroll
    for (int t = 0; t < U; ++t) {
      const int q = q0 + t * UPD_THREADS;
      w4[t] = make_float4(0.f, 0.f, 0.f, 0.f);
      g4[t] = w4[t]; a4[t] = w4[t]; b4[t] = w4[t]; c4[t] = w4[t]; r4[t] = w4[t];
      if (q < nvec) {
        const int i = head + 4 * q;
        w4[t] = *reinterpret_cast<const float4*>(p + i);
        g4[t] = *reinterpret_cast<const float4*>(g + i);
        if (ns > 0) a4[t] = upd_ld4(st0 + i, a_al);
        if (ns > 1) b4[t] = upd_ld4(st1 + i, b_al);
        if (ns > 2) c4[t] = upd_ld4(st2 + i, c_al);
        if (res) r4[t] = upd_ld4(res + i, r_al);
      }
    }
#pragma unroll
    for (int t = 0; t < U; ++t) {
      const int q = q0 + t * UPD_THREADS;
      if (q >= nvec) continue;
      const int i = head + 4 * q;
      float w[4] = {w4[t].x, w4[t].y, w4[t].z, w4[t].w}, gr[4] = {g4[t].x, g4[t].y, g4[t].z, g4[t].w};
      float a[4] = {a4[t].x, a4[t].y, a4[t].z, a4[t].w}, b[4] = {b4[t].x, b4[t].y, b4[t].z, b4[t].w},
            c[4] = {c4[t].x, c4[t].y, c4[t].z, c4[t].w}, u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) u[j] = updater_step(sg, h, w[j], gr[j] * grad_scale, a + j, b + j, c + j);
      if (ns > 0) upd_st4(st0 + i, make_float4(a[0], a[1], a[2], a[3]), a_al);
      if (ns > 1) upd_st4(st1 + i, make_float4(b[0], b[1], b[2], b[3]), b_al);
      if (ns > 2) upd_st4(st2 + i, make_float4(c[0], c[1], c[2], c[3]), c_al);
      if (res) {
        upd_st4(res + i, make_float4(r4[t].x + u[0], r4[t].y + u[1], r4[t].z + u[2], r4[t].w + u[3]), r_al);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] -= u[j];
        *reinterpret_cast<float4*>(p + i) = make_float4(w[0], w[1], w[2], w[3]);
        if (sh) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(w[0], w[1]), hi = __floats2bfloat162_rn(w[2], w[3]);
          if (s_al) {
            *reinterpret_cast<uint2*>(sh + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          } else {
            sh[i] = lo.x; sh[i + 1] = lo.y; sh[i + 2] = hi.x; sh[i + 3] = hi.y;
          }
        }
      }
      if (zero_grads) *reinterpret_cast<float4*>(g + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // scalar head and tail
  const int tail0 = head + 4 * nvec;
  for (int k = threadIdx.x; k < head + (ch.count - tail0); k += UPD_THREADS) {
    const int i = k < head ? k : tail0 + (k - head);
    float w = p[i];
    const float u = updater_step(sg, h, w, g[i] * grad_scale, st0 + i, st1 + i, st2 + i);
    if (res) {
      res[i] += u;
    } else {
      w -= u;
      p[i] = w;
      if (sh) sh[i] = __float2bfloat16(w);
    }
    if (zero_grads) g[i] = 0.f;
  }
}

// fp32 -> bf16 shadow copy of the parameter buffer (used once after init / setParams)
__global__ void cast_f32_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, long long n) {
  long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (; i + 3 < n; i += stride) {
    const float4 v = *reinterpret_cast<const float4*>(in + i);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    *reinterpret_cast<uint2*>(out + i) = u;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long j = n & ~3LL; j < n; ++j) out[j] = __float2bfloat16(in[j]);
}

// ----------------------------------------------------------------------------- threshold codec
constexpr int ENC_THREADS = 256;
constexpr int ENC_PER_THREAD = 8;
constexpr int ENC_TILE = ENC_THREADS * ENC_PER_THREAD;

// Sparse encode: every |x[i]| >= tau becomes +-(i+1) in msg[4..], x[i] moves towards zero by tau.
// msg[0] is the atomic slot counter (must be zero on entry); entries beyond `capacity` are not
// encoded and their residual is left untouched.  Order inside a tile is ascending.
__global__ void __launch_bounds__(ENC_THREADS)
threshold_encode_kernel(float* __restrict__ x, long long n, float tau, int* __restrict__ msg, int capacity) {
  __shared__ int warp_tot[ENC_THREADS / 32];
  __shared__ int tile_base;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    msg[1] = (int)n;
    msg[2] = __float_as_int(tau);
    msg[3] = 0;
  }
  const long long tiles = (n + ENC_TILE - 1) / ENC_TILE;
  for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
    const long long base = t * ENC_TILE + (long long)threadIdx.x * ENC_PER_THREAD;
    float v[ENC_PER_THREAD];
    int flags = 0, cnt = 0;
    if (base + ENC_PER_THREAD <= n) {
      const float4 a = *reinterpret_cast<const float4*>(x + base);
      const float4 b = *reinterpret_cast<const float4*>(x + base + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < ENC_PER_THREAD; ++j) v[j] = (base + j < n) ? x[base + j] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < ENC_PER_THREAD; ++j)
      if (fabsf(v[j]) >= tau) { flags |= 1 << j; ++cnt; }
    // block exclusive scan of cnt
    int incl = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    if (lane == 31) warp_tot[wid] = incl;
    __syncthreads();
    int woff = 0, total = 0;
#pragma unroll
    for (int w = 0; w < ENC_THREADS / 32; ++w) {
      const int c = warp_tot[w];
      if (w < wid) woff += c;
      total += c;
    }
    if (threadIdx.x == 0) tile_base = total ? atomicAdd(&msg[0], total) : 0;
    __syncthreads();
    int slot = tile_base + woff + incl - cnt;
    if (flags) {
      bool touched = false;
#pragma unroll
      for (int j = 0; j < ENC_PER_THREAD; ++j) {
        if (flags & (1 << j)) {
          if (slot < capacity) {
            const bool neg = v[j] < 0.f;
            const int idx = (int)(base + j) + 1;
            msg[4 + slot] = neg ? -idx : idx;
            v[j] += neg ? tau : -tau;
            touched = true;
          }
          ++slot;
        }
      }
      if (touched) {
        if (base + ENC_PER_THREAD <= n) {
          *reinterpret_cast<float4*>(x + base) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(x + base + 4) = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
          for (int j = 0; j < ENC_PER_THREAD; ++j) if (base + j < n) x[base + j] = v[j];
        }
      }
    }
    __syncthreads();
  }
}

// Sparse decode: target[|e|-1] += sign(e) * scale * tau for the first min(msg[0], capacity) entries.
__global__ void threshold_decode_kernel(const int* __restrict__ msg, int capacity, float* __restrict__ target,
                                        long long n_target, float scale, int use_atomics, int* status) {
  int k = msg[0];
  if (k > capacity) k = capacity;
  const float tau = __int_as_float(msg[2]) * scale;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < k; j += gridDim.x * blockDim.x) {
    const int e = msg[4 + j];
    const int idx = (e < 0 ? -e : e) - 1;
    if (idx < 0 || idx >= n_target) { if (status) atomicCAS(status, 0, DL4J_ERR_BOUNDS); continue; }
    const float d = e < 0 ? -tau : tau;
    if (use_atomics) atomicAdd(target + idx, d); else target[idx] += d;
  }
}

// Bitmap encode: word w covers elements [16w, 16w+16): bit b = |x| >= tau, bit b+16 = negative; a
// negative value with tau/2 <= |x| < tau sets only the sign bit and moves by +tau/2.
__global__ void bitmap_encode_kernel(float* __restrict__ x, long long n, float tau, int* __restrict__ msg) {
  __shared__ int block_cnt;
  if (threadIdx.x == 0) block_cnt = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    msg[1] = (int)n;
    msg[2] = __float_as_int(tau);
    msg[3] = 1;
  }
  __syncthreads();
  const long long words = (n + 15) / 16;
  int cnt = 0;
  const float half = tau * 0.5f;
  for (long long w = blockIdx.x * (long long)blockDim.x + threadIdx.x; w < words; w += (long long)gridDim.x * blockDim.x) {
    const long long base = w * 16;
    float v[16];
    const bool full = base + 16 <= n;
    if (full) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 a = *reinterpret_cast<const float4*>(x + base + 4 * q);
        v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = (base + j < n) ? x[base + j] : 0.f;
    }
    int word = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = fabsf(v[j]);
      if (a >= tau) {
        word |= 1 << j;
        ++cnt;
        if (v[j] < 0.f) { word |= 1 << (j + 16); v[j] += tau; } else { v[j] -= tau; }
      } else if (a >= half && v[j] < 0.f) {
        word |= 1 << (j + 16);
        ++cnt;
        v[j] += half;
      }
    }
    msg[4 + w] = word;
    if (word) {
      if (full) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<float4*>(x + base + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) if (base + j < n) x[base + j] = v[j];
      }
    }
  }
  cnt = (int)warp_sum((float)cnt);   // counts per warp stay far below 2^24: exact in fp32
  if ((threadIdx.x & 31) == 0 && cnt) atomicAdd(&block_cnt, cnt);
  __syncthreads();
  if (threadIdx.x == 0 && block_cnt) atomicAdd(&msg[0], block_cnt);
}

__global__ void bitmap_decode_kernel(const int* __restrict__ msg, float* __restrict__ target, long long n, float scale) {
  const float tau = __int_as_float(msg[2]) * scale;
  const float half = tau * 0.5f;
  const long long words = (n + 15) / 16;
  for (long long w = blockIdx.x * (long long)blockDim.x + threadIdx.x; w < words; w += (long long)gridDim.x * blockDim.x) {
    const int word = msg[4 + w];
    if (!word) continue;
    const long long base = w * 16;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (base + j >= n) break;
      const bool bit = word & (1 << j), sign = word & (1 << (j + 16));
      if (bit) target[base + j] += sign ? -tau : tau;
      else if (sign) target[base + j] -= half;
    }
  }
}

}  // namespace dl4j

using namespace dl4j;

DL4J_API int dl4j_fused_update(float* params, float* grads, float* state, void* shadow_bf16, float* residual,
                               const void* chunks, int n_chunks, const void* segs, const float* hyper, int n_hyper,
                               float grad_scale, int zero_grads, void* stream) {
  if (n_chunks <= 0) return 0;
  if (n_hyper > UPD_MAX_HYPER) return -DL4J_ERR_BAD_ARG;
  UpdHyperTable ht;
  memset(&ht, 0, sizeof(ht));
  memcpy(&ht, hyper, sizeof(UpdHyper) * n_hyper);
  fused_update_kernel<<<n_chunks, UPD_THREADS, 0, (cudaStream_t)stream>>>(
      params, grads, state, reinterpret_cast<__nv_bfloat16*>(shadow_bf16), residual, reinterpret_cast<const UpdChunk*>(chunks),
      reinterpret_cast<const UpdSegment*>(segs), ht, grad_scale, zero_grads);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_cast_f32_bf16(const float* in, void* out, long long n, void* stream) {
  if (n <= 0) return 0;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  cast_f32_bf16_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(in, reinterpret_cast<__nv_bfloat16*>(out), n);
  return (int)cudaGetLastError();
}

// msg must hold 4 + capacity ints and msg[0] must be zero on entry (the call zeroes it on the stream).
DL4J_API int dl4j_threshold_encode(float* x, long long n, float tau, int* msg, int capacity, void* stream) {
  if (n <= 0 || n >= 2147483647LL) return -DL4J_ERR_BAD_ARG;
  cudaMemsetAsync(msg, 0, sizeof(int), (cudaStream_t)stream);
  long long tiles = (n + ENC_TILE - 1) / ENC_TILE;
  int grid = (int)(tiles < 148 * 8 ? tiles : 148 * 8);
  threshold_encode_kernel<<<grid, ENC_THREADS, 0, (cudaStream_t)stream>>>(x, n, tau, msg, capacity);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_threshold_decode(const int* msg, int capacity, float* target, long long n_target, float scale,
                                   int use_atomics, void* stream) {
  int dev = 0;
  cudaGetDevice(&dev);
  int grid = capacity / 256 + 1;
  if (grid > 148 * 8) grid = 148 * 8;
  threshold_decode_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(msg, capacity, target, n_target, scale, use_atomics,
                                                                  dl4j_status_word(dev));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_bitmap_encode(float* x, long long n, float tau, int* msg, void* stream) {
  if (n <= 0 || n >= 2147483647LL) return -DL4J_ERR_BAD_ARG;
  cudaMemsetAsync(msg, 0, sizeof(int), (cudaStream_t)stream);
  long long words = (n + 15) / 16;
  long long blocks = (words + 255) / 256;
  int grid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  bitmap_encode_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(x, n, tau, msg);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_bitmap_decode(const int* msg, float* target, long long n, float scale, void* stream) {
  long long words = (n + 15) / 16;
  long long blocks = (words + 255) / 256;
  int grid = (int)(blocks < 148 * 8 ? blocks : 148 * 8);
  if (grid < 1) grid = 1;
  bitmap_decode_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(msg, target, n, scale);
  return (int)cudaGetLastError();
}
