// Fused gradient-sharing kernels over NVLink / NVSwitch peer memory (one rank per GPU, up to 8 ranks).
//
// The reference's multi-GPU primitives are single-process kernels that dereference an array of per-device
// pointers (libnd4j/include/loops/cuda/specials/averagingKernel.cu:29-76, accumulateKernel.cu:38-70) plus the
// threshold/bitmap codec (loops/cuda/type_conversions.cu:215-500); the training-side logic that used them
// (parameter averaging, threshold-encoded gradient sharing) is rebuilt here as two persistent kernels:
//
//  * allreduce_update_kernel ("dense averaging"): reduce-scatter of the gradients by peer loads (or
//    multimem.ld_reduce through the switch) -> regularisation + updater + step on the owned slice ->
//    all-gather of the new parameters (fp32 master + bf16 shadow) by peer stores (or multimem.st), then the
//    local gradient buffer is cleared.  One launch per step instead of allreduce + updater + broadcast.
//  * threshold_share_kernel ("shared gradients"): updater on the local gradient, accumulate into the
//    residual, bitmap-encode the residual into this rank's message slot, exchange by peer loads, decode the
//    sum of every rank's message and apply it to the local parameters.
//
// Synchronisation: cross-GPU barriers are release/acquire flags in every rank's signal pad, grid-wide
// barriers are atomic counters in local scratch.  Every wait is bounded; on expiry the kernel records
// DL4J_ERR_TIMEOUT_PEER in the status word, skips the remaining phases and returns.
// No TMA is used here at all (and in particular no cluster-multicast load of peer memory).
#include <cooperative_groups.h>

#include "common.cuh"
#include "updater_math.cuh"

namespace dl4j {

constexpr int MAX_RANKS = 8;
constexpr int COMM_THREADS = 512;

struct CommCtx {
  int rank, world;
  float* grads[MAX_RANKS];
  float* params[MAX_RANKS];
  __nv_bfloat16* shadow[MAX_RANKS];
  uint32_t* signal[MAX_RANKS];     // per rank: [slots][MAX_RANKS] flags
  int* msg[MAX_RANKS];             // threshold sharing: per rank message slot
  float* mc_grads;                 // multicast (NVLS) addresses, null when unavailable
  float* mc_params;
  __nv_bfloat16* mc_shadow;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float ld_peer_f(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_peer_i(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st_b64(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)) : "memory");
}

// Cross-GPU barrier executed by block 0: thread t signals rank t and waits for rank t's signal.
// `epoch` must increase monotonically per slot.  Returns false (for the whole block) on timeout.
__device__ bool peer_barrier(const CommCtx& c, int slot, uint32_t epoch, int* status) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.signal[threadIdx.x] + slot * MAX_RANKS + c.rank, epoch);
    const uint32_t* mine = c.signal[c.rank] + slot * MAX_RANKS + threadIdx.x;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && (clock64() - t0 > 2000000000LL || *((volatile int*)status) != 0)) {
        atomicCAS(status, 0, DL4J_ERR_TIMEOUT_PEER);
        ok_flag = 0;
        break;
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// Grid-wide barrier on a monotonically increasing counter in local scratch (all blocks co-resident:
// cooperative launch).  `target` = gridDim.x * (number of barriers passed so far + 1).
__device__ bool grid_barrier(unsigned int* counter, unsigned int target, int* status) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    ok_flag = 1;
    __threadfence();
    atomicAdd(counter, 1u);
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (*((volatile unsigned int*)counter) < target) {
      if ((++spins & 0xff) == 0 && (clock64() - t0 > 4000000000LL || *((volatile int*)status) != 0)) {
        atomicCAS(status, 0, DL4J_ERR_TIMEOUT_PEER);
        ok_flag = 0;
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  return ok_flag != 0;
}

// One owned chunk of a dense-averaging step: sum of every rank's gradient (peer loads or one multimem.ld_reduce), the
// updater on the sum, and the new fp32 parameters written to every rank (peer stores or multimem.st) plus this rank's
// bf16 shadow.  Shared by the whole-buffer kernel and the per-bucket kernel.
__device__ __forceinline__ void reduce_update_chunk(const CommCtx& c, float* __restrict__ state, const UpdChunk* __restrict__ chunks,
                                                    const UpdSegment* __restrict__ segs, const UpdHyperTable& ht, float grad_scale,
                                                    int use_multimem, int ci) {
  float* my_params = c.params[c.rank];
  const int NT = (int)blockDim.x;
  const UpdChunk ch = chunks[ci];
  const UpdSegment sg = segs[ch.seg];
  const UpdHyper h = ht.h[sg.hyper];
  const long long rel0 = ch.offset - sg.block_start;
  float* st0 = state + sg.state_off + rel0;
  float* st1 = st0 + sg.block_numel;
  float* st2 = st1 + sg.block_numel;
  const long long sh0 = sg.shadow_off + (ch.offset - sg.offset);
  const int ns = upd_n_state(sg.kernel_id);
  __nv_bfloat16* my_shadow = c.shadow[c.rank];
  // gradients and parameters (peer or multicast accesses) need the 16-byte grid; the state slots sit block_numel elements apart
  // (DL4J's [m | v] layout) and are moved with four 4-byte accesses when they are off it
  const bool vec_ok = (ch.offset & 3) == 0;
  const bool a_al = (reinterpret_cast<uintptr_t>(st0) & 15) == 0, b_al = (reinterpret_cast<uintptr_t>(st1) & 15) == 0,
             c_al = (reinterpret_cast<uintptr_t>(st2) & 15) == 0;
  const bool sh_vec = ((sh0 & 3) == 0);
  const int nvec = vec_ok ? ch.count / 4 : 0;
  // two vectors per thread and iteration: every load of both (peer gradients, parameters, state) is issued
  // before the first use so that enough bytes are in flight to cover the NVLink round trip
  constexpr int U = 2;
  for (int v0 = threadIdx.x; v0 < nvec; v0 += NT * U) {
    float4 g[U], w[U], a4[U], b4[U], c4[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * NT;
      g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      w[u] = g[u]; a4[u] = g[u]; b4[u] = g[u]; c4[u] = g[u];
      if (v < nvec) {
        const long long i = ch.offset + 4LL * v;
        if (use_multimem) {
          g[u] = multimem_ld_reduce_f4(c.mc_grads + i);
        } else {
#pragma unroll
          for (int r = 0; r < MAX_RANKS; ++r) {
            if (r < c.world) {
              const float4 t = ld_peer_f4(c.grads[(c.rank + r) % c.world] + i);
              g[u].x += t.x; g[u].y += t.y; g[u].z += t.z; g[u].w += t.w;
            }
          }
        }
        w[u] = *reinterpret_cast<const float4*>(my_params + i);
        if (ns > 0) a4[u] = upd_ld4(st0 + 4 * v, a_al);
        if (ns > 1) b4[u] = upd_ld4(st1 + 4 * v, b_al);
        if (ns > 2) c4[u] = upd_ld4(st2 + 4 * v, c_al);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * NT;
      if (v >= nvec) continue;
      const long long i = ch.offset + 4LL * v;
      float wv[4] = {w[u].x, w[u].y, w[u].z, w[u].w}, gv[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
      if (sg.kernel_id != 9) {
        float sa[4] = {a4[u].x, a4[u].y, a4[u].z, a4[u].w}, sb[4] = {b4[u].x, b4[u].y, b4[u].z, b4[u].w},
              sc[4] = {c4[u].x, c4[u].y, c4[u].z, c4[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) wv[j] -= updater_step(sg, h, wv[j], gv[j] * grad_scale, sa + j, sb + j, sc + j);
        if (ns > 0) upd_st4(st0 + 4 * v, make_float4(sa[0], sa[1], sa[2], sa[3]), a_al);
        if (ns > 1) upd_st4(st1 + 4 * v, make_float4(sb[0], sb[1], sb[2], sb[3]), b_al);
        if (ns > 2) upd_st4(st2 + 4 * v, make_float4(sc[0], sc[1], sc[2], sc[3]), c_al);
      }
      const float4 wn = make_float4(wv[0], wv[1], wv[2], wv[3]);
      if (use_multimem) {
        multimem_st_f4(c.mc_params + i, wn);
      } else {
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < c.world) *reinterpret_cast<float4*>(c.params[(c.rank + r) % c.world] + i) = wn;
      }
      // only the fp32 master crosses the link; every rank derives its own bf16 shadow (here for the owned chunks,
      // in the last phase for the others)
      if (my_shadow) {
        __nv_bfloat16* sp = my_shadow + sh0 + 4LL * v;
        if (sh_vec) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(wv[0], wv[1]), hi = __floats2bfloat162_rn(wv[2], wv[3]);
          *reinterpret_cast<uint2*>(sp) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) sp[j] = __float2bfloat16(wv[j]);
        }
      }
    }
  }
  // scalar tail (and whole chunk when its offset is not 16-byte aligned)
  for (int e = nvec * 4 + threadIdx.x; e < ch.count; e += NT) {
    const long long i = ch.offset + e;
    float g = 0.f;
    for (int r = 0; r < c.world; ++r) g += ld_peer_f(c.grads[r] + i);
    float w = my_params[i];
    if (sg.kernel_id != 9) w -= updater_step(sg, h, w, g * grad_scale, st0 + e, st1 + e, st2 + e);
    for (int r = 0; r < c.world; ++r) c.params[r][i] = w;
    if (my_shadow) my_shadow[sh0 + e] = __float2bfloat16(w);
  }
    }

// ------------------------------------------------------------------------------------------------ K2
// scratch[0] = grid barrier counter (zeroed by the host before every launch)
__global__ void __launch_bounds__(COMM_THREADS)
allreduce_update_kernel(const CommCtx c, float* __restrict__ state, const UpdChunk* __restrict__ chunks, int n_chunks,
                        const UpdSegment* __restrict__ segs, const UpdHyperTable ht, float grad_scale, long long n_total,
                        uint32_t epoch, unsigned int* scratch, int use_multimem, int* status) {
  unsigned int bar = 0;
  bool ok = true;
  // ---- phase 0: every rank has finished writing its gradients
  if (blockIdx.x == 0) ok = peer_barrier(c, 0, epoch, status);
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok && *((volatile int*)status) == 0;

  if (ok) {
    // ---- phase 1: owned chunks: reduce -> updater -> broadcast
    const int c0 = (int)((long long)n_chunks * c.rank / c.world), c1 = (int)((long long)n_chunks * (c.rank + 1) / c.world);
    for (int ci = c0 + blockIdx.x; ci < c1; ci += gridDim.x) {
      reduce_update_chunk(c, state, chunks, segs, ht, grad_scale, use_multimem, ci);
    }
    __threadfence_system();
  }
  // ---- phase 2: all ranks have read my gradients and written my parameters
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok;
  if (blockIdx.x == 0 && ok) ok = peer_barrier(c, 1, epoch, status);
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok && *((volatile int*)status) == 0;
  // ---- phase 3: clear the local gradient buffer for the next backward pass
  if (ok) {
    float4* g4 = reinterpret_cast<float4*>(c.grads[c.rank]);
    const long long n4 = n_total / 4;
    for (long long i = blockIdx.x * (long long)COMM_THREADS + threadIdx.x; i < n4; i += (long long)gridDim.x * COMM_THREADS)
      g4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (blockIdx.x == 0)
      for (long long i = n4 * 4 + threadIdx.x; i < n_total; i += COMM_THREADS) c.grads[c.rank][i] = 0.f;
    // bf16 shadow of the chunks that other ranks own, from the fp32 values they stored here in phase 1
    __nv_bfloat16* my_shadow = c.shadow[c.rank];
    if (my_shadow) {
      const int c0 = (int)((long long)n_chunks * c.rank / c.world), c1 = (int)((long long)n_chunks * (c.rank + 1) / c.world);
      const float* my_params = c.params[c.rank];
      const int n_other = n_chunks - (c1 - c0);
      for (int k = blockIdx.x; k < n_other; k += gridDim.x) {
        const int ci = k < c0 ? k : k + (c1 - c0);
        const UpdChunk ch = chunks[ci];
        const UpdSegment sg = segs[ch.seg];
        const long long sh0 = sg.shadow_off + (ch.offset - sg.offset);
        const float* src = my_params + ch.offset;
        __nv_bfloat16* dst = my_shadow + sh0;
        const bool vec = ((ch.offset & 3) == 0) && ((sh0 & 3) == 0);
        const int nvec = vec ? ch.count / 4 : 0;
        for (int v = threadIdx.x; v < nvec; v += COMM_THREADS) {
          const float4 w = __ldcg(reinterpret_cast<const float4*>(src) + v);
          __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
          reinterpret_cast<uint2*>(dst)[v] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        }
        for (int e = nvec * 4 + threadIdx.x; e < ch.count; e += COMM_THREADS) dst[e] = __float2bfloat16(__ldcg(src + e));
      }
    }
  }
}


// ------------------------------------------------------------------------------------------------ parameter averaging
// ParallelWrapper's classic mode with averagingFrequency > 1: every rank trained on its own for k steps, now the replicas'
// parameters are replaced by their mean.  Rank r averages the r-th slice (sum of every replica's values by peer loads or one
// multimem.ld_reduce, times 1 / W) and writes it into every replica (peer stores or multimem.st); after the closing barrier each
// rank derives its own bf16 shadow from the fp32 values it now holds.
__global__ void __launch_bounds__(COMM_THREADS)
param_average_kernel(const CommCtx c, const UpdChunk* __restrict__ chunks, int n_chunks, const UpdSegment* __restrict__ segs,
                     long long n_total, uint32_t epoch, unsigned int* scratch, int use_multimem, int* status) {
  unsigned int bar = 0;
  bool ok = true;
  if (blockIdx.x == 0) ok = peer_barrier(c, 0, epoch, status);           // every replica's parameters are final
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok && *((volatile int*)status) == 0;
  if (ok) {
    const float inv = 1.f / (float)c.world;
    const long long n4 = n_total / 4;
    const long long lo = n4 * c.rank / c.world, hi = n4 * (c.rank + 1) / c.world;
    for (long long v = lo + blockIdx.x * (long long)COMM_THREADS + threadIdx.x; v < hi; v += (long long)gridDim.x * COMM_THREADS) {
      const long long i = 4 * v;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      if (use_multimem) {
        a = multimem_ld_reduce_f4(c.mc_params + i);
      } else {
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < c.world) {
            const float4 t = ld_peer_f4(c.params[(c.rank + r) % c.world] + i);
            a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
          }
      }
      a.x *= inv; a.y *= inv; a.z *= inv; a.w *= inv;
      if (use_multimem) {
        multimem_st_f4(c.mc_params + i, a);
      } else {
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r)
          if (r < c.world) *reinterpret_cast<float4*>(c.params[(c.rank + r) % c.world] + i) = a;
      }
    }
    if (c.rank == c.world - 1 && blockIdx.x == 0)                          // the tail that is not a multiple of four elements
      for (long long i = n4 * 4 + threadIdx.x; i < n_total; i += COMM_THREADS) {
        float a = 0.f;
        for (int r = 0; r < c.world; ++r) a += ld_peer_f(c.params[r] + i);
        a *= inv;
        for (int r = 0; r < c.world; ++r) c.params[r][i] = a;
      }
    __threadfence_system();
  }
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok;
  if (blockIdx.x == 0 && ok) ok = peer_barrier(c, 1, epoch, status);      // every replica holds every slice
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok && *((volatile int*)status) == 0;
  __nv_bfloat16* my_shadow = c.shadow[c.rank];
  if (ok && my_shadow) {
    const float* my_params = c.params[c.rank];
    for (int ci = blockIdx.x; ci < n_chunks; ci += gridDim.x) {
      const UpdChunk ch = chunks[ci];
      const UpdSegment sg = segs[ch.seg];
      const long long sh0 = sg.shadow_off + (ch.offset - sg.offset);
      for (int e = threadIdx.x; e < ch.count; e += COMM_THREADS) my_shadow[sh0 + e] = __float2bfloat16(__ldcg(my_params + ch.offset + e));
    }
  }
}


// ------------------------------------------------------------------------------------------------ K2, per bucket
// Dense averaging bucket by bucket, so that the exchange of the layers whose gradients are already final runs while
// the backward pass of the earlier layers is still computing (the reference steps only once the whole gradient is
// complete: deeplearning4j-nn/.../optimize/solvers/StochasticGradientDescent.java:47-57).
//
// One launch per bucket (a contiguous range of updater chunks) on a side stream, after an event that follows the last
// kernel writing into the bucket's gradients.  The grid is small (it shares the SMs with the backward GEMMs) and not
// cooperative: nothing in it waits for another CTA of the same launch -- every CTA polls the peers' "ready" flags
// itself, and the CTA that takes the last ticket publishes this rank's "done" flag.  The step count, the
// hyper-parameters and the flag epoch are read from device memory (written by the host before the step), so the
// launch can sit in a captured CUDA graph.  Gradient clearing and the bf16 shadow of the chunks that other ranks own
// are left to bucket_finish_kernel, which runs once after the last bucket.
// Signal-pad slots: 4 + 2 b = ready flag of bucket b, 5 + 2 b = done flag.
struct StepVars {            // device copy, refreshed by the host before every step
  UpdHyperTable ht;
  uint32_t epoch;
  float grad_scale;
};

__device__ __forceinline__ bool wait_peer_flags(const CommCtx& c, int slot, uint32_t epoch, int* status) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const uint32_t* mine = c.signal[c.rank] + slot * MAX_RANKS + threadIdx.x;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && (clock64() - t0 > 2000000000LL || *((volatile int*)status) != 0)) {
        atomicCAS(status, 0, DL4J_ERR_TIMEOUT_PEER);
        ok_flag = 0;
        break;
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// Block size of the per-bucket kernel.  Two forms were measured on BERT-base at 2 GPUs against the whole-buffer kernel after backward
// (16.7 ms per step): 512-thread CTAs (17.4 ms; they cannot share an SM with a GEMM CTA, whose 192 threads x 232 registers leave
// room for about 12 K registers, so they run between GEMM launches) and 128-thread CTAs that do fit next to a GEMM CTA (20.2 ms
// with 148 CTAs, 25.1 with 64, 34.3 with 32: with so few threads too few bytes are in flight to cover the NVLink round trip, and
// the exchange outlasts the backward pass).  The 512-thread form stays; the bucketed exchange stays off by default.
constexpr int BUCKET_THREADS = COMM_THREADS;

__global__ void __launch_bounds__(BUCKET_THREADS)
bucket_allreduce_update_kernel(const CommCtx c, float* __restrict__ state, const UpdChunk* __restrict__ chunks, int chunk0, int chunk1,
                               const UpdSegment* __restrict__ segs, const StepVars* __restrict__ vars, int bucket,
                               unsigned int* tickets, int use_multimem, int* status) {
  __shared__ UpdHyperTable ht;
  __shared__ unsigned int my_ticket;
  const uint32_t epoch = vars->epoch;
  const float grad_scale = vars->grad_scale;
  for (int i = threadIdx.x; i < (int)(sizeof(UpdHyperTable) / 4); i += BUCKET_THREADS)
    reinterpret_cast<float*>(&ht)[i] = reinterpret_cast<const float*>(&vars->ht)[i];
  const int slot_ready = 4 + 2 * bucket, slot_done = slot_ready + 1;
  // this rank's gradients of the bucket are final (the launch is ordered after the kernels that wrote them)
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.signal[threadIdx.x] + slot_ready * MAX_RANKS + c.rank, epoch);
  }
  bool ok = wait_peer_flags(c, slot_ready, epoch, status) && *((volatile int*)status) == 0;
  if (ok) {
    const int n = chunk1 - chunk0;
    const int c0 = chunk0 + (int)((long long)n * c.rank / c.world), c1 = chunk0 + (int)((long long)n * (c.rank + 1) / c.world);
    for (int ci = c0 + blockIdx.x; ci < c1; ci += gridDim.x) reduce_update_chunk(c, state, chunks, segs, ht, grad_scale, use_multimem, ci);
  }
  // the CTA that finishes last tells every peer that this rank has read their gradients and written their parameters
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) my_ticket = atomicAdd(&tickets[bucket], 1u);
  __syncthreads();
  if (my_ticket == gridDim.x - 1) {
    if (threadIdx.x == 0) tickets[bucket] = 0u;          // ready for the next step (launches of one bucket are stream-ordered)
    if (ok && threadIdx.x < c.world) {
      __threadfence_system();
      st_release_sys(c.signal[threadIdx.x] + slot_done * MAX_RANKS + c.rank, epoch);
    }
  }
}

// After the last bucket: waits until every peer has finished every bucket (their reads of this rank's gradients and their
// writes of the parameters they own), then clears the local gradients and derives the bf16 shadow of the chunks other ranks own.
__global__ void __launch_bounds__(COMM_THREADS)
bucket_finish_kernel(const CommCtx c, const UpdChunk* __restrict__ chunks, const UpdSegment* __restrict__ segs,
                     const int* __restrict__ bucket_chunk0, int n_buckets, const StepVars* __restrict__ vars, long long n_total,
                     int* status) {
  __shared__ int ok_flag;
  const uint32_t epoch = vars->epoch;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  for (int f = threadIdx.x; f < n_buckets * c.world; f += COMM_THREADS) {
    const int b = f / c.world, r = f - b * c.world;
    const uint32_t* flag = c.signal[c.rank] + (5 + 2 * b) * MAX_RANKS + r;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && (clock64() - t0 > 2000000000LL || *((volatile int*)status) != 0)) {
        atomicCAS(status, 0, DL4J_ERR_TIMEOUT_PEER);
        ok_flag = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!ok_flag || *((volatile int*)status) != 0) return;      // gradients stay as they are: the host drops them
  float4* g4 = reinterpret_cast<float4*>(c.grads[c.rank]);
  const long long n4 = n_total / 4;
  for (long long i = blockIdx.x * (long long)COMM_THREADS + threadIdx.x; i < n4; i += (long long)gridDim.x * COMM_THREADS)
    g4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (blockIdx.x == 0)
    for (long long i = n4 * 4 + threadIdx.x; i < n_total; i += COMM_THREADS) c.grads[c.rank][i] = 0.f;
  __nv_bfloat16* my_shadow = c.shadow[c.rank];
  if (!my_shadow) return;
  const float* my_params = c.params[c.rank];
  const int total_chunks = bucket_chunk0[n_buckets];
  for (int ci = blockIdx.x; ci < total_chunks; ci += gridDim.x) {
    // owner of chunk ci inside its bucket
    int b = 0;
    while (b + 1 < n_buckets && bucket_chunk0[b + 1] <= ci) ++b;
    const int k0 = bucket_chunk0[b], n = bucket_chunk0[b + 1] - k0;
    const int c0 = k0 + (int)((long long)n * c.rank / c.world), c1 = k0 + (int)((long long)n * (c.rank + 1) / c.world);
    if (ci >= c0 && ci < c1) continue;                     // own chunks got their shadow in the bucket kernel
    const UpdChunk ch = chunks[ci];
    const UpdSegment sg = segs[ch.seg];
    const long long sh0 = sg.shadow_off + (ch.offset - sg.offset);
    const float* src = my_params + ch.offset;
    __nv_bfloat16* dst = my_shadow + sh0;
    const bool vec = ((ch.offset & 3) == 0) && ((sh0 & 3) == 0);
    const int nvec = vec ? ch.count / 4 : 0;
    for (int v = threadIdx.x; v < nvec; v += COMM_THREADS) {
      const float4 w = __ldcg(reinterpret_cast<const float4*>(src) + v);
      __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
      reinterpret_cast<uint2*>(dst)[v] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
    for (int e = nvec * 4 + threadIdx.x; e < ch.count; e += COMM_THREADS) dst[e] = __float2bfloat16(__ldcg(src + e));
  }
}

// ------------------------------------------------------------------------------------------------ K1
// Threshold ("shared gradients") step in one launch.
//
// Message slot of a rank (int32, double-buffered by step parity):
//   [0] k = elements sent   [1] N   [2] bits(tau)   [3] form: 1 = bitmap, 0 = index list   [4] number of list segments
//   [5] capacity of one list segment   [6..63] unused   [64 .. 64 + segments) entries written per segment
//   payload at thr_payload(segments): bitmap = one word per 16 elements (bit b = |r| >= tau, bit b + 16 = negative; a negative
//   value in [tau/2, tau) sets only the sign bit and moves by tau/2 -- the reference's bitmap format,
//   libnd4j/include/loops/cuda/type_conversions.cu:380-500), or index list = one segment per updater chunk holding
//   +-(index + 1) for every |r| >= tau of that chunk (the reference's primary "flexible" form, type_conversions.cu:215-311,
//   without its global prefix scan: the segment of a chunk sits at the chunk's own word range, so it holds count / 16
//   entries, and the CTA working on the chunk appends through a shared-memory cursor; what does not fit stays in the
//   residual and goes out in a later step, as with the reference's encoding boundary).
// Phase 1 is a single sweep: updater on the local gradient, add into the residual, encode from registers, write the
// remainder back, clear the gradient.  Phase 2 sums every rank's message into the parameters and writes the bf16 shadow of what
// it touched in the same loop (bitmap messages: one word per thread, vector read-modify-write; list messages: atomics,
// then a pass over the same entries for the shadow).  The form is chosen by the host from the density of the previous step.
constexpr int THR_HEADER = 64;
__host__ __device__ __forceinline__ long long thr_payload(int segments) { return THR_HEADER + (segments + 63) / 64 * 64; }

struct EncodeOut {
  int* words;           // bitmap payload
  int* seg;             // this CTA's list segment
  int seg_cap;
  int form;             // 1 bitmap, 0 list
};

// Encodes one element held in a register; returns the 2-bit code (bit 0 magnitude, bit 1 sign) for the bitmap form.
__device__ __forceinline__ int encode_one(float& r, float tau, float half, int form, long long idx, const EncodeOut& eo, int* cursor,
                                          int& sent) {
  const float a = fabsf(r);
  if (a >= tau) {
    const bool neg = r < 0.f;
    if (form == 0) {
      const int pos = atomicAdd(cursor, 1);
      if (pos >= eo.seg_cap) return 0;                 // segment full: the value stays in the residual
      eo.seg[pos] = neg ? -(int)(idx + 1) : (int)(idx + 1);
    }
    r += neg ? tau : -tau;
    ++sent;
    return neg ? 3 : 1;
  }
  if (form == 1 && a >= half && r < 0.f) {
    r += half;
    ++sent;
    return 2;
  }
  return 0;
}

__device__ __forceinline__ int find_segment(const UpdSegment* __restrict__ segs, int n_segs, long long idx) {
  int lo = 0, hi = n_segs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (segs[mid].offset <= idx) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(COMM_THREADS)
threshold_share_kernel(const CommCtx c, float* __restrict__ state, float* __restrict__ residual,
                       const UpdChunk* __restrict__ chunks, int n_chunks, const UpdSegment* __restrict__ segs, int n_segs,
                       const UpdHyperTable ht, float grad_scale, float tau, long long n_total, uint32_t epoch,
                       unsigned int* scratch, int msg_parity, long long msg_stride_ints, int form, int* status) {
  __shared__ int cursor;            // entries appended to this CTA's list segment
  __shared__ int cta_sent;
  unsigned int bar = 0;
  bool ok = true;
  float* grads = c.grads[c.rank];
  float* params = c.params[c.rank];
  __nv_bfloat16* shadow = c.shadow[c.rank];
  int* my_msg = c.msg[c.rank] + (long long)msg_parity * msg_stride_ints;
  const int n_seg = n_chunks;
  const long long payload = thr_payload(n_seg);
  const float half = tau * 0.5f;
  EncodeOut eo;
  eo.words = my_msg + payload;
  eo.seg = eo.words;
  eo.seg_cap = 0;
  eo.form = form;
  if (threadIdx.x == 0) cta_sent = 0;
  const int lane = threadIdx.x & 31;

  // ---- phase 1: updater -> residual -> encode -> residual remainder, gradient cleared (one sweep)
  int sent = 0;
  for (int ci = blockIdx.x; ci < n_chunks; ci += gridDim.x) {
    const UpdChunk ch = chunks[ci];
    const UpdSegment sg = segs[ch.seg];
    const UpdHyper h = ht.h[sg.hyper];
    const long long rel0 = ch.offset - sg.block_start;
    float* st0 = state + sg.state_off + rel0;
    float* st1 = st0 + sg.block_numel;
    float* st2 = st1 + sg.block_numel;
    const int ns = upd_n_state(sg.kernel_id);
    const bool vec_ok = (ch.offset & 15) == 0;        // chunk starts on a word boundary; state slots off the 16-byte grid use 4-byte accesses
    const bool a_al = (reinterpret_cast<uintptr_t>(st0) & 15) == 0, b_al = (reinterpret_cast<uintptr_t>(st1) & 15) == 0,
               c_al = (reinterpret_cast<uintptr_t>(st2) & 15) == 0;
    const int nvec = vec_ok ? ch.count / 4 : 0;
    // this chunk's list segment: the words that lie wholly inside the chunk
    const long long seg0 = (ch.offset + 15) >> 4;
    eo.seg = eo.words + seg0;
    eo.seg_cap = (int)max(0LL, ((ch.offset + ch.count) >> 4) - seg0);
    __syncthreads();                                  // previous chunk's appends are done
    if (threadIdx.x == 0) cursor = 0;
    __syncthreads();
    // every load of a vector is issued before the first use
    constexpr int U = 1;      // (two vectors per thread cost a second resident CTA per SM: 117 registers, measured slower)
    for (int vb = (threadIdx.x & ~31); vb < nvec; vb += COMM_THREADS * U) {
      float4 g4[U], w4[U], r4[U], a4[U], b4[U], c4[U];
      bool valid[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = vb + u * COMM_THREADS + lane;
        valid[u] = v < nvec;
        g4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        w4[u] = g4[u]; r4[u] = g4[u]; a4[u] = g4[u]; b4[u] = g4[u]; c4[u] = g4[u];
        if (valid[u]) {
          const long long i = ch.offset + 4LL * v;
          g4[u] = *reinterpret_cast<const float4*>(grads + i);
          w4[u] = *reinterpret_cast<const float4*>(params + i);
          r4[u] = *reinterpret_cast<const float4*>(residual + i);
          if (sg.kernel_id != 9) {
            if (ns > 0) a4[u] = upd_ld4(st0 + 4 * v, a_al);
            if (ns > 1) b4[u] = upd_ld4(st1 + 4 * v, b_al);
            if (ns > 2) c4[u] = upd_ld4(st2 + 4 * v, c_al);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = vb + u * COMM_THREADS + lane;
        int part = 0;
        if (valid[u]) {
          const long long i = ch.offset + 4LL * v;
          float gv[4] = {g4[u].x, g4[u].y, g4[u].z, g4[u].w}, wv[4] = {w4[u].x, w4[u].y, w4[u].z, w4[u].w},
                rv[4] = {r4[u].x, r4[u].y, r4[u].z, r4[u].w};
          if (sg.kernel_id != 9) {
            float sa[4] = {a4[u].x, a4[u].y, a4[u].z, a4[u].w}, sb[4] = {b4[u].x, b4[u].y, b4[u].z, b4[u].w},
                  sc[4] = {c4[u].x, c4[u].y, c4[u].z, c4[u].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) rv[j] += updater_step(sg, h, wv[j], gv[j] * grad_scale, sa + j, sb + j, sc + j);
            if (ns > 0) upd_st4(st0 + 4 * v, make_float4(sa[0], sa[1], sa[2], sa[3]), a_al);
            if (ns > 1) upd_st4(st1 + 4 * v, make_float4(sb[0], sb[1], sb[2], sb[3]), b_al);
            if (ns > 2) upd_st4(st2 + 4 * v, make_float4(sc[0], sc[1], sc[2], sc[3]), c_al);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int code = encode_one(rv[j], tau, half, form, i + j, eo, &cursor, sent);
            part |= ((code & 1) << (4 * (lane & 3) + j)) | (((code >> 1) & 1) << (16 + 4 * (lane & 3) + j));
          }
          *reinterpret_cast<float4*>(residual + i) = make_float4(rv[0], rv[1], rv[2], rv[3]);
          *reinterpret_cast<float4*>(grads + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (form == 1 && vb + u * COMM_THREADS < nvec) {          // warp-uniform
          // four neighbouring lanes hold the four nibbles of one word
          part |= __shfl_xor_sync(0xffffffffu, part, 1);
          part |= __shfl_xor_sync(0xffffffffu, part, 2);
          if (valid[u] && (lane & 3) == 0) {
            const long long wi = (ch.offset + 4LL * v) >> 4;
            if (4 * (v + 4) <= ch.count) eo.words[wi] = part;            // whole word inside the chunk
            else if (part) atomicOr(eo.words + wi, part);                  // shared with the next chunk
          }
        }
      }
    }
    // scalar tail (and whole chunk when it is not aligned): bits go in with atomics (the payload was zeroed before the launch)
    for (int e = nvec * 4 + threadIdx.x; e < ch.count; e += COMM_THREADS) {
      const long long i = ch.offset + e;
      float r = residual[i];
      if (sg.kernel_id != 9) r += updater_step(sg, h, params[i], grads[i] * grad_scale, st0 + e, st1 + e, st2 + e);
      const int code = encode_one(r, tau, half, form, i, eo, &cursor, sent);
      if (form == 1 && code) atomicOr(eo.words + (i >> 4), ((code & 1) << (i & 15)) | (((code >> 1) & 1) << (16 + (i & 15))));
      residual[i] = r;
      grads[i] = 0.f;
    }
    __syncthreads();
    if (threadIdx.x == 0) my_msg[THR_HEADER + ci] = min(cursor, eo.seg_cap);
  }
  // element count of this CTA -> header
  for (int o = 16; o > 0; o >>= 1) sent += __shfl_xor_sync(0xffffffffu, sent, o);
  if (lane == 0 && sent) atomicAdd(&cta_sent, sent);
  __syncthreads();
  if (threadIdx.x == 0 && cta_sent) atomicAdd(reinterpret_cast<int*>(scratch) + 1, cta_sent);
  __threadfence_system();
  // ---- exchange: every rank's message is complete
  ok = grid_barrier(scratch, gridDim.x * (++bar), status);
  if (blockIdx.x == 0 && threadIdx.x == 0 && ok) {
    my_msg[0] = *((volatile int*)scratch + 1);
    my_msg[1] = (int)n_total; my_msg[2] = __float_as_int(tau); my_msg[3] = form; my_msg[4] = n_seg; my_msg[5] = 0;
    __threadfence_system();
  }
  if (blockIdx.x == 0 && ok) ok = peer_barrier(c, 2, epoch, status);
  ok = grid_barrier(scratch, gridDim.x * (++bar), status) && ok && *((volatile int*)status) == 0;
  if (!ok) return;

  // ---- phase 2a: bitmap messages, chunk by chunk (a word per thread; vector read-modify-write; shadow written in the same loop)
  __shared__ int peer_form[MAX_RANKS], peer_segs[MAX_RANKS];
  if (threadIdx.x < c.world) {
    const int* pm = c.msg[threadIdx.x] + (long long)msg_parity * msg_stride_ints;
    peer_form[threadIdx.x] = ld_peer_i(pm + 3);
    peer_segs[threadIdx.x] = ld_peer_i(pm + 4);
  }
  __syncthreads();
  bool any_bitmap = false, any_list = false;
  for (int r = 0; r < c.world; ++r) { any_bitmap |= peer_form[r] == 1; any_list |= peer_form[r] == 0; }
  if (any_bitmap) {
    for (int ci = blockIdx.x; ci < n_chunks; ci += gridDim.x) {
      const UpdChunk ch = chunks[ci];
      const UpdSegment sg = segs[ch.seg];
      const long long sh0 = sg.shadow_off + (ch.offset - sg.offset);
      const bool vec = ((ch.offset & 15) == 0);
      const int nvec = vec ? ch.count / 4 : 0;
      // A warp covers 128 consecutive float4 (32 message words) per iteration: lane L fetches word L of every bitmap peer -- one
      // full 128-byte request per peer, which is what keeps the NVLink loads efficient at eight ranks -- and the float4 with
      // index 32 j + L takes its nibble from the word held by lane 8 j + L / 4.
      const int n_iter = (nvec + 127) / 128;
      for (int itw = (threadIdx.x >> 5); itw < n_iter; itw += COMM_THREADS / 32) {
        const int v_base = itw * 128;
        const long long w_base = (ch.offset >> 4) + (v_base >> 2);
        int wr[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) {
          wr[r] = 0;
          if (r < c.world && peer_form[r] == 1 && v_base + 4 * lane < nvec)
            wr[r] = ld_peer_i(c.msg[r] + (long long)msg_parity * msg_stride_ints + thr_payload(peer_segs[r]) + w_base + lane);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int v = v_base + 32 * j + lane;
          const int src = 8 * j + (lane >> 2), sh = 4 * (lane & 3);
          float d[4] = {0.f, 0.f, 0.f, 0.f};
          int any = 0;
#pragma unroll
          for (int r = 0; r < MAX_RANKS; ++r) {
            if (r < c.world && peer_form[r] == 1) {          // uniform: the shuffle is executed by the whole warp
              const int w = __shfl_sync(0xffffffffu, wr[r], src);
              const int mag = (w >> sh) & 15, sgn = (w >> (16 + sh)) & 15;
              any |= mag | sgn;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const bool bit = mag & (1 << e), sign = sgn & (1 << e);
                if (bit) d[e] += sign ? -tau : tau;
                else if (sign) d[e] -= half;
              }
            }
          }
          if (!any || v >= nvec) continue;
          const long long i = ch.offset + 4LL * v;
          float4* pp = reinterpret_cast<float4*>(params + i);
          float4 pv = *pp;
          pv.x -= d[0]; pv.y -= d[1]; pv.z -= d[2]; pv.w -= d[3];
          *pp = pv;
          if (shadow) {
            __nv_bfloat16* sp = shadow + sh0 + 4LL * v;
            if ((reinterpret_cast<uintptr_t>(sp) & 7) == 0) {
              __nv_bfloat162 lo = __floats2bfloat162_rn(pv.x, pv.y), hi = __floats2bfloat162_rn(pv.z, pv.w);
              *reinterpret_cast<uint2*>(sp) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            } else {
              sp[0] = __float2bfloat16(pv.x); sp[1] = __float2bfloat16(pv.y); sp[2] = __float2bfloat16(pv.z); sp[3] = __float2bfloat16(pv.w);
            }
          }
        }
      }
      // scalar tail (and whole chunk when it does not start on a word boundary)
      for (int e = nvec * 4 + threadIdx.x; e < ch.count; e += COMM_THREADS) {
        const long long i = ch.offset + e;
        float dj = 0.f;
        for (int r = 0; r < c.world; ++r) {
          if (peer_form[r] != 1) continue;
          const int wr = ld_peer_i(c.msg[r] + (long long)msg_parity * msg_stride_ints + thr_payload(peer_segs[r]) + (i >> 4));
          const bool bit = wr & (1 << (i & 15)), sign = wr & (1 << ((i & 15) + 16));
          if (bit) dj += sign ? -tau : tau;
          else if (sign) dj -= half;
        }
        if (dj == 0.f) continue;
        const float nw = params[i] - dj;
        params[i] = nw;
        if (shadow) shadow[sh0 + e] = __float2bfloat16(nw);
      }
    }
  }
  if (!any_list) return;                       // uniform over the grid: every CTA read the same headers
  // ---- phase 2b: index-list messages, after the bitmap pass (both write the parameters).  One peer at a time in rank order with a
  // grid barrier in between: within one message an index occurs once, so plain read-modify-writes do, and every rank adds the
  // same terms in the same order -- the replicas stay bit-identical (atomics would add them in arrival order).
  for (int r = 0; r < c.world; ++r) {
    if (peer_form[r] != 0) continue;                 // uniform: every CTA read the same headers
    ok = grid_barrier(scratch, gridDim.x * (++bar), status);
    if (!ok) return;
    const int* pm = c.msg[r] + (long long)msg_parity * msg_stride_ints;
    const int* pl = pm + thr_payload(peer_segs[r]);
    for (int sgm = blockIdx.x; sgm < min(peer_segs[r], n_chunks); sgm += gridDim.x) {
      const long long seg0 = (chunks[sgm].offset + 15) >> 4;
      const int cnt = ld_peer_i(pm + THR_HEADER + sgm);
      for (int e = threadIdx.x; e < cnt; e += COMM_THREADS) {
        const int code = ld_peer_i(pl + seg0 + e);
        const long long idx = (code < 0 ? -code : code) - 1;
        if (idx >= 0 && idx < n_total) params[idx] += code < 0 ? tau : -tau;
      }
    }
  }
  if (!shadow) return;
  // ---- phase 2c: shadow of the touched elements from the final parameter values
  ok = grid_barrier(scratch, gridDim.x * (++bar), status);
  if (!ok) return;
  for (int r = 0; r < c.world; ++r) {
    if (peer_form[r] != 0) continue;
    const int* pm = c.msg[r] + (long long)msg_parity * msg_stride_ints;
    const int* pl = pm + thr_payload(peer_segs[r]);
    for (int sgm = blockIdx.x; sgm < min(peer_segs[r], n_chunks); sgm += gridDim.x) {
      const long long seg0 = (chunks[sgm].offset + 15) >> 4;
      const int cnt = ld_peer_i(pm + THR_HEADER + sgm);
      for (int e = threadIdx.x; e < cnt; e += COMM_THREADS) {
        const int code = ld_peer_i(pl + seg0 + e);
        const long long idx = (code < 0 ? -code : code) - 1;
        if (idx < 0 || idx >= n_total) continue;
        const UpdSegment sg = segs[find_segment(segs, n_segs, idx)];
        shadow[sg.shadow_off + (idx - sg.offset)] = __float2bfloat16(__ldcg(params + idx));
      }
    }
  }
}

// Refreshes the bf16 shadow from the fp32 parameters following the segment table (used after a
// threshold-sharing step, whose decode works on flat indices).
__global__ void shadow_refresh_kernel(const float* __restrict__ params, __nv_bfloat16* __restrict__ shadow,
                                      const UpdChunk* __restrict__ chunks, const UpdSegment* __restrict__ segs) {
  const UpdChunk ch = chunks[blockIdx.x];
  const UpdSegment sg = segs[ch.seg];
  const long long sh0 = sg.shadow_off + (ch.offset - sg.offset);
  for (int e = threadIdx.x; e < ch.count; e += blockDim.x) shadow[sh0 + e] = __float2bfloat16(params[ch.offset + e]);
}

}  // namespace dl4j

using namespace dl4j;

struct HostCommArgs {      // mirrors the ctypes structure built in parallel/fused.py
  int rank, world;
  void* grads[MAX_RANKS];
  void* params[MAX_RANKS];
  void* shadow[MAX_RANKS];
  void* signal[MAX_RANKS];
  void* msg[MAX_RANKS];
  void* mc_grads;
  void* mc_params;
  void* mc_shadow;
};

static CommCtx make_ctx(const HostCommArgs* a) {
  CommCtx c;
  c.rank = a->rank; c.world = a->world;
  for (int i = 0; i < MAX_RANKS; ++i) {
    c.grads[i] = (float*)a->grads[i]; c.params[i] = (float*)a->params[i]; c.shadow[i] = (__nv_bfloat16*)a->shadow[i];
    c.signal[i] = (uint32_t*)a->signal[i]; c.msg[i] = (int*)a->msg[i];
  }
  c.mc_grads = (float*)a->mc_grads; c.mc_params = (float*)a->mc_params; c.mc_shadow = (__nv_bfloat16*)a->mc_shadow;
  return c;
}

template <typename K>
static int coop_grid(K kernel, int threads) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1) return 0;
  if (per_sm > 2) per_sm = 2;
  return sms * per_sm;
}

DL4J_API int dl4j_allreduce_update(const void* comm_args, float* state, const void* chunks, int n_chunks, const void* segs,
                                   const float* hyper, int n_hyper, float grad_scale, long long n_total, unsigned int epoch,
                                   void* scratch, int use_multimem, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const HostCommArgs* a = reinterpret_cast<const HostCommArgs*>(comm_args);
  if (a->world < 1 || a->world > MAX_RANKS || n_hyper > UPD_MAX_HYPER) return -DL4J_ERR_BAD_ARG;
  if (use_multimem && (!a->mc_grads || !a->mc_params)) return -DL4J_ERR_BAD_ARG;
  CommCtx c = make_ctx(a);
  UpdHyperTable ht;
  memset(&ht, 0, sizeof(ht));
  memcpy(&ht, hyper, sizeof(UpdHyper) * n_hyper);
  int dev = 0;
  cudaGetDevice(&dev);
  int* status = dl4j_status_word(dev);
  const int grid = coop_grid(allreduce_update_kernel, COMM_THREADS);
  if (grid < 1) return -DL4J_ERR_BAD_ARG;
  cudaMemsetAsync(scratch, 0, 16, stream);
  const UpdChunk* ch = reinterpret_cast<const UpdChunk*>(chunks);
  const UpdSegment* sg = reinterpret_cast<const UpdSegment*>(segs);
  unsigned int* sc = reinterpret_cast<unsigned int*>(scratch);
  void* args[] = {(void*)&c, (void*)&state, (void*)&ch, (void*)&n_chunks, (void*)&sg, (void*)&ht, (void*)&grad_scale,
                  (void*)&n_total, (void*)&epoch, (void*)&sc, (void*)&use_multimem, (void*)&status};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)allreduce_update_kernel, dim3(grid), dim3(COMM_THREADS), args, 0, stream);
  return (int)e;
}


// Mean of the replicas' parameters written into every replica (+ this rank's bf16 shadow); cooperative launch, bounded waits.
DL4J_API int dl4j_param_average(const void* comm_args, const void* chunks, int n_chunks, const void* segs, long long n_total,
                                unsigned int epoch, void* scratch, int use_multimem, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const HostCommArgs* a = reinterpret_cast<const HostCommArgs*>(comm_args);
  if (a->world < 1 || a->world > MAX_RANKS || n_total < 0) return -DL4J_ERR_BAD_ARG;
  if (use_multimem && !a->mc_params) return -DL4J_ERR_BAD_ARG;
  CommCtx c = make_ctx(a);
  int dev = 0;
  cudaGetDevice(&dev);
  int* status = dl4j_status_word(dev);
  const int grid = coop_grid(param_average_kernel, COMM_THREADS);
  if (grid < 1) return -DL4J_ERR_BAD_ARG;
  cudaMemsetAsync(scratch, 0, 16, stream);
  const UpdChunk* ch = reinterpret_cast<const UpdChunk*>(chunks);
  const UpdSegment* sg = reinterpret_cast<const UpdSegment*>(segs);
  unsigned int* sc = reinterpret_cast<unsigned int*>(scratch);
  void* args[] = {(void*)&c, (void*)&ch, (void*)&n_chunks, (void*)&sg, (void*)&n_total, (void*)&epoch, (void*)&sc, (void*)&use_multimem,
                  (void*)&status};
  return (int)cudaLaunchCooperativeKernel((void*)param_average_kernel, dim3(grid), dim3(COMM_THREADS), args, 0, stream);
}


// Per-bucket dense averaging (see bucket_allreduce_update_kernel).  `vars` is the device StepVars block, `tickets` a zeroed
// device array of one counter per bucket; `grid` CTAs (small: the launch shares the SMs with the backward pass).
DL4J_API int dl4j_bucket_allreduce_update(const void* comm_args, float* state, const void* chunks, int chunk0, int chunk1,
                                          const void* segs, const void* vars, int bucket, void* tickets, int use_multimem,
                                          int grid, void* stream_) {
  const HostCommArgs* a = reinterpret_cast<const HostCommArgs*>(comm_args);
  if (a->world < 1 || a->world > MAX_RANKS || bucket < 0 || bucket >= 64 || chunk1 < chunk0 || grid < 1) return -DL4J_ERR_BAD_ARG;
  if (use_multimem && (!a->mc_grads || !a->mc_params)) return -DL4J_ERR_BAD_ARG;
  CommCtx c = make_ctx(a);
  int dev = 0;
  cudaGetDevice(&dev);
  bucket_allreduce_update_kernel<<<grid, BUCKET_THREADS, 0, (cudaStream_t)stream_>>>(
      c, state, reinterpret_cast<const UpdChunk*>(chunks), chunk0, chunk1, reinterpret_cast<const UpdSegment*>(segs),
      reinterpret_cast<const StepVars*>(vars), bucket, reinterpret_cast<unsigned int*>(tickets), use_multimem, dl4j_status_word(dev));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_bucket_finish(const void* comm_args, const void* chunks, const void* segs, const int* bucket_chunk0, int n_buckets,
                                const void* vars, long long n_total, void* stream_) {
  const HostCommArgs* a = reinterpret_cast<const HostCommArgs*>(comm_args);
  if (a->world < 1 || a->world > MAX_RANKS || n_buckets < 1 || n_buckets > 64) return -DL4J_ERR_BAD_ARG;
  CommCtx c = make_ctx(a);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  bucket_finish_kernel<<<sms * 2, COMM_THREADS, 0, (cudaStream_t)stream_>>>(
      c, reinterpret_cast<const UpdChunk*>(chunks), reinterpret_cast<const UpdSegment*>(segs), bucket_chunk0, n_buckets,
      reinterpret_cast<const StepVars*>(vars), n_total, dl4j_status_word(dev));
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_step_vars_bytes() { return (int)sizeof(StepVars); }

DL4J_API int dl4j_threshold_share(const void* comm_args, float* state, float* residual, const void* chunks, int n_chunks,
                                  const void* segs, int n_segs, const float* hyper, int n_hyper, float grad_scale, float tau,
                                  long long n_total, unsigned int epoch, void* scratch, int msg_parity,
                                  long long msg_stride_ints, int form, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const HostCommArgs* a = reinterpret_cast<const HostCommArgs*>(comm_args);
  if (a->world < 1 || a->world > MAX_RANKS || n_hyper > UPD_MAX_HYPER || n_total >= 2147483647LL || n_segs < 1) return -DL4J_ERR_BAD_ARG;
  CommCtx c = make_ctx(a);
  UpdHyperTable ht;
  memset(&ht, 0, sizeof(ht));
  memcpy(&ht, hyper, sizeof(UpdHyper) * n_hyper);
  int dev = 0;
  cudaGetDevice(&dev);
  int* status = dl4j_status_word(dev);
  const int grid = coop_grid(threshold_share_kernel, COMM_THREADS);
  if (grid < 1) return -DL4J_ERR_BAD_ARG;
  const long long words = (n_total + 15) / 16;
  if (thr_payload(n_chunks) + words > msg_stride_ints) return -DL4J_ERR_BAD_ARG;
  cudaMemsetAsync(scratch, 0, 16, stream);
  // bitmap bits of chunk edges and unaligned chunks are OR-ed in: this step's payload starts from zero
  if (form == 1)
    cudaMemsetAsync(reinterpret_cast<int*>(a->msg[a->rank]) + (long long)msg_parity * msg_stride_ints + thr_payload(n_chunks), 0,
                    (size_t)words * 4, stream);
  const UpdChunk* ch = reinterpret_cast<const UpdChunk*>(chunks);
  const UpdSegment* sg = reinterpret_cast<const UpdSegment*>(segs);
  unsigned int* sc = reinterpret_cast<unsigned int*>(scratch);
  void* args[] = {(void*)&c, (void*)&state, (void*)&residual, (void*)&ch, (void*)&n_chunks, (void*)&sg, (void*)&n_segs, (void*)&ht,
                  (void*)&grad_scale, (void*)&tau, (void*)&n_total, (void*)&epoch, (void*)&sc, (void*)&msg_parity,
                  (void*)&msg_stride_ints, (void*)&form, (void*)&status};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)threshold_share_kernel, dim3(grid), dim3(COMM_THREADS), args, 0, stream);
  return (int)e;
}

// Ints a message slot must hold for a buffer of n_total elements (header + segment table + payload), for any grid this library uses.
DL4J_API long long dl4j_threshold_msg_ints(long long n_total, int n_chunks) { return thr_payload(n_chunks) + (n_total + 15) / 16 + 64; }

DL4J_API int dl4j_shadow_refresh(const float* params, void* shadow, const void* chunks, int n_chunks, const void* segs, void* stream) {
  if (n_chunks <= 0) return 0;
  shadow_refresh_kernel<<<n_chunks, 256, 0, (cudaStream_t)stream>>>(params, reinterpret_cast<__nv_bfloat16*>(shadow),
                                                                    reinterpret_cast<const UpdChunk*>(chunks),
                                                                    reinterpret_cast<const UpdSegment*>(segs));
  return (int)cudaGetLastError();
}
