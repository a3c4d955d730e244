// Persistent LSTM sequence kernel: all time steps of one layer in a single cooperative launch.
//
// Math per step (DL4J gate order a|f|o|g along the 4n axis, libnd4j lstmLayer / LSTMHelpers.java):
//   z_t = zx_t + h_{t-1} RW          zx_t = x_t W + b is computed beforehand by one large GEMM
//   a = tanh(z_a)  f = sigm(z_f)  o = sigm(z_o)  g = sigm(z_g)
//   c_t = f * c_{t-1} + g * a        h_t = o * tanh(c_t)
//
// Work split: CTA j owns hidden units [16 j, 16 j + 16) and keeps their 64 recurrent weight rows
// (4 gates x 16 units, each row = n bf16 values) resident in shared memory for the whole sequence, so the
// recurrent weights are read from HBM once per launch instead of once per step.  Per step the CTA streams
// h_{t-1} ([mb, n] bf16, L2 resident) through a multi-stage TMA ring as the M operand of tcgen05.mma
// (M = 128 batch rows, zero filled beyond mb; N = 64 gate rows; K = n) issued by three warps that take every third
// k-block each (a single thread cannot issue MMAs fast enough for N this small), accumulates in TMEM, and its four
// epilogue warps (one thread per batch row) apply the cell non-linearities with c_t held in registers across
// steps, then publish their slice of h_t.  Steps are separated by a grid-wide arrive/wait on a global counter;
// every wait is bounded and reports through the status word.
#include "common.cuh"

namespace dl4j {

constexpr int LS_UNITS = 16;                 // hidden units per CTA
constexpr int LS_N = 4 * LS_UNITS;           // MMA N: gate rows per CTA
constexpr int LS_M = 128;                    // MMA M: batch rows (zero padded)
constexpr int LS_BK = 64;                    // K elements per stage (128 bytes, SWIZZLE_128B)
constexpr int LS_ISSUERS = 3;                // MMA-issuing warps.  One thread gets at most one tcgen05.mma into the pipe per ~150 clocks
                                             // whatever the instruction's shape (measured: 150 clk for N = 8 .. 256), while an
                                             // M 128 x N 64 x K 16 instruction occupies the tensor core for ~48 clocks and N = 16 for
                                             // less; three issuers, each with every third k-block, bring an N = 64 instruction down to ~50 clocks, and
                                             // with the producer warp and four epilogue warps the CTA stays at 256 threads (a ninth warp
                                             // would cut the register budget to 168 and spill the epilogue).
constexpr int LS_ACCS = LS_ISSUERS;          // one TMEM accumulator per issuer (MMAs of different threads never share one); the
                                             // epilogue sums them
constexpr int LS_TMEM_COLS = 256;            // allocation sizes are powers of two >= 32: LS_ACCS x LS_N = 192 columns used
static_assert(LS_ACCS * LS_N <= LS_TMEM_COLS, "forward accumulators exceed the TMEM allocation");
constexpr int LS_MAX_STAGES = 16;             // ring depth is chosen at launch from the shared memory left beside the weights
constexpr int LS_B_KB = LS_N * LS_BK * 2;    // 8 KB per k-block of resident weights
constexpr int LS_EPI_WARP0 = 1 + LS_ISSUERS; // warp 0 TMA, warps 1..3 MMA issuers, warps 4-7 epilogue
constexpr int LS_THREADS = 32 * (LS_EPI_WARP0 + 4);

struct LstmSeqParams {
  const __nv_bfloat16* zx;   // [T, mb, 4n]
  __nv_bfloat16* h_all;      // [T + 1, mb, n]; slot 0 holds h_0, step s writes slot s + 1
  const float* c0;           // [mb, n]
  float* cs;                 // [T, mb, n]  c_t (time index, not step index)
  __nv_bfloat16* gates;      // [T, mb, 4n] activated gates (for the backward pass)
  int T, mb, n, reverse;
  int stages, a_stage;       // TMA ring: number of stages and bytes per stage (batch rows rounded up to 8, x 128 B)
  unsigned int* counter;     // zero on entry
  int* status;
  long long* trace;          // optional [T][32] clock64 stamps written by the middle CTA (null = off); see dl4j_lstm_set_trace
};

// Named barrier over the four epilogue warps (barrier 0 is __syncthreads).
__device__ __forceinline__ void epilogue_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Acquire loads: once the target is seen, the other CTAs' stores that preceded their (fenced) arrivals are visible to this thread;
// no separate fence is needed after the wait.
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(unsigned int* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ bool wait_counter(const unsigned int* counter, unsigned int target, int* status) {
  if (ld_acquire_gpu(counter) >= target) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (ld_acquire_gpu(counter) < target) {
    if ((++spins & 0xff) == 0 && (clock64() - t0 > 4000000000LL || *((volatile int*)status) != 0)) {
      atomicCAS(status, 0, DL4J_ERR_TIMEOUT_PEER);
      return false;
    }
  }
  return true;
}

// Timeline of one CTA: slot `i` of step `s` receives this SM's clock.  Slots: 0 producer saw the step's grid barrier open,
// 1 producer issued the step's last load, 2..17 MMA thread saw k-block (slot - 2) land (first 16 k-blocks), 18 MMA thread
// committed the accumulator, 19 epilogue saw the accumulator, 20 after the TMEM loads, 21 after the global stores, 22 after the
// fences, 23 after the barrier arrive.
__device__ __forceinline__ void ls_stamp(long long* trace, int s, int slot) {
  if (trace != nullptr && blockIdx.x == gridDim.x / 2) trace[s * 32 + slot] = clock64();
}

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid(x) = 0.5 tanh(x / 2) + 0.5: one special-function instruction
__device__ __forceinline__ float sigm_fast(float x) { return fmaf(0.5f, tanh_fast(0.5f * x), 0.5f); }

__device__ __forceinline__ void unpack8(const uint4& u, float* o) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return u;
}

__global__ void __launch_bounds__(LS_THREADS, 1)
lstm_seq_fwd_kernel(const __grid_constant__ CUtensorMap tmap_h, const __grid_constant__ CUtensorMap tmap_w, const LstmSeqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int kblocks = p.n / LS_BK;
  uint8_t* w_smem = smem;                                   // kblocks x 8 KB, resident
  uint8_t* a_smem = w_smem + kblocks * LS_B_KB;             // ring of p.stages x p.a_stage bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(a_smem + p.stages * p.a_stage);
  uint64_t* full_bar = bars;                  // [LS_MAX_STAGES]
  uint64_t* empty_bar = bars + LS_MAX_STAGES;     // [LS_MAX_STAGES]
  uint64_t* w_full = bars + 2 * LS_MAX_STAGES;
  uint64_t* acc_full = w_full + 1;
  uint64_t* acc_empty = w_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_full + 3);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit0 = blockIdx.x * LS_UNITS;
  const unsigned int arrivals_per_step = gridDim.x;         // one arrive per CTA

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_h);
    prefetch_tmap(&tmap_w);
    for (int i = 0; i < p.stages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    mbar_init(w_full, 1);
    mbar_init(acc_full, (uint32_t)min(LS_ISSUERS, kblocks));      // one commit per issuer that has k-blocks
    mbar_init(acc_empty, 4);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, LS_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // resident weights: per k-block four boxes of 16 rows (one per gate) placed 2 KB apart
      mbar_expect_tx(w_full, (uint32_t)(kblocks * LS_B_KB));
      for (int kb = 0; kb < kblocks; ++kb)
#pragma unroll
        for (int g = 0; g < 4; ++g)
          tma_load_4d(w_smem + kb * LS_B_KB + g * (LS_UNITS * 128), &tmap_w, w_full, kb * LS_BK, g * p.n + unit0, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int s = 0; s < p.T && ok; ++s) {
        if (s > 0) {
          ok = wait_counter(p.counter, arrivals_per_step * (unsigned)s, p.status);   // every CTA published h of step s-1
          if (!ok) break;
          fence_proxy_async_all();       // generic-proxy stores of other CTAs -> async-proxy (TMA) reads below
        }
        ls_stamp(p.trace, s, 0);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], (uint32_t)p.a_stage);
          tma_load_4d(a_smem + stage * p.a_stage, &tmap_h, &full_bar[stage], kb * LS_BK, 0, s, 0);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        ls_stamp(p.trace, s, 1);
      }
    }
  } else if (warp < LS_EPI_WARP0) {
    const int me = warp - 1;                      // issuer index: k-blocks me, me + LS_ISSUERS, ... of every step
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 0, 0, LS_M, LS_N);
      const uint32_t acc = tmem_base + (uint32_t)(me * LS_N);
      bool ok = mbar_wait_bounded(w_full, 0, p.status, DL4J_ERR_TIMEOUT_MMA);
      tc_fence_after();
      for (int s = 0; s < p.T && ok; ++s) {
        if (!mbar_wait_bounded(acc_empty, (uint32_t)((s & 1) ^ 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        // Sequence position g of a k-block decides its issuer (g mod LS_ISSUERS) and its ring stage (g mod stages); the ring depth
        // is a multiple of LS_ISSUERS, so a stage always belongs to the same issuer, which therefore sees every phase of that
        // stage's barrier in order (a thread that skipped a phase could mistake the previous completion for the one it waits for).
        const int g0 = s * kblocks;
        const int kb_first = (me + LS_ISSUERS - g0 % LS_ISSUERS) % LS_ISSUERS;
        for (int kb = kb_first; kb < kblocks; kb += LS_ISSUERS) {
          const int g = g0 + kb;
          const int stage = g % p.stages;
          const uint32_t phase = (uint32_t)((g / p.stages) & 1);
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          if (kb < 16) ls_stamp(p.trace, s, 2 + kb);
          tc_fence_after();
          const uint64_t da = make_smem_desc_sw128(smem_u32(a_smem + stage * p.a_stage), 16, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_u32(w_smem + kb * LS_B_KB), 16, 1024);
#pragma unroll
          for (int k = 0; k < LS_BK / 16; ++k)
            umma_f16(acc, da + ((uint64_t)(k * 32) >> 4), db + ((uint64_t)(k * 32) >> 4), idesc, (kb > kb_first || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
        }
        if (ok && kb_first < kblocks) umma_commit(acc_full);
        if (me == 0) ls_stamp(p.trace, s, 18);
      }
    }
  } else {
    const int q = warp & 3;                       // TMEM lane quadrant of this warp
    const int b = q * 32 + lane;                  // batch row handled by this thread
    const bool row_ok = b < p.mb;
    const long n4 = 4L * p.n;
    float c[LS_UNITS];
#pragma unroll
    for (int u = 0; u < LS_UNITS; ++u) c[u] = 0.f;
    if (row_ok) {
      const float4* cp = reinterpret_cast<const float4*>(p.c0 + (long)b * p.n + unit0);
#pragma unroll
      for (int i = 0; i < LS_UNITS / 4; ++i) { const float4 v = cp[i]; c[4 * i] = v.x; c[4 * i + 1] = v.y; c[4 * i + 2] = v.z; c[4 * i + 3] = v.w; }
    }
    bool ok = true;
    for (int s = 0; s < p.T && ok; ++s) {
      const int t = p.reverse ? p.T - 1 - s : s;
      // input contribution of this step, fetched before the accumulator is ready
      uint4 zraw[8];
      if (row_ok) {
        const __nv_bfloat16* zrow = p.zx + ((long)t * p.mb + b) * n4 + unit0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4* src = reinterpret_cast<const uint4*>(zrow + (long)g * p.n);
          zraw[2 * g] = __ldg(src);
          zraw[2 * g + 1] = __ldg(src + 1);
        }
      }
      if (!mbar_wait_bounded(acc_full, (uint32_t)(s & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      if (threadIdx.x == 32 * LS_EPI_WARP0) ls_stamp(p.trace, s, 19);
      tc_fence_after();
      uint32_t r0[32], r1[32];
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll
      for (int i = 0; i < 32; ++i) { r0[i] = 0u; r1[i] = 0u; }
      const int g0m = (s * kblocks) % LS_ISSUERS;
#pragma unroll
      for (int j = 0; j < LS_ACCS; ++j) {          // fold the issuers' partial accumulators
        // issuer j wrote its accumulator in this step only if one of the step's k-blocks fell to it (always, once n >= 192)
        if ((j + LS_ISSUERS - g0m) % LS_ISSUERS >= kblocks) continue;
        uint32_t t0[32], t1[32];
        tmem_ld_32x32(taddr + j * LS_N, t0);
        tmem_ld_32x32(taddr + j * LS_N + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          r0[i] = __float_as_uint(__uint_as_float(r0[i]) + __uint_as_float(t0[i]));
          r1[i] = __float_as_uint(__uint_as_float(r1[i]) + __uint_as_float(t1[i]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);      // accumulator drained: the next step's MMAs may overwrite it
      if (threadIdx.x == 32 * LS_EPI_WARP0) ls_stamp(p.trace, s, 20);
      uint4 gp[8];                                 // activated gates, packed: stored after h_t has been published
      if (row_ok) {
        float za[16], zf[16], zo[16], zg[16];
        unpack8(zraw[0], za); unpack8(zraw[1], za + 8);
        unpack8(zraw[2], zf); unpack8(zraw[3], zf + 8);
        unpack8(zraw[4], zo); unpack8(zraw[5], zo + 8);
        unpack8(zraw[6], zg); unpack8(zraw[7], zg + 8);
        float h[16];
#pragma unroll
        for (int u = 0; u < LS_UNITS; ++u) {
          const float a = tanh_fast(za[u] + __uint_as_float(r0[u]));
          const float f = sigm_fast(zf[u] + __uint_as_float(r0[16 + u]));
          const float o = sigm_fast(zo[u] + __uint_as_float(r1[u]));
          const float g = sigm_fast(zg[u] + __uint_as_float(r1[16 + u]));
          c[u] = fmaf(f, c[u], g * a);
          h[u] = o * tanh_fast(c[u]);
          za[u] = a; zf[u] = f; zo[u] = o; zg[u] = g;
        }
        gp[0] = pack8(za); gp[1] = pack8(za + 8); gp[2] = pack8(zf); gp[3] = pack8(zf + 8);
        gp[4] = pack8(zo); gp[5] = pack8(zo + 8); gp[6] = pack8(zg); gp[7] = pack8(zg + 8);
        // h_t is what the other CTAs wait for: publish it first, then write what only the backward pass reads
        uint4* hd = reinterpret_cast<uint4*>(p.h_all + ((long)(s + 1) * p.mb + b) * p.n + unit0);
        hd[0] = pack8(h);
        hd[1] = pack8(h + 8);
      }
      if (threadIdx.x == 32 * LS_EPI_WARP0) ls_stamp(p.trace, s, 21);
      fence_proxy_async_all();
      epilogue_bar_sync();                         // every epilogue thread's stores precede the barrier; the one fence below is cumulative
      if (threadIdx.x == 32 * LS_EPI_WARP0) {
        ls_stamp(p.trace, s, 22);
        red_release_add(p.counter);                // one arrive per CTA; the release orders every epilogue thread's stores
                                                   // (they precede the barrier above) before the increment becomes visible
      }
      if (threadIdx.x == 32 * LS_EPI_WARP0) ls_stamp(p.trace, s, 23);
      if (row_ok) {
        __nv_bfloat16* grow = p.gates + ((long)t * p.mb + b) * n4 + unit0;
        uint4* gd;
        gd = reinterpret_cast<uint4*>(grow);               gd[0] = gp[0]; gd[1] = gp[1];
        gd = reinterpret_cast<uint4*>(grow + (long)p.n);     gd[0] = gp[2]; gd[1] = gp[3];
        gd = reinterpret_cast<uint4*>(grow + 2L * p.n);      gd[0] = gp[4]; gd[1] = gp[5];
        gd = reinterpret_cast<uint4*>(grow + 3L * p.n);      gd[0] = gp[6]; gd[1] = gp[7];
        float4* cd = reinterpret_cast<float4*>(p.cs + ((long)t * p.mb + b) * p.n + unit0);
#pragma unroll
        for (int i = 0; i < LS_UNITS / 4; ++i) cd[i] = make_float4(c[4 * i], c[4 * i + 1], c[4 * i + 2], c[4 * i + 3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, LS_TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------- backward
// Walks the steps in reverse inside one cooperative launch.  CTA j owns the same 16 hidden units as in the forward
// kernel and keeps RW[units, :] (16 rows x 4n gate columns, K-major) resident in shared memory.  Per step it forms
//   dh_s[:, units] = dout_t[:, units] + dz_{s+1} RW[units, :]^T        (tcgen05, M = 128 batch rows, N = 16, K = 4n)
// streaming dz_{s+1} ([mb, 4n] bf16, written by all CTAs in the previous step) through the TMA ring, then applies the
// cell gradient with dc carried in registers and publishes its 64 columns of dz_s.  One extra MMA round after step 0
// yields the gradient of the initial hidden state.
struct LstmSeqBwdParams {
  const __nv_bfloat16* dout;   // [T, mb, n]
  const __nv_bfloat16* gates;  // [T, mb, 4n]
  const float* cs;             // [T, mb, n]
  const float* c0;             // [mb, n]
  const float* dc_last;        // [mb, n] or null
  __nv_bfloat16* dzx;          // [T, mb, 4n]
  __nv_bfloat16* dh0;          // [mb, n] or null
  float* dc0;                  // [mb, n] or null
  int T, mb, n, reverse;
  int stages, a_stage;       // TMA ring: number of stages and bytes per stage (batch rows rounded up to 8, x 128 B)
  unsigned int* counter;
  int* status;
  long long* trace;
};

constexpr int LB_N = LS_UNITS;               // MMA N
constexpr int LB_B_KB = LB_N * LS_BK * 2;    // 2 KB of resident weights per k-block
static_assert(LS_ISSUERS >= 2 && LS_ISSUERS <= 4, "the backward epilogue folds two to four accumulators out of 64 TMEM columns");
constexpr int LB_TMEM_COLS = 64;           // LS_ACCS partial accumulators (one per issuer) of LB_N columns each

__global__ void __launch_bounds__(LS_THREADS, 1)
lstm_seq_bwd_kernel(const __grid_constant__ CUtensorMap tmap_dz, const __grid_constant__ CUtensorMap tmap_w, const LstmSeqBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int kblocks = 4 * p.n / LS_BK;
  uint8_t* w_smem = smem;
  uint8_t* a_smem = w_smem + kblocks * LB_B_KB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(a_smem + p.stages * p.a_stage);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + LS_MAX_STAGES;
  uint64_t* w_full = bars + 2 * LS_MAX_STAGES;
  uint64_t* acc_full = w_full + 1;
  uint64_t* acc_empty = w_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_full + 3);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit0 = blockIdx.x * LS_UNITS;
  const unsigned int arrivals_per_step = gridDim.x;
  const int rounds = p.T - 1 + (p.dh0 ? 1 : 0);     // MMA rounds: one per step except the last one in time, plus dh0

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_dz);
    prefetch_tmap(&tmap_w);
    for (int i = 0; i < p.stages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    mbar_init(w_full, 1);
    mbar_init(acc_full, LS_ISSUERS);             // 4n / 64 >= 4 k-blocks: every issuer has work in every round
    mbar_init(acc_empty, 4);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, LB_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(w_full, (uint32_t)(kblocks * LB_B_KB));
      for (int kb = 0; kb < kblocks; ++kb) tma_load_4d(w_smem + kb * LB_B_KB, &tmap_w, w_full, kb * LS_BK, unit0, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        const int s_src = p.T - 1 - r;                         // step whose dz feeds this round
        const int t_src = p.reverse ? p.T - 1 - s_src : s_src;
        ok = wait_counter(p.counter, arrivals_per_step * (unsigned)(r + 1), p.status);
        if (!ok) break;
        fence_proxy_async_all();
        ls_stamp(p.trace, r, 0);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], (uint32_t)p.a_stage);
          tma_load_4d(a_smem + stage * p.a_stage, &tmap_dz, &full_bar[stage], kb * LS_BK, 0, t_src, 0);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        ls_stamp(p.trace, r, 1);
      }
    }
  } else if (warp < LS_EPI_WARP0) {
    const int me = warp - 1;                      // issuer index: k-blocks me, me + LS_ISSUERS, ... of every round
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 0, 0, LS_M, LB_N);
      const uint32_t acc = tmem_base + (uint32_t)(me * LB_N);
      bool ok = mbar_wait_bounded(w_full, 0, p.status, DL4J_ERR_TIMEOUT_MMA);
      tc_fence_after();
      for (int r = 0; r < rounds && ok; ++r) {
        if (!mbar_wait_bounded(acc_empty, (uint32_t)((r & 1) ^ 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const int g0 = r * kblocks;                  // issuer and stage by sequence position, as in the forward kernel
        const int kb_first = (me + LS_ISSUERS - g0 % LS_ISSUERS) % LS_ISSUERS;
        for (int kb = kb_first; kb < kblocks; kb += LS_ISSUERS) {
          const int g = g0 + kb;
          const int stage = g % p.stages;
          const uint32_t phase = (uint32_t)((g / p.stages) & 1);
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          if (me == 0 && (kb & 3) == 0 && kb < 64) ls_stamp(p.trace, r, 2 + (kb >> 2));       // every fourth k-block
          tc_fence_after();
          const uint64_t da = make_smem_desc_sw128(smem_u32(a_smem + stage * p.a_stage), 16, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_u32(w_smem + kb * LB_B_KB), 16, 1024);
#pragma unroll
          for (int k = 0; k < LS_BK / 16; ++k)
            umma_f16(acc, da + ((uint64_t)(k * 32) >> 4), db + ((uint64_t)(k * 32) >> 4), idesc, (kb > kb_first || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
        }
        if (ok) umma_commit(acc_full);
        if (me == 0) ls_stamp(p.trace, r, 18);
      }
    }
  } else {
    const int q = warp & 3;
    const int b = q * 32 + lane;
    const bool row_ok = b < p.mb;
    const long n4 = 4L * p.n;
    float dc[LS_UNITS];
#pragma unroll
    for (int u = 0; u < LS_UNITS; ++u) dc[u] = 0.f;
    if (row_ok && p.dc_last) {
      const float4* cp = reinterpret_cast<const float4*>(p.dc_last + (long)b * p.n + unit0);
#pragma unroll
      for (int i = 0; i < LS_UNITS / 4; ++i) { const float4 v = cp[i]; dc[4 * i] = v.x; dc[4 * i + 1] = v.y; dc[4 * i + 2] = v.z; dc[4 * i + 3] = v.w; }
    }
    bool ok = true;
    for (int s = p.T - 1; s >= -1 && ok; --s) {
      if (s < 0 && !p.dh0) break;
      const int r = p.T - 2 - s;                     // MMA round that produced this step's recurrent gradient (none for s = T-1)
      const int t = p.reverse ? p.T - 1 - s : s;
      uint4 graw[8], draw[2];
      float ct[LS_UNITS], cp_[LS_UNITS];
      if (row_ok && s >= 0) {
        const __nv_bfloat16* grow = p.gates + ((long)t * p.mb + b) * n4 + unit0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4* src = reinterpret_cast<const uint4*>(grow + (long)g * p.n);
          graw[2 * g] = __ldg(src);
          graw[2 * g + 1] = __ldg(src + 1);
        }
        const uint4* dsrc = reinterpret_cast<const uint4*>(p.dout + ((long)t * p.mb + b) * p.n + unit0);
        draw[0] = __ldg(dsrc);
        draw[1] = __ldg(dsrc + 1);
        const float4* c4 = reinterpret_cast<const float4*>(p.cs + ((long)t * p.mb + b) * p.n + unit0);
        const int tp = p.reverse ? t + 1 : t - 1;
        const float4* p4 = reinterpret_cast<const float4*>((s > 0 ? p.cs + ((long)tp * p.mb + b) * p.n : p.c0 + (long)b * p.n) + unit0);
#pragma unroll
        for (int i = 0; i < LS_UNITS / 4; ++i) {
          const float4 v = __ldg(c4 + i), w = __ldg(p4 + i);
          ct[4 * i] = v.x; ct[4 * i + 1] = v.y; ct[4 * i + 2] = v.z; ct[4 * i + 3] = v.w;
          cp_[4 * i] = w.x; cp_[4 * i + 1] = w.y; cp_[4 * i + 2] = w.z; cp_[4 * i + 3] = w.w;
        }
      }
      uint32_t acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0u;
      if (r >= 0) {
        if (!mbar_wait_bounded(acc_full, (uint32_t)(r & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
        if (threadIdx.x == 32 * LS_EPI_WARP0) ls_stamp(p.trace, r, 19);
        tc_fence_after();
        uint32_t hi[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16), acc);
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + 32, hi);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < LS_UNITS; ++u) {         // fold the issuers' accumulators (columns u, 16 + u, 32 + u, 48 + u)
          float v = __uint_as_float(acc[u]) + __uint_as_float(acc[16 + u]);
          if (LS_ISSUERS > 2) v += __uint_as_float(hi[u]);
          if (LS_ISSUERS > 3) v += __uint_as_float(hi[16 + u]);
          acc[u] = __float_as_uint(v);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty);
      }
      if (s < 0) {
        if (row_ok) {
          float h[16];
#pragma unroll
          for (int u = 0; u < LS_UNITS; ++u) h[u] = __uint_as_float(acc[u]);
          uint4* hd = reinterpret_cast<uint4*>(p.dh0 + (long)b * p.n + unit0);
          hd[0] = pack8(h);
          hd[1] = pack8(h + 8);
        }
        break;
      }
      if (row_ok) {
        float ga[16], gf[16], go[16], gg[16], dh[16];
        unpack8(graw[0], ga); unpack8(graw[1], ga + 8);
        unpack8(graw[2], gf); unpack8(graw[3], gf + 8);
        unpack8(graw[4], go); unpack8(graw[5], go + 8);
        unpack8(graw[6], gg); unpack8(graw[7], gg + 8);
        unpack8(draw[0], dh); unpack8(draw[1], dh + 8);
#pragma unroll
        for (int u = 0; u < LS_UNITS; ++u) {
          const float a = ga[u], f = gf[u], o = go[u], g = gg[u];
          const float dhv = dh[u] + __uint_as_float(acc[u]);
          const float tc = tanh_fast(ct[u]);
          const float dcv = dc[u] + dhv * o * (1.f - tc * tc);
          ga[u] = dcv * g * (1.f - a * a);
          gf[u] = dcv * cp_[u] * f * (1.f - f);
          go[u] = dhv * tc * o * (1.f - o);
          gg[u] = dcv * a * g * (1.f - g);
          dc[u] = dcv * f;
        }
        __nv_bfloat16* drow = p.dzx + ((long)t * p.mb + b) * n4 + unit0;
        uint4* gd;
        gd = reinterpret_cast<uint4*>(drow);               gd[0] = pack8(ga); gd[1] = pack8(ga + 8);
        gd = reinterpret_cast<uint4*>(drow + (long)p.n);     gd[0] = pack8(gf); gd[1] = pack8(gf + 8);
        gd = reinterpret_cast<uint4*>(drow + 2L * p.n);      gd[0] = pack8(go); gd[1] = pack8(go + 8);
        gd = reinterpret_cast<uint4*>(drow + 3L * p.n);      gd[0] = pack8(gg); gd[1] = pack8(gg + 8);
      }
      if (threadIdx.x == 32 * LS_EPI_WARP0 && r >= 0) ls_stamp(p.trace, r, 21);
      fence_proxy_async_all();
      epilogue_bar_sync();
      if (threadIdx.x == 32 * LS_EPI_WARP0) {
        if (r >= 0) ls_stamp(p.trace, r, 22);
        red_release_add(p.counter);
      }
    }
    if (row_ok && p.dc0) {
      float4* cd = reinterpret_cast<float4*>(p.dc0 + (long)b * p.n + unit0);
#pragma unroll
      for (int i = 0; i < LS_UNITS / 4; ++i) cd[i] = make_float4(dc[4 * i], dc[4 * i + 1], dc[4 * i + 2], dc[4 * i + 3]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, LB_TMEM_COLS);
  }
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// release at cluster scope: the stores above are visible to the peer thread that observes this arrival with an acquire
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 0x3ff) == 0 && (clock64() - t0 > 4000000000LL || *((volatile int*)status) != 0)) {
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}
// shared memory of this CTA -> shared memory of a CTA of the cluster; the bytes are counted on that CTA's mbarrier
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_cluster), "r"(src_cta),
               "r"(bytes), "r"(bar_cluster)
               : "memory");
}
// every thread of every CTA of the cluster
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Cluster form of the backward kernel: the CS (2 or 4) CTAs of a cluster own 16 CS hidden units together and split the reduction
// over the 4n gate columns.  CTA `rank` keeps RW[16 CS units, its 1/CS of the columns] resident (the same 128 KB as 16 units x all
// columns), streams only its share of dz per step (the L2 -> SM stream is what bounds the single-CTA form) and issues N = 16 CS
// instructions.  Each CTA finishes 16 of the units: the other columns of its partial sums are staged in shared memory and copied
// into the owners' shared memory by bulk copies that complete on the owner's mbarrier (cp.async.bulk.shared::cluster), and it waits
// for the CS - 1 slices that the peers send to it.
template <int CS>
__global__ void __launch_bounds__(LS_THREADS, 1)
lstm_seq_bwd_cluster_kernel(const __grid_constant__ CUtensorMap tmap_dz, const __grid_constant__ CUtensorMap tmap_w, const LstmSeqBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int GN = CS * LS_UNITS;                 // MMA N: the cluster's units
  constexpr int G_B_KB = GN * LS_BK * 2;            // resident weights per k-block
  constexpr int G_TMEM = CS == 2 ? 128 : 256;       // LS_ISSUERS accumulators of GN columns, rounded up to a power of two
  static_assert(LS_ISSUERS * GN <= G_TMEM, "accumulators exceed the TMEM allocation");
  const int kblocks = 4 * p.n / LS_BK / CS;         // this CTA's share of the reduction
  const uint32_t rank = cluster_ctarank();
  const int rows_x = p.a_stage / 128;               // batch rows (rounded up to 8) that take part in the exchange
  const int kb_base = (int)rank * kblocks;
  uint8_t* w_smem = smem;
  uint8_t* a_smem = w_smem + kblocks * G_B_KB;
  float* xbuf = reinterpret_cast<float*>(a_smem + p.stages * p.a_stage);      // [2 parities][CS - 1 senders][rows_x][16]: the peers' partial sums
  float* sbuf = xbuf + 2 * (CS - 1) * rows_x * LS_UNITS;                       // [CS - 1 receivers][rows_x][16]: staging of what this CTA sends
  uint64_t* bars = reinterpret_cast<uint64_t*>(sbuf + (CS - 1) * rows_x * LS_UNITS);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + LS_MAX_STAGES;
  uint64_t* w_full = bars + 2 * LS_MAX_STAGES;
  uint64_t* acc_full = w_full + 1;
  uint64_t* acc_empty = w_full + 2;
  uint64_t* x_full = w_full + 3;               // [2]: the peers' slices have landed in xbuf[parity]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_full + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int unit0 = blockIdx.x * LS_UNITS;                 // the 16 units this CTA finishes
  const int grp_unit0 = (int)(blockIdx.x / CS) * CS * LS_UNITS;     // the cluster's units (MMA N)
  const unsigned int arrivals_per_step = gridDim.x;
  const int rounds = p.T - 1 + (p.dh0 ? 1 : 0);     // MMA rounds: one per step except the last one in time, plus dh0

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_dz);
    prefetch_tmap(&tmap_w);
    for (int i = 0; i < p.stages; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
    mbar_init(w_full, 1);
    mbar_init(acc_full, LS_ISSUERS);             // 4n / 64 >= 4 k-blocks: every issuer has work in every round
    mbar_init(acc_empty, 4);
    mbar_init(&x_full[0], 1);                    // one local arrive with the expected byte count per round
    mbar_init(&x_full[1], 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, G_TMEM);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                               // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(w_full, (uint32_t)(kblocks * G_B_KB));
      for (int kb = 0; kb < kblocks; ++kb) tma_load_4d(w_smem + kb * G_B_KB, &tmap_w, w_full, (kb_base + kb) * LS_BK, grp_unit0, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        const int s_src = p.T - 1 - r;                         // step whose dz feeds this round
        const int t_src = p.reverse ? p.T - 1 - s_src : s_src;
        ok = wait_counter(p.counter, arrivals_per_step * (unsigned)(r + 1), p.status);
        if (!ok) break;
        fence_proxy_async_all();
        ls_stamp(p.trace, r, 0);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], (uint32_t)p.a_stage);
          tma_load_4d(a_smem + stage * p.a_stage, &tmap_dz, &full_bar[stage], (kb_base + kb) * LS_BK, 0, t_src, 0);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        ls_stamp(p.trace, r, 1);
      }
    }
  } else if (warp < LS_EPI_WARP0) {
    const int me = warp - 1;                      // issuer index: k-blocks me, me + LS_ISSUERS, ... of every round
    if (lane == 0) {
      const uint32_t idesc = make_idesc(1, 0, 0, LS_M, GN);
      const uint32_t acc = tmem_base + (uint32_t)(me * GN);
      bool ok = mbar_wait_bounded(w_full, 0, p.status, DL4J_ERR_TIMEOUT_MMA);
      tc_fence_after();
      for (int r = 0; r < rounds && ok; ++r) {
        if (!mbar_wait_bounded(acc_empty, (uint32_t)((r & 1) ^ 1), p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const int g0 = r * kblocks;                  // issuer and stage by sequence position, as in the forward kernel
        const int kb_first = (me + LS_ISSUERS - g0 % LS_ISSUERS) % LS_ISSUERS;
        for (int kb = kb_first; kb < kblocks; kb += LS_ISSUERS) {
          const int g = g0 + kb;
          const int stage = g % p.stages;
          const uint32_t phase = (uint32_t)((g / p.stages) & 1);
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          if (me == 0 && (kb & 3) == 0 && kb < 64) ls_stamp(p.trace, r, 2 + (kb >> 2));       // every fourth k-block
          tc_fence_after();
          const uint64_t da = make_smem_desc_sw128(smem_u32(a_smem + stage * p.a_stage), 16, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_u32(w_smem + kb * G_B_KB), 16, 1024);
#pragma unroll
          for (int k = 0; k < LS_BK / 16; ++k)
            umma_f16(acc, da + ((uint64_t)(k * 32) >> 4), db + ((uint64_t)(k * 32) >> 4), idesc, (kb > kb_first || k > 0) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
        }
        if (ok) umma_commit(acc_full);
        if (me == 0) ls_stamp(p.trace, r, 18);
      }
    }
  } else {
    const int q = warp & 3;
    const int b = q * 32 + lane;
    const bool row_ok = b < p.mb;
    const long n4 = 4L * p.n;
    float dc[LS_UNITS];
#pragma unroll
    for (int u = 0; u < LS_UNITS; ++u) dc[u] = 0.f;
    if (row_ok && p.dc_last) {
      const float4* cp = reinterpret_cast<const float4*>(p.dc_last + (long)b * p.n + unit0);
#pragma unroll
      for (int i = 0; i < LS_UNITS / 4; ++i) { const float4 v = cp[i]; dc[4 * i] = v.x; dc[4 * i + 1] = v.y; dc[4 * i + 2] = v.z; dc[4 * i + 3] = v.w; }
    }
    bool ok = true;
    for (int s = p.T - 1; s >= -1 && ok; --s) {
      if (s < 0 && !p.dh0) break;
      const int r = p.T - 2 - s;                     // MMA round that produced this step's recurrent gradient (none for s = T-1)
      const int t = p.reverse ? p.T - 1 - s : s;
      uint4 graw[8], draw[2];
      float ct[LS_UNITS], cp_[LS_UNITS];
      if (row_ok && s >= 0) {
        const __nv_bfloat16* grow = p.gates + ((long)t * p.mb + b) * n4 + unit0;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint4* src = reinterpret_cast<const uint4*>(grow + (long)g * p.n);
          graw[2 * g] = __ldg(src);
          graw[2 * g + 1] = __ldg(src + 1);
        }
        const uint4* dsrc = reinterpret_cast<const uint4*>(p.dout + ((long)t * p.mb + b) * p.n + unit0);
        draw[0] = __ldg(dsrc);
        draw[1] = __ldg(dsrc + 1);
        const float4* c4 = reinterpret_cast<const float4*>(p.cs + ((long)t * p.mb + b) * p.n + unit0);
        const int tp = p.reverse ? t + 1 : t - 1;
        const float4* p4 = reinterpret_cast<const float4*>((s > 0 ? p.cs + ((long)tp * p.mb + b) * p.n : p.c0 + (long)b * p.n) + unit0);
#pragma unroll
        for (int i = 0; i < LS_UNITS / 4; ++i) {
          const float4 v = __ldg(c4 + i), w = __ldg(p4 + i);
          ct[4 * i] = v.x; ct[4 * i + 1] = v.y; ct[4 * i + 2] = v.z; ct[4 * i + 3] = v.w;
          cp_[4 * i] = w.x; cp_[4 * i + 1] = w.y; cp_[4 * i + 2] = w.z; cp_[4 * i + 3] = w.w;
        }
      }
      uint32_t acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = 0u;
      if (r >= 0) {
        if (threadIdx.x == 32 * LS_EPI_WARP0)        // this round's slices from the CS - 1 peers
          mbar_expect_tx(&x_full[r & 1], (uint32_t)((CS - 1) * rows_x * LS_UNITS * 4));
        if (!mbar_wait_bounded(acc_full, (uint32_t)(r & 1), p.status, DL4J_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
        if (threadIdx.x == 32 * LS_EPI_WARP0) ls_stamp(p.trace, r, 19);
        tc_fence_after();
        // Partial sums over this CTA's share of the gate columns for the cluster's units (one accumulator per issuer), 32 columns
        // at a time: the 16 columns of this CTA's own units stay in registers, the others are staged for their owners.
        const int par = r & 1;
        if (lane == 0) bulk_wait_read<0>();          // the previous round's copies have read the staging buffer
        __syncwarp();
        uint32_t keep[LS_UNITS];
#pragma unroll
        for (int i = 0; i < LS_UNITS; ++i) keep[i] = 0u;
#pragma unroll
        for (int half = 0; half < GN / 32; ++half) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + half * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 1; j < LS_ISSUERS; ++j) {
            uint32_t t2[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + j * GN + half * 32, t2);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(t2[i]));
          }
#pragma unroll
          for (int gg = 0; gg < 2; ++gg) {
            const int g = half * 2 + gg;             // 16-column group = rank of the CTA that finishes these units
            if (g == (int)rank) {
#pragma unroll
              for (int i = 0; i < LS_UNITS; ++i) keep[i] = v[16 * gg + i];
            } else if (b < rows_x) {
              const int d = (g - (int)rank + CS) % CS;                       // 1 .. CS - 1
              uint4* dst = reinterpret_cast<uint4*>(sbuf + ((size_t)(d - 1) * rows_x + b) * LS_UNITS);
#pragma unroll
              for (int j = 0; j < LS_UNITS / 4; ++j)
                dst[j] = make_uint4(v[16 * gg + 4 * j], v[16 * gg + 4 * j + 1], v[16 * gg + 4 * j + 2], v[16 * gg + 4 * j + 3]);
            }
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();                    // staging stores -> the bulk copies below
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(acc_empty);                    // accumulators drained: the next round's MMAs may start
          const int nrows = min(32, rows_x - q * 32);
          if (nrows > 0) {
#pragma unroll
            for (int d = 1; d < CS; ++d) {
              const uint32_t peer = (rank + (uint32_t)d) % CS;
              const int slot = CS - d - 1;           // at the receiver, slot j holds the slice of rank (receiver + j + 1) % CS
              const uint32_t src = smem_u32(sbuf + ((size_t)(d - 1) * rows_x + q * 32) * LS_UNITS);
              const uint32_t dst = mapa_cluster(smem_u32(xbuf + ((size_t)(par * (CS - 1) + slot) * rows_x + q * 32) * LS_UNITS), peer);
              bulk_copy_to_cluster(dst, src, (uint32_t)nrows * LS_UNITS * 4u, mapa_cluster(smem_u32(&x_full[par]), peer));
            }
            bulk_commit();
          }
        }
        if (!mbar_wait_bounded(&x_full[par], (uint32_t)((r >> 1) & 1), p.status, DL4J_ERR_TIMEOUT_PEER)) { ok = false; break; }
#pragma unroll
        for (int i = 0; i < LS_UNITS; ++i) acc[i] = keep[i];
        if (b < rows_x) {
#pragma unroll
          for (int sl = 0; sl < CS - 1; ++sl) {
            const float4* in = reinterpret_cast<const float4*>(xbuf + ((size_t)(par * (CS - 1) + sl) * rows_x + b) * LS_UNITS);
#pragma unroll
            for (int j = 0; j < LS_UNITS / 4; ++j) {
              const float4 x4 = in[j];
              acc[4 * j] = __float_as_uint(__uint_as_float(acc[4 * j]) + x4.x);
              acc[4 * j + 1] = __float_as_uint(__uint_as_float(acc[4 * j + 1]) + x4.y);
              acc[4 * j + 2] = __float_as_uint(__uint_as_float(acc[4 * j + 2]) + x4.z);
              acc[4 * j + 3] = __float_as_uint(__uint_as_float(acc[4 * j + 3]) + x4.w);
            }
          }
        }
      }
      if (s < 0) {
        if (row_ok) {
          float h[16];
#pragma unroll
          for (int u = 0; u < LS_UNITS; ++u) h[u] = __uint_as_float(acc[u]);
          uint4* hd = reinterpret_cast<uint4*>(p.dh0 + (long)b * p.n + unit0);
          hd[0] = pack8(h);
          hd[1] = pack8(h + 8);
        }
        break;
      }
      if (row_ok) {
        float ga[16], gf[16], go[16], gg[16], dh[16];
        unpack8(graw[0], ga); unpack8(graw[1], ga + 8);
        unpack8(graw[2], gf); unpack8(graw[3], gf + 8);
        unpack8(graw[4], go); unpack8(graw[5], go + 8);
        unpack8(graw[6], gg); unpack8(graw[7], gg + 8);
        unpack8(draw[0], dh); unpack8(draw[1], dh + 8);
#pragma unroll
        for (int u = 0; u < LS_UNITS; ++u) {
          const float a = ga[u], f = gf[u], o = go[u], g = gg[u];
          const float dhv = dh[u] + __uint_as_float(acc[u]);
          const float tc = tanh_fast(ct[u]);
          const float dcv = dc[u] + dhv * o * (1.f - tc * tc);
          ga[u] = dcv * g * (1.f - a * a);
          gf[u] = dcv * cp_[u] * f * (1.f - f);
          go[u] = dhv * tc * o * (1.f - o);
          gg[u] = dcv * a * g * (1.f - g);
          dc[u] = dcv * f;
        }
        __nv_bfloat16* drow = p.dzx + ((long)t * p.mb + b) * n4 + unit0;
        uint4* gd;
        gd = reinterpret_cast<uint4*>(drow);               gd[0] = pack8(ga); gd[1] = pack8(ga + 8);
        gd = reinterpret_cast<uint4*>(drow + (long)p.n);     gd[0] = pack8(gf); gd[1] = pack8(gf + 8);
        gd = reinterpret_cast<uint4*>(drow + 2L * p.n);      gd[0] = pack8(go); gd[1] = pack8(go + 8);
        gd = reinterpret_cast<uint4*>(drow + 3L * p.n);      gd[0] = pack8(gg); gd[1] = pack8(gg + 8);
      }
      if (threadIdx.x == 32 * LS_EPI_WARP0 && r >= 0) ls_stamp(p.trace, r, 21);
      fence_proxy_async_all();
      epilogue_bar_sync();
      if (threadIdx.x == 32 * LS_EPI_WARP0) {
        if (r >= 0) ls_stamp(p.trace, r, 22);
        red_release_add(p.counter);
      }
    }
    if (row_ok && p.dc0) {
      float4* cd = reinterpret_cast<float4*>(p.dc0 + (long)b * p.n + unit0);
#pragma unroll
      for (int i = 0; i < LS_UNITS / 4; ++i) cd[i] = make_float4(dc[4 * i], dc[4 * i + 1], dc[4 * i + 2], dc[4 * i + 3]);
    }
  }

  if (warp >= LS_EPI_WARP0 && lane == 0) bulk_wait<0>();     // this CTA's copies have completed before it may exit
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, G_TMEM);
  }
  cluster_sync_all();                               // neither CTA leaves while the other may still write into it
}

}  // namespace dl4j

using namespace dl4j;

// CTAs per cluster in the backward kernel: 4 unless DL4J_LSTM_CLUSTER says 1 (single-CTA form) or 2
static int lstm_cluster_size() {
  static const int cs = [] { const char* e = getenv("DL4J_LSTM_CLUSTER"); const int v = e ? atoi(e) : 4; return v >= 4 ? 4 : (v >= 2 ? 2 : 1); }();
  return cs;
}

// Device buffer of at least T x 32 int64 that the next launches' middle CTA fills with its timeline (null switches it off).
static long long* g_lstm_trace = nullptr;
DL4J_API void dl4j_lstm_set_trace(void* buf) { g_lstm_trace = reinterpret_cast<long long*>(buf); }

// Shared memory plan: resident weights, then as many ring stages as fit (stage = batch rows rounded up to 8 x 128 B: rows
// beyond the batch are never loaded, the MMA reads whatever those rows of the tile hold and their accumulator rows are
// ignored), then the barriers.  Returns the dynamic shared memory size, 0 when fewer than two stages fit.
static size_t ls_ring(size_t weight_bytes, int mb, int* a_rows, int* stages) {
  const int rows = (mb + 7) / 8 * 8;
  // the M = 128 MMA reads a full 16 KB tile from every stage base: keep that much allocated behind the last stage
  const size_t tail = (size_t)(LS_M - rows) * 128;
  const size_t stage = (size_t)rows * 128, limit = 227 * 1024, fixed = weight_bytes + 1024 + 512 + tail;
  if (fixed + 2 * stage > limit) return 0;
  size_t s = (limit - fixed) / stage;
  if (s > LS_MAX_STAGES) s = LS_MAX_STAGES;
  s -= s % LS_ISSUERS;                 // a stage must always fall to the same issuing warp (see the kernels)
  if (s < (size_t)LS_ISSUERS) return 0;
  *a_rows = rows;
  *stages = (int)s;
  return fixed + s * stage;
}

static int ls_encode(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t nb1, uint64_t row_stride_bytes,
                     uint64_t sb1_bytes, uint32_t box_inner, uint32_t box_outer) {
  dl4j_PFN_encodeTiled enc = dl4j_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[4] = {inner, outer, nb1, 1};
  cuuint64_t strides[3] = {row_stride_bytes, sb1_bytes, sb1_bytes * nb1};
  cuuint32_t box[4] = {box_inner, box_outer, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// zx [T, mb, 4n] bf16; rw [4n, n] bf16 (row g*n + j = recurrent weights into gate g of unit j); h_all [T+1, mb, n] bf16 with slot 0 = h_0;
// c0 [mb, n] fp32; cs [T, mb, n] fp32; gates [T, mb, 4n] bf16; counter: one unsigned int of device scratch.
// Limits: n % 64 == 0, n <= 1216 (weights resident in shared memory), n / 16 <= SM count, 1 <= mb <= 128.
DL4J_API int dl4j_lstm_seq_fwd(const void* zx, const void* rw, void* h_all, const float* c0, float* cs, void* gates, int T, int mb, int n,
                               int reverse, unsigned int* counter, void* stream_) {
  if (T < 1 || mb < 1 || mb > LS_M || n < 64 || n % 64 != 0) return -DL4J_ERR_BAD_ARG;
  const int kblocks = n / LS_BK;
  int a_rows, stages;
  const size_t smem = ls_ring((size_t)kblocks * LS_B_KB, mb, &a_rows, &stages);
  if (!smem) return -DL4J_ERR_BAD_ARG;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = n / LS_UNITS;
  if (grid > sms) return -DL4J_ERR_BAD_ARG;
  cudaStream_t stream = (cudaStream_t)stream_;
  CUtensorMap th, tw;
  int r = ls_encode(&th, h_all, (uint64_t)n, (uint64_t)mb, (uint64_t)T + 1, (uint64_t)n * 2, (uint64_t)mb * n * 2, LS_BK, (uint32_t)a_rows);
  if (r) return -1000 - r;
  r = ls_encode(&tw, rw, (uint64_t)n, (uint64_t)4 * n, 1, (uint64_t)n * 2, (uint64_t)4 * n * n * 2, LS_BK, LS_UNITS);
  if (r) return -1000 - r;
  LstmSeqParams p;
  p.zx = reinterpret_cast<const __nv_bfloat16*>(zx);
  p.h_all = reinterpret_cast<__nv_bfloat16*>(h_all);
  p.c0 = c0; p.cs = cs;
  p.gates = reinterpret_cast<__nv_bfloat16*>(gates);
  p.T = T; p.mb = mb; p.n = n; p.reverse = reverse;
  p.stages = stages; p.a_stage = a_rows * 128;
  p.counter = counter;
  p.status = dl4j_status_word(dev);
  p.trace = g_lstm_trace;
  cudaError_t e = cudaMemsetAsync(counter, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return (int)e;
  e = cudaFuncSetAttribute(lstm_seq_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  void* args[] = {(void*)&th, (void*)&tw, (void*)&p};
  e = cudaLaunchCooperativeKernel((void*)lstm_seq_fwd_kernel, dim3(grid), dim3(LS_THREADS), args, smem, stream);
  return (int)e;
}

// dout [T, mb, n] bf16; gates [T, mb, 4n] bf16; cs [T, mb, n] fp32; c0 [mb, n] fp32; rwt [n, 4n] bf16 row-major (row j = weights
// from unit j into every gate column); dzx [T, mb, 4n] bf16 out; dc_last / dh0 / dc0 optional.  Same limits as the forward entry.
// One attempt with `csz` CTAs per cluster (1 = the single-CTA form).  Returns 1 when this form cannot be set up for the problem
// (shape, shared memory), a CUDA error code when the launch itself was refused, 0 when the kernel is in the stream.
static int lstm_bwd_launch(int csz, const void* dout, const void* gates, const float* cs, const float* c0, const void* rwt, void* dzx,
                           const float* dc_last, void* dh0, float* dc0, int T, int mb, int n, int reverse, unsigned int* counter,
                           cudaStream_t stream) {
  const int kblocks = 4 * n / LS_BK;
  if (csz > 1 && !((n / LS_UNITS) % csz == 0 && kblocks % csz == 0 && kblocks / csz >= LS_ISSUERS)) return 1;   // every issuer needs a k-block per round
  int a_rows = 0, stages = 0;
  const int rows8 = (mb + 7) / 8 * 8;
  const size_t xchg_bytes = (size_t)3 * (csz - 1) * rows8 * LS_UNITS * sizeof(float);     // two receive parities + one staging buffer
  const size_t smem = csz > 1 ? ls_ring((size_t)(kblocks / csz) * (csz * LS_UNITS * LS_BK * 2) + xchg_bytes, mb, &a_rows, &stages)
                              : ls_ring((size_t)kblocks * LB_B_KB, mb, &a_rows, &stages);
  if (!smem) return 1;
  int dev = 0;
  cudaGetDevice(&dev);
  const int grid = n / LS_UNITS;
  CUtensorMap td, tw;
  int r = ls_encode(&td, dzx, (uint64_t)4 * n, (uint64_t)mb, (uint64_t)T, (uint64_t)4 * n * 2, (uint64_t)mb * 4 * n * 2, LS_BK, (uint32_t)a_rows);
  if (r) return -1000 - r;
  r = ls_encode(&tw, rwt, (uint64_t)4 * n, (uint64_t)n, 1, (uint64_t)4 * n * 2, (uint64_t)4 * n * n * 2, LS_BK, (uint32_t)(csz * LS_UNITS));
  if (r) return -1000 - r;
  LstmSeqBwdParams p;
  p.dout = reinterpret_cast<const __nv_bfloat16*>(dout);
  p.gates = reinterpret_cast<const __nv_bfloat16*>(gates);
  p.cs = cs; p.c0 = c0; p.dc_last = dc_last;
  p.dzx = reinterpret_cast<__nv_bfloat16*>(dzx);
  p.dh0 = reinterpret_cast<__nv_bfloat16*>(dh0);
  p.dc0 = dc0;
  p.T = T; p.mb = mb; p.n = n; p.reverse = reverse;
  p.stages = stages; p.a_stage = a_rows * 128;
  p.counter = counter;
  p.status = dl4j_status_word(dev);
  p.trace = g_lstm_trace;
  void* kern = csz == 4 ? (void*)lstm_seq_bwd_cluster_kernel<4> : csz == 2 ? (void*)lstm_seq_bwd_cluster_kernel<2> : (void*)lstm_seq_bwd_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(counter, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) return (int)e;
  void* args[] = {(void*)&td, (void*)&tw, (void*)&p};
  if (csz == 1) return (int)cudaLaunchCooperativeKernel(kern, dim3(grid), dim3(LS_THREADS), args, smem, stream);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(LS_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = (unsigned)csz; attrs[0].val.clusterDim.y = 1; attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeCooperative;
  attrs[1].val.cooperative = 1;
  cfg.attrs = attrs; cfg.numAttrs = 2;
  return (int)cudaLaunchKernelExC(&cfg, kern, args);
}

DL4J_API int dl4j_lstm_seq_bwd(const void* dout, const void* gates, const float* cs, const float* c0, const void* rwt, void* dzx,
                               const float* dc_last, void* dh0, float* dc0, int T, int mb, int n, int reverse, unsigned int* counter,
                               void* stream_) {
  if (T < 1 || mb < 1 || mb > LS_M || n < 64 || n % 64 != 0) return -DL4J_ERR_BAD_ARG;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (n / LS_UNITS > sms) return -DL4J_ERR_BAD_ARG;
  // Cluster form first (CS CTAs share 16 CS units and split the gate columns: the same resident bytes, 1 / CS of the L2 -> SM stream
  // per CTA); a form that does not fit the problem, or whose launch the driver refuses (a cooperative launch needs every cluster
  // resident at once, which a partly occupied device or a profiler may not grant), gives way to the next smaller one.
  int rc = 1;
  for (int csz = lstm_cluster_size(); csz >= 1; csz /= 2) {
    rc = lstm_bwd_launch(csz, dout, gates, cs, c0, rwt, dzx, dc_last, dh0, dc0, T, mb, n, reverse, counter, (cudaStream_t)stream_);
    if (rc == 0) return 0;
    if (rc < 0) return rc;                       // tensor-map encoding failed: not a matter of the form
    if (rc != 1) (void)cudaGetLastError();       // a refused launch leaves a (non-sticky) error behind
    if (csz == 1) break;
  }
  return rc == 1 ? -DL4J_ERR_BAD_ARG : rc;
}
