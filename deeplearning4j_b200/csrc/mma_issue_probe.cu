// Issue-rate probe for tcgen05.mma (cta_group::1, bf16, K = 16): one CTA, operands fixed in shared memory, `issuers` warps
// each issuing `iters` instructions into accumulators of their own.  Reports the clocks one issuer spent per instruction.
//
// What it measures on a B200: a single thread completes one instruction per ~150 clocks whatever the shape (M 64 / 128,
// N 8 .. 256), while two issuers reach ~127 clocks per M 128 x N 256 instruction each (the tensor core's own rate), four reach
// 64 at N 128 and 48 at N 64.  Kernels whose instructions are small (the persistent LSTM: N = 64 forward, N = 16 backward)
// therefore spread the issue over several warps.
#include "common.cuh"

namespace dl4j {

constexpr int PROBE_A_BYTES = 32768, PROBE_B_BYTES = 65536;

__global__ void __launch_bounds__(128, 1) mma_issue_probe_kernel(long long* out, int M, int N, int iters, int accs, int issuers, int mn_major) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // K-major: A = 128 rows x 128 B, B = 256 rows x 128 B (one SWIZZLE_128B k-block each).  MN-major: 64-element column groups
  // 16 KB apart (A two, B up to four), 16 reduction rows = 2 KB per instruction.
  uint8_t* a_s = smem;
  uint8_t* b_s = smem + PROBE_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PROBE_A_BYTES + PROBE_B_BYTES);
  uint32_t* slot = reinterpret_cast<uint32_t*>(bars + 4);
  for (int i = threadIdx.x; i < (PROBE_A_BYTES + PROBE_B_BYTES) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(bars + i, 1);
    mbar_fence_init();
  }
  if (threadIdx.x < 32) { tmem_alloc(slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot;
  const int w = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0 && w < issuers) {
    const uint32_t idesc = make_idesc(1, mn_major, mn_major, M, N);
    const uint64_t da = make_smem_desc_sw128(smem_u32(a_s), mn_major ? 16384 : 16, 1024);
    const uint64_t db = make_smem_desc_sw128(smem_u32(b_s), mn_major ? 16384 : 16, 1024);
    const uint64_t kstep = (uint64_t)((mn_major ? 2048 : 32) >> 4);
    for (int rep = 0; rep < 3; ++rep) {            // the last repetition is reported
      const long long t0 = clock64();
      for (int i = 0; i < iters; ++i) {
        const int k = i & 3;
        umma_f16(tmem + (uint32_t)((w * accs + i % accs) * N), da + k * kstep, db + k * kstep, idesc,
                 i >= accs ? 1u : 0u);
      }
      const long long t1 = clock64();
      umma_commit(bars + w);
      const bool ok = mbar_wait_bounded(bars + w, (uint32_t)(rep & 1), nullptr, 0);
      const long long t2 = clock64();
      if (w == 0) { out[0] = t1 - t0; out[1] = ok ? t2 - t0 : -1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace dl4j

using namespace dl4j;

// out[0] = clocks issuer 0 spent issuing `iters` instructions, out[1] = clocks until they had completed (-1: the wait gave up).
// mn_major != 0: both operands MN-major (the layout of transposed tiles) instead of K-major.
// Limits: M in {64, 128}; N a multiple of 16 in 16 .. 256; issuers 1 .. 4; issuers * accs * N <= 512 tensor-memory columns.
DL4J_API int dl4j_mma_issue_probe(int M, int N, int iters, int accs, int issuers, int mn_major, long long* out_host) {
  if ((M != 64 && M != 128) || N < 16 || N > 256 || N % 16 || issuers < 1 || issuers > 4 || accs < 1 || issuers * accs * N > 512 || iters < 1)
    return -DL4J_ERR_BAD_ARG;
  long long* d = nullptr;
  cudaError_t e = cudaMalloc(&d, 2 * sizeof(long long));
  if (e != cudaSuccess) return (int)e;
  const int smem = PROBE_A_BYTES + PROBE_B_BYTES + 1024 + 64;
  e = cudaFuncSetAttribute(mma_issue_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess) {
    mma_issue_probe_kernel<<<1, 128, smem>>>(d, M, N, iters, accs, issuers, mn_major ? 1 : 0);
    e = cudaMemcpy(out_host, d, 2 * sizeof(long long), cudaMemcpyDeviceToHost);
  }
  cudaFree(d);
  return (int)e;
}
