// bf16 / fp16 GEMM on pairs of SMs: the cta_group::2 form of gemm_tcgen05.cu (same warp roles, same epilogue).
//
// Two CTAs of a cluster work on one 256 x 256 output tile.  Each stages its own 128 rows of A and 128 columns of B per
// 64-wide K slice (32 KB a stage instead of 48), the leader CTA's single MMA thread issues tcgen05.mma.cta_group::2 for
// both (M = 256: each CTA's tensor core produces its own 128 rows into its own tensor memory and reads the other half of B
// from the partner's shared memory), and each CTA's four epilogue warps drain and store their own rows.
// Synchronisation across the pair:
//   * loads are plain TMA loads that complete on the loading CTA's own barrier; a thread of the peer forwards "stage landed"
//     to the leader with a remote mbarrier arrive (no cluster-multicast load, no cta_group qualifier on loads);
//   * tcgen05.commit arrives on the "stage free" and "accumulator ready" barriers of both CTAs (two commits, one per CTA);
//   * the peer's epilogue warps release the accumulator on the leader's barrier (remote arrive).
// Every wait is bounded, as in the single-CTA kernel.
#include "common.cuh"

namespace dl4j {
namespace pair {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;         // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

struct PairParams {
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

// one CTA of the pair: its 128 rows of A and its 128 of the 256 columns of B per stage
struct PairSmem {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = 128 * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int EPI_SLAB = 32 * 128;
  static constexpr int EPI_BYTES = 4 * 2 * EPI_SLAB;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 512;
};

constexpr int BLOCK_N = 256;          // columns of the pair's tile (each CTA stages half of them)

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A * B over the CTA pair: 256 rows (128 per CTA), N columns (each CTA stages N / 2 of B)
__device__ __forceinline__ void umma2_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the mbarrier at shared::cluster address `bar` once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

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
__device__ __forceinline__ float load_bias(const PairParams& p, int col) {
  if (col >= p.N) return 0.f;
  return p.bias_fp32 ? __ldg(reinterpret_cast<const float*>(p.bias) + col)
                     : unpack_lo((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.bias) + col), p.fmt);
}
__device__ __forceinline__ float unpack_hi(uint32_t u, int fmt) {
  uint32_t h = u >> 16;
  if (fmt == 1) return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&h));
  return __half2float(*reinterpret_cast<__half*>(&h));
}


template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_aux,
                 const __grid_constant__ CUtensorMap tmap_ones, const __grid_constant__ CUtensorMap tmap_bias,
                 const PairParams p) {
  using S = PairSmem;
  constexpr int STAGES = S::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + S::EPI_BYTES);
  uint64_t* full_bar = bars;                          // [STAGES] this CTA's own loads
  uint64_t* peer_full = bars + STAGES;                // [STAGES] (leader) the peer's loads of the same stage have landed
  uint64_t* empty_bar = bars + 2 * STAGES;            // [STAGES] the pair's MMAs have read the stage (both CTAs)
  uint64_t* tmem_full = bars + 3 * STAGES;            // [2] accumulator ready (both CTAs)
  uint64_t* tmem_empty = bars + 3 * STAGES + 2;       // [2] (leader) both CTAs' epilogues have drained the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();            // 0 = leader (issues the MMAs), 1 = peer
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  const int tiles_m = (p.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int kb_total = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int kb_per_split = (kb_total + p.splits - 1) / p.splits;
  const int num_work = tiles_m * tiles_n * p.splits;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&peer_full[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);       // four epilogue warps of each CTA
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 2 * BLOCK_N);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                     // both CTAs' barriers exist before anybody arrives on a remote one
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_empty_leader = mapa(smem_u32(tmem_empty), 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs: own A rows, own half of B)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cluster_id; w < num_work && ok; w += num_clusters) {
        const int tile = w / p.splits, split = w % p.splits;
        int mt, nt;
        tile_coords(tile, tiles_m, tiles_n, p.raster_gn, mt, nt);
        const int m0 = mt * (2 * BLOCK_M) + (int)rank * BLOCK_M;
        const int n0 = nt * BLOCK_N + (int)rank * 128;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kb_total);
        if (p.bias_mma) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, p.status, DL4J_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], (BLOCK_M / 64 + 128 / 64) * (64 * UMMA_K * 2));
#pragma unroll
          for (int i = 0; i < BLOCK_M / 64; ++i)
            tma_load_4d(sa + i * (64 * BLOCK_K * 2), &tmap_ones, &full_bar[stage], i * 64, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < 128 / 64; ++i)
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
            tma_load_4d(sa, &tmap_a, &full_bar[stage], k0, m0, 0, 0);
          } else {
#pragma unroll
            for (int i = 0; i < BLOCK_M / 64; ++i)
              tma_load_4d(sa + i * (64 * BLOCK_K * 2), &tmap_a, &full_bar[stage], m0 + i * 64, k0, 0, 0);
          }
          if (!B_MN) {
            tma_load_4d(sb, &tmap_b, &full_bar[stage], k0, n0, 0, 0);
          } else {
#pragma unroll
            for (int i = 0; i < 128 / 64; ++i)
              tma_load_4d(sb + i * (64 * BLOCK_K * 2), &tmap_b, &full_bar[stage], n0 + i * 64, k0, 0, 0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank != 0) {
      // ------------------------------------------------------------------ peer: tell the leader when a stage has landed here
      // (the loads carry no cta_group qualifier, so each CTA's loads complete on its own barrier)
      const uint32_t leader_peer_full = mapa(smem_u32(peer_full), 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cluster_id; w < num_work && ok; w += num_clusters) {
        const int split = w % p.splits;
        const int kb0 = split * kb_per_split;
        const int n_it = min(kb0 + kb_per_split, kb_total) - kb0 + (p.bias_mma ? 1 : 0);
        for (int i = 0; i < n_it; ++i) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          mbar_arrive_cluster(leader_peer_full + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    } else if (lane == 0) {
      // ------------------------------------------------------------------ leader: MMA issuer for the pair
      const uint32_t idesc = make_idesc(p.fmt, A_MN ? 1 : 0, B_MN ? 1 : 0, 2 * BLOCK_M, BLOCK_N);
      constexpr uint32_t LBO_A = A_MN ? 64 * BLOCK_K * 2 : 16, LBO_B = B_MN ? 64 * BLOCK_K * 2 : 16;
      constexpr uint32_t KSTEP_A = A_MN ? UMMA_K * 128 : UMMA_K * 2, KSTEP_B = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t empty_local = smem_u32(empty_bar), empty_peer = mapa(empty_local, 1);
      const uint32_t tfull_local = smem_u32(tmem_full), tfull_peer = mapa(tfull_local, 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int w = cluster_id; w < num_work && ok; w += num_clusters, ++it) {
        const int split = w % p.splits;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(kb0 + kb_per_split, kb_total);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait_bounded(&tmem_empty[buf], acc_phase ^ 1, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BLOCK_N;
        if (p.bias_mma) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA) ||
              !mbar_wait_bounded(&peer_full[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          umma2_f16(tmem_d, make_smem_desc_sw128(sa, 64 * BLOCK_K * 2, 1024), make_smem_desc_sw128(sb, 64 * BLOCK_K * 2, 1024),
                    make_idesc(p.fmt, 1, 1, 2 * BLOCK_M, BLOCK_N), 0u);
          umma2_commit(empty_local + stage * 8);
          umma2_commit(empty_peer + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA) ||
              !mbar_wait_bounded(&peer_full[stage], phase, p.status, DL4J_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, LBO_A, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, LBO_B, 1024);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
            umma2_f16(tmem_d, da + ((uint64_t)(k * KSTEP_A) >> 4), db + ((uint64_t)(k * KSTEP_B) >> 4), idesc,
                      (kb > kb0 || k > 0 || p.bias_mma) ? 1u : 0u);
          }
          umma2_commit(empty_local + stage * 8);      // frees the stage in both CTAs once these MMAs have read it
          umma2_commit(empty_peer + stage * 8);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma2_commit(tfull_local + buf * 8);          // accumulator ready: each CTA drains its own 128 rows
        umma2_commit(tfull_peer + buf * 8);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quadrant this warp may access
    int it = 0;
    bool ok = true;
    for (int w = cluster_id; w < num_work && ok; w += num_clusters, ++it) {
      const long c_off = 0;
      const int tile = w / p.splits, split = w % p.splits;
      int mt, nt;
      tile_coords(tile, tiles_m, tiles_n, p.raster_gn, mt, nt);
      const int m0 = mt * (2 * BLOCK_M) + (int)rank * BLOCK_M, n0 = nt * BLOCK_N;
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
        const int b1 = 0, b2 = 0;
        uint8_t* ring = epi_smem + q * (2 * PairSmem::EPI_SLAB);
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
          uint8_t* slab_out = my_row0 + (want_aux ? PairSmem::EPI_SLAB : ring_idx * PairSmem::EPI_SLAB);
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
                  v[j] += unpack_lo(u.x, p.fmt); v[j + 1] += unpack_hi(u.x, p.fmt);
                  v[j + 2] += unpack_lo(u.y, p.fmt); v[j + 3] += unpack_hi(u.y, p.fmt);
                  v[j + 4] += unpack_lo(u.z, p.fmt); v[j + 5] += unpack_hi(u.z, p.fmt);
                  v[j + 6] += unpack_lo(u.w, p.fmt); v[j + 7] += unpack_hi(u.w, p.fmt);
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (col0 + j < p.N) v[j] += unpack_lo((uint32_t)rs[j], p.fmt);
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
              uint8_t* src = ring + (want_aux ? PairSmem::EPI_SLAB : ring_idx * PairSmem::EPI_SLAB);
              if (p.atomic_out) tma_reduce_add_4d(&tmap_c, src, n0 + c, r0, b1, b2);
              else tma_store_4d(&tmap_c, src, n0 + c, r0, b1, b2);
            }
            bulk_commit();
          }
          ring_idx ^= 1;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tmem_empty_leader + buf * 8);
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
                v[j] += unpack_lo(u.x, p.fmt); v[j + 1] += unpack_hi(u.x, p.fmt);
                v[j + 2] += unpack_lo(u.y, p.fmt); v[j + 3] += unpack_hi(u.y, p.fmt);
                v[j + 4] += unpack_lo(u.z, p.fmt); v[j + 5] += unpack_hi(u.z, p.fmt);
                v[j + 6] += unpack_lo(u.w, p.fmt); v[j + 7] += unpack_hi(u.w, p.fmt);
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) v[j] += unpack_lo((uint32_t)rs[j], p.fmt);
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
      if (lane == 0) mbar_arrive_cluster(tmem_empty_leader + buf * 8);
    }
    if (lane == 0) bulk_wait<0>();          // staged tiles must have left shared memory before the CTA exits
  }


  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                     // the peer's shared memory and tensor memory stay alive until the pair is done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 2 * BLOCK_N);
  }
}

}  // namespace pair
}  // namespace dl4j

// =============================================================================== host side
using namespace dl4j;
using namespace dl4j::pair;

static int encode_2d_pair(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                          uint32_t box_inner, uint32_t box_outer, CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
  dl4j_PFN_encodeTiled enc = dl4j_get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[4] = {inner, outer, 1, 1};
  cuuint64_t strides[3] = {row_stride_bytes, row_stride_bytes * outer, row_stride_bytes * outer};
  cuuint32_t box[4] = {box_inner, box_outer, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

#define DL4J_REP8(x) x, x, x, x, x, x, x, x
#define DL4J_REP128(x) DL4J_REP8(DL4J_REP8(x)), DL4J_REP8(DL4J_REP8(x))
static __device__ __align__(128) uint16_t g_pair_ones_bf16[128] = {DL4J_REP128(0x3F80)};
static __device__ __align__(128) uint16_t g_pair_ones_f16[128] = {DL4J_REP128(0x3C00)};

template <bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tx,
                       const CUtensorMap& tones, const CUtensorMap& tbias, const PairParams& p, int clusters, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = PairSmem::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tx, tones, tbias, p);
  return (int)e;
}

// C[M,N] = act(alpha * A B + bias) (+ residual) on CTA pairs: one 256 x 256 tile per pair of SMs (tcgen05.mma.cta_group::2),
// each CTA staging its own 128 rows of A and its own 128 of the tile's 256 columns of B, so a stage is 32 KB per SM instead of
// 48 KB and the tensor core fetches half of B from the partner's shared memory.  Same arguments and contract as dl4j_gemm
// (no batch dimensions).  The loads are plain per-CTA TMA loads (no cluster multicast).
DL4J_API int dl4j_gemm_pair(const void* A, const void* B, void* C, void* aux, const void* bias, const void* residual, int M,
                            int N, int K, long lda, long ldb, long ldc, long ld_aux, long ld_res, int a_mn, int b_mn, int fmt,
                            int bias_fp32, int out_fp32, int act, int atomic_out, int splits, float alpha, int num_sms,
                            void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7)) return -DL4J_ERR_BAD_ARG;
  if (splits < 1) splits = 1;
  if (splits > 1 && !(atomic_out && out_fp32)) return -DL4J_ERR_BAD_ARG;
  int dev = 0;
  cudaGetDevice(&dev);
  PairParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.ld_aux = ld_aux; p.ld_res = ld_res; p.C = C; p.aux = aux; p.bias = bias;
  p.residual = residual; p.bias_fp32 = bias_fp32; p.out_fp32 = out_fp32; p.act = act; p.atomic_out = atomic_out;
  p.splits = splits; p.fmt = fmt; p.alpha = alpha; p.status = dl4j_status_word(dev);
  p.batch1 = 1; p.batch2 = 1;
  const CUtensorMapDataType dt_in = fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = encode_2d_pair(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BLOCK_K, BLOCK_M, dt_in);
  else       r = encode_2d_pair(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BLOCK_K, dt_in);
  if (r) return r > 0 ? -1000 - r : r;
  if (!b_mn) r = encode_2d_pair(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BLOCK_K, 128, dt_in);
  else       r = encode_2d_pair(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BLOCK_K, dt_in);
  if (r) return r > 0 ? -1000 - r : r;
  CUtensorMap tc, tx;
  memset(&tc, 0, sizeof(tc));
  memset(&tx, 0, sizeof(tx));
  const int esz = out_fp32 ? 4 : 2;
  p.tma_store = 0; p.tma_aux = 0;
  if (!(reinterpret_cast<uintptr_t>(C) & 15) && ((ldc * esz) % 16 == 0) &&
      (!aux || (!(reinterpret_cast<uintptr_t>(aux) & 15) && (ld_aux * 2) % 16 == 0))) {
    r = encode_2d_pair(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * esz, out_fp32 ? 32 : 64, 32,
                       out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : dt_in);
    if (r == 0) p.tma_store = 1;
    if (r == 0 && aux) {
      r = encode_2d_pair(&tx, aux, (uint64_t)N, (uint64_t)M, (uint64_t)ld_aux * 2, 64, 32, dt_in);
      if (r == 0) p.tma_aux = 1; else p.tma_store = 0;
    }
  }
  CUtensorMap tones, tbias;
  memset(&tones, 0, sizeof(tones));
  memset(&tbias, 0, sizeof(tbias));
  p.bias_mma = 0;
  if (bias && !bias_fp32 && alpha == 1.0f && splits == 1 && !(reinterpret_cast<uintptr_t>(bias) & 15)) {
    void* ones = nullptr;
    cudaError_t ce = fmt == 1 ? cudaGetSymbolAddress(&ones, g_pair_ones_bf16) : cudaGetSymbolAddress(&ones, g_pair_ones_f16);
    if (ce == cudaSuccess && encode_2d_pair(&tones, ones, 128, 1, 256, 64, UMMA_K, dt_in) == 0 &&
        encode_2d_pair(&tbias, bias, (uint64_t)N, 1, (uint64_t)((N + 7) / 8 * 8) * 2, 64, UMMA_K, dt_in) == 0)
      p.bias_mma = 1;
  }
  const int tm = (M + 255) / 256, tn = (N + 255) / 256;
  p.raster_gn = tn < 16 ? tn : 16;
  const long tiles_l = (long)tm * tn * splits;
  if (tiles_l > 0x7fffffffL) return -DL4J_ERR_BAD_ARG;
  if (num_sms <= 0) num_sms = 148;
  const int max_clusters = num_sms / 2;
  const int clusters = tiles_l < max_clusters ? (int)tiles_l : max_clusters;
#define DL4J_PAIR_CASE(AM, BM) \
  if (a_mn == AM && b_mn == BM) return launch_pair<AM != 0, BM != 0>(ta, tb, tc, tx, tones, tbias, p, clusters, stream);
  DL4J_PAIR_CASE(0, 0) DL4J_PAIR_CASE(0, 1) DL4J_PAIR_CASE(1, 0) DL4J_PAIR_CASE(1, 1)
#undef DL4J_PAIR_CASE
  return -DL4J_ERR_BAD_ARG;
}
