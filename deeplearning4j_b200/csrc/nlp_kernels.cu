// Word2vec output-layer updates (skip-gram and CBOW with hierarchical softmax and / or negative sampling) for a whole batch of
// training examples in one launch, and the Barnes-Hut t-SNE edge forces.
//
// The reference walks a batch on the host and launches one single-thread kernel per Huffman node or negative sample
// (helpers/cuda/sg_cb.cu: hSoftmaxKernel / nSamplingKernel under skipgramBatchExec_ / cbowBatchExec_).  Here one warp owns one
// training example: the input vector (a syn0 row, or the mean of the context rows for CBOW) and the accumulated error live in
// shared memory, every output row is read once for the dot product and once for the update, updates of the shared tables are
// fire-and-forget fp32 reductions (rows that several examples of the batch touch accumulate, the "hogwild" behaviour of the
// original algorithm), and the negative samples come from the same 64-bit linear congruential sequence per example.
#include "common.cuh"

namespace dl4j {

constexpr int NLP_WARPS = 4;
constexpr float NLP_MAX_EXP = 6.0f;

struct W2vParams {
  float* syn0;                  // [V, D]
  float* syn1;                  // [V - 1, D] inner Huffman nodes, or null
  float* syn1neg;               // [V, D], or null
  const int* neg_table;         // unigram table or null (then samples are taken modulo V)
  long long neg_table_len;
  const int* target;            // [B] skip-gram: row of syn0 that is trained; CBOW: the predicted word (only used as ngStarter default)
  const int* ng_starter;        // [B] positive word of the negative-sampling rounds, or null
  const int* points;            // [B, L] Huffman inner nodes (-1 = padding), or null
  const signed char* codes;     // [B, L]
  const int* context;           // CBOW: [B, W] context rows (-1 = padding); null for skip-gram
  const float* alpha;           // [B] (or [1])
  const long long* random;      // [B] (or [1]) starting value of the sample sequence
  int n_alpha, n_random;
  int B, L, W, D, V, ns_rounds, train_words;
};

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// one output row: returns after adding g * row to `err` and g * in to the row
__device__ __forceinline__ void w2v_row(float* __restrict__ row, const float* __restrict__ in, float* __restrict__ err, int D, int lane,
                                        float code, float alpha, bool hierarchic) {
  float dot = 0.f;
  for (int d = lane; d < D; d += 32) dot = fmaf(in[d], row[d], dot);
  dot = warp_sum_f(dot);
  float g;
  if (hierarchic) {
    if (dot < -NLP_MAX_EXP || dot >= NLP_MAX_EXP) return;             // saturated node: no update (hSoftmaxKernel)
    g = (1.f - code - 1.f / (1.f + __expf(-dot))) * alpha;
  } else if (dot > NLP_MAX_EXP) {
    g = (code - 1.f) * alpha;
  } else if (dot < -NLP_MAX_EXP) {
    g = code * alpha;
  } else {
    g = (code - 1.f / (1.f + __expf(-dot))) * alpha;
  }
  for (int d = lane; d < D; d += 32) {
    const float r = row[d];
    err[d] = fmaf(g, r, err[d]);
    atomicAdd(row + d, g * in[d]);
  }
}

__global__ void __launch_bounds__(NLP_WARPS * 32)
w2v_batch_kernel(const W2vParams p) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* in = sh + (size_t)warp * 2 * p.D;
  float* err = in + p.D;
  for (int b = blockIdx.x * NLP_WARPS + warp; b < p.B; b += gridDim.x * NLP_WARPS) {
    const int tgt = p.target[b];
    int n_ctx = 0;
    if (p.context) {
      for (int d = lane; d < p.D; d += 32) in[d] = 0.f;
      for (int w = 0; w < p.W; ++w) {
        const int c = p.context[(long long)b * p.W + w];
        if (c < 0 || c >= p.V) continue;
        ++n_ctx;
        const float* r = p.syn0 + (long long)c * p.D;
        for (int d = lane; d < p.D; d += 32) in[d] += r[d];
      }
      if (n_ctx == 0) continue;
      const float inv = 1.f / (float)n_ctx;
      for (int d = lane; d < p.D; d += 32) in[d] *= inv;
    } else {
      if (tgt < 0 || tgt >= p.V) continue;
      const float* r = p.syn0 + (long long)tgt * p.D;
      for (int d = lane; d < p.D; d += 32) in[d] = r[d];
    }
    for (int d = lane; d < p.D; d += 32) err[d] = 0.f;
    __syncwarp();
    const float alpha = p.alpha[b % p.n_alpha];
    if (p.points && p.syn1) {
      for (int l = 0; l < p.L; ++l) {
        const int node = p.points[(long long)b * p.L + l];
        if (node < 0 || node >= p.V) continue;
        w2v_row(p.syn1 + (long long)node * p.D, in, err, p.D, lane, (float)p.codes[(long long)b * p.L + l], alpha, true);
        __syncwarp();
      }
    }
    const int starter = p.ng_starter ? p.ng_starter[b] : -1;
    if (p.ns_rounds > 0 && p.syn1neg && starter >= 0 && starter < p.V) {
      unsigned long long rnd = (unsigned long long)p.random[b % p.n_random];
      for (int r = 0; r <= p.ns_rounds; ++r) {
        int row = starter;
        if (r > 0) {
          rnd = rnd * 25214903917ULL + 11ULL;
          const unsigned long long pick = rnd >> 16;
          row = p.neg_table && p.neg_table_len > 0 ? p.neg_table[pick % (unsigned long long)p.neg_table_len] : (int)(pick % (unsigned long long)p.V);
          if (row == starter || row < 0 || row >= p.V) continue;
        }
        w2v_row(p.syn1neg + (long long)row * p.D, in, err, p.D, lane, r == 0 ? 1.f : 0.f, alpha, false);
        __syncwarp();
      }
    }
    // the accumulated error goes to the trained input rows
    if (p.context) {
      if (p.train_words) {
        // as in the original algorithm (and cbow_ of helpers/cuda/sg_cb.cu) every context row receives the whole error
        for (int w = 0; w < p.W; ++w) {
          const int c = p.context[(long long)b * p.W + w];
          if (c < 0 || c >= p.V) continue;
          float* r = p.syn0 + (long long)c * p.D;
          for (int d = lane; d < p.D; d += 32) atomicAdd(r + d, err[d]);
        }
      }
    } else {
      float* r = p.syn0 + (long long)tgt * p.D;
      for (int d = lane; d < p.D; d += 32) atomicAdd(r + d, err[d]);
    }
    __syncwarp();
  }
}

// Attractive forces of Barnes-Hut t-SNE over the sparse P (CSR): out[i] = sum_j P_ij (y_i - y_j) / (1 + |y_i - y_j|^2)
// (helpers/cuda/BarnesHutTsne.cu: edgeForces).  One warp per row, lanes over the row's neighbours, D <= 8 output dimensions.
__global__ void __launch_bounds__(128)
barnes_edge_forces_kernel(const int* __restrict__ row_p, const int* __restrict__ col_p, const float* __restrict__ val_p,
                          const float* __restrict__ y, float* __restrict__ out, int N, int D) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (i >= N) return;
  float yi[8], acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) { yi[d] = d < D ? y[(long long)i * D + d] : 0.f; acc[d] = 0.f; }
  for (int e = row_p[i] + lane; e < row_p[i + 1]; e += 32) {
    const int j = col_p[e];
    if (j < 0 || j >= N) continue;
    float diff[8], q = 1.f;
#pragma unroll
    for (int d = 0; d < 8; ++d) { diff[d] = d < D ? yi[d] - y[(long long)j * D + d] : 0.f; q = fmaf(diff[d], diff[d], q); }
    const float w = val_p[e] / q;
#pragma unroll
    for (int d = 0; d < 8; ++d) acc[d] = fmaf(w, diff[d], acc[d]);
  }
#pragma unroll
  for (int d = 0; d < 8; ++d) acc[d] = warp_sum_f(acc[d]);
  if (lane == 0)
    for (int d = 0; d < D; ++d) out[(long long)i * D + d] = acc[d];
}

}  // namespace dl4j

using namespace dl4j;

// One launch for a batch of word2vec examples.  `context` null: skip-gram (row target[b] of syn0 is the input and receives the
// error); non-null [B, W]: CBOW (the mean of the context rows is the input; with train_words the error goes back to each of them).
// Tables are fp32; index arrays int32; codes int8; alpha fp32 [n_alpha]; random int64 [n_random].
DL4J_API int dl4j_w2v_batch(float* syn0, float* syn1, float* syn1neg, const int* neg_table, long long neg_table_len, const int* target,
                            const int* ng_starter, const int* points, const signed char* codes, const int* context, const float* alpha,
                            int n_alpha, const long long* random, int n_random, int B, int L, int W, int D, int V, int ns_rounds,
                            int train_words, void* stream) {
  if (!syn0 || !target || !alpha || !random || B < 1 || D < 1 || V < 1 || n_alpha < 1 || n_random < 1) return -DL4J_ERR_BAD_ARG;
  if ((size_t)NLP_WARPS * 2 * D * sizeof(float) > 200 * 1024) return -DL4J_ERR_BAD_ARG;
  W2vParams p;
  p.syn0 = syn0; p.syn1 = syn1; p.syn1neg = syn1neg; p.neg_table = neg_table; p.neg_table_len = neg_table_len;
  p.target = target; p.ng_starter = ng_starter; p.points = points; p.codes = codes; p.context = context;
  p.alpha = alpha; p.random = random; p.n_alpha = n_alpha; p.n_random = n_random;
  p.B = B; p.L = L; p.W = W; p.D = D; p.V = V; p.ns_rounds = ns_rounds; p.train_words = train_words;
  const size_t smem = (size_t)NLP_WARPS * 2 * D * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(w2v_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int blocks = (B + NLP_WARPS - 1) / NLP_WARPS;
  if (blocks > 148 * 8) blocks = 148 * 8;
  w2v_batch_kernel<<<blocks, NLP_WARPS * 32, smem, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}

DL4J_API int dl4j_barnes_edge_forces(const int* row_p, const int* col_p, const float* val_p, const float* y, float* out, int N, int D,
                                     void* stream) {
  if (N < 1 || D < 1 || D > 8) return -DL4J_ERR_BAD_ARG;
  barnes_edge_forces_kernel<<<(N + 3) / 4, 128, 0, (cudaStream_t)stream>>>(row_p, col_p, val_p, y, out, N, D);
  return (int)cudaGetLastError();
}
