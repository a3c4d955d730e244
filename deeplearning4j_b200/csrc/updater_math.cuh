// Updater tables and per-element math shared by the single-GPU fused updater and the fused
// gradient-sharing kernels.  Formulas: libnd4j/include/ops/declarable/helpers/cuda/updater*.cu.
#pragma once
#include "common.cuh"

namespace dl4j {

struct UpdSegment {     // one per parameter array (56 bytes)
  long long offset;     // into params / grads
  long long block_start;// first element of the updater block this parameter belongs to
  long long block_numel;
  long long state_off;  // block's offset into the state buffer
  long long shadow_off; // this parameter's offset into the (16-byte aligned per parameter) bf16 shadow buffer
  float l1, l2, wd;     // wd already multiplied by lr when applyLR
  int kernel_id;        // see IUpdater.KERNEL_ID
  int hyper;            // index into UpdHyper table
  int pad;
};

struct UpdHyper {       // per updater block, refreshed each iteration (passed by value)
  float lr, b1, b2, eps, eps_t, mb1t, mu, rho;
};

struct UpdChunk { long long offset; int count; int seg; };

constexpr int UPD_MAX_HYPER = 8;
struct UpdHyperTable { UpdHyper h[UPD_MAX_HYPER]; };

__device__ __forceinline__ float sgnf(float x) { return (x > 0.f) - (x < 0.f); }

// state arrays per parameter element, by kernel id (0 Sgd, 1 Nesterovs, 2 Adam, 3 AdaMax, 4 Nadam, 5 AMSGrad,
// 6 AdaBelief, 7 AdaGrad, 8 RmsProp, 9 NoOp, 10 AdaDelta)
__device__ __forceinline__ int upd_n_state(int kernel_id) {
  switch (kernel_id) {
    case 0: case 9: return 0;
    case 1: case 7: case 8: return 1;
    case 5: return 3;
    default: return 2;
  }
}

// One element of regularisation + updater + weight decay.  `gr` is the (already scaled) gradient, `w` the
// parameter; st0/st1/st2 point at this element's state slots.  Returns the update (params -= update).
__device__ __forceinline__ float updater_step(const UpdSegment& sg, const UpdHyper& h, float w, float gr, float* st0,
                                              float* st1, float* st2) {
  if (sg.l2 != 0.f) gr += sg.l2 * w;
  if (sg.l1 != 0.f) gr += sg.l1 * sgnf(w);
  float u;
  switch (sg.kernel_id) {
    case 0: u = h.lr * gr; break;                                            // Sgd
    case 1: {                                                                 // Nesterovs
      const float prev = h.mu * *st0;
      const float v = prev - h.lr * gr;
      *st0 = v;
      u = prev + (-h.mu - 1.f) * v;
    } break;
    case 2: {                                                                 // Adam
      const float m = h.b1 * *st0 + (1.f - h.b1) * gr;
      const float v = h.b2 * *st1 + (1.f - h.b2) * gr * gr;
      *st0 = m; *st1 = v;
      u = m * h.eps_t / (sqrtf(v) + h.eps);
    } break;
    case 3: {                                                                 // AdaMax
      const float m = h.b1 * *st0 + (1.f - h.b1) * gr;
      const float uu = fmaxf(h.b2 * *st1, fabsf(gr)) + 1e-32f;
      *st0 = m; *st1 = uu;
      u = m * h.eps_t / uu;
    } break;
    case 4: {                                                                 // Nadam
      const float omg = (1.f - h.b1) * gr;
      const float m = h.b1 * *st0 + omg;
      const float v = h.b2 * *st1 + (1.f - h.b2) * gr * gr;
      *st0 = m; *st1 = v;
      u = (h.lr * ((m * h.b1 + omg) / h.mb1t)) / (sqrtf(v) + h.eps);
    } break;
    case 5: {                                                                 // AMSGrad
      const float m = h.b1 * *st0 + (1.f - h.b1) * gr;
      const float v = h.b2 * *st1 + (1.f - h.b2) * gr * gr;
      const float hh = fmaxf(*st2, v);
      *st0 = m; *st1 = v; *st2 = hh;
      u = h.eps_t * m / (sqrtf(hh) + h.eps);
    } break;
    case 6: {                                                                 // AdaBelief
      const float m = h.b1 * *st0 + (1.f - h.b1) * gr;
      const float d = gr - m;
      const float s = h.b2 * *st1 + (1.f - h.b2) * d * d + h.eps;
      *st0 = m; *st1 = s;
      u = m * h.eps_t / (sqrtf(s) + h.eps);
    } break;
    case 7: {                                                                 // AdaGrad
      const float s = *st0 + gr * gr;
      *st0 = s;
      u = h.lr * gr / (sqrtf(s) + h.eps);
    } break;
    case 8: {                                                                 // RmsProp
      const float s = *st0 * h.rho + gr * gr * (1.f - h.rho);
      *st0 = s;
      u = h.lr * gr / (sqrtf(s) + h.eps);
    } break;
    case 10: {                                                                // AdaDelta
      const float msg = h.rho * *st0 + (1.f - h.rho) * gr * gr;
      u = gr * (sqrtf(*st1 + h.eps) / sqrtf(msg + h.eps));
      *st0 = msg;
      *st1 = h.rho * *st1 + (1.f - h.rho) * u * u;
    } break;
    default: u = 0.f;
  }
  if (sg.wd != 0.f) u += sg.wd * w;
  return u;
}

// four consecutive floats: one 16-byte access when the address allows it
__device__ __forceinline__ float4 upd_ld4(const float* q, bool aligned) {
  if (aligned) return *reinterpret_cast<const float4*>(q);
  return make_float4(q[0], q[1], q[2], q[3]);
}
__device__ __forceinline__ void upd_st4(float* q, const float4 v, bool aligned) {
  if (aligned) { *reinterpret_cast<float4*>(q) = v; return; }
  q[0] = v.x; q[1] = v.y; q[2] = v.z; q[3] = v.w;
}


}  // namespace dl4j
