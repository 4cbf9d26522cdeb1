// Sigma-delta family as row-scan ops: the sigma decoder (a running sum), the
// delta encoder (a thresholded difference with a residual) and the fused
// sigma -> bias -> ReLU -> delta neuron.  Floating-point recurrences, one row
// per lane, in the reference's operation order.
#pragma once
#include "ops.cuh"

namespace sb {

// ===========================================================================
// Sigma forward: dendrite/sigma.py:38-72
//   out[t] = float(sum_{s<=t} x[s]) + pre_state
// torch.cumsum on a CPU float tensor accumulates in double and rounds every
// output to float; the persistent state is added afterwards in float.
// ===========================================================================
struct SigmaFwd {
  static constexpr int NIN = 1, NOUT = 1;
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  SB_PIPE(3, 3, 32);
  struct Params {
    const float* state;   // [rows] or null
    float* final_state;   // [rows] or null: out[..., -1]
  };
  double acc;
  float pre, last;
  __device__ __forceinline__ void init(const Params& p, const RowGeom&, int64_t row, bool valid) {
    acc = 0.0; last = 0.f;
    pre = (valid && p.state) ? __ldg(p.state + row) : 0.f;
  }
  __device__ __forceinline__ void step(const float (&a)[1], float (&b)[1]) {
    acc += (double)a[0];
    last = __fadd_rn((float)acc, pre);
    b[0] = last;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (p.final_state && valid) p.final_state[row] = last;
  }
};

// Sigma backward: the adjoint of cumsum, a cumsum over reversed time
// (autograd: grad.flip(-1).cumsum(-1).flip(-1)), double accumulation again.
struct SigmaBwd {
  static constexpr int NIN = 1, NOUT = 1;
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  SB_PIPE(3, 3, 32);
  struct Params {};
  double acc;
  __device__ __forceinline__ void init(const Params&, const RowGeom&, int64_t, bool) { acc = 0.0; }
  __device__ __forceinline__ void step(const float (&a)[1], float (&b)[1]) {
    acc += (double)a[0];
    b[0] = (float)acc;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params&, const RowGeom&, int64_t, bool, int, int64_t) {}
};

// ===========================================================================
// Delta forward: axon/delta.py:44-54 (cum_error = False) + the floor
// quantisation of Delta.forward (delta.py:316)
//   d[t] = (x[t] - pre) + residual;  y[t] = d[t] if |d[t]| >= thr else 0 * d[t]
//   residual = d[t] - y[t];  pre = x[t];  out[t] = floor(y[t] / step) * step
// ===========================================================================
struct DeltaParams {
  DecayVec thr;            // 1 or C thresholds
  const float* pre;        // [rows] or null
  const float* residual;   // [rows] or null
  float* final_residual;   // [rows] or null
  float step;              // quantisation step 1 / scale as fp32; 0 disables
  float inv_step;          // scale when it is a power of two (y / step == y * scale exactly), else 0
};

struct DeltaState {
  float pre, res, thr, qstep, qinv;
  __device__ __forceinline__ void init(const DeltaParams& p, const RowGeom& g, int64_t row, bool valid) {
    pre = (valid && p.pre) ? __ldg(p.pre + row) : 0.f;
    res = (valid && p.residual) ? __ldg(p.residual + row) : 0.f;
    thr = valid ? load_decay(p.thr, g, row) : 0.f;
    qstep = p.step;
    qinv = p.inv_step;
  }
  // returns the quantised output; d receives the un-thresholded difference
  __device__ __forceinline__ float step(float x, float& d) {
    d = __fadd_rn(__fsub_rn(x, pre), res);
    const float y = fabsf(d) >= thr ? d : __fmul_rn(0.f, d);
    res = __fsub_rn(d, y);
    pre = x;
    // An IEEE divide takes its slow path for the zeros that make up most of y; for a power-of-two
    // scale the multiplication gives the same bits.
    if (qinv > 0.f) return __fmul_rn(floorf(__fmul_rn(y, qinv)), qstep);
    return qstep > 0.f ? __fmul_rn(floorf(__fdiv_rn(y, qstep)), qstep) : y;
  }
};

template <bool SAVE_DELTA>
struct DeltaFwd {
  static constexpr int NIN = 1, NOUT = SAVE_DELTA ? 2 : 1;
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  SB_PIPE(3, (SAVE_DELTA ? 1 : 3), 32);
  typedef DeltaParams Params;
  DeltaState s;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    s.init(p, g, row, valid);
  }
  __device__ __forceinline__ void step(const float (&a)[1], float (&b)[NOUT]) {
    float d;
    b[0] = s.step(a[0], d);
    if (SAVE_DELTA) b[1] = d;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (p.final_residual && valid) p.final_residual[row] = s.res;
  }
};

// ===========================================================================
// Delta backward: axon/delta.py:77-122
//   grad_x[t] = g[t] - g[t+1]   (g[T] = 0)
//   grad_thr  = sum ( |d| - thr > 0 ? -d * scale * exp(-| |d| - thr | / tau) / thr : -sign(d) ) * g
// ===========================================================================
template <bool TGRAD>
struct DeltaBwd {
  static constexpr int NIN = TGRAD ? 2 : 1, NOUT = 1;
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  SB_PIPE(3, (TGRAD ? 1 : 3), 32);
  struct Params {
    DecayVec thr;
    float tau, scale;
    double* partial;
  };
  float gnext, thr, tau, scale;
  GradAcc acc;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    gnext = 0.f; acc.reset();
    thr = (TGRAD && valid) ? load_decay(p.thr, g, row) : 1.f;
    tau = p.tau; scale = p.scale;
  }
  __device__ __forceinline__ void step(const float (&in)[NIN], float (&b)[1]) {
    b[0] = __fsub_rn(in[0], gnext);
    gnext = in[0];
    if (TGRAD) {
      const float d = in[1];
      const float sub = __fsub_rn(fabsf(d), thr);
      float gt;
      if (sub > 0.f) {
        const float nd = __fmul_rn(scale, expf(__fdiv_rn(-fabsf(sub), tau)));
        gt = __fdiv_rn(__fmul_rn(-d, nd), thr);
      } else {
        gt = d > 0.f ? -1.f : (d < 0.f ? 1.f : -d);   // -sign(d)
      }
      acc.add(__fmul_rn(gt, in[0]));
    }
  }
  __device__ __forceinline__ void tile_end() { if (TGRAD) acc.flush(); }
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int lane,
                                         int64_t warp_id) {
    if (TGRAD) store_partial(p.partial, p.thr.n <= 1, acc.d, valid, lane, row, warp_id);
  }
};

// ===========================================================================
// Sigma-delta ReLU neuron, forward only: neuron/sigma_delta.py:171-219 with
// activation = relu and no normalisation, one pass:
//   s[t] = float(cumsum x) + sigma_state;  a[t] = relu(s[t] + bias);  out = delta(a)
// bias: one value, or one per neuron as set_bias() stores it (sigma_delta.py:152-165)
// ===========================================================================
// SAVE = 0: inference (8 B per step).  SAVE = 1 also writes the activation (what the backward's
// ReLU mask needs), SAVE = 2 the delta unit's difference as well (threshold gradient).
template <int SAVE>
struct SdnnFwd {
  static constexpr int NIN = 1, NOUT = 1 + SAVE;
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  SB_PIPE((SAVE == 0 ? 5 : 3), 1, 32);   // five stages of one box: 0.77 -> 0.88 of copy bandwidth (three boxes, three stages)
  struct Params {
    DeltaParams delta;
    const float* sigma_state;   // [rows] or null
    DecayVec bias;              // nullable (v == null): no bias; 1 value or one per neuron (rows_per_batch)
    float* final_sigma;         // [rows] or null
    float* final_pre;           // [rows] or null: the delta unit's next pre_state (last activation)
  };
  DeltaState s;
  double acc;
  float spre, bias, last_sigma;
  bool has_bias;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    s.init(p.delta, g, row, valid);
    acc = 0.0; last_sigma = 0.f;
    spre = (valid && p.sigma_state) ? __ldg(p.sigma_state + row) : 0.f;
    has_bias = p.bias.v != nullptr;
    bias = (valid && has_bias) ? __ldg(p.bias.v + (p.bias.n <= 1 ? 0 : row % g.rows_per_batch)) : 0.f;
  }
  __device__ __forceinline__ void step(const float (&a)[1], float (&b)[NOUT]) {
    acc += (double)a[0];
    last_sigma = __fadd_rn((float)acc, spre);
    const float z = has_bias ? __fadd_rn(last_sigma, bias) : last_sigma;
    const float act = fmaxf(z, 0.f);
    float d;
    b[0] = s.step(act, d);
    if (SAVE >= 1) b[1] = act;
    if (SAVE >= 2) b[NOUT - 1] = d;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (!valid) return;
    if (p.final_sigma) p.final_sigma[row] = last_sigma;
    if (p.final_pre) p.final_pre[row] = s.pre;
    if (p.delta.final_residual) p.delta.final_residual[row] = s.res;
  }
};

// ===========================================================================
// Backward of the same neuron in one reverse pass:
//   gd[t] = g[t] - g[t+1]                      (delta, delta.py:103-107)
//   gz[t] = gd[t] if act[t] > 0 else 0          (ReLU)
//   gx[t] = float(sum_{s>=t} gz[s])             (adjoint of the running sum, double accumulation)
// and, with TGRAD, the threshold gradient of the delta unit from its saved difference.
// ===========================================================================
template <bool TGRAD>
struct SdnnBwd {
  static constexpr int NIN = TGRAD ? 3 : 2, NOUT = 1;
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  SB_PIPE(3, 2, 32);   // 0.86 -> 0.95
  typedef typename DeltaBwd<TGRAD>::Params Params;
  DeltaBwd<TGRAD> dl;
  double acc;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    dl.init(p, g, row, valid);
    acc = 0.0;
  }
  __device__ __forceinline__ void step(const float (&in)[NIN], float (&b)[1]) {
    float gd[1];
    if (TGRAD) {
      const float din[2] = {in[0], in[2]};
      dl.step(reinterpret_cast<const float(&)[DeltaBwd<TGRAD>::NIN]>(din), gd);
    } else {
      const float din[1] = {in[0]};
      dl.step(reinterpret_cast<const float(&)[DeltaBwd<TGRAD>::NIN]>(din), gd);
    }
    acc += (double)(in[1] > 0.f ? gd[0] : 0.f);
    b[0] = (float)acc;
  }
  __device__ __forceinline__ void tile_end() { dl.tile_end(); }
  __device__ __forceinline__ void finish(const Params& p, const RowGeom& g, int64_t row, bool valid, int lane,
                                         int64_t warp_id) {
    dl.finish(p, g, row, valid, lane, warp_id);
  }
};

}  // namespace sb
