// Per-step arithmetic of every time-recurrent op on the SLAYER hot path.
// Each struct plugs into the row-scan skeleton (rowscan.cuh): init() loads the
// per-row state and parameters into registers, step() advances one time bin,
// tile_end() runs once per 32 steps, finish() writes per-row results.
//
// The arithmetic restates the CPU loops of lava-dl
// (src/lava/lib/dl/slayer/neuron/dynamics/*.py, spike/*.py); each op cites the
// lines it follows.  States are int32 with 64-bit products, i.e. exact while
// every state stays inside int32 (Loihi states are 24 bit); fused ops skip the
// float round trip between stages, which is the identity for |state| < 2^24 and
// a power-of-two w_scale (the host only fuses in that case).
//
// Every op also states the pipeline shape its TMA kernel runs with: STAGES per
// warp, BOXES of TILE steps per stage (shared memory per warp = STAGES *
// max(NIN, NOUT - NBIT) * BOXES * TILE * 128 B).  The values were picked by
// sweeping shapes on a B200; where a comment beside SB_PIPE gives two numbers
// they are fractions of the measured copy bandwidth before and after.  The
// pattern: one-stream ops want long row segments (three or four boxes per
// stage) and three stages; ops that write two full-width streams per input
// stream want five or six stages of one box; ops with two input tiles want two
// boxes and three or four stages; ops with four or more full-width streams fall
// to 16-step tiles only when 32-step tiles would leave fewer than four warps
// per SM.
#pragma once

#include "common.cuh"

namespace sb {

#define SB_PIPE(S, B, T) static constexpr int STAGES = S, BOXES = B, TILE = T

// ---------------------------------------------------------------------------
// Parameter blocks shared by several ops
// ---------------------------------------------------------------------------
struct DecayVec {       // un-scaled integer-valued floats, 1 or C entries
  const float* v;
  int64_t n;
};

struct Scale {
  float w;      // w_scale as float
  float inv_w;  // exact reciprocal when w_scale is a power of two
};

__device__ __forceinline__ float load_decay(const DecayVec& d, const RowGeom& g, int64_t row) {
  return __ldg(d.v + param_index(g, row, d.n));
}

// Surrogate gradient of the spike function, spike/spike.py:10-23.
//   binary: scale_rho / 2 / tau_rho * exp(-|v - thr| / tau_rho)
//   graded: scale_rho * exp(min(v - thr, 0) / tau_rho)
// exp(x / tau) is evaluated as 2^(x * log2(e) / tau) with the constant folded
// on the host: one multiply and one MUFU.EX2 instead of an IEEE divide plus
// expf.  The result differs from the divide-then-exp form by at most
// (2 + |x / tau|) ulp, far inside the 1e-5 relative bound on gradients, and
// the backward kernels drop from 36 to about 24 instructions per step.
struct Surrogate {
  float c0;        // binary: (scale_rho / 2) / tau_rho ; graded: scale_rho
  float k2;        // log2(e) / tau_rho
};
template <bool GRADED>
__device__ __forceinline__ float surrogate(const Surrogate& s, float v, float thr) {
  const float d = __fsub_rn(v, thr);
  const float x = GRADED ? fminf(d, 0.f) : -fabsf(d);
  return __fmul_rn(s.c0, exp2f(__fmul_rn(x, s.k2)));
}

// Gradients of the phase-threshold (complex) spike, spike/complex.py:144-167.
struct CSurrogate {
  float k2;             // log2(e) / tau_rho
  float scale_rho;
  float half_over_tau;  // (1 / 2) / tau_rho
  float two_tau;        // 2 * tau_rho
  float neg_scale_over_tau;  // -scale_rho / tau_rho
};
__device__ __forceinline__ float sgnf(float x) { return (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : 0.f); }
template <bool GRADED>
__device__ __forceinline__ void csurrogate(const CSurrogate& s, float re, float im, float thr, float& d_re,
                                           float& d_im) {
  float delta_real;
  if (GRADED) delta_real = exp2f(__fmul_rn(-fmaxf(__fsub_rn(thr, re), 0.f), s.k2));
  else delta_real = __fmul_rn(s.half_over_tau, exp2f(__fmul_rn(-fabsf(__fsub_rn(re, thr)), s.k2)));
  const float delta_imag = __fmul_rn(s.half_over_tau, exp2f(__fmul_rn(-fabsf(im), s.k2)));
  const float step_real = __fmul_rn(
      0.5f, __fadd_rn(1.f, __fmul_rn(sgnf(__fsub_rn(re, thr)), __fsub_rn(1.f, __fmul_rn(s.two_tau, delta_real)))));
  d_re = __fmul_rn(__fmul_rn(s.scale_rho, delta_real), delta_imag);
  d_im = __fmul_rn(__fmul_rn(__fmul_rn(s.neg_scale_over_tau, sgnf(im)), delta_imag), step_real);
}

// Per-thread accumulator for parameter gradients: fp32 inside a 32-step tile,
// fp64 across tiles (keeps the sum of up to 10^9 terms within 1e-5 relative).
struct GradAcc {
  float f;
  double d;
  __device__ __forceinline__ void reset() { f = 0.f; d = 0.0; }
  __device__ __forceinline__ void add(float x) { f = __fadd_rn(f, x); }
  __device__ __forceinline__ void flush() { d += (double)f; f = 0.f; }
};

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Writes one parameter-gradient partial.  Shared parameter: warp shuffle, one
// slot per warp.  Per-channel parameter: one slot per row (lanes of a warp may
// belong to different channels).  reduce_param_grad() folds the slots.
__device__ __forceinline__ void store_partial(double* partial, bool shared, double v, bool valid, int lane,
                                              int64_t row, int64_t warp_id) {
  if (shared) {
    const double s = warp_sum(valid ? v : 0.0);
    if (lane == 0) partial[warp_id] = s;
  } else if (valid) {
    partial[row] = v;
  }
}

// ===========================================================================
// Leaky integrator forward: leaky_integrator.py:210-231
//   y[t] = rshift0(y_old * (4096 - int(decay)), 12) + int(w * x[t])
//   y_old = 0 where float(y[t]) >= thr * w (only when thr * w > 0) else y[t]
// ===========================================================================
template <bool RESET, bool POW2>
struct LiFwd {
  static constexpr int NIN = 1, NOUT = 1;
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  static constexpr bool HAS_FAST = true;
  SB_PIPE(3, 3, 32);
  struct Params {
    DecayVec decay;
    const float* state;   // [rows]
    float* final_state;   // [rows] or null: y[..., -1]
    int k_reset;          // smallest int whose fp32 value reaches thr * w
    Scale sc;
  };
  // dy is the state already decayed for the next step (0 after a reset): the reset select then sits
  // behind the multiply instead of in front of it, and the compare leaves the serial chain.
  int dy, mul, k_reset, last;
  float w, inv_w;
  bool fast_;

  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w; k_reset = p.k_reset;
    int y = 0;
    mul = 4096; last = 0;
    if (valid) {
      mul = 4096 - (int)load_decay(p.decay, g, row);
      y = to_fixed(w, __ldg(p.state + row));
    }
    fast_ = __all_sync(0xffffffffu, mul_is_decay(mul));
    dy = mul_shift12(y, mul);
    if (fast_) mul <<= 4;
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[1], float (&b)[1]) {
    const int yn = dy + to_fixed(w, a[0]);
    b[0] = from_fixed<POW2>(yn, w, inv_w);
    last = yn;
    const int d = FAST ? mul_shift12_pos(yn, mul) : mul_shift12(yn, mul);
    dy = (RESET && yn >= k_reset) ? 0 : d;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (p.final_state && valid) p.final_state[row] = from_fixed<POW2>(last, w, inv_w);
  }
};

// ===========================================================================
// Leaky integrator backward: leaky_integrator.py:234-259
//   g[t] = (1 - decay / 4096) * g[t+1] + go[t]   (reset ignored)
//   grad_decay = sum g[t+1] * y[t]
// ===========================================================================
template <bool DGRAD>
struct LiBwd {
  static constexpr int NIN = DGRAD ? 2 : 1, NOUT = 1;
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  SB_PIPE((DGRAD ? 4 : 3), (DGRAD ? 2 : 4), 32);   // with the decay gradient (two input tiles): 0.86 -> 0.95
  struct Params {
    DecayVec decay;
    double* partial;  // scratch, see store_partial()
  };
  float a, gcur;
  GradAcc acc;

  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    gcur = 0.f; acc.reset();
    a = valid ? __fsub_rn(1.f, __fdiv_rn(load_decay(p.decay, g, row), 4096.f)) : 0.f;
  }
  __device__ __forceinline__ void step(const float (&in)[NIN], float (&b)[1]) {
    if (DGRAD) acc.add(__fmul_rn(gcur, in[NIN - 1]));
    gcur = __fadd_rn(__fmul_rn(a, gcur), in[0]);
    b[0] = gcur;
  }
  __device__ __forceinline__ void tile_end() { if (DGRAD) acc.flush(); }
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int lane,
                                         int64_t warp_id) {
    if (DGRAD) store_partial(p.partial, p.decay.n <= 1, acc.d, valid, lane, row, warp_id);
  }
};

// ===========================================================================
// Adaptive threshold + refractory state machine shared by several ops:
// adaptive_threshold.py:237-274 (and the same lines inside
// adaptive_phase_th.py:234-283, adaptive_resonator.py:379-436)
// ===========================================================================
struct AthParams {
  DecayVec ref_decay, th_decay;
  const float* ref_state;  // [rows]
  const float* th_state;   // [rows]
  int th_step;             // int(th_scale * w_scale)
  int th0;                 // int(th0 * w_scale)
};
struct AthState {
  int th, ref, th_mul, ref_mul, th0, th_step;
  int th_new, ref_new;
  __device__ __forceinline__ void init(const AthParams& p, const RowGeom& g, int64_t row, bool valid, float w) {
    th0 = p.th0; th_step = p.th_step;
    th = th0; ref = 0; th_mul = 4096; ref_mul = 4096; th_new = th0; ref_new = 0;
    if (valid) {
      th = to_fixed(w, __ldg(p.th_state + row));
      ref = to_fixed(w, __ldg(p.ref_state + row));
      th_mul = 4096 - (int)load_decay(p.th_decay, g, row);
      ref_mul = 4096 - (int)load_decay(p.ref_decay, g, row);
    }
  }
  // true when every lane's multipliers allow the short truncating multiply; the caller then
  // calls use_fast() once and decay<true>() from there on
  __device__ __forceinline__ bool fast_ok() const {
    return __all_sync(0xffffffffu, mul_is_decay(th_mul) && mul_is_decay(ref_mul));
  }
  __device__ __forceinline__ void use_fast() { th_mul <<= 4; ref_mul <<= 4; }
  template <bool FAST = false>
  __device__ __forceinline__ void decay() {
    ref_new = FAST ? mul_shift12_pos(ref, ref_mul) : mul_shift12(ref, ref_mul);
    th_new = (FAST ? mul_shift12_pos(th - th0, th_mul) : mul_shift12(th - th0, th_mul)) + th0;
  }
  __device__ __forceinline__ void commit(bool spike) {
    th = th_new + (spike ? th_step : 0);
    ref = ref_new + (spike ? 2 * th_new : 0);
  }
};

template <bool POW2>
struct AthFwd {
  static constexpr int NIN = 1, NOUT = 2;  // out: threshold, refractory
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  static constexpr bool HAS_FAST = true;
  SB_PIPE(5, 1, 32);   // 0.75 -> 0.80 of copy bandwidth against three stages
  struct Params {
    AthParams ath;
    Scale sc;
  };
  AthState s;
  float w, inv_w;
  bool fast_;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w;
    s.init(p.ath, g, row, valid, w);
    fast_ = s.fast_ok();
    if (fast_) s.use_fast();
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[1], float (&b)[2]) {
    s.template decay<FAST>();
    const int x = to_fixed(w, a[0]);
    b[0] = from_fixed<POW2>(s.th_new, w, inv_w);
    b[1] = from_fixed<POW2>(s.ref_new, w, inv_w);
    s.commit(x >= s.th_new + s.ref_new);
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params&, const RowGeom&, int64_t, bool, int, int64_t) {}
};

// Adaptive phase threshold: adaptive_phase_th.py:234-283
template <bool POW2>
struct ApthFwd {
  static constexpr int NIN = 2, NOUT = 2;  // in: re, im; out: threshold, refractory
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  static constexpr bool HAS_FAST = true;
  SB_PIPE(6, 1, 32);   // 0.79 -> 0.85
  struct Params {
    AthParams ath;
    const float* im_state;  // [rows]
    Scale sc;
  };
  AthState s;
  int im_old;
  float w, inv_w;
  bool fast_;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w;
    s.init(p.ath, g, row, valid, w);
    im_old = valid ? to_fixed(w, __ldg(p.im_state + row)) : 0;
    fast_ = s.fast_ok();
    if (fast_) s.use_fast();
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[2], float (&b)[2]) {
    s.template decay<FAST>();
    const int re = to_fixed(w, a[0]);
    const int im = to_fixed(w, a[1]);
    b[0] = from_fixed<POW2>(s.th_new, w, inv_w);
    b[1] = from_fixed<POW2>(s.ref_new, w, inv_w);
    s.commit(re >= s.th_new + s.ref_new && im >= 0 && im_old < 0);
    im_old = im;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params&, const RowGeom&, int64_t, bool, int, int64_t) {}
};

// ===========================================================================
// Resonator state machine: resonator.py:333-376
//   re[t] = rshift0(cos*re_o,12) - rshift0(sin*im_o,12) + int(w*re_in[t])
//   im[t] = rshift0(sin*re_o,12) + rshift0(cos*im_o,12) + int(w*im_in[t])
//   Izhikevich reset (thr*w >= 0): where float(im[t]) >= thr*w:
//     re_o = 0, im_o = int(float(thr*w - 1)); elsewhere im_o passes through fp32
// ===========================================================================
struct ResParams {
  DecayVec sin_decay, cos_decay;  // already scaled integer-valued floats, same count
  const float* re_state;
  const float* im_state;
};
struct ResState {
  int re, im, sn, cs, re_new, im_new;
  __device__ __forceinline__ void init(const ResParams& p, const RowGeom& g, int64_t row, bool valid, float w) {
    re = im = sn = cs = re_new = im_new = 0;
    if (valid) {
      sn = (int)load_decay(p.sin_decay, g, row);
      cs = (int)load_decay(p.cos_decay, g, row);
      re = to_fixed(w, __ldg(p.re_state + row));
      im = to_fixed(w, __ldg(p.im_state + row));
    }
  }
  // sin/cos small enough for the pre-shifted multiplier (always, for decays scaled by 4096)
  __device__ __forceinline__ bool fast_ok() const {
    return __all_sync(0xffffffffu, sn > -(1 << 27) && sn < (1 << 27) && cs > -(1 << 27) && cs < (1 << 27));
  }
  __device__ __forceinline__ void use_fast() { sn <<= 4; cs <<= 4; }
  template <bool FAST = false>
  __device__ __forceinline__ void advance(float w, float re_in, float im_in) {
    if (FAST) {
      re_new = mul_shift12_sym(re, cs) - mul_shift12_sym(im, sn) + to_fixed(w, re_in);
      im_new = mul_shift12_sym(re, sn) + mul_shift12_sym(im, cs) + to_fixed(w, im_in);
    } else {
      re_new = mul_shift12(cs, re) - mul_shift12(sn, im) + to_fixed(w, re_in);
      im_new = mul_shift12(sn, re) + mul_shift12(cs, im) + to_fixed(w, im_in);
    }
  }
  __device__ __forceinline__ void keep() { re = re_new; im = im_new; }
};

template <bool RESET, bool POW2>
struct ResFwd {
  static constexpr int NIN = 2, NOUT = 2;
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  static constexpr bool HAS_FAST = true;
  SB_PIPE(3, 2, 32);   // two boxes per stage: 0.83 -> 0.91
  struct Params {
    ResParams res;
    int k_thr;     // smallest int whose fp32 value reaches thr * w
    int im_reset;  // int(float(thr * w - 1))
    Scale sc;
  };
  ResState s;
  int k_thr, im_reset;
  float w, inv_w;
  bool fast_;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w; k_thr = p.k_thr; im_reset = p.im_reset;
    s.init(p.res, g, row, valid, w);
    fast_ = s.fast_ok();
    if (fast_) s.use_fast();
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[2], float (&b)[2]) {
    s.template advance<FAST>(w, a[0], a[1]);
    b[0] = from_fixed<POW2>(s.re_new, w, inv_w);
    b[1] = from_fixed<POW2>(s.im_new, w, inv_w);
    if (RESET) {
      const bool spk = s.im_new >= k_thr;
      s.re = spk ? 0 : s.re_new;
      s.im = spk ? im_reset : __float2int_rz(__int2float_rn(s.im_new));
    } else {
      s.keep();
    }
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params&, const RowGeom&, int64_t, bool, int, int64_t) {}
};

// Resonator backward: resonator.py:379-467 (also adaptive_resonator.py:439-525)
template <bool PGRAD>
struct ResBwd {
  static constexpr int NIN = PGRAD ? 4 : 2, NOUT = 2;  // in: g_re, g_im, [re, im]
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  SB_PIPE((PGRAD ? 3 : 4), 2, 32);   // two boxes per stage: 0.80 -> 0.92 (four stages), 0.89 -> 0.93 with sin / cos gradients (three)
  struct Params {
    DecayVec sin_decay, cos_decay;
    double* partial_sin;
    double* partial_cos;
  };
  float sn, cs, gre, gim;
  GradAcc asin_, acos_;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    gre = gim = 0.f; sn = cs = 0.f; asin_.reset(); acos_.reset();
    if (valid) {
      sn = __fdiv_rn(load_decay(p.sin_decay, g, row), 4096.f);
      cs = __fdiv_rn(load_decay(p.cos_decay, g, row), 4096.f);
    }
  }
  __device__ __forceinline__ void scan(float go_re, float go_im, float re, float im) {
    if (PGRAD) {
      asin_.add(__fadd_rn(__fmul_rn(-gre, im), __fmul_rn(gim, re)));
      acos_.add(__fadd_rn(__fmul_rn(gre, re), __fmul_rn(gim, im)));
    }
    const float nre = __fadd_rn(__fadd_rn(__fmul_rn(cs, gre), __fmul_rn(sn, gim)), go_re);
    const float nim = __fadd_rn(__fadd_rn(__fmul_rn(-sn, gre), __fmul_rn(cs, gim)), go_im);
    gre = nre; gim = nim;
  }
  __device__ __forceinline__ void step(const float (&a)[NIN], float (&b)[2]) {
    scan(a[0], a[1], PGRAD ? a[NIN - 2] : 0.f, PGRAD ? a[NIN - 1] : 0.f);
    b[0] = gre; b[1] = gim;
  }
  __device__ __forceinline__ void tile_end() { if (PGRAD) { asin_.flush(); acos_.flush(); } }
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int lane,
                                         int64_t warp_id) {
    if (PGRAD) {
      const bool shared = p.sin_decay.n <= 1;
      store_partial(p.partial_sin, shared, asin_.d, valid, lane, row, warp_id);
      store_partial(p.partial_cos, shared, acos_.d, valid, lane, row, warp_id);
    }
  }
};

// Adaptive resonator forward: adaptive_resonator.py:379-436
template <bool POW2>
struct AdResFwd {
  static constexpr int NIN = 2, NOUT = 4;  // out: re, im, threshold, refractory
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = 0;
  static constexpr bool HAS_FAST = true;
  SB_PIPE(3, 1, 32);   // 32-step tiles although that leaves four warps per SM: 0.66 -> 0.79 against 16-step tiles
  struct Params {
    ResParams res;
    AthParams ath;
    Scale sc;
  };
  ResState r;
  AthState s;
  float w, inv_w;
  bool fast_;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w;
    r.init(p.res, g, row, valid, w);
    s.init(p.ath, g, row, valid, w);
    const bool fr = r.fast_ok(), fs = s.fast_ok();
    fast_ = fr && fs;
    if (fast_) { r.use_fast(); s.use_fast(); }
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[2], float (&b)[4]) {
    s.template decay<FAST>();
    r.template advance<FAST>(w, a[0], a[1]);
    b[0] = from_fixed<POW2>(r.re_new, w, inv_w);
    b[1] = from_fixed<POW2>(r.im_new, w, inv_w);
    b[2] = from_fixed<POW2>(s.th_new, w, inv_w);
    b[3] = from_fixed<POW2>(s.ref_new, w, inv_w);
    s.commit(r.im_new >= s.th_new + s.ref_new);
    r.keep();
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params&, const RowGeom&, int64_t, bool, int, int64_t) {}
};

// ===========================================================================
// Fused CUBA neuron forward: neuron/cuba.py:274-421 with norm=None
//   current = LI(x), voltage = LI(current, reset at threshold), spike(voltage)
// Outputs (in tile order): [current], voltage, [spike]
// ===========================================================================
template <bool OUT_CUR, bool OUT_SPK, bool GRADED, bool OUT_VOL = true>
struct CubaFwd {
  static_assert(OUT_VOL || (OUT_SPK && !GRADED && !OUT_CUR), "without the voltage series only binary spikes leave");
  static constexpr int NIN = 1, NOUT = (OUT_VOL ? 1 : 0) + (OUT_CUR ? 1 : 0) + (OUT_SPK ? 1 : 0);
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = (OUT_SPK && !GRADED) ? 1 : 0;  // binary spikes leave as bits
  static constexpr bool HAS_FAST = true;
  // boxes per stage by the number of tiles a stage holds: 3 for one (spikes + voltage), 2 for two (training:
  // current + voltage; 3.44 -> 3.12 ms at [64,8192,2000]), else 1; with no output tile at all (spikes only:
  // the stage holds the input) 2 boxes, 0.85 -> 0.89 of copy bandwidth against 3
  SB_PIPE(3, ((NOUT - NBIT) == 0 ? 2 : ((NOUT - NBIT) <= 1 ? 3 : ((NOUT - NBIT) == 2 ? 2 : 1))), 32);
  static constexpr int IV = OUT_CUR ? 1 : 0, IS = IV + (OUT_VOL ? 1 : 0);
  struct Params {
    DecayVec cdecay, vdecay;
    const float* cstate;
    const float* vstate;
    float* final_c;  // current[..., -1] or null
    float* final_v;  // voltage[..., -1] (before reset) or null
    float* final_s;  // spike[..., -1] or null
    int k_reset;     // reset when v >= k_reset  (float(v) >= f32(thr * w))
    int k_spike;     // spike when v >= k_spike  (float(v) / w >= f32(thr))
    float spike_scale;
    Scale sc;
  };
  // dv is the voltage already decayed for the next step (0 after a reset): the reset select then sits
  // behind the multiply instead of in front of it, and the compare leaves the serial chain.
  // The fast path (every multiplier of the warp in 0 .. 4096, one integer threshold for spike and reset)
  // uses the short truncating multiply and a single compare.
  int c, dv, cmul, vmul, k_reset, k_spike, last_v;
  float w, inv_w, spike_scale, last_s;
  bool fast_;

  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w; k_reset = p.k_reset; k_spike = p.k_spike; spike_scale = p.spike_scale;
    int v = 0;
    c = last_v = 0; cmul = vmul = 4096; last_s = 0.f;
    if (valid) {
      cmul = 4096 - (int)load_decay(p.cdecay, g, row);
      vmul = 4096 - (int)load_decay(p.vdecay, g, row);
      c = to_fixed(w, __ldg(p.cstate + row));
      v = to_fixed(w, __ldg(p.vstate + row));
    }
    fast_ = __all_sync(0xffffffffu, mul_is_decay(cmul) && mul_is_decay(vmul)) && (!OUT_SPK || k_spike == k_reset);
    dv = mul_shift12(v, vmul);
    if (fast_) { cmul <<= 4; vmul <<= 4; }
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[1], float (&b)[NOUT]) {
    c = (FAST ? mul_shift12_pos(c, cmul) : mul_shift12(c, cmul)) + to_fixed(w, a[0]);
    const int vn = dv + c;
    const float vf = from_fixed<true>(vn, w, inv_w);
    if (OUT_CUR) b[0] = from_fixed<true>(c, w, inv_w);
    if (OUT_VOL) b[IV] = vf;
    const bool rs = vn >= k_reset;
    if (OUT_SPK) {
      const bool s = FAST ? rs : (vn >= k_spike);
      last_s = GRADED ? __fdiv_rn(__fmul_rn(s ? 1.f : 0.f, vf), spike_scale) : (s ? 1.f : 0.f);
      b[IS] = last_s;
    }
    last_v = vn;
    const int d = FAST ? mul_shift12_pos(vn, vmul) : mul_shift12(vn, vmul);
    dv = rs ? 0 : d;
  }
  // one step outside the row-scan skeleton (the recurrent walk): picks the path per call
  __device__ __forceinline__ void step(const float (&a)[1], float (&b)[NOUT]) {
    if (fast_) step_t<true>(a, b); else step_t<false>(a, b);
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (!valid) return;
    if (p.final_c) p.final_c[row] = from_fixed<true>(c, w, inv_w);
    if (p.final_v) p.final_v[row] = from_fixed<true>(last_v, w, inv_w);
    if (OUT_SPK && p.final_s) p.final_s[row] = last_s;
  }
};

// ===========================================================================
// Fused backward of CUBA / ALIF forward: spike surrogate (spike/spike.py:112-126)
// then two reverse leaky-integrator scans (leaky_integrator.py:234-259).
// Inputs (tile order): g_spike, voltage, [threshold tensor], [current]
// Output: g_x
// ===========================================================================
template <bool TENSOR_THR, bool GRADED, bool DGRAD>
struct CubaBwd {
  static constexpr int NIN = 2 + (TENSOR_THR ? 1 : 0) + (DGRAD ? 1 : 0), NOUT = 1;
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  // Six stages of one 32-step box measured best without decay gradients (cuba_bwd 0.86 -> 0.90,
  // alif_bwd 0.84 -> 0.89 of copy bandwidth): the reverse scan is short of loads in flight, not of warps.
  // With decay gradients (CUBA: three input tiles) two 32-step boxes and three stages (3.03 -> 2.74 ms).
  SB_PIPE((DGRAD ? 3 : 6), ((DGRAD && NIN == 3) ? 2 : 1), ((DGRAD && NIN > 3) ? 16 : 32));
  static constexpr int ITH = 2, ICUR = 2 + (TENSOR_THR ? 1 : 0);
  struct Params {
    DecayVec cdecay, vdecay;
    Surrogate sg;
    float thr;            // scalar threshold (fp32), ignored with a tensor threshold
    double* partial_c;    // scratch for grad of current decay
    double* partial_v;    // scratch for grad of voltage decay
    int spike_delay;      // 1: the forward wrote spikes one step late, so g_spike[t] is read from t + 1
  };
  float ac, av, gv, gx, thr, gnext;
  bool delayed;
  Surrogate sg;
  GradAcc accc, accv;

  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    gv = gx = 0.f; ac = av = 0.f; thr = p.thr; sg = p.sg; accc.reset(); accv.reset();
    gnext = 0.f; delayed = p.spike_delay != 0;
    if (valid) {
      ac = __fsub_rn(1.f, __fdiv_rn(load_decay(p.cdecay, g, row), 4096.f));
      av = __fsub_rn(1.f, __fdiv_rn(load_decay(p.vdecay, g, row), 4096.f));
    }
  }
  __device__ __forceinline__ void step(const float (&a)[NIN], float (&b)[1]) {
    const float vol = a[1];
    const float th = TENSOR_THR ? a[ITH] : thr;
    // the scan runs backwards, so the gradient of the delayed spike (time t + 1) was the previous input
    const float gin = delayed ? gnext : a[0];
    gnext = a[0];
    const float gs = __fmul_rn(surrogate<GRADED>(sg, vol, th), gin);
    if (DGRAD) {
      accv.add(__fmul_rn(gv, vol));
      accc.add(__fmul_rn(gx, a[ICUR]));
    }
    gv = __fadd_rn(__fmul_rn(av, gv), gs);
    gx = __fadd_rn(__fmul_rn(ac, gx), gv);
    b[0] = gx;
  }
  __device__ __forceinline__ void tile_end() { if (DGRAD) { accc.flush(); accv.flush(); } }
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int lane,
                                         int64_t warp_id) {
    if (DGRAD) {
      store_partial(p.partial_c, p.cdecay.n <= 1, accc.d, valid, lane, row, warp_id);
      store_partial(p.partial_v, p.vdecay.n <= 1, accv.d, valid, lane, row, warp_id);
    }
  }
};

// ===========================================================================
// Fused ALIF forward: neuron/alif.py:383-591 with norm=None
//   current = LI(x); voltage = LI(current) (no reset); (th, ref) = ATh(voltage)
//   spike = voltage >= th + ref   (fp32 comparison of the returned series)
// DYN: outputs current, voltage, threshold, refractory (what dynamics() returns)
// else: outputs voltage, threshold + refractory, spike (what forward() needs)
// LEAN: binary spikes only (forward() when nothing will be differentiated: the
//       voltage and threshold series are what the backward pass reads)
// MARGIN: outputs voltage - (threshold + refractory), spike.  The surrogate gradient of the spike reads
//       nothing but that difference (spike/spike.py:10-23), and without learnable decays the reverse
//       scans read nothing else of the forward pass: one series instead of two, in both directions.
// ===========================================================================
template <bool DYN, bool GRADED, bool LEAN = false, bool MARGIN = false>
struct AlifFwd {
  static_assert(!LEAN || (!DYN && !GRADED), "spikes only: forward mode, binary spikes");
  static_assert(!MARGIN || (!DYN && !LEAN), "the margin form is a forward mode");
  static constexpr int NIN = 1, NOUT = LEAN ? 1 : (MARGIN ? 2 : (DYN ? 4 : 3));
  static constexpr bool REVERSE = false;
  // binary spikes leave as bits (which is what lets the block's one-step delay ride on the store);
  // with two boxes per stage that runs as fast as spikes on a TMA tile with four stages of one box
  // (0.777 against 0.779 of copy bandwidth; one box per stage: 0.72)
  static constexpr int NBIT = (!DYN && !GRADED) ? 1 : 0;
  static constexpr bool HAS_FAST = true;
  // LEAN: the stage holds the input only and the step chain, not memory, sets the pace: one box per stage, so that
  // 18 warps fit an SM (0.57 -> 0.68 of copy bandwidth at 8 bytes per step against two boxes)
  // MARGIN (one output tile per stage): five stages of one box, 0.73 -> 0.76 against three stages of three
  SB_PIPE(((MARGIN && NBIT) ? 5 : (DYN ? 3 : (NBIT ? 3 : 4))), ((!DYN && NBIT && !LEAN && !MARGIN) ? 2 : 1), (DYN ? 16 : 32));
  struct Params {
    DecayVec cdecay, vdecay;
    const float* cstate;
    const float* vstate;
    AthParams ath;
    float* final_c; float* final_v; float* final_th; float* final_ref; float* final_s;  // [rows] or null
    float spike_scale;
    Scale sc;
  };
  int c, v, cmul, vmul;
  AthState s;
  float w, inv_w, spike_scale, last_s;
  bool fast_;

  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w; spike_scale = p.spike_scale;
    c = v = 0; cmul = vmul = 4096; last_s = 0.f;
    s.init(p.ath, g, row, valid, w);
    if (valid) {
      cmul = 4096 - (int)load_decay(p.cdecay, g, row);
      vmul = 4096 - (int)load_decay(p.vdecay, g, row);
      c = to_fixed(w, __ldg(p.cstate + row));
      v = to_fixed(w, __ldg(p.vstate + row));
    }
    const bool fs = s.fast_ok();
    fast_ = __all_sync(0xffffffffu, mul_is_decay(cmul) && mul_is_decay(vmul)) && fs;
    if (fast_) { cmul <<= 4; vmul <<= 4; s.use_fast(); }
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[1], float (&b)[NOUT]) {
    c = (FAST ? mul_shift12_pos(c, cmul) : mul_shift12(c, cmul)) + to_fixed(w, a[0]);
    v = (FAST ? mul_shift12_pos(v, vmul) : mul_shift12(v, vmul)) + c;
    s.template decay<FAST>();
    if constexpr ((LEAN || MARGIN) && !GRADED) {
      // The spike compares voltage / w with threshold / w + refractory / w in fp32; w is a power of two here, and
      // scaling by a power of two commutes with fp32 rounding, so the comparison (and the margin, scaled once
      // at the end) is taken on the unscaled conversions: the same bits with two or three multiplies fewer.
      const float vi = __int2float_rn(v);
      const float ti = __fadd_rn(__int2float_rn(s.th_new), __int2float_rn(s.ref_new));
      last_s = (vi >= ti) ? 1.f : 0.f;
      if constexpr (LEAN) {
        b[0] = last_s;
      } else {
        b[0] = __fmul_rn(__fsub_rn(vi, ti), inv_w); b[1] = last_s;
      }
      s.commit(v >= s.th_new + s.ref_new);
      return;
    }
    const float vf = from_fixed<true>(v, w, inv_w);
    const float thf = from_fixed<true>(s.th_new, w, inv_w);
    const float reff = from_fixed<true>(s.ref_new, w, inv_w);
    if (DYN) {
      b[0] = from_fixed<true>(c, w, inv_w); b[1] = vf; b[2] = thf; b[3] = reff;
    } else {
      const float thsum = __fadd_rn(thf, reff);
      const bool sp = vf >= thsum;
      last_s = GRADED ? __fdiv_rn(__fmul_rn(sp ? 1.f : 0.f, vf), spike_scale) : (sp ? 1.f : 0.f);
      if constexpr (LEAN) {
        b[0] = last_s;
      } else if constexpr (MARGIN) {
        b[0] = __fsub_rn(vf, thsum); b[1] = last_s;
      } else {
        b[0] = vf; b[1] = thsum; b[NOUT - 1] = last_s;
      }
    }
    s.commit(v >= s.th_new + s.ref_new);
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (!valid) return;
    if (p.final_c) p.final_c[row] = from_fixed<true>(c, w, inv_w);
    if (p.final_v) p.final_v[row] = from_fixed<true>(v, w, inv_w);
    if (p.final_th) p.final_th[row] = from_fixed<true>(s.th_new, w, inv_w);
    if (p.final_ref) p.final_ref[row] = from_fixed<true>(s.ref_new, w, inv_w);
    if (!DYN && p.final_s) p.final_s[row] = last_s;
  }
};

// ===========================================================================
// Fused resonate-and-fire forward.
//   ADAPT = false: neuron/rf.py (resonator, scalar threshold, complex spike)
//   ADAPT = true : neuron/adrf.py:439-652 (resonator -> adaptive_phase_th ->
//                  complex spike with tensor threshold th + ref)
// Complex spike: spike/complex.py:66-92
//   spike = (re >= thr) * (im[t-1] < 0) * (im >= 0),  im[-1] = imag state
// DYN (ADAPT only): outputs re, im, threshold, refractory
// else            : outputs re, im, [threshold + refractory], spike
// LEAN            : binary spikes only (forward() when nothing will be differentiated)
// MARGIN (ADAPT)  : outputs re - (threshold + refractory), im, spike: the gradient of the complex spike
//                   reads re only through that difference (spike/complex.py:144-167), and without sin / cos
//                   gradients the reverse scan reads nothing else of the forward pass
// ===========================================================================
template <bool ADAPT, bool DYN, bool GRADED, bool LEAN = false, bool MARGIN = false>
struct RfFwd {
  static_assert(ADAPT || !DYN, "DYN needs ADAPT");
  static_assert(!LEAN || (!DYN && !GRADED), "spikes only: forward mode, binary spikes");
  static_assert(!MARGIN || (ADAPT && !DYN && !LEAN), "the margin form belongs to the adaptive forward");
  static constexpr int NIN = 2, NOUT = LEAN ? 1 : (MARGIN ? 3 : (ADAPT ? 4 : 3));
  static constexpr bool REVERSE = false;
  static constexpr int NBIT = (!DYN && !GRADED) ? 1 : 0;
  static constexpr bool HAS_FAST = true;
  // three tiles per stage (adaptive forward): four stages measured best (adrf_fwd 0.78 -> 0.81 of copy bandwidth)
  // LEAN (two input tiles per stage, no output tile): two stages of one box, 14 warps per SM (0.46 -> 0.62)
  // MARGIN (two output tiles): four stages, 0.77 -> 0.82
  SB_PIPE((LEAN ? 2 : (((NOUT - NBIT) == 3 || MARGIN) ? 4 : 3)), 1, ((NOUT - NBIT) >= 4 ? 16 : 32));
  struct Params {
    ResParams res;
    AthParams ath;    // ADAPT only
    int k_spike;      // !ADAPT: spike needs re >= k_spike (float(re)/w >= f32(thr))
    float* final_re; float* final_im; float* final_th; float* final_ref; float* final_s;
    float spike_scale;
    Scale sc;
  };
  ResState r;
  AthState s;
  int k_spike, im_old_i;
  bool im_prev_neg, fast_;
  float w, inv_w, spike_scale, last_s;

  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    w = p.sc.w; inv_w = p.sc.inv_w; k_spike = p.k_spike; spike_scale = p.spike_scale; last_s = 0.f;
    r.init(p.res, g, row, valid, w);
    if (ADAPT) s.init(p.ath, g, row, valid, w);
    im_old_i = r.im;  // int(w * imag_state): adaptive_phase_th.py:258
    im_prev_neg = valid ? (__ldg(p.res.im_state + row) < 0.f) : false;  // complex.py:72
    const bool fr = r.fast_ok();
    bool fs = true;
    if (ADAPT) fs = s.fast_ok();
    fast_ = fr && fs;
    if (fast_) { r.use_fast(); if (ADAPT) s.use_fast(); }
  }
  __device__ __forceinline__ bool fast() const { return fast_; }
  template <bool FAST>
  __device__ __forceinline__ void step_t(const float (&a)[2], float (&b)[NOUT]) {
    r.template advance<FAST>(w, a[0], a[1]);
    r.keep();
    const float ref_ = from_fixed<true>(r.re, w, inv_w);
    const float imf = from_fixed<true>(r.im, w, inv_w);
    if constexpr (ADAPT && (LEAN || MARGIN) && !GRADED) {
      // as in the ALIF kernel: compare (and subtract) before the power-of-two scaling, the same bits
      s.template decay<FAST>();
      const float rei = __int2float_rn(r.re);
      const float ti = __fadd_rn(__int2float_rn(s.th_new), __int2float_rn(s.ref_new));
      const bool sp = (rei >= ti) && im_prev_neg && (r.im >= 0);
      last_s = sp ? 1.f : 0.f;
      if constexpr (LEAN) {
        b[0] = last_s;
      } else {
        b[0] = __fmul_rn(__fsub_rn(rei, ti), inv_w); b[1] = imf; b[2] = last_s;
      }
      s.commit(r.re >= s.th_new + s.ref_new && r.im >= 0 && im_old_i < 0);
      im_old_i = r.im;
      im_prev_neg = r.im < 0;
      return;
    }
    if (ADAPT) {
      s.template decay<FAST>();
      const float thf = from_fixed<true>(s.th_new, w, inv_w);
      const float rff = from_fixed<true>(s.ref_new, w, inv_w);
      if (DYN) {
        b[0] = ref_; b[1] = imf; b[2] = thf; b[3] = rff;
      } else {
        const float thsum = __fadd_rn(thf, rff);
        const bool sp = (ref_ >= thsum) && im_prev_neg && (r.im >= 0);
        last_s = GRADED ? __fdiv_rn(__fmul_rn(sp ? 1.f : 0.f, ref_), spike_scale) : (sp ? 1.f : 0.f);
        if constexpr (LEAN) {
          b[0] = last_s;
        } else if constexpr (MARGIN) {
          b[0] = __fsub_rn(ref_, thsum); b[1] = imf; b[2] = last_s;
        } else {
          b[0] = ref_; b[1] = imf; b[NOUT - 2] = thsum; b[NOUT - 1] = last_s;
        }
      }
      s.commit(r.re >= s.th_new + s.ref_new && r.im >= 0 && im_old_i < 0);
      im_old_i = r.im;
    } else {
      const bool sp = (r.re >= k_spike) && im_prev_neg && (r.im >= 0);
      last_s = GRADED ? __fdiv_rn(__fmul_rn(sp ? 1.f : 0.f, ref_), spike_scale) : (sp ? 1.f : 0.f);
      if constexpr (LEAN) {
        b[0] = last_s;
      } else {
        b[0] = ref_; b[1] = imf; b[NOUT - 1] = last_s;
      }
    }
    im_prev_neg = r.im < 0;
  }
  __device__ __forceinline__ void tile_end() {}
  __device__ __forceinline__ void finish(const Params& p, const RowGeom&, int64_t row, bool valid, int, int64_t) {
    if (!valid) return;
    if (p.final_re) p.final_re[row] = from_fixed<true>(r.re, w, inv_w);
    if (p.final_im) p.final_im[row] = from_fixed<true>(r.im, w, inv_w);
    if (ADAPT && p.final_th) p.final_th[row] = from_fixed<true>(s.th_new, w, inv_w);
    if (ADAPT && p.final_ref) p.final_ref[row] = from_fixed<true>(s.ref_new, w, inv_w);
    if (!DYN && p.final_s) p.final_s[row] = last_s;
  }
};

// ===========================================================================
// Fused backward of RfFwd: complex-spike gradient (spike/complex.py:144-167)
// followed by the reverse rotation scan (resonator.py:379-467).
// Inputs: g_spike, re, im, [threshold tensor]; outputs: g_re_in, g_im_in
// ===========================================================================
template <bool TENSOR_THR, bool GRADED, bool PGRAD>
struct RfBwd {
  static constexpr int NIN = 3 + (TENSOR_THR ? 1 : 0), NOUT = 2;
  static constexpr bool REVERSE = true;
  static constexpr int NBIT = 0;
  // six stages of 16 steps measured best with a threshold series and no sin/cos gradients (0.82 -> 0.87); with a scalar
  // threshold (three input tiles: the plain resonator, and the adaptive one's margin form) four stages of 32 steps (0.85 -> 0.88)
  SB_PIPE((PGRAD ? 3 : (TENSOR_THR ? 6 : 4)), 1, ((PGRAD || TENSOR_THR) ? 16 : 32));
  struct Params {
    DecayVec sin_decay, cos_decay;
    CSurrogate sg;
    float thr;
    double* partial_sin;
    double* partial_cos;
    int spike_delay;      // 1: the forward wrote spikes one step late, so g_spike[t] is read from t + 1
  };
  ResBwd<PGRAD> scan;
  CSurrogate sg;
  float thr, gnext;
  bool delayed;
  __device__ __forceinline__ void init(const Params& p, const RowGeom& g, int64_t row, bool valid) {
    typename ResBwd<PGRAD>::Params rp{p.sin_decay, p.cos_decay, p.partial_sin, p.partial_cos};
    scan.init(rp, g, row, valid);
    sg = p.sg; thr = p.thr; gnext = 0.f; delayed = p.spike_delay != 0;
  }
  __device__ __forceinline__ void step(const float (&a)[NIN], float (&b)[2]) {
    float dre, dim;
    csurrogate<GRADED>(sg, a[1], a[2], TENSOR_THR ? a[NIN - 1] : thr, dre, dim);
    // the scan runs backwards, so the gradient of the delayed spike (time t + 1) was the previous input
    const float gin = delayed ? gnext : a[0];
    gnext = a[0];
    scan.scan(__fmul_rn(gin, dre), __fmul_rn(gin, dim), a[1], a[2]);
    b[0] = scan.gre; b[1] = scan.gim;
  }
  __device__ __forceinline__ void tile_end() { scan.tile_end(); }
  __device__ __forceinline__ void finish(const Params& p, const RowGeom& g, int64_t row, bool valid, int lane,
                                         int64_t warp_id) {
    typename ResBwd<PGRAD>::Params rp{p.sin_decay, p.cos_decay, p.partial_sin, p.partial_cos};
    scan.finish(rp, g, row, valid, lane, warp_id);
  }
};

}  // namespace sb
