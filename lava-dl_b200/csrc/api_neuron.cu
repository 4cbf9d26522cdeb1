// Entry points for the fused neuron passes: what Neuron.forward() /
// Neuron.dynamics() of neuron/{cuba,alif,rf,adrf}.py compute with several
// dynamics calls plus a spike function, done in one walk over time.
#include <limits.h>

#include "api_util.cuh"
#include "reduce.cuh"
#include "recurrent.cuh"
#include "rowscan.cuh"

using namespace sb;

static int64_t maxn(std::initializer_list<int64_t> v) {
  int64_t m = 1;
  for (int64_t x : v) m = x > m ? x : m;
  return m;
}
static bool counts_ok(std::initializer_list<int64_t> v, int64_t nmax) {
  for (int64_t x : v)
    if (!(x == 1 || x == nmax)) return false;
  return true;
}

static Surrogate make_surrogate(float tau_rho, float scale_rho, bool graded) {
  // fp32 arithmetic in the order spike/spike.py:10-23 applies it to 0-dim fp32 tensors
  Surrogate s;
  s.k2 = (float)(1.4426950408889634 / (double)tau_rho);
  volatile float half = scale_rho / 2.0f;
  volatile float c = half / tau_rho;
  s.c0 = graded ? scale_rho : c;
  return s;
}

static CSurrogate make_csurrogate(float tau_rho, float scale_rho) {
  // spike/complex.py:144-167, again in fp32
  CSurrogate s;
  s.k2 = (float)(1.4426950408889634 / (double)tau_rho);
  s.scale_rho = scale_rho;
  volatile float a = 0.5f / tau_rho;
  volatile float b = 2.0f * tau_rho;
  volatile float c = (-scale_rho) / tau_rho;
  s.half_over_tau = a;
  s.two_tau = b;
  s.neg_scale_over_tau = c;
  return s;
}

extern "C" {

int sb_cuba_fwd(const float* x, const float* cdecay, int64_t n_cdecay, const float* vdecay, int64_t n_vdecay,
                const float* cstate, const float* vstate, float* current, float* voltage, float* spike,
                float* final_c, float* final_v, float* final_s, const sb_geom* g, double threshold,
                int w_scale, int graded, float spike_scale, int spike_delay, const float* delay_head,
                const float* axon_delay, int64_t n_axon_delay, float axon_delay_ts, void* stream) {
  RowGeom rg;
  SB_REQUIRE(spike_delay == 0 || (spike_delay == 1 && spike != nullptr && !graded),
             "the fused one-step delay needs binary spike output");
  SB_REQUIRE(axon_delay == nullptr || (spike != nullptr && !graded && n_axon_delay > 0 && axon_delay_ts != 0.f),
             "the fused axonal delay needs binary spike output, a delay table and a non-zero sampling time");
  const BitDelay bd{spike_delay, delay_head, axon_delay, n_axon_delay, axon_delay_ts};
  SB_TRY(check_count(n_cdecay, "current decay"));
  SB_TRY(check_count(n_vdecay, "voltage decay"));
  const int64_t nmax = maxn({n_cdecay, n_vdecay});
  SB_TRY(check_geom(g, &rg, nmax));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(counts_ok({n_cdecay, n_vdecay}, nmax), "decay counts disagree");
  SB_REQUIRE(w_scale > 0 && is_pow2(w_scale), "fused kernels need a power-of-two w_scale (got %d)", w_scale);
  SB_REQUIRE(cdecay && vdecay && cstate && vstate, "null parameter pointer");
  SB_REQUIRE(voltage != nullptr || (spike != nullptr && !graded && current == nullptr),
             "without the voltage series only binary spikes can be returned");
  const Scale sc = make_scale(w_scale);
  // reset: int64 voltage >= Python float (thr * w_scale), evaluated in fp32 (leaky_integrator.py:218-225)
  const float thr_scaled = (float)(threshold * (double)w_scale);
  const int k_reset = thr_scaled > 0.f ? int_threshold_ge(thr_scaled) : INT_MAX;
  // spike: fp32 voltage >= fp32(threshold) (spike/spike.py:86-88)
  const int k_spike = int_threshold_ge_scaled((float)threshold, sc.w);
  cudaStream_t st = (cudaStream_t)stream;
  const float* in[1] = {x};
#define SB_GO(C, S, G)                                                                              \
  {                                                                                                 \
    typename CubaFwd<C, S, G>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate,     \
                                        final_c, final_v, final_s, k_reset, k_spike, spike_scale, sc}; \
    float* out[3];                                                                                  \
    int no = 0;                                                                                     \
    if (C) out[no++] = current;                                                                     \
    out[no++] = voltage;                                                                            \
    if (S) out[no++] = spike;                                                                       \
    return launch_rowscan<CubaFwd<C, S, G>>(p, rg, in, out, st, bd);                                \
  }
  if (voltage == nullptr) {
    // inference: spikes only (x in, fp32 spikes out, 8 bytes per neuron-step instead of 12)
    typename CubaFwd<false, true, false, false>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate,
                                                           final_c, final_v, final_s, k_reset, k_spike, spike_scale, sc};
    float* out[1] = {spike};
    return launch_rowscan<CubaFwd<false, true, false, false>>(p, rg, in, out, st, bd);
  }
  if (current) {
    if (spike) { if (graded) SB_GO(true, true, true) else SB_GO(true, true, false) }
    else SB_GO(true, false, false)
  } else {
    if (spike) { if (graded) SB_GO(false, true, true) else SB_GO(false, true, false) }
    else SB_GO(false, false, false)
  }
#undef SB_GO
}

int sb_cuba_fwd_packed(const float* x, const float* cdecay, int64_t n_cdecay, const float* vdecay,
                       int64_t n_vdecay, const float* cstate, const float* vstate, float* voltage,
                       uint32_t* spike_bits, float* final_c, float* final_v, float* final_s, const sb_geom* g,
                       double threshold, int w_scale, int spike_delay, const float* delay_head, void* stream) {
  RowGeom rg;
  SB_REQUIRE(spike_delay == 0 || spike_delay == 1, "spike_delay is 0 or 1");
  SB_TRY(check_count(n_cdecay, "current decay"));
  SB_TRY(check_count(n_vdecay, "voltage decay"));
  const int64_t nmax = maxn({n_cdecay, n_vdecay});
  SB_TRY(check_geom(g, &rg, nmax));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  SB_REQUIRE(counts_ok({n_cdecay, n_vdecay}, nmax), "decay counts disagree");
  SB_REQUIRE(w_scale > 0 && is_pow2(w_scale), "fused kernels need a power-of-two w_scale (got %d)", w_scale);
  SB_REQUIRE(cdecay && vdecay && cstate && vstate, "null parameter pointer");
  SB_REQUIRE(spike_bits != nullptr, "the packed spike output is required");
  SB_REQUIRE((reinterpret_cast<uintptr_t>(spike_bits) & 3u) == 0, "spike_bits must be 4-byte aligned");
  const Scale sc = make_scale(w_scale);
  const float thr_scaled = (float)(threshold * (double)w_scale);
  const int k_reset = thr_scaled > 0.f ? int_threshold_ge(thr_scaled) : INT_MAX;
  const int k_spike = int_threshold_ge_scaled((float)threshold, sc.w);
  BitDelay bd{spike_delay, delay_head, nullptr, 0, 1.f};
  bd.packed = spike_bits;
  cudaStream_t st = (cudaStream_t)stream;
  const float* in[1] = {x};
  if (voltage != nullptr) {
    typename CubaFwd<false, true, false, true>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate,
                                                          final_c, final_v, final_s, k_reset, k_spike, 1.f, sc};
    float* out[2] = {voltage, nullptr};
    return launch_rowscan<CubaFwd<false, true, false, true>>(p, rg, in, out, st, bd);
  }
  typename CubaFwd<false, true, false, false>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate,
                                                         final_c, final_v, final_s, k_reset, k_spike, 1.f, sc};
  float* out[1] = {nullptr};
  return launch_rowscan<CubaFwd<false, true, false, false>>(p, rg, in, out, st, bd);
}

int sb_cuba_bwd(const float* grad_spike, const float* voltage, const float* thr_tensor, float thr,
                const float* current, const float* cdecay, int64_t n_cdecay, const float* vdecay,
                int64_t n_vdecay, float* grad_x, float* grad_cdecay, float* grad_vdecay, void* scratch_c,
                void* scratch_v, const sb_geom* g, float tau_rho, float scale_rho, int graded, int spike_delay,
                void* stream) {
  RowGeom rg;
  SB_REQUIRE(spike_delay == 0 || spike_delay == 1, "spike_delay is 0 or 1");
  SB_TRY(check_count(n_cdecay, "current decay"));
  SB_TRY(check_count(n_vdecay, "voltage decay"));
  const int64_t nmax = maxn({n_cdecay, n_vdecay});
  SB_TRY(check_geom(g, &rg, nmax));
  SB_REQUIRE(counts_ok({n_cdecay, n_vdecay}, nmax), "decay counts disagree");
  SB_REQUIRE(cdecay && vdecay, "null parameter pointer");
  SB_REQUIRE((grad_cdecay == nullptr) == (grad_vdecay == nullptr), "decay gradients come together");
  const bool dgrad = grad_cdecay != nullptr;
  if (dgrad)
    SB_REQUIRE(current && scratch_c && scratch_v && scratch_c != scratch_v,
               "decay gradients need the saved current and two scratch areas");
  cudaStream_t st = (cudaStream_t)stream;
  if (dgrad && (rg.rows == 0 || rg.T == 0)) {
    SB_CUDA(cudaMemsetAsync(grad_cdecay, 0, sizeof(float) * n_cdecay, st));
    SB_CUDA(cudaMemsetAsync(grad_vdecay, 0, sizeof(float) * n_vdecay, st));
    return SB_OK;
  }
  const Surrogate sg = make_surrogate(tau_rho, scale_rho, graded != 0);
  float* out[1] = {grad_x};
#define SB_GO(TT, G, D)                                                                             \
  {                                                                                                 \
    typename CubaBwd<TT, G, D>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, sg, thr,           \
                                         (double*)scratch_c, (double*)scratch_v, spike_delay};      \
    const float* in[4];                                                                             \
    int ni = 0;                                                                                     \
    in[ni++] = grad_spike;                                                                          \
    in[ni++] = voltage;                                                                             \
    if (TT) in[ni++] = thr_tensor;                                                                  \
    if (D) in[ni++] = current;                                                                      \
    SB_TRY((launch_rowscan<CubaBwd<TT, G, D>>(p, rg, in, out, st)));                                \
  }
  const bool tt = thr_tensor != nullptr;
  if (tt) {
    if (graded) { if (dgrad) SB_GO(true, true, true) else SB_GO(true, true, false) }
    else        { if (dgrad) SB_GO(true, false, true) else SB_GO(true, false, false) }
  } else {
    if (graded) { if (dgrad) SB_GO(false, true, true) else SB_GO(false, true, false) }
    else        { if (dgrad) SB_GO(false, false, true) else SB_GO(false, false, false) }
  }
#undef SB_GO
  if (dgrad) {
    SB_TRY(fold_param_grad((double*)scratch_c, grad_cdecay, rg, n_cdecay, st));
    SB_TRY(fold_param_grad((double*)scratch_v, grad_vdecay, rg, n_vdecay, st));
  }
  return SB_OK;
}

int sb_alif_fwd(const float* x, const float* cdecay, int64_t n_cdecay, const float* vdecay, int64_t n_vdecay,
                const float* ref_decay, int64_t n_ref_decay, const float* th_decay, int64_t n_th_decay,
                const float* cstate, const float* vstate, const float* ref_state, const float* th_state,
                float* out0, float* out1, float* out2, float* out3, float* final_c, float* final_v,
                float* final_th, float* final_ref, float* final_s, const sb_geom* g, int th_step, int th0,
                int w_scale, int mode, int graded, float spike_scale, int spike_delay, const float* delay_head,
                void* stream) {
  RowGeom rg;
  SB_REQUIRE(spike_delay == 0 || (spike_delay == 1 && mode == 0 && !graded),
             "the fused one-step delay needs forward mode and binary spikes");
  const BitDelay bd{spike_delay, delay_head, nullptr, 0, 1.f};
  SB_TRY(check_count(n_cdecay, "current decay"));
  SB_TRY(check_count(n_vdecay, "voltage decay"));
  SB_TRY(check_count(n_ref_decay, "refractory decay"));
  SB_TRY(check_count(n_th_decay, "threshold decay"));
  const int64_t nmax = maxn({n_cdecay, n_vdecay, n_ref_decay, n_th_decay});
  SB_TRY(check_geom(g, &rg, nmax));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(counts_ok({n_cdecay, n_vdecay, n_ref_decay, n_th_decay}, nmax), "decay counts disagree");
  SB_REQUIRE(w_scale > 0 && is_pow2(w_scale), "fused kernels need a power-of-two w_scale (got %d)", w_scale);
  SB_REQUIRE(cdecay && vdecay && ref_decay && th_decay && cstate && vstate && ref_state && th_state,
             "null parameter pointer");
  SB_REQUIRE(mode == 0 || mode == 1, "mode must be 0 (forward) or 1 (dynamics)");
  const Scale sc = make_scale(w_scale);
  AthParams ap{{ref_decay, n_ref_decay}, {th_decay, n_th_decay}, ref_state, th_state, th_step, th0};
  cudaStream_t st = (cudaStream_t)stream;
  const float* in[1] = {x};
  // kernel order in forward mode: voltage, threshold + refractory, spike
  float* out[4] = {out0, out1, out2, out3};
  if (mode == 0) { out[0] = out1; out[1] = out2; out[2] = out0; out[3] = nullptr; }
#define SB_GO(D, G)                                                                                  \
  {                                                                                                  \
    typename AlifFwd<D, G>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate, ap,     \
                                     final_c, final_v, final_th, final_ref, final_s, spike_scale, sc}; \
    return launch_rowscan<AlifFwd<D, G>>(p, rg, in, out, st, bd);                                    \
  }
  if (mode == 0 && out1 == nullptr && out2 == nullptr) {
    // inference: spikes only (voltage and threshold series are what the backward pass reads)
    SB_REQUIRE(!graded && out0 != nullptr, "without the voltage and threshold series only binary spikes can be returned");
    typename AlifFwd<false, false, true>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate, ap,
                                                    final_c, final_v, final_th, final_ref, final_s, spike_scale, sc};
    float* lean[1] = {out0};
    return launch_rowscan<AlifFwd<false, false, true>>(p, rg, in, lean, st, bd);
  }
  if (mode == 0 && out1 != nullptr && out2 == nullptr) {
    // training without learnable decays: out1 = voltage - (threshold + refractory), all the backward pass reads
    float* two[2] = {out1, out0};
    if (graded) {
      typename AlifFwd<false, true, false, true>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate, ap,
                                                           final_c, final_v, final_th, final_ref, final_s, spike_scale, sc};
      return launch_rowscan<AlifFwd<false, true, false, true>>(p, rg, in, two, st, bd);
    }
    typename AlifFwd<false, false, false, true>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate, ap,
                                                          final_c, final_v, final_th, final_ref, final_s, spike_scale, sc};
    return launch_rowscan<AlifFwd<false, false, false, true>>(p, rg, in, two, st, bd);
  }
  if (mode == 1) SB_GO(true, false)
  else if (graded) SB_GO(false, true)
  else SB_GO(false, false)
#undef SB_GO
}

int sb_rf_fwd(const float* re_in, const float* im_in, const float* sin_decay, const float* cos_decay,
              int64_t n_decay, const float* ref_decay, int64_t n_ref_decay, const float* th_decay,
              int64_t n_th_decay, const float* re_state, const float* im_state, const float* ref_state,
              const float* th_state, float* out0, float* out1, float* out2, float* out3, float* final_re,
              float* final_im, float* final_th, float* final_ref, float* final_s, const sb_geom* g,
              float threshold, int th_step, int th0, int w_scale, int adapt, int mode, int graded,
              float spike_scale, int spike_delay, const float* delay_head, void* stream) {
  RowGeom rg;
  SB_REQUIRE(spike_delay == 0 || (spike_delay == 1 && mode == 0 && !graded),
             "the fused one-step delay needs forward mode and binary spikes");
  const BitDelay bd{spike_delay, delay_head, nullptr, 0, 1.f};
  SB_TRY(check_count(n_decay, "sin/cos decay"));
  if (!adapt) { n_ref_decay = 1; n_th_decay = 1; }
  SB_TRY(check_count(n_ref_decay, "refractory decay"));
  SB_TRY(check_count(n_th_decay, "threshold decay"));
  const int64_t nmax = maxn({n_decay, n_ref_decay, n_th_decay});
  SB_TRY(check_geom(g, &rg, nmax));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(counts_ok({n_decay, n_ref_decay, n_th_decay}, nmax), "parameter counts disagree");
  SB_REQUIRE(w_scale > 0 && is_pow2(w_scale), "fused kernels need a power-of-two w_scale (got %d)", w_scale);
  SB_REQUIRE(sin_decay && cos_decay && re_state && im_state, "null parameter pointer");
  SB_REQUIRE(!adapt || (ref_decay && th_decay && ref_state && th_state), "null adaptive parameter pointer");
  SB_REQUIRE(mode == 0 || (mode == 1 && adapt), "mode 1 (dynamics) exists only for the adaptive neuron");
  const Scale sc = make_scale(w_scale);
  ResParams rp{{sin_decay, n_decay}, {cos_decay, n_decay}, re_state, im_state};
  AthParams ap{{ref_decay, n_ref_decay}, {th_decay, n_th_decay}, ref_state, th_state, th_step, th0};
  const int k_spike = int_threshold_ge_scaled(threshold, sc.w);
  cudaStream_t st = (cudaStream_t)stream;
  const float* in[2] = {re_in, im_in};
  // kernel order in forward mode: re, im, [threshold + refractory], spike
  float* out[4] = {out0, out1, out2, out3};
  if (mode == 0) {
    if (adapt) { out[0] = out1; out[1] = out2; out[2] = out3; out[3] = out0; }
    else { out[0] = out1; out[1] = out2; out[2] = out0; out[3] = nullptr; }
  }
#define SB_GO(A, D, G)                                                                               \
  {                                                                                                  \
    typename RfFwd<A, D, G>::Params p{rp, ap, k_spike, final_re, final_im, final_th, final_ref,      \
                                      final_s, spike_scale, sc};                                     \
    return launch_rowscan<RfFwd<A, D, G>>(p, rg, in, out, st, bd);                                   \
  }
  if (mode == 0 && out1 == nullptr && out2 == nullptr && out3 == nullptr) {
    // inference: spikes only
    SB_REQUIRE(!graded && out0 != nullptr, "without the state series only binary spikes can be returned");
    float* lean[1] = {out0};
    if (adapt) {
      typename RfFwd<true, false, false, true>::Params p{rp, ap, k_spike, final_re, final_im, final_th, final_ref,
                                                          final_s, spike_scale, sc};
      return launch_rowscan<RfFwd<true, false, false, true>>(p, rg, in, lean, st, bd);
    }
    typename RfFwd<false, false, false, true>::Params p{rp, ap, k_spike, final_re, final_im, final_th, final_ref,
                                                         final_s, spike_scale, sc};
    return launch_rowscan<RfFwd<false, false, false, true>>(p, rg, in, lean, st, bd);
  }
  if (adapt && mode == 0 && out1 != nullptr && out2 != nullptr && out3 == nullptr) {
    // training without sin / cos gradients: out1 = re - (threshold + refractory), out2 = im
    float* three[3] = {out1, out2, out0};
    if (graded) {
      typename RfFwd<true, false, true, false, true>::Params p{rp, ap, k_spike, final_re, final_im, final_th, final_ref,
                                                                final_s, spike_scale, sc};
      return launch_rowscan<RfFwd<true, false, true, false, true>>(p, rg, in, three, st, bd);
    }
    typename RfFwd<true, false, false, false, true>::Params p{rp, ap, k_spike, final_re, final_im, final_th, final_ref,
                                                               final_s, spike_scale, sc};
    return launch_rowscan<RfFwd<true, false, false, false, true>>(p, rg, in, three, st, bd);
  }
  if (adapt) {
    if (mode == 1) SB_GO(true, true, false)
    else if (graded) SB_GO(true, false, true)
    else SB_GO(true, false, false)
  } else {
    if (graded) SB_GO(false, false, true)
    else SB_GO(false, false, false)
  }
#undef SB_GO
}

int sb_rf_bwd(const float* grad_spike, const float* re, const float* im, const float* thr_tensor, float thr,
              const float* sin_decay, const float* cos_decay, int64_t n_decay, float* grad_re_in,
              float* grad_im_in, float* grad_sin, float* grad_cos, void* scratch_sin, void* scratch_cos,
              const sb_geom* g, float tau_rho, float scale_rho, int graded, int spike_delay, void* stream) {
  RowGeom rg;
  SB_REQUIRE(spike_delay == 0 || spike_delay == 1, "spike_delay is 0 or 1");
  SB_TRY(check_count(n_decay, "sin/cos decay"));
  SB_TRY(check_geom(g, &rg, n_decay));
  SB_REQUIRE(sin_decay && cos_decay, "null parameter pointer");
  SB_REQUIRE((grad_sin == nullptr) == (grad_cos == nullptr), "grad_sin and grad_cos come together");
  const bool pgrad = grad_sin != nullptr;
  if (pgrad)
    SB_REQUIRE(scratch_sin && scratch_cos && scratch_sin != scratch_cos, "parameter gradients need two scratch areas");
  cudaStream_t st = (cudaStream_t)stream;
  if (pgrad && (rg.rows == 0 || rg.T == 0)) {
    SB_CUDA(cudaMemsetAsync(grad_sin, 0, sizeof(float) * n_decay, st));
    SB_CUDA(cudaMemsetAsync(grad_cos, 0, sizeof(float) * n_decay, st));
    return SB_OK;
  }
  const CSurrogate sg = make_csurrogate(tau_rho, scale_rho);
  float* out[2] = {grad_re_in, grad_im_in};
#define SB_GO(TT, G, P)                                                                              \
  {                                                                                                  \
    typename RfBwd<TT, G, P>::Params p{{sin_decay, n_decay}, {cos_decay, n_decay}, sg, thr,          \
                                       (double*)scratch_sin, (double*)scratch_cos, spike_delay};     \
    const float* in[4] = {grad_spike, re, im, thr_tensor};                                           \
    SB_TRY((launch_rowscan<RfBwd<TT, G, P>>(p, rg, in, out, st)));                                   \
  }
  const bool tt = thr_tensor != nullptr;
  if (tt) {
    if (graded) { if (pgrad) SB_GO(true, true, true) else SB_GO(true, true, false) }
    else        { if (pgrad) SB_GO(true, false, true) else SB_GO(true, false, false) }
  } else {
    if (graded) { if (pgrad) SB_GO(false, true, true) else SB_GO(false, true, false) }
    else        { if (pgrad) SB_GO(false, false, true) else SB_GO(false, false, false) }
  }
#undef SB_GO
  if (pgrad) {
    SB_TRY(fold_param_grad((double*)scratch_sin, grad_sin, rg, n_decay, st));
    SB_TRY(fold_param_grad((double*)scratch_cos, grad_cos, rg, n_decay, st));
  }
  return SB_OK;
}

int sb_cuba_recurrent_fwd(const float* z, const float* rec_t, const float* cdecay, int64_t n_cdecay,
                          const float* vdecay, int64_t n_vdecay, const float* cstate, const float* vstate,
                          float* voltage, float* spike, float* final_c, float* final_v, float* final_s,
                          int64_t batch, int64_t neurons, int64_t T, double threshold, int w_scale, int graded,
                          float spike_scale, void* stream) {
  SB_REQUIRE(batch >= 0 && neurons >= 0 && T >= 0 && T <= INT_MAX, "negative or oversized extent");
  if (batch == 0 || neurons == 0 || T == 0) return SB_OK;
  SB_REQUIRE(neurons <= 1024, "the recurrent kernel holds one neuron per thread: at most 1024 neurons (got %lld)",
             (long long)neurons);
  SB_REQUIRE(batch <= INT_MAX, "batch too large");
  SB_TRY(check_count(n_cdecay, "current decay"));
  SB_TRY(check_count(n_vdecay, "voltage decay"));
  SB_REQUIRE((n_cdecay == 1 || n_cdecay == neurons) && (n_vdecay == 1 || n_vdecay == neurons),
             "decays are shared or one per neuron");
  SB_REQUIRE(w_scale > 0 && is_pow2(w_scale), "fused kernels need a power-of-two w_scale (got %d)", w_scale);
  SB_REQUIRE(z && rec_t && cdecay && vdecay && cstate && vstate && voltage && spike, "null pointer");
  const RowGeom rg{batch * neurons, neurons, 1, (int)T};
  const Scale sc = make_scale(w_scale);
  // Every step of the reference is a Neuron call with T = 1, so the reset between steps is the state
  // hand-over voltage * (1 - spike) (leaky_integrator.py persistent_state), i.e. the spike criterion.
  const int k_spike = int_threshold_ge_scaled((float)threshold, sc.w);
  const int k_reset = k_spike;
  const int C = (int)neurons, threads = (C + 31) / 32 * 32;
  const size_t smem = rec_fwd_smem(C);
  cudaStream_t st = (cudaStream_t)stream;
#define SB_GO(G)                                                                                             \
  {                                                                                                          \
    typename CubaFwd<false, true, G>::Params p{{cdecay, n_cdecay}, {vdecay, n_vdecay}, cstate, vstate,        \
                                               final_c, final_v, final_s, k_reset, k_spike, spike_scale, sc}; \
    SB_CUDA(cudaFuncSetAttribute(cuba_recurrent_fwd_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                 (int)smem));                                                                \
    cuba_recurrent_fwd_kernel<G><<<(unsigned)batch, threads, smem, st>>>(p, rg, z, rec_t, voltage, spike, C); \
  }
  if (graded) SB_GO(true) else SB_GO(false)
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_cuba_recurrent_bwd(const float* grad_spike, const float* voltage, const float* rec, float* grad_z,
                          int64_t batch, int64_t neurons, int64_t T, float threshold, float tau_rho,
                          float scale_rho, int graded, void* stream) {
  SB_REQUIRE(batch >= 0 && neurons >= 0 && T >= 0 && T <= INT_MAX, "negative or oversized extent");
  if (batch == 0 || neurons == 0 || T == 0) return SB_OK;
  SB_REQUIRE(neurons <= 1024, "the recurrent kernel holds one neuron per thread: at most 1024 neurons (got %lld)",
             (long long)neurons);
  SB_REQUIRE(batch <= INT_MAX, "batch too large");
  SB_REQUIRE(grad_spike && voltage && rec && grad_z, "null pointer");
  const RowGeom rg{batch * neurons, neurons, 1, (int)T};
  const Surrogate sg = make_surrogate(tau_rho, scale_rho, graded != 0);
  const int C = (int)neurons, threads = (C + 31) / 32 * 32;
  // Two samples per CTA share every load of R.  One CTA's walk gets about 1.2x slower that way (measured at
  // batch 128, 512 neurons: 5.5 -> 6.6 ms), so it pays only when it saves a wave of CTAs: batch > SM count.
  const int S = (batch > sm_count() && rec_bwd_smem(C, 2) <= 200 * 1024) ? 2 : 1;
  const size_t smem = rec_bwd_smem(C, S);
  const unsigned grid = (unsigned)((batch + S - 1) / S);
  cudaStream_t st = (cudaStream_t)stream;
  // 16-byte loads of R need whole column quads and an aligned matrix; partial sums are 16-byte stores too
  const bool vec = (C % 4 == 0) && ((reinterpret_cast<uintptr_t>(rec) & 15u) == 0);
#define SB_GO(G, SS, V)                                                                                     \
  {                                                                                                         \
    SB_CUDA(cudaFuncSetAttribute(cuba_recurrent_bwd_kernel<G, SS, V>,                                       \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                  \
    cuba_recurrent_bwd_kernel<G, SS, V><<<grid, threads, smem, st>>>(sg, threshold, rg, grad_spike, voltage, \
                                                                     rec, grad_z, C, (int)batch);           \
  }
#define SB_GO2(G, SS) { if (vec) SB_GO(G, SS, true) else SB_GO(G, SS, false) }
  if (S == 2) { if (graded) SB_GO2(true, 2) else SB_GO2(false, 2) }
  else        { if (graded) SB_GO2(true, 1) else SB_GO2(false, 1) }
#undef SB_GO2
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // extern "C"
