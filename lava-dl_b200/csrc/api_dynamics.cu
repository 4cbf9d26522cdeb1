// Entry points for the un-fused dynamics primitives (what the public
// dynamics(...) functions of lava-dl call one by one).
#include <limits.h>

#include "api_util.cuh"
#include "reduce.cuh"
#include "rowscan.cuh"

namespace sb {

int check_geom(const sb_geom* g, RowGeom* out, int64_t n_max) {
  SB_REQUIRE(g != nullptr, "geometry is null");
  SB_REQUIRE(g->rows >= 0 && g->T >= 0, "negative geometry (rows=%lld, T=%lld)", (long long)g->rows,
             (long long)g->T);
  SB_REQUIRE(g->T <= INT_MAX, "T too large");
  out->rows = g->rows;
  out->T = (int)g->T;
  out->rows_per_batch = g->rows_per_batch > 0 ? g->rows_per_batch : 1;
  out->decay_block = g->decay_block > 0 ? g->decay_block : 1;
  if (n_max > 1) {
    SB_REQUIRE(g->rows_per_batch > 0 && g->decay_block > 0 && g->rows % g->rows_per_batch == 0,
               "per-channel parameters need rows_per_batch/decay_block (rows=%lld rpb=%lld blk=%lld)",
               (long long)g->rows, (long long)g->rows_per_batch, (long long)g->decay_block);
    SB_REQUIRE(g->rows_per_batch == n_max * g->decay_block,
               "parameter count %lld does not match channels %lld", (long long)n_max,
               (long long)(g->rows_per_batch / g->decay_block));
  }
  return SB_OK;
}

Scale make_scale(int w_scale) {
  Scale s;
  s.w = (float)w_scale;
  s.inv_w = 1.0f / (float)w_scale;
  return s;
}

int check_count(int64_t n, const char* name) {
  SB_REQUIRE(n >= 1, "%s count must be >= 1 (got %lld)", name, (long long)n);
  return SB_OK;
}

}  // namespace sb

using namespace sb;

static int64_t max3(int64_t a, int64_t b, int64_t c) { return a > b ? (a > c ? a : c) : (b > c ? b : c); }

extern "C" {

int sb_li_fwd(const float* x, const float* decay, int64_t n_decay, const float* state, float* y,
              float* final_state, const sb_geom* g, float thr_scaled, int w_scale, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_decay, "decay"));
  SB_TRY(check_geom(g, &rg, n_decay));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(w_scale > 0, "w_scale must be positive");
  SB_REQUIRE(decay && state, "null parameter pointer");
  const bool reset = thr_scaled > 0.f;
  const bool pow2 = is_pow2(w_scale);
  const float* in[1] = {x};
  float* out[1] = {y};
  cudaStream_t st = (cudaStream_t)stream;
#define SB_GO(R, P)                                                                      \
  {                                                                                      \
    typename LiFwd<R, P>::Params p{{decay, n_decay}, state, final_state,                 \
                                   reset ? int_threshold_ge(thr_scaled) : INT_MAX, make_scale(w_scale)}; \
    return launch_rowscan<LiFwd<R, P>>(p, rg, in, out, st);                              \
  }
  if (reset) { if (pow2) SB_GO(true, true) else SB_GO(true, false) }
  else       { if (pow2) SB_GO(false, true) else SB_GO(false, false) }
#undef SB_GO
}

int sb_li_bwd(const float* grad_y, const float* y, const float* decay, int64_t n_decay, float* grad_x,
              float* grad_decay, void* scratch, const sb_geom* g, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_decay, "decay"));
  SB_TRY(check_geom(g, &rg, n_decay));
  SB_REQUIRE(decay, "null decay");
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_decay) {
    SB_REQUIRE(y && scratch, "grad_decay needs the saved output and scratch");
    if (rg.rows == 0 || rg.T == 0) {
      SB_CUDA(cudaMemsetAsync(grad_decay, 0, sizeof(float) * n_decay, st));
      return SB_OK;
    }
    const float* in[2] = {grad_y, y};
    float* out[1] = {grad_x};
    LiBwd<true>::Params p{{decay, n_decay}, (double*)scratch};
    SB_TRY((launch_rowscan<LiBwd<true>>(p, rg, in, out, st)));
    return fold_param_grad((double*)scratch, grad_decay, rg, n_decay, st);
  }
  const float* in[1] = {grad_y};
  float* out[1] = {grad_x};
  LiBwd<false>::Params p{{decay, n_decay}, nullptr};
  return launch_rowscan<LiBwd<false>>(p, rg, in, out, st);
}

int sb_ath_fwd(const float* x, const float* ref_state, const float* ref_decay, int64_t n_ref_decay,
               const float* th_state, const float* th_decay, int64_t n_th_decay, float* threshold,
               float* refractory, const sb_geom* g, int th_step, int th0, int w_scale, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_ref_decay, "ref_decay"));
  SB_TRY(check_count(n_th_decay, "th_decay"));
  SB_TRY(check_geom(g, &rg, n_ref_decay > n_th_decay ? n_ref_decay : n_th_decay));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(n_ref_decay == 1 || n_th_decay == 1 || n_ref_decay == n_th_decay, "decay counts disagree");
  SB_REQUIRE(w_scale > 0, "w_scale must be positive");
  SB_REQUIRE(ref_state && ref_decay && th_state && th_decay, "null parameter pointer");
  const float* in[1] = {x};
  float* out[2] = {threshold, refractory};
  AthParams ap{{ref_decay, n_ref_decay}, {th_decay, n_th_decay}, ref_state, th_state, th_step, th0};
  cudaStream_t st = (cudaStream_t)stream;
  if (is_pow2(w_scale)) {
    AthFwd<true>::Params p{ap, make_scale(w_scale)};
    return launch_rowscan<AthFwd<true>>(p, rg, in, out, st);
  }
  AthFwd<false>::Params p{ap, make_scale(w_scale)};
  return launch_rowscan<AthFwd<false>>(p, rg, in, out, st);
}

int sb_apth_fwd(const float* re, const float* im, const float* im_state, const float* ref_state,
                const float* ref_decay, int64_t n_ref_decay, const float* th_state, const float* th_decay,
                int64_t n_th_decay, float* threshold, float* refractory, const sb_geom* g, int th_step, int th0,
                int w_scale, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_ref_decay, "ref_decay"));
  SB_TRY(check_count(n_th_decay, "th_decay"));
  SB_TRY(check_geom(g, &rg, n_ref_decay > n_th_decay ? n_ref_decay : n_th_decay));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(n_ref_decay == 1 || n_th_decay == 1 || n_ref_decay == n_th_decay, "decay counts disagree");
  SB_REQUIRE(w_scale > 0, "w_scale must be positive");
  SB_REQUIRE(im_state && ref_state && ref_decay && th_state && th_decay, "null parameter pointer");
  const float* in[2] = {re, im};
  float* out[2] = {threshold, refractory};
  AthParams ap{{ref_decay, n_ref_decay}, {th_decay, n_th_decay}, ref_state, th_state, th_step, th0};
  cudaStream_t st = (cudaStream_t)stream;
  if (is_pow2(w_scale)) {
    ApthFwd<true>::Params p{ap, im_state, make_scale(w_scale)};
    return launch_rowscan<ApthFwd<true>>(p, rg, in, out, st);
  }
  ApthFwd<false>::Params p{ap, im_state, make_scale(w_scale)};
  return launch_rowscan<ApthFwd<false>>(p, rg, in, out, st);
}

int sb_res_fwd(const float* re_in, const float* im_in, const float* sin_decay, const float* cos_decay,
               int64_t n_decay, const float* re_state, const float* im_state, float* re, float* im,
               const sb_geom* g, int reset, float thr_scaled, int im_reset, int w_scale, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_decay, "sin/cos decay"));
  SB_TRY(check_geom(g, &rg, n_decay));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE(w_scale > 0, "w_scale must be positive");
  SB_REQUIRE(sin_decay && cos_decay && re_state && im_state, "null parameter pointer");
  const float* in[2] = {re_in, im_in};
  float* out[2] = {re, im};
  ResParams rp{{sin_decay, n_decay}, {cos_decay, n_decay}, re_state, im_state};
  const bool pow2 = is_pow2(w_scale);
  cudaStream_t st = (cudaStream_t)stream;
#define SB_GO(R, P)                                                                                   \
  {                                                                                                   \
    typename ResFwd<R, P>::Params p{rp, reset ? int_threshold_ge(thr_scaled) : INT_MAX, im_reset,     \
                                    make_scale(w_scale)};                                             \
    return launch_rowscan<ResFwd<R, P>>(p, rg, in, out, st);                                          \
  }
  if (reset) { if (pow2) SB_GO(true, true) else SB_GO(true, false) }
  else       { if (pow2) SB_GO(false, true) else SB_GO(false, false) }
#undef SB_GO
}

int sb_res_bwd(const float* grad_re, const float* grad_im, const float* re, const float* im,
               const float* sin_decay, const float* cos_decay, int64_t n_decay, float* grad_re_in,
               float* grad_im_in, float* grad_sin, float* grad_cos, void* scratch_sin, void* scratch_cos,
               const sb_geom* g, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_decay, "sin/cos decay"));
  SB_TRY(check_geom(g, &rg, n_decay));
  SB_REQUIRE(sin_decay && cos_decay, "null parameter pointer");
  SB_REQUIRE((grad_sin == nullptr) == (grad_cos == nullptr), "grad_sin and grad_cos come together");
  cudaStream_t st = (cudaStream_t)stream;
  float* out[2] = {grad_re_in, grad_im_in};
  if (grad_sin) {
    SB_REQUIRE(re && im && scratch_sin && scratch_cos && scratch_sin != scratch_cos,
               "parameter gradients need re, im and two scratch areas");
    if (rg.rows == 0 || rg.T == 0) {
      SB_CUDA(cudaMemsetAsync(grad_sin, 0, sizeof(float) * n_decay, st));
      SB_CUDA(cudaMemsetAsync(grad_cos, 0, sizeof(float) * n_decay, st));
      return SB_OK;
    }
    const float* in[4] = {grad_re, grad_im, re, im};
    ResBwd<true>::Params p{{sin_decay, n_decay}, {cos_decay, n_decay}, (double*)scratch_sin, (double*)scratch_cos};
    SB_TRY((launch_rowscan<ResBwd<true>>(p, rg, in, out, st)));
    SB_TRY(fold_param_grad((double*)scratch_sin, grad_sin, rg, n_decay, st));
    return fold_param_grad((double*)scratch_cos, grad_cos, rg, n_decay, st);
  }
  const float* in[2] = {grad_re, grad_im};
  ResBwd<false>::Params p{{sin_decay, n_decay}, {cos_decay, n_decay}, nullptr, nullptr};
  return launch_rowscan<ResBwd<false>>(p, rg, in, out, st);
}

int sb_adres_fwd(const float* re_in, const float* im_in, const float* sin_decay, const float* cos_decay,
                 int64_t n_decay, const float* ref_decay, int64_t n_ref_decay, const float* th_decay,
                 int64_t n_th_decay, const float* re_state, const float* im_state, const float* ref_state,
                 const float* th_state, float* re, float* im, float* threshold, float* refractory,
                 const sb_geom* g, int th_step, int th0, int w_scale, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_decay, "sin/cos decay"));
  SB_TRY(check_count(n_ref_decay, "ref_decay"));
  SB_TRY(check_count(n_th_decay, "th_decay"));
  const int64_t nmax = max3(n_decay, n_ref_decay, n_th_decay);
  SB_TRY(check_geom(g, &rg, nmax));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;  // nothing to do, pointers may be null
  SB_REQUIRE((n_decay == 1 || n_decay == nmax) && (n_ref_decay == 1 || n_ref_decay == nmax) &&
                 (n_th_decay == 1 || n_th_decay == nmax),
             "parameter counts disagree");
  SB_REQUIRE(w_scale > 0, "w_scale must be positive");
  SB_REQUIRE(sin_decay && cos_decay && ref_decay && th_decay && re_state && im_state && ref_state && th_state,
             "null parameter pointer");
  const float* in[2] = {re_in, im_in};
  float* out[4] = {re, im, threshold, refractory};
  ResParams rp{{sin_decay, n_decay}, {cos_decay, n_decay}, re_state, im_state};
  AthParams ap{{ref_decay, n_ref_decay}, {th_decay, n_th_decay}, ref_state, th_state, th_step, th0};
  cudaStream_t st = (cudaStream_t)stream;
  if (is_pow2(w_scale)) {
    AdResFwd<true>::Params p{rp, ap, make_scale(w_scale)};
    return launch_rowscan<AdResFwd<true>>(p, rg, in, out, st);
  }
  AdResFwd<false>::Params p{rp, ap, make_scale(w_scale)};
  return launch_rowscan<AdResFwd<false>>(p, rg, in, out, st);
}

}  // extern "C"
