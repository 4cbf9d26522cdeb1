// Entry points of the sigma-delta family (dendrite/sigma.py, axon/delta.py,
// neuron/sigma_delta.py): the same one-row-per-lane TMA-pipelined scan as the
// spiking dynamics, with floating-point recurrences.
#include "api_util.cuh"
#include "ops_sigma_delta.cuh"
#include "reduce.cuh"
#include "rowscan.cuh"

using namespace sb;

namespace {

// 1 / scale as fp32 and, when scale is a power of two, scale itself
void quant_steps(double scale, float* step, float* inv_step) {
  *step = scale > 0.0 ? (float)(1.0 / scale) : 0.f;
  const int64_t is = (int64_t)scale;
  *inv_step = (scale > 0.0 && (double)is == scale && is <= (1 << 24) && is_pow2(is)) ? (float)scale : 0.f;
}

int plain_geom(int64_t rows, int64_t T, RowGeom* rg) {
  sb_geom g{rows, T, 1, 1};
  return check_geom(&g, rg, 1);
}

}  // namespace

extern "C" {

int sb_sigma_fwd(const float* x, const float* state, float* out, float* final_state, int64_t rows, int64_t T,
                 void* stream) {
  RowGeom rg;
  SB_TRY(plain_geom(rows, T, &rg));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  const float* in[1] = {x};
  float* o[1] = {out};
  SigmaFwd::Params p{state, final_state};
  return launch_rowscan<SigmaFwd>(p, rg, in, o, (cudaStream_t)stream);
}

int sb_sigma_bwd(const float* grad_out, float* grad_x, int64_t rows, int64_t T, void* stream) {
  RowGeom rg;
  SB_TRY(plain_geom(rows, T, &rg));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  const float* in[1] = {grad_out};
  float* o[1] = {grad_x};
  SigmaBwd::Params p{};
  return launch_rowscan<SigmaBwd>(p, rg, in, o, (cudaStream_t)stream);
}

int sb_delta_fwd(const float* x, const float* threshold, int64_t n_threshold, const float* pre_state,
                 const float* residual_state, float* out, float* delta_input, float* final_residual,
                 const sb_geom* g, double scale, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_threshold, "threshold"));
  SB_TRY(check_geom(g, &rg, n_threshold));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  SB_REQUIRE(threshold != nullptr, "null threshold");
  SB_REQUIRE(scale >= 0.0, "scale must be positive (0 leaves the output unquantised)");
  float step, inv_step;
  quant_steps(scale, &step, &inv_step);
  DeltaParams p{{threshold, n_threshold}, pre_state, residual_state, final_residual, step, inv_step};
  const float* in[1] = {x};
  if (delta_input) {
    float* o[2] = {out, delta_input};
    return launch_rowscan<DeltaFwd<true>>(p, rg, in, o, (cudaStream_t)stream);
  }
  float* o[1] = {out};
  return launch_rowscan<DeltaFwd<false>>(p, rg, in, o, (cudaStream_t)stream);
}

int sb_delta_bwd(const float* grad_out, const float* delta_input, const float* threshold, int64_t n_threshold,
                 float* grad_x, float* grad_threshold, void* scratch, const sb_geom* g, float tau_grad,
                 float scale_grad, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_threshold, "threshold"));
  SB_TRY(check_geom(g, &rg, n_threshold));
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_threshold) {
    SB_REQUIRE(delta_input && threshold && scratch, "grad_threshold needs the saved difference, the threshold and scratch");
    SB_REQUIRE(tau_grad != 0.f, "tau_grad must be non-zero");
    if (rg.rows == 0 || rg.T == 0) {
      SB_CUDA(cudaMemsetAsync(grad_threshold, 0, sizeof(float) * n_threshold, st));
      return SB_OK;
    }
    const float* in[2] = {grad_out, delta_input};
    float* o[1] = {grad_x};
    DeltaBwd<true>::Params p{{threshold, n_threshold}, tau_grad, scale_grad, (double*)scratch};
    SB_TRY((launch_rowscan<DeltaBwd<true>>(p, rg, in, o, st)));
    return fold_param_grad((double*)scratch, grad_threshold, rg, n_threshold, st);
  }
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  const float* in[1] = {grad_out};
  float* o[1] = {grad_x};
  DeltaBwd<false>::Params p{{nullptr, 1}, 1.f, 1.f, nullptr};
  return launch_rowscan<DeltaBwd<false>>(p, rg, in, o, st);
}

int sb_sdnn_relu_fwd(const float* x, const float* sigma_state, const float* bias, int64_t n_bias,
                     const float* threshold, int64_t n_threshold, const float* pre_state,
                     const float* residual_state, float* out, float* activation, float* delta_input,
                     float* final_sigma, float* final_pre, float* final_residual, const sb_geom* g, double scale,
                     void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_threshold, "threshold"));
  if (bias) SB_TRY(check_count(n_bias, "bias"));
  const int64_t nb = bias ? n_bias : 1;
  SB_TRY(check_geom(g, &rg, n_threshold));
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  SB_REQUIRE(threshold != nullptr, "null threshold");
  SB_REQUIRE(nb == 1 || nb == rg.rows_per_batch, "bias needs 1 value or one per neuron (%lld), got %lld",
             (long long)rg.rows_per_batch, (long long)nb);
  SB_REQUIRE(scale >= 0.0, "scale must be positive (0 leaves the output unquantised)");
  SB_REQUIRE(delta_input == nullptr || activation != nullptr, "saving the difference also saves the activation");
  float step, inv_step;
  quant_steps(scale, &step, &inv_step);
  const DeltaParams dp{{threshold, n_threshold}, pre_state, residual_state, final_residual, step, inv_step};
  const float* in[1] = {x};
  cudaStream_t st = (cudaStream_t)stream;
  if (delta_input) {
    SdnnFwd<2>::Params p{dp, sigma_state, {bias, nb}, final_sigma, final_pre};
    float* o[3] = {out, activation, delta_input};
    return launch_rowscan<SdnnFwd<2>>(p, rg, in, o, st);
  }
  if (activation) {
    SdnnFwd<1>::Params p{dp, sigma_state, {bias, nb}, final_sigma, final_pre};
    float* o[2] = {out, activation};
    return launch_rowscan<SdnnFwd<1>>(p, rg, in, o, st);
  }
  SdnnFwd<0>::Params p{dp, sigma_state, {bias, nb}, final_sigma, final_pre};
  float* o[1] = {out};
  return launch_rowscan<SdnnFwd<0>>(p, rg, in, o, st);
}

int sb_sdnn_relu_bwd(const float* grad_out, const float* activation, const float* delta_input,
                     const float* threshold, int64_t n_threshold, float* grad_x, float* grad_threshold,
                     void* scratch, const sb_geom* g, float tau_grad, float scale_grad, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_threshold, "threshold"));
  SB_TRY(check_geom(g, &rg, n_threshold));
  cudaStream_t st = (cudaStream_t)stream;
  if (grad_threshold) {
    SB_REQUIRE(delta_input && threshold && scratch, "grad_threshold needs the saved difference, the threshold and scratch");
    SB_REQUIRE(tau_grad != 0.f, "tau_grad must be non-zero");
    if (rg.rows == 0 || rg.T == 0) {
      SB_CUDA(cudaMemsetAsync(grad_threshold, 0, sizeof(float) * n_threshold, st));
      return SB_OK;
    }
    const float* in[3] = {grad_out, activation, delta_input};
    float* o[1] = {grad_x};
    SdnnBwd<true>::Params p{{threshold, n_threshold}, tau_grad, scale_grad, (double*)scratch};
    SB_TRY((launch_rowscan<SdnnBwd<true>>(p, rg, in, o, st)));
    return fold_param_grad((double*)scratch, grad_threshold, rg, n_threshold, st);
  }
  if (rg.rows == 0 || rg.T == 0) return SB_OK;
  const float* in[2] = {grad_out, activation};
  float* o[1] = {grad_x};
  SdnnBwd<false>::Params p{{nullptr, 1}, 1.f, 1.f, nullptr};
  return launch_rowscan<SdnnBwd<false>>(p, rg, in, o, st);
}

}  // extern "C"
