/*
 * slayer_b200.h -- C ABI of the B200 (sm_100a) implementation of lava-dl's SLAYER
 * hot path: Loihi-quantised neuron dynamics, spike functions, time shift and
 * the causal temporal filter.
 *
 * This is the boundary a binding of lava-dl (ctypes today; pybind, cffi, ...)
 * attaches to.  It replaces the seven JIT-compiled torch extensions of the
 * reference (src/lava/lib/dl/slayer/neuron/dynamics/{leaky_integrator,
 * adaptive_threshold,resonator,adaptive_resonator,adaptive_phase_th}.cu,
 * src/lava/lib/dl/slayer/utils/time/shift.cu, src/lava/lib/dl/slayer/utils/
 * filter/conv.cu) and the Python loops that run when those are not used.
 *
 * Conventions
 *  - Every tensor is fp32, contiguous, device memory of the CURRENT device,
 *    shaped [rows, T] with time contiguous: rows = batch * prod(spatial dims).
 *    The caller owns all memory, including scratch; the library allocates
 *    nothing and keeps no per-call state.
 *  - Per-row vectors (states, final states) are float[rows].
 *  - Decay-like parameters are float[n] with n == 1 (shared) or n == channels;
 *    row r uses entry (r % rows_per_batch) / decay_block, where rows_per_batch
 *    = prod(spatial dims) and decay_block = prod(spatial dims after the
 *    channel dim).  Decays are the reference's "un-scaled integer" values
 *    (0..4096), sin/cos are already scaled by 4096.
 *  - Integer semantics follow the reference's CPU code path (int64 tensors,
 *    truncation toward zero); states are held as int32, so results are exact
 *    while every state magnitude stays below 2^31 (Loihi states are 24 bit).
 *  - `stream` is a cudaStream_t passed as void*; kernels are launched on it
 *    and nothing synchronises.
 *  - Return value: SB_OK or a negative SB_ERR_*; sb_last_error_string() gives
 *    the text for the calling thread.  Launch errors are checked after every
 *    launch (the reference checks none, leaky_integrator.cu:140-150).
 */
#ifndef SLAYER_B200_H_
#define SLAYER_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_OK 0
#define SB_ERR_INVALID_ARG (-1)
#define SB_ERR_CUDA (-2)
#define SB_ERR_UNSUPPORTED (-3)

/* bits of sb_device_status() */
#define SB_DEV_TMA_TIMEOUT 1u /* a bulk tensor load did not arrive within the bounded wait */
#define SB_DEV_BAD_DELAY 2u   /* a fused axonal delay was outside 0..62 steps and was clamped */

/* Row geometry shared by all time-recurrent entry points. */
typedef struct sb_geom {
  int64_t rows;           /* batch * prod(spatial) */
  int64_t T;              /* time steps (contiguous axis) */
  int64_t rows_per_batch; /* prod(spatial); only used when a parameter has n > 1 */
  int64_t decay_block;    /* prod(spatial[1:]); only used when a parameter has n > 1 */
} sb_geom;

/* ---- library -------------------------------------------------------------- */
int sb_version(void);
const char* sb_last_error_string(void);
/* Reads and clears the sticky device status word of the current device
 * (synchronises the device). */
int sb_device_status(unsigned int* bits);
/* Bytes of scratch a backward call needs per parameter-gradient output
 * (decay, sin, cos ...).  n is that parameter's element count. */
int64_t sb_param_grad_scratch_bytes(int64_t rows, int64_t n);
/* 1 when this [rows, T] problem takes the TMA-tiled kernels (T % 4 == 0, T >= 32,
 * 16-byte aligned bases), 0 when it takes the plain-load kernels. */
int sb_uses_tma(const void* base, int64_t T);

/* ---- leaky integrator ------------------------------------------------------
 * Replaces leaky_integrator.cu:112-153 (LIDynamicsFwd) / leaky_integrator.py:210-231.
 * thr_scaled = fp32(threshold * w_scale); <= 0 disables the reset.
 * final_state (nullable) receives y[..., -1]. */
int sb_li_fwd(const float* x, const float* decay, int64_t n_decay, const float* state, float* y,
              float* final_state, const sb_geom* g, float thr_scaled, int w_scale, void* stream);
/* Replaces leaky_integrator.cu:155-200 (LIDynamicsBwd) / leaky_integrator.py:234-259.
 * grad_decay (nullable, float[n_decay]) needs `y` (saved forward output) and
 * `scratch` of sb_param_grad_scratch_bytes(rows, n_decay) bytes. */
int sb_li_bwd(const float* grad_y, const float* y, const float* decay, int64_t n_decay, float* grad_x,
              float* grad_decay, void* scratch, const sb_geom* g, void* stream);

/* No counterpart in the reference.  Same computation as sb_li_bwd with
 * grad_decay, for callers that cannot provide scratch memory because they
 * cannot allocate (ahead-of-time planned runtimes that give a custom op only
 * its inputs and outputs, processes whose pool already owns the whole GPU,
 * latency-bound loops that cannot take the device sync of an allocation).
 * The scratch is a SB_NOALLOC_SCRATCH_BYTES array inside the library, resident
 * on every GPU that loads it.  Limits: shared decay up to 32 * (capacity/8 - 64)
 * rows; per-channel decay rows + 64 * n_decay <= capacity/8.  Larger problems
 * return SB_ERR_INVALID_ARG.  The first call on a device looks the array up
 * (do it outside stream capture; the per-device lookup is safe to race from several
 * threads).  Calls share the array: calls overlapping on the GPU race.  If
 * sb_device_status reports SB_DEV_TMA_TIMEOUT after a call, that call's grad_x and
 * grad_decay are incomplete.  Allocates nothing. */
#define SB_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
int sb_li_bwd_noalloc(const float* grad_y, const float* y, const float* decay, int64_t n_decay, float* grad_x,
                      float* grad_decay, const sb_geom* g, void* stream);

/* ---- adaptive threshold ----------------------------------------------------
 * Replaces adaptive_threshold.cu:81-129 / adaptive_threshold.py:237-274.
 * th_step = int(th_scale * w_scale), th0 = int(th0 * w_scale) (host ints). */
int sb_ath_fwd(const float* x, const float* ref_state, const float* ref_decay, int64_t n_ref_decay,
               const float* th_state, const float* th_decay, int64_t n_th_decay, float* threshold,
               float* refractory, const sb_geom* g, int th_step, int th0, int w_scale, void* stream);

/* ---- adaptive phase threshold ----------------------------------------------
 * Replaces adaptive_phase_th.cu:89-143 / adaptive_phase_th.py:234-283. */
int sb_apth_fwd(const float* re, const float* im, const float* im_state, const float* ref_state,
                const float* ref_decay, int64_t n_ref_decay, const float* th_state, const float* th_decay,
                int64_t n_th_decay, float* threshold, float* refractory, const sb_geom* g, int th_step, int th0,
                int w_scale, void* stream);

/* ---- resonator -------------------------------------------------------------
 * Replaces resonator.cu:151-198 / resonator.py:333-376.
 * reset != 0 enables the Izhikevich reset; then thr_scaled = fp32(threshold *
 * w_scale) and im_reset = int(fp32(threshold * w_scale - 1)) (host computes
 * the subtraction in double, as Python does). */
int sb_res_fwd(const float* re_in, const float* im_in, const float* sin_decay, const float* cos_decay,
               int64_t n_decay, const float* re_state, const float* im_state, float* re, float* im,
               const sb_geom* g, int reset, float thr_scaled, int im_reset, int w_scale, void* stream);
/* Replaces resonator.cu:200-263 / resonator.py:379-467; also the backward of
 * the adaptive resonator (adaptive_resonator.cu:245-308).  grad_sin/grad_cos
 * (nullable, both or none) need re, im and two scratch areas. */
int sb_res_bwd(const float* grad_re, const float* grad_im, const float* re, const float* im,
               const float* sin_decay, const float* cos_decay, int64_t n_decay, float* grad_re_in,
               float* grad_im_in, float* grad_sin, float* grad_cos, void* scratch_sin, void* scratch_cos,
               const sb_geom* g, void* stream);

/* ---- adaptive resonator ----------------------------------------------------
 * Replaces adaptive_resonator.cu:178-243 / adaptive_resonator.py:379-436. */
int sb_adres_fwd(const float* re_in, const float* im_in, const float* sin_decay, const float* cos_decay,
                 int64_t n_decay, const float* ref_decay, int64_t n_ref_decay, const float* th_decay,
                 int64_t n_th_decay, const float* re_state, const float* im_state, const float* ref_state,
                 const float* th_state, float* re, float* im, float* threshold, float* refractory,
                 const sb_geom* g, int th_step, int th0, int w_scale, void* stream);

/* ---- spike functions (element-wise) ----------------------------------------
 * Replace the ATen op chains of spike/spike.py:64-126.  thr_tensor (nullable)
 * is a per-element threshold of n floats, else thr is used. */
int sb_spike_fwd(const float* v, const float* thr_tensor, float thr, float* spike, int64_t n, int graded,
                 float scale, void* stream);
int sb_spike_bwd(const float* v, const float* thr_tensor, float thr, const float* grad_spike, float* grad_v,
                 int64_t n, float tau_rho, float scale_rho, int graded, void* stream);
/* spike/complex.py:49-167.  imag_last is float[rows] (im at t = -1). */
int sb_cspike_fwd(const float* re, const float* im, const float* thr_tensor, float thr, const float* imag_last,
                  float* spike, int64_t rows, int64_t T, int graded, float scale, void* stream);
int sb_cspike_bwd(const float* re, const float* im, const float* thr_tensor, float thr, const float* grad_spike,
                  float* grad_re, float* grad_im, int64_t n, float tau_rho, float scale_rho, int graded,
                  void* stream);

/* ---- fused neurons -----------------------------------------------------------
 * One pass for what neuron/{cuba,alif,rf,adrf}.py compute with several calls
 * (dynamics ... spike) when no normalisation sits in between.  Require a
 * power-of-two w_scale.  Nullable outputs are skipped.
 *
 * CUBA (neuron/cuba.py:274-421): thr = fp32(threshold + eps).
 * Outputs: current (nullable), voltage, spike (nullable);
 * final_c/final_v/final_s (nullable float[rows]) = last time bin of
 * current, voltage (before reset) and spike.  voltage may be null when only
 * binary spikes are wanted (current null, graded 0): what Neuron.forward
 * returns when nothing will be differentiated, 8 B per neuron-step instead of 12.
 * spike_delay = 1 (binary spikes only) writes the spike series one step late,
 * spike_out[t] = spike[t-1], which is the one-step inter-layer delay of the
 * blocks (block/base.py:15-39) at no extra memory traffic; delay_head
 * (nullable float[rows]) supplies spike_out[0], else 0.  final_s stays the
 * undelayed last spike.
 * axon_delay (nullable float[n_axon_delay], n_axon_delay = rows_per_batch;
 * binary spikes only) folds the block's axonal delay (axon/delay.py:150-175,
 * applied after the step delay at block/base.py:551-552) into the same store:
 * row r is written int(axon_delay[r % n] / axon_delay_ts) steps later still,
 * zero filled.  Delays must lie in 0..62 steps; others are clamped and
 * SB_DEV_BAD_DELAY is set in the device status word. */
int sb_cuba_fwd(const float* x, const float* cdecay, int64_t n_cdecay, const float* vdecay, int64_t n_vdecay,
                const float* cstate, const float* vstate, float* current, float* voltage, float* spike,
                float* final_c, float* final_v, float* final_s, const sb_geom* g, double threshold,
                int w_scale, int graded, float spike_scale, int spike_delay, const float* delay_head,
                const float* axon_delay, int64_t n_axon_delay, float axon_delay_ts, void* stream);
/* Inference form of sb_cuba_fwd with the spikes as bits (no counterpart in the
 * reference, whose Neuron.forward returns fp32 0/1 values, neuron/cuba.py:423-440):
 * spike_bits is uint32[rows][ceil(T / 32)], word w of row r holding steps
 * 32 w .. 32 w + 31 of that row (bit i = step 32 w + i; bits past T are 0).
 * The fp32 spike tensor is not written, and neither is the voltage series when
 * voltage is null: 4 B read and 1/8 B written per neuron-step instead of 12 B,
 * and a device-to-host copy of the result that is 32 times smaller.
 * Binary spikes only; spike_delay / delay_head as in sb_cuba_fwd. */
int sb_cuba_fwd_packed(const float* x, const float* cdecay, int64_t n_cdecay, const float* vdecay,
                       int64_t n_vdecay, const float* cstate, const float* vstate, float* voltage,
                       uint32_t* spike_bits, float* final_c, float* final_v, float* final_s, const sb_geom* g,
                       double threshold, int w_scale, int spike_delay, const float* delay_head, void* stream);

/* Backward of CUBA and ALIF forward: surrogate gradient + both integrators.
 * thr_tensor (nullable): per-element threshold (ALIF passes th + ref).
 * grad_cdecay/grad_vdecay (nullable, both or none) need `current` and scratch.
 * spike_delay = 1: grad_spike is the gradient of the one-step-late series. */
/* Host side of sb_cuba_fwd_packed: expands spike_bits (host memory, uint32[rows][ceil(T / 32)]) into
 * the fp32 0 / 1 tensor out (host memory, float[rows][T]) that Neuron.forward returns, on `threads`
 * CPU threads (0 = all).  stream_ordered = 0: done on return.  stream_ordered = 1: enqueued on
 * `stream` as a host function, i.e. after the copy of the bits that was queued there before it and
 * before whatever is queued after it; both buffers must stay alive until the stream reaches it. */
int sb_unpack_spikes_host(const uint32_t* spike_bits, float* out, int64_t rows, int64_t T, int threads,
                          int stream_ordered, void* stream);

int sb_cuba_bwd(const float* grad_spike, const float* voltage, const float* thr_tensor, float thr,
                const float* current, const float* cdecay, int64_t n_cdecay, const float* vdecay,
                int64_t n_vdecay, float* grad_x, float* grad_cdecay, float* grad_vdecay, void* scratch_c,
                void* scratch_v, const sb_geom* g, float tau_rho, float scale_rho, int graded, int spike_delay,
                void* stream);

/* ALIF (neuron/alif.py:383-591).  mode 0: forward() -> spike, voltage,
 * thsum = threshold + refractory.  mode 1: dynamics() -> current, voltage,
 * threshold, refractory (out0..out3).  spike_delay = 1 (mode 0, binary spikes):
 * the spike series is written one step late, delay_head (nullable float[rows])
 * supplying its first step, as in sb_cuba_fwd; sb_cuba_bwd undoes it.
 * Mode 0 with out1 and out2 null (binary spikes): only the spikes are written,
 * what Neuron.forward returns when nothing will be differentiated.  Mode 0 with
 * out2 null: out1 receives voltage - (threshold + refractory) instead of the
 * voltage; sb_cuba_bwd on it with the scalar threshold 0 gives the same input
 * gradient as on the two series (the surrogate reads only their difference). */
int sb_alif_fwd(const float* x, const float* cdecay, int64_t n_cdecay, const float* vdecay, int64_t n_vdecay,
                const float* ref_decay, int64_t n_ref_decay, const float* th_decay, int64_t n_th_decay,
                const float* cstate, const float* vstate, const float* ref_state, const float* th_state,
                float* out0, float* out1, float* out2, float* out3, float* final_c, float* final_v,
                float* final_th, float* final_ref, float* final_s, const sb_geom* g, int th_step, int th0,
                int w_scale, int mode, int graded, float spike_scale, int spike_delay, const float* delay_head,
                void* stream);

/* RF (neuron/rf.py) and ADRF (neuron/adrf.py:439-652).  adapt = 0: outputs
 * spike, re, im (out0..out2) with scalar threshold.  adapt = 1, mode 0:
 * spike, re, im, th + ref.  adapt = 1, mode 1: re, im, threshold, refractory.
 * spike_delay / delay_head (mode 0, binary spikes) as in sb_cuba_fwd; sb_rf_bwd
 * takes the same spike_delay to read the gradient of the late series.
 * Mode 0 with out1, out2 (and out3) null (binary spikes): only the spikes are written.
 * adapt = 1, mode 0 with out3 null: out1 receives re - (threshold + refractory) instead of
 * re; sb_rf_bwd on it with the scalar threshold 0 and no sin / cos gradients gives the same
 * input gradients (the spike's gradient reads re only through that difference). */
int sb_rf_fwd(const float* re_in, const float* im_in, const float* sin_decay, const float* cos_decay,
              int64_t n_decay, const float* ref_decay, int64_t n_ref_decay, const float* th_decay,
              int64_t n_th_decay, const float* re_state, const float* im_state, const float* ref_state,
              const float* th_state, float* out0, float* out1, float* out2, float* out3, float* final_re,
              float* final_im, float* final_th, float* final_ref, float* final_s, const sb_geom* g,
              float threshold, int th_step, int th0, int w_scale, int adapt, int mode, int graded,
              float spike_scale, int spike_delay, const float* delay_head, void* stream);
int sb_rf_bwd(const float* grad_spike, const float* re, const float* im, const float* thr_tensor, float thr,
              const float* sin_decay, const float* cos_decay, int64_t n_decay, float* grad_re_in,
              float* grad_im_in, float* grad_sin, float* grad_cos, void* scratch_sin, void* scratch_cos,
              const sb_geom* g, float tau_rho, float scale_rho, int graded, int spike_delay, void* stream);

/* ---- time shift --------------------------------------------------------------
 * Replaces shift.cu:80-175 / utils/time/shift.py:46-143:
 * out[r, t] = in[r, t - d], zero fill, d = int(shift / sampling_time)
 * (truncation toward zero, negative allowed).  lut (nullable, float[n_lut],
 * n_lut = rows_per_batch) gives one shift per neuron, else `shift`. */
int sb_shift(const float* x, const float* lut, int64_t n_lut, float shift, float sampling_time, float* out,
             int64_t rows, int64_t T, void* stream);

/* ---- causal temporal filter ----------------------------------------------------
 * Replaces conv.cu:80-172 / utils/filter/conv.py:48-97.
 * conv: out[r,t] = Ts * sum_{i<K} f[i] * in[r, t-i];  corr: ... in[r, t+i]. */
int sb_fir_conv(const float* x, const float* filter, int64_t K, float sampling_time, float* out, int64_t rows,
                int64_t T, void* stream);
/* 1 when a filter call of this size (bases 16-byte aligned) runs as a banded
 * matrix product on the tensor cores (tcgen05, three TF32 products per term:
 * K <= 64, T % 4 == 0, T >= 32, rows >= 128), 0 when it runs the FP32 sliding
 * window kernel.  The reference has one kernel (conv.cu:24-78). */
int sb_fir_uses_tensor_cores(int64_t K, int64_t rows, int64_t T);
int sb_fir_corr(const float* x, const float* filter, int64_t K, float sampling_time, float* out, int64_t rows,
                int64_t T, void* stream);
/* Fused delay + filter (forward): conv(shift(x, lut), f); and its adjoint
 * (backward): shift(corr(g, f), -lut).  One read and one write per element. */
int sb_shift_fir_fwd(const float* x, const float* lut, int64_t n_lut, float shift, float shift_ts,
                     const float* filter, int64_t K, float sampling_time, float* out, int64_t rows, int64_t T,
                     void* stream);
int sb_shift_fir_bwd(const float* grad_out, const float* lut, int64_t n_lut, float shift, float shift_ts,
                     const float* filter, int64_t K, float sampling_time, float* grad_x, int64_t rows,
                     int64_t T, void* stream);

/* ---- sigma-delta family (next to the path: the same serial-in-time shape) -------
 * Sigma decoder, replaces dendrite/sigma.py:38-72 (torch.cumsum + persistent
 * state): out[r,t] = float(sum_{s<=t} x[r,s], accumulated in double as
 * torch.cumsum does on a CPU float tensor) + state[r] (nullable = 0).
 * final_state (nullable float[rows]) receives out[r, T-1].
 * sb_sigma_bwd is its adjoint: the same sum over reversed time. */
int sb_sigma_fwd(const float* x, const float* state, float* out, float* final_state, int64_t rows, int64_t T,
                 void* stream);
int sb_sigma_bwd(const float* grad_out, float* grad_x, int64_t rows, int64_t T, void* stream);
/* Delta encoder, replaces axon/delta.py:13-76 (cum_error = False, the Python
 * loop over time) and the floor quantisation of Delta.forward (delta.py:316):
 *   d[t] = (x[t] - pre) + residual;  y[t] = d[t] if |d[t]| >= threshold else 0;
 *   residual = d[t] - y[t];  pre = x[t];  out[t] = floor(y[t] * scale) / scale.
 * threshold: 1 or C values.  pre_state / residual_state (nullable float[rows]).
 * delta_input (nullable) receives d (saved for the threshold gradient);
 * final_residual (nullable float[rows]).  scale = 0 leaves out unquantised. */
int sb_delta_fwd(const float* x, const float* threshold, int64_t n_threshold, const float* pre_state,
                 const float* residual_state, float* out, float* delta_input, float* final_residual,
                 const sb_geom* g, double scale, void* stream);
/* Replaces axon/delta.py:77-122: grad_x[t] = g[t] - g[t+1]; grad_threshold
 * (nullable; needs delta_input and scratch of sb_param_grad_scratch_bytes) =
 * sum over batch, space and time of
 *   (|d| - thr > 0 ? -d * scale_grad * exp(-(|d| - thr) / tau_grad) / thr : -sign(d)) * g.
 * (The reference's per-channel reduction fails on its own shapes; here it sums
 * per channel as its comment intends.) */
int sb_delta_bwd(const float* grad_out, const float* delta_input, const float* threshold, int64_t n_threshold,
                 float* grad_x, float* grad_threshold, void* scratch, const sb_geom* g, float tau_grad,
                 float scale_grad, void* stream);
/* Sigma-delta ReLU neuron: neuron/sigma_delta.py:171-219 with activation = relu
 * and no normalisation, one pass each way:
 * sigma -> + bias (nullable; 1 value or one per neuron, rows_per_batch values, as
 * set_bias stores it) -> relu -> delta -> floor.  8 bytes per step for inference;
 * activation (nullable) saves the ReLU output for the backward pass, delta_input
 * (nullable, needs activation) the delta unit's difference for the threshold
 * gradient.  final_sigma / final_pre / final_residual (nullable float[rows]) are
 * the persistent states of the sigma and delta units after the call.
 * Backward: grad_x[t] = float(sum_{s>=t} (g[s] - g[s+1]) * (activation[s] > 0)),
 * grad_threshold as sb_delta_bwd.  No bias gradient. */
int sb_sdnn_relu_fwd(const float* x, const float* sigma_state, const float* bias, int64_t n_bias,
                     const float* threshold, int64_t n_threshold, const float* pre_state,
                     const float* residual_state, float* out, float* activation, float* delta_input,
                     float* final_sigma, float* final_pre, float* final_residual, const sb_geom* g, double scale,
                     void* stream);
int sb_sdnn_relu_bwd(const float* grad_out, const float* activation, const float* delta_input,
                     const float* threshold, int64_t n_threshold, float* grad_x, float* grad_threshold,
                     void* scratch, const sb_geom* g, float tau_grad, float scale_grad, void* stream);

/* ---- sum-pooling synapse (next to the path: what feeds the neurons in conv networks) ----
 * Replaces the Conv3d call of synapse/layer.py:438-508 for the default pooling
 * geometry (stride = kernel, no padding, no dilation).  x is [NC, H, W, T] with
 * NC = batch * channels, y is [NC, Ho, Wo, T], weight is the (kh, kw) kernel
 * (after the pre-hook), row-major.  Windows reaching past H or W read zeros,
 * as the reference's zero padding of odd sizes does.
 * y[nc,ho,wo,t] = sum_ij w[i,j] * x[nc, ho*kh+i, wo*kw+j, t]; bwd is its adjoint. */
int sb_pool_fwd(const float* x, const float* weight, float* y, int64_t NC, int64_t H, int64_t W, int64_t Ho,
                int64_t Wo, int64_t kh, int64_t kw, int64_t T, void* stream);
int sb_pool_bwd(const float* grad_y, const float* weight, float* grad_x, int64_t NC, int64_t H, int64_t W,
                int64_t Ho, int64_t Wo, int64_t kh, int64_t kw, int64_t T, void* stream);

/* Convolution synapse, forward (replaces the Conv3d call of synapse/layer.py:297-323
 * for stride 1, dilation 1, one group).  x [N, Ci, H, W, T], weight [Co, Ci, kh, kw]
 * (after the pre-hook), y [N, Co, H+2ph-kh+1, W+2pw-kw+1, T].
 * Two kernels: an implicit GEMM on the tensor cores (tcgen05, operands split into TF32 pairs so
 * that the result keeps fp32 accuracy; bit-exact for spikes and weights on a 1/32 grid) for 1x1,
 * 3x3 and 5x5 kernels with T a multiple of 4 and >= 32 and 16-byte aligned tensors (a layer too
 * wide for its shared memory runs in blocks of input channels, one launch each), and an fp32
 * kernel for every shape with N * Ho <= 65535 and the weights of 16 output channels in 96 KB.
 * sb_conv_fwd picks the tensor cores when the shape allows and the contraction is long enough to
 * pay for them (Ci * kh * kw >= 64); sb_conv_fwd_path takes the choice from the caller:
 * path 0 = fp32 kernel, 1 = tensor cores (SB_ERR_UNSUPPORTED if the shape does not fit), -1 = as
 * sb_conv_fwd.  sb_conv_uses_tensor_cores says what sb_conv_fwd would do. */
int sb_conv_fwd(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co, int64_t H,
                int64_t W, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T, void* stream);
int sb_conv_fwd_path(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co, int64_t H,
                     int64_t W, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T, int path, void* stream);
int sb_conv_uses_tensor_cores(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw,
                              int64_t ph, int64_t pw, int64_t T);
/* 1 when the tensor-core kernel can take the geometry at all (what path = 1 needs). */
int sb_conv_fits_tensor_cores(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw,
                              int64_t ph, int64_t pw, int64_t T);

/* 1 when sb_conv_wgrad takes the problem (accumulator tiles of one CTA, one output row staged in
 * shared memory, T % 4 == 0), else 0: the caller then falls back (the mirror package uses ATen's
 * convolution backward). */
int sb_conv_wgrad_fits(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw,
                       int64_t ph, int64_t pw, int64_t T);
/* Weight gradient of the same convolution (what convolution_backward returns for
 * the weight of the Conv3d at synapse/layer.py:297-323), fp32:
 *   grad_weight[co,ci,i,j] = sum_{n,ho,wo,t} grad_y[n,co,ho,wo,t] * x[n,ci,ho+i-ph,wo+j-pw,t].
 * scratch: sb_conv_wgrad_scratch_bytes(...) bytes (one partial per output row,
 * summed in a fixed order).  Needs T % 4 == 0, 16-byte aligned tensors and
 * ceil(Co / 8) * ceil(Ci * kh * kw / 8) <= 384.  The input gradient is
 * sb_conv_fwd of grad_y with the flipped, transposed weight and padding
 * (kh - 1 - ph, kw - 1 - pw). */
int64_t sb_conv_wgrad_scratch_bytes(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t kh, int64_t kw,
                                    int64_t ph);
int sb_conv_wgrad(const float* x, const float* grad_y, float* grad_weight, void* scratch, int64_t N, int64_t Ci,
                  int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T,
                  void* stream);

/* ---- gradient plumbing ------------------------------------------------------------
 * No counterpart in the reference: out[i] = *value (a device scalar) for i < n.
 * Autograd hands the backward of sum() / mean() one number broadcast to the
 * tensor's shape; the backward entry points want a dense tensor, and this fills
 * it at memory speed without reading the number on the host. */
int sb_broadcast_fill(const float* value, float* out, int64_t n, void* stream);

/* ---- dense recurrent CUBA layer ---------------------------------------------------
 * Replaces the per-step Python loops of slayer/utils/recurrent.py:45-112 (forward
 * :54-77, backward :79-112), the caller being block/base.py:1460-1488.
 * z [batch, neurons, T] is the output of the input synapse; rec_t [neurons, neurons]
 * is the (already quantised) recurrent matrix transposed, rec the same matrix as is.
 *   spike[t] = CUBA(z[t] + R spike[t-1]), the neuron state carried from step to step
 *   (cstate/vstate in, final_* out, one value per [batch, neuron]).
 * Backward: every step was a Neuron call with T = 1 on a detached state, so
 *   grad_z[t] = surrogate(voltage[t]) * (grad_spike[t] + R^T grad_z[t+1]);
 * the decay gradients of such calls are zero; grad of R is the plain product
 * grad_z[..., 1:] x spike[..., :-1] and is left to the caller's GEMM.
 * One neuron per thread: neurons <= 1024.  Decays: 1 or `neurons` values. */
int sb_cuba_recurrent_fwd(const float* z, const float* rec_t, const float* cdecay, int64_t n_cdecay,
                          const float* vdecay, int64_t n_vdecay, const float* cstate, const float* vstate,
                          float* voltage, float* spike, float* final_c, float* final_v, float* final_s,
                          int64_t batch, int64_t neurons, int64_t T, double threshold, int w_scale, int graded,
                          float spike_scale, void* stream);
int sb_cuba_recurrent_bwd(const float* grad_spike, const float* voltage, const float* rec, float* grad_z,
                          int64_t batch, int64_t neurons, int64_t T, float threshold, float tau_rho,
                          float scale_rho, int graded, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SLAYER_B200_H_ */
