"""Functional layer between the torch-facing API and the C ABI.

Every function takes/returns torch tensors, derives the row geometry the
kernels need from the tensor shape, allocates outputs with torch and launches on
the current stream.  Nothing here differentiates; autograd wiring lives in the
``slayer`` sub-modules.
"""

import math
from ctypes import c_void_p

import numpy as np
import torch

from . import _native as N


def _rows_T(x):
    T = x.shape[-1]
    rows = x.numel() // T if T > 0 else 0
    return rows, T


def geom(x, *counts):
    """``sb_geom`` of a ``[B, C, ..., T]`` tensor for parameters with the given
    element counts (1 = shared, C = per channel)."""
    rows, T = _rows_T(x)
    rpb, blk = 1, 1
    if x.dim() >= 3:
        rpb = int(np.prod(x.shape[1:-1]))
        blk = int(np.prod(x.shape[2:-1])) if x.dim() > 3 else 1
    nmax = max(counts) if counts else 1
    if nmax > 1:
        if x.dim() < 3 or x.shape[1] != nmax:
            raise ValueError(
                f'per-channel parameter of {nmax} elements does not match input shape {tuple(x.shape)}'
            )
    return N.Geom(rows, T, rpb, blk)


def _c(t):
    """Contiguous view or copy.  A tensor that is one value broadcast to a shape (the gradient
    autograd hands back for a ``sum()`` or ``mean()`` loss) is materialised with a fill: the
    strided copy kernel ``contiguous()`` would run moves 2 TB/s, the fill runs at memory speed."""
    if t.is_contiguous():
        return t
    if t.numel() > 0 and t.is_cuda and t.dtype == torch.float32 and all(st == 0 for st in t.stride()):
        out = torch.empty(t.shape, dtype=t.dtype, device=t.device)
        N.call('sb_broadcast_fill', out, c_void_p(t.data_ptr()), N.ptr(out), out.numel(), N.stream_of(out))
        return out
    return t.contiguous()


def _param(p, like):
    """Flatten a decay-like parameter to contiguous fp32 on the input's device."""
    p = p.detach().to(device=like.device, dtype=torch.float32).reshape(-1)
    return _c(p)


def row_state(state, x):
    """Broadcast a state to one value per row (``state * ones(x.shape[:-1])``)."""
    lead = x.shape[:-1]
    s = state.detach().to(device=x.device, dtype=torch.float32)
    if s.numel() == 1:
        return s.reshape(1).expand(int(np.prod(lead)) if len(lead) else 1).contiguous()
    if tuple(s.shape) != tuple(lead):
        s = s.expand(lead)
    return _c(s).reshape(-1)


def is_pow2(v):
    v = int(v)
    return v > 0 and (v & (v - 1)) == 0


def f32(v):
    return float(np.float32(v))


# --------------------------------------------------------------------------
# leaky integrator
# --------------------------------------------------------------------------
def li_fwd(x, decay, state, w_scale, threshold=None, want_final=False):
    N.require_cuda(x)
    x = _c(x)
    decay = _param(decay, x)
    st = row_state(state, x)
    y = torch.empty_like(x)
    fin = torch.empty(x.shape[:-1], device=x.device, dtype=torch.float32) if want_final else None
    thr = -1.0 if threshold is None else float(threshold)
    thr_scaled = thr * w_scale  # Python double, then fp32 at the boundary
    g = geom(x, decay.numel())
    N.call('sb_li_fwd', x, N.ptr(x), N.ptr(decay), decay.numel(), N.ptr(st), N.ptr(y), N.ptr(fin), g,
           f32(thr_scaled) if thr_scaled > 0 else -1.0, int(w_scale), N.stream_of(x))
    return (y, fin) if want_final else y


def li_bwd(grad_y, y, decay, need_decay_grad):
    N.require_cuda(grad_y)
    grad_y = _c(grad_y)
    dec = _param(decay, grad_y)
    grad_x = torch.empty_like(grad_y)
    g = geom(grad_y, dec.numel())
    if need_decay_grad:
        y = _c(y)
        gd = torch.empty(dec.numel(), device=grad_y.device, dtype=torch.float32)
        scr = N.scratch(g.rows, dec.numel(), grad_y.device)
        N.call('sb_li_bwd', grad_y, N.ptr(grad_y), N.ptr(y), N.ptr(dec), dec.numel(), N.ptr(grad_x), N.ptr(gd),
               N.ptr(scr), g, N.stream_of(grad_y))
        return grad_x, gd.reshape(decay.shape)
    N.call('sb_li_bwd', grad_y, N.ptr(grad_y), None, N.ptr(dec), dec.numel(), N.ptr(grad_x), None, None, g,
           N.stream_of(grad_y))
    return grad_x, None


# --------------------------------------------------------------------------
# adaptive threshold / phase threshold
# --------------------------------------------------------------------------
def ath_fwd(x, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale):
    N.require_cuda(x)
    x = _c(x)
    rd, td = _param(ref_decay, x), _param(th_decay, x)
    rs, ts = row_state(ref_state, x), row_state(th_state, x)
    th = torch.empty_like(x)
    ref = torch.empty_like(x)
    g = geom(x, rd.numel(), td.numel())
    N.call('sb_ath_fwd', x, N.ptr(x), N.ptr(rs), N.ptr(rd), rd.numel(), N.ptr(ts), N.ptr(td), td.numel(),
           N.ptr(th), N.ptr(ref), g, int(th_scale * w_scale), int(th0 * w_scale), int(w_scale), N.stream_of(x))
    return th, ref


def apth_fwd(re, im, im_state, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale):
    N.require_cuda(re, im)
    re, im = _c(re), _c(im)
    rd, td = _param(ref_decay, re), _param(th_decay, re)
    ims, rs, ts = row_state(im_state, re), row_state(ref_state, re), row_state(th_state, re)
    th = torch.empty_like(re)
    ref = torch.empty_like(re)
    g = geom(re, rd.numel(), td.numel())
    N.call('sb_apth_fwd', re, N.ptr(re), N.ptr(im), N.ptr(ims), N.ptr(rs), N.ptr(rd), rd.numel(), N.ptr(ts),
           N.ptr(td), td.numel(), N.ptr(th), N.ptr(ref), g, int(th_scale * w_scale), int(th0 * w_scale),
           int(w_scale), N.stream_of(re))
    return th, ref


# --------------------------------------------------------------------------
# resonator / adaptive resonator
# --------------------------------------------------------------------------
def res_fwd(re_in, im_in, sin_decay, cos_decay, re_state, im_state, w_scale, threshold=None):
    N.require_cuda(re_in, im_in)
    re_in, im_in = _c(re_in), _c(im_in)
    sd, cd = _param(sin_decay, re_in), _param(cos_decay, re_in)
    if sd.numel() != cd.numel():
        raise ValueError('sin_decay and cos_decay must have the same number of elements')
    rs, ims = row_state(re_state, re_in), row_state(im_state, im_in)
    re = torch.empty_like(re_in)
    im = torch.empty_like(im_in)
    thr = -1.0 if threshold is None else float(threshold)
    thr_scaled = thr * w_scale
    reset = thr_scaled >= 0
    im_reset = int(np.float32(thr_scaled - 1)) if reset else 0
    g = geom(re_in, sd.numel())
    N.call('sb_res_fwd', re_in, N.ptr(re_in), N.ptr(im_in), N.ptr(sd), N.ptr(cd), sd.numel(), N.ptr(rs),
           N.ptr(ims), N.ptr(re), N.ptr(im), g, int(reset), f32(thr_scaled), im_reset, int(w_scale),
           N.stream_of(re_in))
    return re, im


def res_bwd(grad_re, grad_im, re, im, sin_decay, cos_decay, need_param_grad):
    N.require_cuda(grad_re, grad_im)
    grad_re, grad_im = _c(grad_re), _c(grad_im)
    sd, cd = _param(sin_decay, grad_re), _param(cos_decay, grad_re)
    gre = torch.empty_like(grad_re)
    gim = torch.empty_like(grad_im)
    g = geom(grad_re, sd.numel())
    if need_param_grad:
        re, im = _c(re), _c(im)
        gs = torch.empty(sd.numel(), device=grad_re.device, dtype=torch.float32)
        gc = torch.empty_like(gs)
        s1 = N.scratch(g.rows, sd.numel(), grad_re.device)
        s2 = N.scratch(g.rows, sd.numel(), grad_re.device)
        N.call('sb_res_bwd', grad_re, N.ptr(grad_re), N.ptr(grad_im), N.ptr(re), N.ptr(im), N.ptr(sd), N.ptr(cd),
               sd.numel(), N.ptr(gre), N.ptr(gim), N.ptr(gs), N.ptr(gc), N.ptr(s1), N.ptr(s2), g,
               N.stream_of(grad_re))
        return gre, gim, gs.reshape(sin_decay.shape), gc.reshape(cos_decay.shape)
    N.call('sb_res_bwd', grad_re, N.ptr(grad_re), N.ptr(grad_im), None, None, N.ptr(sd), N.ptr(cd), sd.numel(),
           N.ptr(gre), N.ptr(gim), None, None, None, None, g, N.stream_of(grad_re))
    return gre, gim, None, None


def adres_fwd(re_in, im_in, sin_decay, cos_decay, ref_decay, th_decay, re_state, im_state, ref_state, th_state,
              th_scale, th0, w_scale):
    N.require_cuda(re_in, im_in)
    re_in, im_in = _c(re_in), _c(im_in)
    sd, cd = _param(sin_decay, re_in), _param(cos_decay, re_in)
    rd, td = _param(ref_decay, re_in), _param(th_decay, re_in)
    rs, ims = row_state(re_state, re_in), row_state(im_state, re_in)
    refs, ths = row_state(ref_state, re_in), row_state(th_state, re_in)
    outs = [torch.empty_like(re_in) for _ in range(4)]
    g = geom(re_in, sd.numel(), rd.numel(), td.numel())
    N.call('sb_adres_fwd', re_in, N.ptr(re_in), N.ptr(im_in), N.ptr(sd), N.ptr(cd), sd.numel(), N.ptr(rd),
           rd.numel(), N.ptr(td), td.numel(), N.ptr(rs), N.ptr(ims), N.ptr(refs), N.ptr(ths), N.ptr(outs[0]),
           N.ptr(outs[1]), N.ptr(outs[2]), N.ptr(outs[3]), g, int(th_scale * w_scale), int(th0 * w_scale),
           int(w_scale), N.stream_of(re_in))
    return tuple(outs)


# --------------------------------------------------------------------------
# spike functions
# --------------------------------------------------------------------------
def _thr_args(threshold, like):
    """(tensor pointer or None, scalar) for a float-or-tensor threshold."""
    if torch.is_tensor(threshold) and threshold.numel() > 1:
        t = threshold.detach().to(device=like.device, dtype=torch.float32)
        if t.shape != like.shape:
            t = t.expand(like.shape)
        return _c(t), 0.0
    if torch.is_tensor(threshold):
        return None, f32(threshold.item())
    return None, f32(threshold)


def spike_fwd(v, threshold, graded, scale):
    N.require_cuda(v)
    v = _c(v)
    tt, ts = _thr_args(threshold, v)
    out = torch.empty_like(v)
    N.call('sb_spike_fwd', v, N.ptr(v), N.ptr(tt), ts, N.ptr(out), v.numel(), int(bool(graded)), float(scale),
           N.stream_of(v))
    return out


def spike_bwd(v, threshold, grad_spike, tau_rho, scale_rho, graded):
    N.require_cuda(v, grad_spike)
    v, grad_spike = _c(v), _c(grad_spike)
    tt, ts = _thr_args(threshold, v)
    out = torch.empty_like(v)
    N.call('sb_spike_bwd', v, N.ptr(v), N.ptr(tt), ts, N.ptr(grad_spike), N.ptr(out), v.numel(), f32(tau_rho),
           f32(scale_rho), int(bool(graded)), N.stream_of(v))
    return out


def cspike_fwd(re, im, threshold, imag_last, graded, scale):
    N.require_cuda(re, im)
    re, im = _c(re), _c(im)
    tt, ts = _thr_args(threshold, re)
    if not torch.is_tensor(imag_last):
        imag_last = torch.tensor(float(imag_last))
    last = row_state(imag_last, im)
    rows, T = _rows_T(re)
    out = torch.empty_like(re)
    N.call('sb_cspike_fwd', re, N.ptr(re), N.ptr(im), N.ptr(tt), ts, N.ptr(last), N.ptr(out), rows, T,
           int(bool(graded)), float(scale), N.stream_of(re))
    return out


def cspike_bwd(re, im, threshold, grad_spike, tau_rho, scale_rho, graded):
    N.require_cuda(re, im, grad_spike)
    re, im, grad_spike = _c(re), _c(im), _c(grad_spike)
    tt, ts = _thr_args(threshold, re)
    gre = torch.empty_like(re)
    gim = torch.empty_like(re)
    N.call('sb_cspike_bwd', re, N.ptr(re), N.ptr(im), N.ptr(tt), ts, N.ptr(grad_spike), N.ptr(gre), N.ptr(gim),
           re.numel(), f32(tau_rho), f32(scale_rho), int(bool(graded)), N.stream_of(re))
    return gre, gim


# --------------------------------------------------------------------------
# shift / temporal filter
# --------------------------------------------------------------------------
def _lut_args(shift_val, x, sampling_time):
    """(lut tensor or None, n_lut, scalar shift, shift sampling time)."""
    if torch.is_tensor(shift_val) and shift_val.numel() > 1:
        n_spatial = int(np.prod(x.shape[1:-1]))
        if n_spatial != shift_val.numel():
            raise Exception(
                f'Expected spatial dimension of input and shift_val to be same. '
                f'Found input.shape={tuple(x.shape)}, shift_val.shape={tuple(shift_val.shape)}.'
            )
        lut = _c(shift_val.detach().to(device=x.device, dtype=torch.float32).reshape(-1))
        return lut, lut.numel(), 0.0, float(sampling_time)
    if torch.is_tensor(shift_val):
        shift_val = shift_val.item()
    # scalar path: int(shift / sampling_time) in Python arithmetic (shift.py:55-56)
    return None, 0, float(int(shift_val / sampling_time)), 1.0


def shift(x, shift_val, sampling_time=1):
    N.require_cuda(x)
    if x.dim() <= 1:
        raise AssertionError(f'Expected input to have at least two dimension. Found input.shape={tuple(x.shape)}.')
    x = _c(x)
    lut, n_lut, sv, ts = _lut_args(shift_val, x, sampling_time)
    rows, T = _rows_T(x)
    out = torch.empty_like(x)
    N.call('sb_shift', x, N.ptr(x), N.ptr(lut), n_lut, sv, ts, N.ptr(out), rows, T, N.stream_of(x))
    return out


def fir(x, filt, sampling_time, corr):
    N.require_cuda(x)
    x = _c(x)
    f = _c(filt.detach().to(device=x.device, dtype=torch.float32).reshape(-1))
    rows, T = _rows_T(x)
    out = torch.empty_like(x)
    N.call('sb_fir_corr' if corr else 'sb_fir_conv', x, N.ptr(x), N.ptr(f), f.numel(), float(sampling_time),
           N.ptr(out), rows, T, N.stream_of(x))
    return out


def shift_fir(x, shift_val, shift_ts, filt, sampling_time, backward):
    N.require_cuda(x)
    x = _c(x)
    f = _c(filt.detach().to(device=x.device, dtype=torch.float32).reshape(-1))
    lut, n_lut, sv, ts = _lut_args(shift_val, x, shift_ts)
    rows, T = _rows_T(x)
    out = torch.empty_like(x)
    N.call('sb_shift_fir_bwd' if backward else 'sb_shift_fir_fwd', x, N.ptr(x), N.ptr(lut), n_lut, sv, ts,
           N.ptr(f), f.numel(), float(sampling_time), N.ptr(out), rows, T, N.stream_of(x))
    return out


# --------------------------------------------------------------------------
# sigma-delta family
# --------------------------------------------------------------------------
def _opt_state(state, x):
    return None if state is None else row_state(state, x)


def sigma_fwd(x, state=None, want_final=False):
    N.require_cuda(x)
    x = _c(x)
    rows, T = _rows_T(x)
    st = _opt_state(state, x)
    out = torch.empty_like(x)
    fin = _vec(x) if want_final else None
    N.call('sb_sigma_fwd', x, N.ptr(x), N.ptr(st), N.ptr(out), N.ptr(fin), rows, T, N.stream_of(x))
    return (out, fin) if want_final else out


def sigma_bwd(grad_out):
    N.require_cuda(grad_out)
    grad_out = _c(grad_out)
    rows, T = _rows_T(grad_out)
    gx = torch.empty_like(grad_out)
    N.call('sb_sigma_bwd', grad_out, N.ptr(grad_out), N.ptr(gx), rows, T, N.stream_of(grad_out))
    return gx


def delta_fwd(x, threshold, pre_state, residual_state, scale, want_delta):
    """Returns (out, delta_input or None, final_residual)."""
    N.require_cuda(x)
    x = _c(x)
    thr = _param(threshold, x)
    pre, res = _opt_state(pre_state, x), _opt_state(residual_state, x)
    out = torch.empty_like(x)
    dlt = torch.empty_like(x) if want_delta else None
    fres = _vec(x)
    g = geom(x, thr.numel())
    N.call('sb_delta_fwd', x, N.ptr(x), N.ptr(thr), thr.numel(), N.ptr(pre), N.ptr(res), N.ptr(out), N.ptr(dlt),
           N.ptr(fres), g, float(scale), N.stream_of(x))
    return out, dlt, fres


def delta_bwd(grad_out, delta_input, threshold, tau_grad, scale_grad, need_threshold_grad):
    N.require_cuda(grad_out)
    grad_out = _c(grad_out)
    thr = _param(threshold, grad_out)
    gx = torch.empty_like(grad_out)
    g = geom(grad_out, thr.numel())
    if need_threshold_grad:
        gthr = torch.empty(thr.numel(), device=grad_out.device, dtype=torch.float32)
        scr = N.scratch(g.rows, thr.numel(), grad_out.device)
        N.call('sb_delta_bwd', grad_out, N.ptr(grad_out), N.ptr(_c(delta_input)), N.ptr(thr), thr.numel(), N.ptr(gx),
               N.ptr(gthr), N.ptr(scr), g, float(tau_grad), float(scale_grad), N.stream_of(grad_out))
        return gx, gthr.reshape(threshold.shape)
    N.call('sb_delta_bwd', grad_out, N.ptr(grad_out), None, N.ptr(thr), thr.numel(), N.ptr(gx), None, None, g,
           float(tau_grad), float(scale_grad), N.stream_of(grad_out))
    return gx, None


def sdnn_relu_fwd(x, threshold, bias, sigma_state, pre_state, residual_state, scale, want_act=False,
                  want_delta=False):
    """Sigma -> bias -> relu -> delta -> floor in one pass.  Returns dict(out, activation, delta_input,
    final_sigma, final_pre, final_residual); the two saved tensors only on request."""
    N.require_cuda(x)
    x = _c(x)
    thr = _param(threshold, x)
    b = None if bias is None else _param(bias, x)
    ss, pre, res = _opt_state(sigma_state, x), _opt_state(pre_state, x), _opt_state(residual_state, x)
    out = torch.empty_like(x)
    act = torch.empty_like(x) if (want_act or want_delta) else None
    dlt = torch.empty_like(x) if want_delta else None
    fs, fp, fr = _vec(x), _vec(x), _vec(x)
    g = geom(x, thr.numel())
    N.call('sb_sdnn_relu_fwd', x, N.ptr(x), N.ptr(ss), N.ptr(b), 0 if b is None else b.numel(), N.ptr(thr),
           thr.numel(), N.ptr(pre), N.ptr(res), N.ptr(out), N.ptr(act), N.ptr(dlt), N.ptr(fs), N.ptr(fp), N.ptr(fr), g,
           float(scale), N.stream_of(x))
    return dict(out=out, activation=act, delta_input=dlt, final_sigma=fs, final_pre=fp, final_residual=fr)


def sdnn_relu_bwd(grad_out, activation, delta_input, threshold, tau_grad, scale_grad, need_threshold_grad):
    N.require_cuda(grad_out)
    grad_out = _c(grad_out)
    thr = _param(threshold, grad_out)
    gx = torch.empty_like(grad_out)
    g = geom(grad_out, thr.numel())
    if need_threshold_grad:
        gthr = torch.empty(thr.numel(), device=grad_out.device, dtype=torch.float32)
        scr = N.scratch(g.rows, thr.numel(), grad_out.device)
        N.call('sb_sdnn_relu_bwd', grad_out, N.ptr(grad_out), N.ptr(activation), N.ptr(delta_input), N.ptr(thr),
               thr.numel(), N.ptr(gx), N.ptr(gthr), N.ptr(scr), g, float(tau_grad), float(scale_grad),
               N.stream_of(grad_out))
        return gx, gthr.reshape(threshold.shape)
    N.call('sb_sdnn_relu_bwd', grad_out, N.ptr(grad_out), N.ptr(activation), None, N.ptr(thr), thr.numel(), N.ptr(gx),
           None, None, g, float(tau_grad), float(scale_grad), N.stream_of(grad_out))
    return gx, None


# --------------------------------------------------------------------------
# fused neurons
# --------------------------------------------------------------------------
def _vec(shape_like):
    return torch.empty(shape_like.shape[:-1], device=shape_like.device, dtype=torch.float32)


def cuba_fwd(x, cdecay, vdecay, cstate, vstate, threshold, w_scale, want_current, want_spike, graded=False,
             spike_scale=1.0, spike_delay=0, delay_head=None, axon_delay=None, axon_delay_ts=1.0, want_voltage=True):
    """Returns dict with current/voltage/spike series and final_c/final_v/final_s.
    ``spike_delay=1`` returns the spike series one step late (``delay_head`` fills t = 0);
    ``axon_delay`` (one value per neuron, 0..62 steps) delays each row further.
    ``want_voltage=False`` (binary spikes only, no current) leaves the voltage series unwritten."""
    N.require_cuda(x)
    x = _c(x)
    cd, vd = _param(cdecay, x), _param(vdecay, x)
    cs, vs = row_state(cstate, x), row_state(vstate, x)
    cur = torch.empty_like(x) if want_current else None
    vol = torch.empty_like(x) if want_voltage else None
    spk = torch.empty_like(x) if want_spike else None
    fc, fv = _vec(x), _vec(x)
    fs = _vec(x) if want_spike else None
    g = geom(x, cd.numel(), vd.numel())
    head = None if delay_head is None else row_state(delay_head, x)
    lut, n_lut = None, 0
    if axon_delay is not None:
        lut = _c(axon_delay.detach().to(device=x.device, dtype=torch.float32).reshape(-1))
        n_lut = lut.numel()
        if n_lut != int(np.prod(x.shape[1:-1])):
            raise ValueError(f'axon_delay needs one value per neuron ({int(np.prod(x.shape[1:-1]))}), got {n_lut}')
    N.call('sb_cuba_fwd', x, N.ptr(x), N.ptr(cd), cd.numel(), N.ptr(vd), vd.numel(), N.ptr(cs), N.ptr(vs),
           N.ptr(cur), N.ptr(vol), N.ptr(spk), N.ptr(fc), N.ptr(fv), N.ptr(fs), g, float(threshold), int(w_scale),
           int(bool(graded)), float(spike_scale), int(spike_delay), N.ptr(head), N.ptr(lut), n_lut,
           float(axon_delay_ts), N.stream_of(x))
    return dict(current=cur, voltage=vol, spike=spk, final_c=fc, final_v=fv, final_s=fs)


def cuba_fwd_packed(x, cdecay, vdecay, cstate, vstate, threshold, w_scale, want_voltage=False, spike_delay=0,
                    delay_head=None):
    """Inference pass with the spikes as bits: ``spike_bits`` is int32 ``x.shape[:-1] + (ceil(T / 32),)``,
    bit ``i`` of word ``w`` = spike at step ``32 w + i`` (``unpack_spikes`` restores the fp32 tensor).
    Returns dict(spike_bits, voltage or None, final_c, final_v, final_s)."""
    N.require_cuda(x)
    x = _c(x)
    cd, vd = _param(cdecay, x), _param(vdecay, x)
    cs, vs = row_state(cstate, x), row_state(vstate, x)
    T = x.shape[-1]
    bits = torch.empty(x.shape[:-1] + ((T + 31) // 32,), device=x.device, dtype=torch.int32)
    vol = torch.empty_like(x) if want_voltage else None
    fc, fv, fs = _vec(x), _vec(x), _vec(x)
    g = geom(x, cd.numel(), vd.numel())
    head = None if delay_head is None else row_state(delay_head, x)
    N.call('sb_cuba_fwd_packed', x, N.ptr(x), N.ptr(cd), cd.numel(), N.ptr(vd), vd.numel(), N.ptr(cs), N.ptr(vs),
           N.ptr(vol), N.ptr(bits), N.ptr(fc), N.ptr(fv), N.ptr(fs), g, float(threshold), int(w_scale),
           int(spike_delay), N.ptr(head), N.stream_of(x))
    return dict(spike_bits=bits, voltage=vol, final_c=fc, final_v=fv, final_s=fs)


def unpack_spikes(bits, T, out=None, stream=None, threads=0):
    """fp32 0/1 tensor ``bits.shape[:-1] + (T,)`` from the packed words of ``cuba_fwd_packed``.

    CUDA ``bits``: plain torch ops on the device.  CPU ``bits`` (the result copied to the host as
    bits, 1/32 of the bytes): expanded by the library on ``threads`` CPU threads (0 = all) into
    ``out`` (allocated when ``None``).  With ``stream`` (a ``torch.cuda.Stream``) the expansion is
    queued on that stream as a host function -- after a non-blocking copy of the bits queued there
    before, before anything queued later -- and ``out`` is complete once the stream has passed it."""
    if bits.is_cuda:
        shifts = torch.arange(32, device=bits.device, dtype=torch.int32)
        b = (bits.unsqueeze(-1) >> shifts) & 1
        return b.reshape(bits.shape[:-1] + (-1,))[..., :T].to(torch.float32)
    if bits.dtype != torch.int32 or not bits.is_contiguous() or bits.shape[-1] != (T + 31) // 32:
        raise ValueError('bits must be a contiguous int32 tensor with ceil(T / 32) words per row')
    shape = tuple(bits.shape[:-1]) + (T,)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32)
    elif tuple(out.shape) != shape or out.dtype != torch.float32 or not out.is_contiguous() or out.is_cuda:
        raise ValueError(f'out must be a contiguous fp32 CPU tensor of shape {shape}')
    rows = bits.numel() // max(bits.shape[-1], 1)
    rc = N.load().sb_unpack_spikes_host(c_void_p(bits.data_ptr()), c_void_p(out.data_ptr()), rows, T, int(threads),
                                        0 if stream is None else 1, c_void_p(0 if stream is None else stream.cuda_stream))
    if rc != 0:
        raise RuntimeError(f'sb_unpack_spikes_host failed ({rc}): {N.last_error()}')
    return out


def cuba_bwd(grad_spike, voltage, threshold, current, cdecay, vdecay, tau_rho, scale_rho, graded, need_decay_grad,
             spike_delay=0):
    N.require_cuda(grad_spike, voltage)
    grad_spike, voltage = _c(grad_spike), _c(voltage)
    cd, vd = _param(cdecay, voltage), _param(vdecay, voltage)
    tt, ts = _thr_args(threshold, voltage)
    gx = torch.empty_like(voltage)
    g = geom(voltage, cd.numel(), vd.numel())
    gcd = gvd = sc = sv = None
    if need_decay_grad:
        current = _c(current)
        gcd = torch.empty(cd.numel(), device=voltage.device, dtype=torch.float32)
        gvd = torch.empty(vd.numel(), device=voltage.device, dtype=torch.float32)
        sc = N.scratch(g.rows, cd.numel(), voltage.device)
        sv = N.scratch(g.rows, vd.numel(), voltage.device)
    N.call('sb_cuba_bwd', voltage, N.ptr(grad_spike), N.ptr(voltage), N.ptr(tt), ts,
           N.ptr(current) if need_decay_grad else None, N.ptr(cd), cd.numel(), N.ptr(vd), vd.numel(), N.ptr(gx),
           N.ptr(gcd), N.ptr(gvd), N.ptr(sc), N.ptr(sv), g, f32(tau_rho), f32(scale_rho), int(bool(graded)),
           int(spike_delay), N.stream_of(voltage))
    if need_decay_grad:
        return gx, gcd.reshape(cdecay.shape), gvd.reshape(vdecay.shape)
    return gx, None, None


def cuba_recurrent_fwd(z, rec, cdecay, vdecay, cstate, vstate, threshold, w_scale, graded=False, spike_scale=1.0):
    """Dense recurrent CUBA layer over ``z`` ``[batch, neurons, time]`` with the (quantised) recurrent
    matrix ``rec`` ``[neurons, neurons]``: one launch for the whole walk over time.  Returns dict with
    spike/voltage series and final_c/final_v/final_s."""
    N.require_cuda(z, rec)
    if z.dim() != 3 or rec.shape != (z.shape[1], z.shape[1]):
        raise ValueError(f'recurrent layer needs [batch, neurons, time] input and a square matrix, got '
                         f'{tuple(z.shape)} and {tuple(rec.shape)}')
    z = _c(z)
    rec_t = _c(rec.detach().to(torch.float32).t())
    cd, vd = _param(cdecay, z), _param(vdecay, z)
    cs, vs = row_state(cstate, z), row_state(vstate, z)
    vol, spk = torch.empty_like(z), torch.empty_like(z)
    fc, fv, fs = _vec(z), _vec(z), _vec(z)
    B, C, T = z.shape
    N.call('sb_cuba_recurrent_fwd', z, N.ptr(z), N.ptr(rec_t), N.ptr(cd), cd.numel(), N.ptr(vd), vd.numel(),
           N.ptr(cs), N.ptr(vs), N.ptr(vol), N.ptr(spk), N.ptr(fc), N.ptr(fv), N.ptr(fs), B, C, T,
           float(threshold), int(w_scale), int(bool(graded)), float(spike_scale), N.stream_of(z))
    return dict(voltage=vol, spike=spk, final_c=fc, final_v=fv, final_s=fs)


def cuba_recurrent_bwd(grad_spike, voltage, rec, threshold, tau_rho, scale_rho, graded=False):
    """Gradient of ``cuba_recurrent_fwd`` with respect to ``z``."""
    N.require_cuda(grad_spike, voltage, rec)
    grad_spike, voltage = _c(grad_spike), _c(voltage)
    rec = _c(rec.detach().to(torch.float32))
    gz = torch.empty_like(voltage)
    B, C, T = voltage.shape
    N.call('sb_cuba_recurrent_bwd', voltage, N.ptr(grad_spike), N.ptr(voltage), N.ptr(rec), N.ptr(gz), B, C, T,
           f32(threshold), f32(tau_rho), f32(scale_rho), int(bool(graded)), N.stream_of(voltage))
    return gz


def alif_fwd(x, cdecay, vdecay, ref_decay, th_decay, cstate, vstate, ref_state, th_state, th_step, th0, w_scale,
             dynamics_mode, graded=False, spike_scale=1.0, spike_delay=0, delay_head=None, spikes_only=False,
             margin=False):
    """``spikes_only`` (forward mode, binary spikes): the voltage and threshold series, which only
    the backward pass reads, are not written; ``outs`` is then ``[spike, None, None]``.
    ``margin`` (forward mode): ``outs`` is ``[spike, voltage - (threshold + refractory), None]`` -- the
    one series the backward pass needs when the decays are not learnt (``cuba_bwd`` on it with threshold 0)."""
    N.require_cuda(x)
    x = _c(x)
    cd, vd = _param(cdecay, x), _param(vdecay, x)
    rd, td = _param(ref_decay, x), _param(th_decay, x)
    cs, vs = row_state(cstate, x), row_state(vstate, x)
    rs, ts = row_state(ref_state, x), row_state(th_state, x)
    outs = [torch.empty_like(x) for _ in range(4 if dynamics_mode else 3)]
    if spikes_only:
        if dynamics_mode or graded:
            raise ValueError('spikes_only needs forward mode and binary spikes')
        outs = [outs[0], None, None]
    elif margin:
        if dynamics_mode:
            raise ValueError('margin needs forward mode')
        outs = [outs[0], outs[1], None]
    fin = [_vec(x) for _ in range(5)]
    g = geom(x, cd.numel(), vd.numel(), rd.numel(), td.numel())
    head = None if delay_head is None else row_state(delay_head, x)
    N.call('sb_alif_fwd', x, N.ptr(x), N.ptr(cd), cd.numel(), N.ptr(vd), vd.numel(), N.ptr(rd), rd.numel(),
           N.ptr(td), td.numel(), N.ptr(cs), N.ptr(vs), N.ptr(rs), N.ptr(ts),
           N.ptr(outs[0]), N.ptr(outs[1]), N.ptr(outs[2]), N.ptr(outs[3]) if dynamics_mode else None,
           N.ptr(fin[0]), N.ptr(fin[1]), N.ptr(fin[2]), N.ptr(fin[3]), None if dynamics_mode else N.ptr(fin[4]),
           g, int(th_step * w_scale), int(th0 * w_scale), int(w_scale), int(bool(dynamics_mode)),
           int(bool(graded)), float(spike_scale), int(spike_delay), N.ptr(head), N.stream_of(x))
    return outs, dict(final_c=fin[0], final_v=fin[1], final_th=fin[2], final_ref=fin[3], final_s=fin[4])


def rf_fwd(re_in, im_in, sin_decay, cos_decay, re_state, im_state, threshold, w_scale, graded=False,
           spike_scale=1.0, adaptive=None, dynamics_mode=False, spike_delay=0, delay_head=None, spikes_only=False,
           margin=False):
    """``adaptive`` = None for RF, else dict(ref_decay, th_decay, ref_state, th_state, th_step, th0).
    ``spikes_only`` (forward mode, binary spikes): the state series, which only the backward pass
    reads, are not written; ``outs`` is then ``[spike, None, ...]``.
    ``margin`` (adaptive, forward mode): ``outs`` is ``[spike, re - (threshold + refractory), im, None]`` -- what
    the backward pass needs when sin / cos are not learnt (``rf_bwd`` on it with threshold 0)."""
    N.require_cuda(re_in, im_in)
    re_in, im_in = _c(re_in), _c(im_in)
    sd, cd = _param(sin_decay, re_in), _param(cos_decay, re_in)
    rs, ims = row_state(re_state, re_in), row_state(im_state, re_in)
    adapt = adaptive is not None
    if adapt:
        rd, td = _param(adaptive['ref_decay'], re_in), _param(adaptive['th_decay'], re_in)
        refs, ths = row_state(adaptive['ref_state'], re_in), row_state(adaptive['th_state'], re_in)
        th_step, th0 = int(adaptive['th_step'] * w_scale), int(adaptive['th0'] * w_scale)
        counts = (sd.numel(), rd.numel(), td.numel())
    else:
        rd = td = refs = ths = None
        th_step = th0 = 0
        counts = (sd.numel(),)
    nout = 4 if adapt else 3
    outs = [torch.empty_like(re_in) for _ in range(nout)]
    if spikes_only:
        if dynamics_mode or graded:
            raise ValueError('spikes_only needs forward mode and binary spikes')
        outs = [outs[0]] + [None] * (nout - 1)
    elif margin:
        if dynamics_mode or not adapt:
            raise ValueError('margin needs the adaptive neuron in forward mode')
        outs = outs[:3] + [None]
    fin = [_vec(re_in) for _ in range(5)]
    g = geom(re_in, *counts)
    head = None if delay_head is None else row_state(delay_head, re_in)
    N.call('sb_rf_fwd', re_in, N.ptr(re_in), N.ptr(im_in), N.ptr(sd), N.ptr(cd), sd.numel(),
           N.ptr(rd), rd.numel() if adapt else 1, N.ptr(td), td.numel() if adapt else 1,
           N.ptr(rs), N.ptr(ims), N.ptr(refs), N.ptr(ths),
           N.ptr(outs[0]), N.ptr(outs[1]), N.ptr(outs[2]), N.ptr(outs[3]) if adapt else None,
           N.ptr(fin[0]), N.ptr(fin[1]), N.ptr(fin[2]) if adapt else None, N.ptr(fin[3]) if adapt else None,
           None if dynamics_mode else N.ptr(fin[4]), g, f32(threshold), th_step, th0, int(w_scale), int(adapt),
           int(bool(dynamics_mode)), int(bool(graded)), float(spike_scale), int(spike_delay), N.ptr(head),
           N.stream_of(re_in))
    return outs, dict(final_re=fin[0], final_im=fin[1], final_th=fin[2], final_ref=fin[3], final_s=fin[4])


def rf_bwd(grad_spike, re, im, threshold, sin_decay, cos_decay, tau_rho, scale_rho, graded, need_param_grad,
           spike_delay=0):
    N.require_cuda(grad_spike, re, im)
    grad_spike, re, im = _c(grad_spike), _c(re), _c(im)
    sd, cd = _param(sin_decay, re), _param(cos_decay, re)
    tt, ts = _thr_args(threshold, re)
    gre = torch.empty_like(re)
    gim = torch.empty_like(re)
    g = geom(re, sd.numel())
    gs = gc = s1 = s2 = None
    if need_param_grad:
        gs = torch.empty(sd.numel(), device=re.device, dtype=torch.float32)
        gc = torch.empty_like(gs)
        s1 = N.scratch(g.rows, sd.numel(), re.device)
        s2 = N.scratch(g.rows, sd.numel(), re.device)
    N.call('sb_rf_bwd', re, N.ptr(grad_spike), N.ptr(re), N.ptr(im), N.ptr(tt), ts, N.ptr(sd), N.ptr(cd),
           sd.numel(), N.ptr(gre), N.ptr(gim), N.ptr(gs), N.ptr(gc), N.ptr(s1), N.ptr(s2), g, f32(tau_rho),
           f32(scale_rho), int(bool(graded)), int(spike_delay), N.stream_of(re))
    if need_param_grad:
        return gre, gim, gs.reshape(sin_decay.shape), gc.reshape(cos_decay.shape)
    return gre, gim, None, None


# --------------------------------------------------------------------------
# sum-pooling synapse
# --------------------------------------------------------------------------
def pool_out_size(size, k):
    """Output length of the reference's pooling: it pads ``size % k`` zeros when the
    size is not a multiple of the window and then strides by the window."""
    padded = size + (size % k)
    return (padded - k) // k + 1 if padded >= k else 0


def pool_fwd(x, weight):
    """x: [N, C, H, W, T]; weight: [..., kh, kw, 1] kernel (already hooked)."""
    N.require_cuda(x)
    x = _c(x)
    n, c, h, w, t = x.shape
    kh, kw = int(weight.shape[-3]), int(weight.shape[-2])
    wgt = _c(weight.detach().to(device=x.device, dtype=torch.float32).reshape(-1))
    ho, wo = pool_out_size(h, kh), pool_out_size(w, kw)
    y = torch.empty((n, c, ho, wo, t), device=x.device, dtype=torch.float32)
    N.call('sb_pool_fwd', x, N.ptr(x), N.ptr(wgt), N.ptr(y), n * c, h, w, ho, wo, kh, kw, t, N.stream_of(x))
    return y


def pool_bwd(grad_y, weight, in_shape):
    N.require_cuda(grad_y)
    grad_y = _c(grad_y)
    n, c, h, w, t = in_shape
    kh, kw = int(weight.shape[-3]), int(weight.shape[-2])
    wgt = _c(weight.detach().to(device=grad_y.device, dtype=torch.float32).reshape(-1))
    gx = torch.empty(in_shape, device=grad_y.device, dtype=torch.float32)
    N.call('sb_pool_bwd', grad_y, N.ptr(grad_y), N.ptr(wgt), N.ptr(gx), n * c, h, w, grad_y.shape[2], grad_y.shape[3],
           kh, kw, t, N.stream_of(grad_y))
    return gx


def conv_fwd_supported(x, weight, stride, padding, dilation, groups):
    """``sb_conv_fwd`` covers stride 1, dilation 1, one group: on the tensor cores for 1x1, 3x3 and
    5x5 kernels with T % 4 == 0, through the fp32 kernel for the other shapes it can launch."""
    if not (x.is_cuda and x.dim() == 5 and x.dtype == torch.float32):
        return False
    if tuple(stride) != (1, 1, 1) or tuple(dilation) != (1, 1, 1) or groups != 1 or padding[2] != 0:
        return False
    n, ci, h, w, t = x.shape
    kh, kw = int(weight.shape[2]), int(weight.shape[3])
    ho = h + 2 * padding[0] - kh + 1
    if ho <= 0 or w + 2 * padding[1] - kw + 1 <= 0:
        return False
    if x.data_ptr() % 16 == 0 and N.load().sb_conv_fits_tensor_cores(
            n, ci, int(weight.shape[0]), h, w, kh, kw, int(padding[0]), int(padding[1]), t):
        return True   # tcgen05 implicit GEMM
    # limits of the fp32 kernel: its launch grid and the weights of 16 output channels in shared memory
    return 0 < n * ho <= 65535 and ci * kh * kw * 16 * 4 <= 96 * 1024


def conv_fwd(x, weight, padding, path=-1):
    """x: [N, Ci, H, W, T]; weight: [Co, Ci, kh, kw, 1] (already hooked); padding (ph, pw).
    ``path``: -1 lets the library choose, 0 forces the fp32 kernel, 1 the tensor cores."""
    N.require_cuda(x)
    x = _c(x)
    n, ci, h, w, t = x.shape
    co, _, kh, kw = weight.shape[:4]
    wgt = _c(weight.detach().to(device=x.device, dtype=torch.float32).reshape(co, -1))
    ph, pw = int(padding[0]), int(padding[1])
    y = torch.empty((n, co, h + 2 * ph - kh + 1, w + 2 * pw - kw + 1, t), device=x.device, dtype=torch.float32)
    if path == -1:
        # shapes only the tensor-core kernel can launch (more than 65535 output rows, wide layers)
        fp32_ok = 0 < n * y.shape[2] <= 65535 and ci * kh * kw * 16 * 4 <= 96 * 1024
        if not fp32_ok:
            path = 1
    N.call('sb_conv_fwd_path', x, N.ptr(x), N.ptr(wgt), N.ptr(y), n, ci, co, h, w, kh, kw, ph, pw, t, int(path),
           N.stream_of(x))
    return y


def conv_wgrad_supported(x, weight, padding=(0, 0)):
    """Whether the weight-gradient kernel takes the layer: ``T % 4 == 0``, at most 384 accumulator
    tiles of 8 x 8, one output row staged within its shared memory (the library decides)."""
    if x.dim() != 5 or x.data_ptr() % 16 != 0:
        return False
    n, ci, h, w, t = x.shape
    co, _, kh, kw = weight.shape[:4]
    return N.load().sb_conv_wgrad_fits(n, ci, co, h, w, kh, kw, int(padding[0]), int(padding[1]), t) == 1


def conv_wgrad(x, grad_y, weight_shape, padding):
    """Gradient of ``conv_fwd`` with respect to the weight; returns a tensor of ``weight_shape``."""
    N.require_cuda(x, grad_y)
    x, grad_y = _c(x), _c(grad_y)
    n, ci, h, w, t = x.shape
    co, _, kh, kw = weight_shape[:4]
    ph, pw = int(padding[0]), int(padding[1])
    gw = torch.empty(tuple(weight_shape), device=x.device, dtype=torch.float32)
    nbytes = N.load().sb_conv_wgrad_scratch_bytes(n, ci, co, h, kh, kw, ph)
    scratch = torch.empty(max(nbytes // 4, 1), device=x.device, dtype=torch.float32)
    N.call('sb_conv_wgrad', x, N.ptr(x), N.ptr(grad_y), N.ptr(gw), N.ptr(scratch), n, ci, co, h, w, kh, kw, ph, pw,
           t, N.stream_of(x))
    return gw


def conv_dgrad(grad_y, weight, padding):
    """Gradient of ``conv_fwd`` with respect to its input: the same kernel on ``grad_y``
    with the weight flipped in space and its channel axes swapped."""
    kh, kw = weight.shape[2], weight.shape[3]
    wt = weight.detach()[:, :, :, :, 0] if weight.dim() == 5 else weight.detach()
    wt = wt.flip(2, 3).transpose(0, 1).contiguous()
    # gradients are not exact in TF32: the tensor-core kernel splits them into TF32 pairs (still faster
    # than the fp32 kernel where the swapped problem fits it); the library chooses
    pad = (kh - 1 - int(padding[0]), kw - 1 - int(padding[1]))
    return conv_fwd(grad_y, wt, pad, path=-1)
