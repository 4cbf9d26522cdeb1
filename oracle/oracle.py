"""numpy front end of the C oracle (``slayer_oracle.c``) plus the neuron-level
call sequences of lava-dl restated on top of it.

TEST INFRASTRUCTURE ONLY.  Arrays are float32 numpy arrays shaped like the
torch tensors of the reference API (``[batch, ..., time]``).  Each function
cites the reference code it follows (paths relative to
``src/lava/lib/dl/slayer/``).
"""

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, '_build', 'libslayer_oracle.so')
_lib = None


def build(force=False):
    src = os.path.join(_HERE, 'slayer_oracle.c')
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        r = subprocess.run(['make', '-C', _HERE] + (['-B'] if force else []), capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f'oracle build failed:\n{r.stdout}\n{r.stderr}')
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
    return _lib


def set_threads(n):
    """Number of OpenMP threads used by the oracle (for the timed baseline)."""
    os.environ['OMP_NUM_THREADS'] = str(n)
    try:
        omp = ctypes.CDLL('libgomp.so.1')
        omp.omp_set_num_threads(int(n))
    except OSError:
        pass


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def _geom(x, *counts):
    T = x.shape[-1]
    rows = x.size // T if T else 0
    rpb = int(np.prod(x.shape[1:-1])) if x.ndim >= 3 else 1
    blk = int(np.prod(x.shape[2:-1])) if x.ndim > 3 else 1
    return rows, T, rpb, blk


def _state(s, x):
    s = np.asarray(s, dtype=np.float32)
    lead = x.shape[:-1]
    if s.size == 1:
        return np.full(int(np.prod(lead)) if len(lead) else 1, s.reshape(-1)[0], dtype=np.float32)
    return _f(np.broadcast_to(s, lead)).reshape(-1)


def _vec(p):
    return _f(np.asarray(p, dtype=np.float32).reshape(-1))


I64 = c_int64


# --------------------------------------------------------------------------
# primitives
# --------------------------------------------------------------------------
def li_fwd(x, decay, state, w_scale, threshold=None):
    """neuron/dynamics/leaky_integrator.py:50-100,210-231"""
    x = _f(x)
    decay = _vec(decay)
    st = _state(state, x)
    y = np.empty_like(x)
    thr = (-1 if threshold is None else threshold) * w_scale
    rows, T, rpb, blk = _geom(x)
    lib().orc_li_fwd(_p(x), _p(decay), I64(decay.size), _p(st), _p(y), I64(rows), I64(T), I64(rpb), I64(blk),
                     c_double(thr), c_int(int(w_scale)))
    return y


def li_bwd(grad_out, out, decay):
    """neuron/dynamics/leaky_integrator.py:234-259; returns (grad_in, grad_decay[float64])"""
    go, out = _f(grad_out), _f(out)
    dec = _vec(decay)
    gi = np.empty_like(go)
    gd = np.zeros(dec.size, dtype=np.float64)
    rows, T, rpb, blk = _geom(go)
    lib().orc_li_bwd(_p(go), _p(out), _p(dec), I64(dec.size), _p(gi), _p(gd), I64(rows), I64(T), I64(rpb), I64(blk))
    return gi, gd


def ath_fwd(x, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale):
    """neuron/dynamics/adaptive_threshold.py:51-126,237-274"""
    x = _f(x)
    rd, td = _vec(ref_decay), _vec(th_decay)
    rs, ts = _state(ref_state, x), _state(th_state, x)
    th, ref = np.empty_like(x), np.empty_like(x)
    rows, T, rpb, blk = _geom(x)
    lib().orc_ath_fwd(_p(x), _p(rs), _p(rd), I64(rd.size), _p(ts), _p(td), I64(td.size), _p(th), _p(ref),
                      I64(rows), I64(T), I64(rpb), I64(blk), I64(int(th_scale * w_scale)),
                      I64(int(th0 * w_scale)), c_int(int(w_scale)))
    return th, ref


def apth_fwd(re, im, im_state, ref_state, ref_decay, th_state, th_decay, th_scale, th0, w_scale):
    """neuron/dynamics/adaptive_phase_th.py:51-132,234-283"""
    re, im = _f(re), _f(im)
    rd, td = _vec(ref_decay), _vec(th_decay)
    ims, rs, ts = _state(im_state, re), _state(ref_state, re), _state(th_state, re)
    th, ref = np.empty_like(re), np.empty_like(re)
    rows, T, rpb, blk = _geom(re)
    lib().orc_apth_fwd(_p(re), _p(im), _p(ims), _p(rs), _p(rd), I64(rd.size), _p(ts), _p(td), I64(td.size),
                       _p(th), _p(ref), I64(rows), I64(T), I64(rpb), I64(blk), I64(int(th_scale * w_scale)),
                       I64(int(th0 * w_scale)), c_int(int(w_scale)))
    return th, ref


def res_fwd(re_in, im_in, sin_decay, cos_decay, re_state, im_state, w_scale, threshold=None):
    """neuron/dynamics/resonator.py:49-132,333-376"""
    re_in, im_in = _f(re_in), _f(im_in)
    sd, cd = _vec(sin_decay), _vec(cos_decay)
    rs, ims = _state(re_state, re_in), _state(im_state, re_in)
    re, im = np.empty_like(re_in), np.empty_like(re_in)
    thr = (-1 if threshold is None else threshold) * w_scale
    rows, T, rpb, blk = _geom(re_in)
    lib().orc_res_fwd(_p(re_in), _p(im_in), _p(sd), _p(cd), I64(sd.size), _p(rs), _p(ims), _p(re), _p(im),
                      I64(rows), I64(T), I64(rpb), I64(blk), c_double(thr), c_int(int(w_scale)))
    return re, im


def res_bwd(g_re, g_im, re, im, sin_decay, cos_decay):
    """neuron/dynamics/resonator.py:379-467; returns grads and float64 sin/cos grads"""
    g_re, g_im, re, im = _f(g_re), _f(g_im), _f(re), _f(im)
    sd, cd = _vec(sin_decay), _vec(cos_decay)
    a, b = np.empty_like(g_re), np.empty_like(g_re)
    gs, gc = np.zeros(sd.size, dtype=np.float64), np.zeros(sd.size, dtype=np.float64)
    rows, T, rpb, blk = _geom(g_re)
    lib().orc_res_bwd(_p(g_re), _p(g_im), _p(re), _p(im), _p(sd), _p(cd), I64(sd.size), _p(a), _p(b), _p(gs),
                      _p(gc), I64(rows), I64(T), I64(rpb), I64(blk))
    return a, b, gs, gc


def adres_fwd(re_in, im_in, sin_decay, cos_decay, ref_decay, th_decay, re_state, im_state, ref_state, th_state,
              th_scale, th0, w_scale):
    """neuron/dynamics/adaptive_resonator.py:49-158,379-436"""
    re_in, im_in = _f(re_in), _f(im_in)
    sd, cd, rd, td = _vec(sin_decay), _vec(cos_decay), _vec(ref_decay), _vec(th_decay)
    rs, ims = _state(re_state, re_in), _state(im_state, re_in)
    refs, ths = _state(ref_state, re_in), _state(th_state, re_in)
    outs = [np.empty_like(re_in) for _ in range(4)]
    rows, T, rpb, blk = _geom(re_in)
    lib().orc_adres_fwd(_p(re_in), _p(im_in), _p(sd), _p(cd), I64(sd.size), _p(rd), I64(rd.size), _p(td),
                        I64(td.size), _p(rs), _p(ims), _p(refs), _p(ths), _p(outs[0]), _p(outs[1]), _p(outs[2]),
                        _p(outs[3]), I64(rows), I64(T), I64(rpb), I64(blk), I64(int(th_scale * w_scale)),
                        I64(int(th0 * w_scale)), c_int(int(w_scale)))
    return tuple(outs)


def _thr(threshold, like):
    if isinstance(threshold, np.ndarray) and threshold.size > 1:
        return _f(np.broadcast_to(threshold, like.shape)), 0.0
    return None, float(np.asarray(threshold, dtype=np.float32).reshape(-1)[0])


def spike_fwd(v, threshold, graded=False, scale=1):
    """spike/spike.py:64-110"""
    v = _f(v)
    tt, ts = _thr(threshold, v)
    out = np.empty_like(v)
    lib().orc_spike_fwd(_p(v), _p(tt), c_float(ts), _p(out), I64(v.size), c_int(int(graded)), c_float(scale))
    return out


def spike_bwd(v, threshold, grad_spike, tau_rho, scale_rho, graded=False):
    """spike/spike.py:10-23,112-126"""
    v, gs = _f(v), _f(grad_spike)
    tt, ts = _thr(threshold, v)
    out = np.empty_like(v)
    lib().orc_spike_bwd(_p(v), _p(tt), c_float(ts), _p(gs), _p(out), I64(v.size),
                        c_float(np.float32(tau_rho)), c_float(np.float32(scale_rho)), c_int(int(graded)))
    return out


def cspike_fwd(re, im, threshold, imag_last, graded=False, scale=1):
    """spike/complex.py:49-116"""
    re, im = _f(re), _f(im)
    tt, ts = _thr(threshold, re)
    last = _state(imag_last, im)
    out = np.empty_like(re)
    rows, T, _, _ = _geom(re)
    lib().orc_cspike_fwd(_p(re), _p(im), _p(tt), c_float(ts), _p(last), _p(out), I64(rows), I64(T),
                         c_int(int(graded)), c_float(scale))
    return out


def cspike_bwd(re, im, threshold, grad_spike, tau_rho, scale_rho, graded=False):
    """spike/complex.py:118-167"""
    re, im, gs = _f(re), _f(im), _f(grad_spike)
    tt, ts = _thr(threshold, re)
    gre, gim = np.empty_like(re), np.empty_like(re)
    lib().orc_cspike_bwd(_p(re), _p(im), _p(tt), c_float(ts), _p(gs), _p(gre), _p(gim), I64(re.size),
                         c_float(np.float32(tau_rho)), c_float(np.float32(scale_rho)), c_int(int(graded)))
    return gre, gim


def shift(x, shift_val, sampling_time=1):
    """utils/time/shift.py:94-143 with int(shift / sampling_time) truncation"""
    x = _f(x)
    if isinstance(shift_val, np.ndarray) and shift_val.size > 1:
        d = (np.asarray(shift_val, dtype=np.float32).reshape(-1) / np.float32(sampling_time)).astype(np.int64)
    else:
        d = np.array([int(float(np.asarray(shift_val).reshape(-1)[0]) / sampling_time)], dtype=np.int64)
    d = np.ascontiguousarray(d)
    out = np.empty_like(x)
    rows, T, _, _ = _geom(x)
    lib().orc_shift(_p(x), _p(d), I64(d.size), _p(out), I64(rows), I64(T))
    return out


def fir(x, filt, sampling_time=1, corr=False):
    """utils/filter/conv.py:48-97"""
    x = _f(x)
    f = _vec(filt)
    out = np.empty_like(x)
    rows, T, _, _ = _geom(x)
    lib().orc_fir(_p(x), _p(f), I64(f.size), c_float(sampling_time), _p(out), I64(rows), I64(T), c_int(int(corr)))
    return out


def conv(x, filt, sampling_time=1):
    return fir(x, filt, sampling_time, corr=False)


def corr(x, filt, sampling_time=1):
    return fir(x, filt, sampling_time, corr=True)


def sigma(x, state=None, reverse=False):
    """dendrite/sigma.py:38-72 (reverse=True: the adjoint, a running sum over reversed time)"""
    x = _f(x)
    st = None if state is None else _state(state, x)
    out = np.empty_like(x)
    rows, T, _, _ = _geom(x)
    lib().orc_sigma(_p(x), _p(st), _p(out), I64(rows), I64(T), c_int(int(reverse)))
    return out


def delta_fwd(x, threshold, pre_state=None, residual_state=None, scale=4096):
    """axon/delta.py:13-76,258-316 with cum_error=False; returns dict(out, delta_input, residual)"""
    x = _f(x)
    thr = _vec(threshold)
    pre = None if pre_state is None else _state(pre_state, x)
    res = None if residual_state is None else _state(residual_state, x)
    out, dlt = np.empty_like(x), np.empty_like(x)
    rows, T, rpb, blk = _geom(x)
    fres = np.empty(rows, dtype=np.float32)
    lib().orc_delta_fwd(_p(x), _p(thr), I64(thr.size), _p(pre), _p(res), _p(out), _p(dlt), _p(fres), I64(rows),
                        I64(T), I64(rpb), I64(blk), c_double(scale))
    return dict(out=out, delta_input=dlt, residual=fres.reshape(x.shape[:-1]))


def delta_bwd(grad_out, delta_input, threshold, tau_grad=1.0, scale_grad=1.0):
    """axon/delta.py:77-122; returns (grad_x, grad_threshold[float64])"""
    go, dlt = _f(grad_out), _f(delta_input)
    thr = _vec(threshold)
    gx = np.empty_like(go)
    gthr = np.zeros(thr.size, dtype=np.float64)
    rows, T, rpb, blk = _geom(go)
    lib().orc_delta_bwd(_p(go), _p(dlt), _p(thr), I64(thr.size), _p(gx), _p(gthr), I64(rows), I64(T), I64(rpb),
                        I64(blk), c_float(tau_grad), c_float(scale_grad))
    return gx, gthr


def sdnn_relu(x, threshold, bias=None, sigma_state=None, pre_state=None, residual_state=None, scale=4096):
    """neuron/sigma_delta.py:171-219 with activation = relu, norm = None:
    sigma -> + bias (per neuron) -> relu -> delta.  Returns dict(out, sigma, act, delta_input, residual)."""
    x = _f(x)
    s = sigma(x, sigma_state)
    z = s
    if bias is not None:
        # one bias per neuron (sigma_delta.py:190-200 adds bias[None, ..., None]) or a single value
        b = np.asarray(bias, dtype=np.float32).reshape(-1)
        z = (s + (b.reshape((1,) + x.shape[1:-1] + (1,)) if b.size > 1 else b[0])).astype(np.float32)
    act = np.maximum(z, np.float32(0)).astype(np.float32)
    r = delta_fwd(act, threshold, pre_state, residual_state, scale)
    r.update(sigma=s, act=act, pre=act[..., -1])
    return r


def quantize(p):
    """utils/quantize.py:18-32 with step 1: round half to even, as torch.round"""
    return np.round(np.asarray(p, dtype=np.float32))


# --------------------------------------------------------------------------
# neuron-level call sequences (forward + backward of loss = sum(spike * g))
# --------------------------------------------------------------------------
def cuba(x, threshold, current_decay, voltage_decay, scale=64, cstate=0., vstate=0., grad_spike=None,
         tau_grad=1, scale_grad=1, graded=False):
    """neuron/cuba.py:274-440.  Decays are the stored parameters (x 4096)."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale
    eps = 0.01 / s_scale
    cd, vd = quantize(current_decay), quantize(voltage_decay)
    current = li_fwd(x, cd, cstate, s_scale)
    voltage = li_fwd(current, vd, vstate, s_scale, thr + eps)
    spike = spike_fwd(voltage, thr + eps, graded, 1)
    out = dict(current=current, voltage=voltage, spike=spike)
    if grad_spike is not None:
        tau_rho, scale_rho = tau_grad * thr * 100, scale_grad * 0.1
        g_v = spike_bwd(voltage, thr + eps, grad_spike, tau_rho, scale_rho, graded)
        g_c, gvd = li_bwd(g_v, voltage, vd)
        g_x, gcd = li_bwd(g_c, current, cd)
        out.update(grad_x=g_x, grad_current_decay=gcd, grad_voltage_decay=gvd)
    return out


def cuba_grad_x_scale(voltage, threshold, grad_spike, current_decay, voltage_decay, scale=64, tau_grad=1,
                      scale_grad=1, graded=False):
    """Comparison scale for the input gradient of ``cuba``: the two reverse scans run on the
    magnitudes of their terms (float64).  An element of grad_x is a sum of signed terms whose
    exponentials differ by an ulp between math libraries; 1e-5 of this sum of magnitudes is the
    forward-error bound such a sum can be held to, and equals 1e-5 relative where nothing cancels."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale + 0.01 / s_scale
    g = np.abs(spike_bwd(voltage, thr, grad_spike, tau_grad * (int(threshold * w_scale) / w_scale) * 100,
                         scale_grad * 0.1, graded)).astype(np.float64)
    for decay in (voltage_decay, current_decay):
        d = quantize(decay).astype(np.float64).reshape(-1)
        a = np.abs(1.0 - d / 4096.0)
        a = a[0] if a.size == 1 else a.reshape((1, -1) + (1,) * (g.ndim - 3))
        acc = np.zeros(g.shape[:-1])
        out = np.empty_like(g)
        for t in range(g.shape[-1] - 1, -1, -1):
            acc = a * acc + g[..., t]
            out[..., t] = acc
        g = out
    return g


def cuba_recurrent(z, rec, threshold, current_decay, voltage_decay, scale=64, cstate=0., vstate=0., grad_spike=None,
                   tau_grad=1, scale_grad=1, graded=False):
    """utils/recurrent.py:45-112: per step, feedback = s[t-1] R^T, one CUBA neuron call
    with T = 1 whose state persists (neuron/cuba.py:396-440), and for the gradient the
    reverse walk in which only R couples the steps.  z [B, C, T], rec [C, C]."""
    z = np.asarray(z, dtype=np.float32)
    rec = np.asarray(rec, dtype=np.float32)
    B, C, T = z.shape
    spike = np.zeros_like(z)
    voltage = np.zeros_like(z)
    cs = np.broadcast_to(np.asarray(cstate, dtype=np.float32), (B, C)).copy()
    vs = np.broadcast_to(np.asarray(vstate, dtype=np.float32), (B, C)).copy()
    s = np.zeros((B, C), dtype=np.float32)
    for t in range(T):
        dend = (z[..., t] + s @ rec.T).astype(np.float32)
        r = cuba(dend[..., None], threshold, current_decay, voltage_decay, scale, cs, vs, graded=graded)
        s = r['spike'][..., 0]
        cs = r['current'][..., 0]
        vs = r['voltage'][..., 0] * (1 - (s > 0))   # leaky_integrator.py persistent_state
        spike[..., t], voltage[..., t] = s, r['voltage'][..., 0]
    out = dict(spike=spike, voltage=voltage, final_c=cs, final_v=vs)
    if grad_spike is not None:
        w_scale, s_scale = scale, scale * 64
        thr = int(threshold * w_scale) / w_scale
        eps = 0.01 / s_scale
        tau_rho, scale_rho = tau_grad * thr * 100, scale_grad * 0.1
        g = np.asarray(grad_spike, dtype=np.float32)
        grad_z = np.zeros_like(z)
        carry = np.zeros((B, C), dtype=np.float32)
        for t in range(T - 1, -1, -1):
            gs = (g[..., t] + carry).astype(np.float32)
            gd = spike_bwd(voltage[..., t:t + 1], thr + eps, gs[..., None], tau_rho, scale_rho, graded)[..., 0]
            grad_z[..., t] = gd
            carry = (gd @ rec).astype(np.float32)
        go = grad_z[..., 1:].transpose(1, 0, 2).reshape(C, -1)
        si = spike[..., :-1].transpose(0, 2, 1).reshape(-1, C)
        out.update(grad_z=grad_z, grad_rec=(go @ si).astype(np.float32))
    return out


def alif(x, threshold, threshold_step, current_decay, voltage_decay, threshold_decay, refractory_decay, scale=64,
         cstate=0., vstate=0., th_state=None, ref_state=0., grad_spike=None, tau_grad=1, scale_grad=1,
         graded=False):
    """neuron/alif.py:383-610.  Decays are the stored parameters (x 4096)."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale
    step = int(threshold_step * w_scale) / w_scale
    cd, vd = quantize(current_decay), quantize(voltage_decay)
    td, rd = quantize(threshold_decay), quantize(refractory_decay)
    current = li_fwd(x, cd, cstate, s_scale)
    voltage = li_fwd(current, vd, vstate, s_scale)
    th, ref = ath_fwd(voltage, ref_state, rd, thr if th_state is None else th_state, td, step, thr, s_scale)
    thsum = th + ref
    spike = spike_fwd(voltage, thsum, graded, 1)
    out = dict(current=current, voltage=voltage, threshold=th, refractory=ref, spike=spike)
    if grad_spike is not None:
        tau_rho, scale_rho = tau_grad * thr * 100, scale_grad * 0.1
        g_v = spike_bwd(voltage, thsum, grad_spike, tau_rho, scale_rho, graded)
        g_c, gvd = li_bwd(g_v, voltage, vd)
        g_x, gcd = li_bwd(g_c, current, cd)
        out.update(grad_x=g_x, grad_current_decay=gcd, grad_voltage_decay=gvd)
    return out


def rf(re_in, im_in, threshold, sin_decay, cos_decay, scale=64, re_state=0., im_state=0., grad_spike=None,
       tau_grad=1, scale_grad=1, graded=False):
    """neuron/rf.py:340-500.  sin/cos decays are the stored parameters."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale
    sd, cd = quantize(sin_decay), quantize(cos_decay)
    re, im = res_fwd(re_in, im_in, sd, cd, re_state, im_state, s_scale)
    spike = cspike_fwd(re, im, thr, im_state, graded, 1)
    out = dict(real=re, imag=im, spike=spike)
    if grad_spike is not None:
        tau_rho, scale_rho = tau_grad * thr * 0.5, scale_grad * 10
        g_re, g_im = cspike_bwd(re, im, thr, grad_spike, tau_rho, scale_rho, graded)
        a, b, gs, gc = res_bwd(g_re, g_im, re, im, sd, cd)
        out.update(grad_re=a, grad_im=b, grad_sin_decay=gs, grad_cos_decay=gc)
    return out


def adrf(re_in, im_in, threshold, threshold_step, sin_decay, cos_decay, threshold_decay, refractory_decay,
         scale=64, re_state=0., im_state=0., th_state=None, ref_state=0., grad_spike=None, tau_grad=1,
         scale_grad=1, graded=False):
    """neuron/adrf.py:439-677.  Decays are the stored parameters (x 4096)."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale
    step = int(threshold_step * w_scale) / w_scale
    sd, cd = quantize(sin_decay), quantize(cos_decay)
    td, rd = quantize(threshold_decay), quantize(refractory_decay)
    re, im = res_fwd(re_in, im_in, sd, cd, re_state, im_state, s_scale)
    th, ref = apth_fwd(re, im, im_state, ref_state, rd, thr if th_state is None else th_state, td, step, thr,
                       s_scale)
    thsum = th + ref
    spike = cspike_fwd(re, im, thsum, im_state, graded, 1)
    out = dict(real=re, imag=im, threshold=th, refractory=ref, spike=spike)
    if grad_spike is not None:
        tau_rho, scale_rho = tau_grad * thr * 100, scale_grad * 0.1
        g_re, g_im = cspike_bwd(re, im, thsum, grad_spike, tau_rho, scale_rho, graded)
        a, b, gs, gc = res_bwd(g_re, g_im, re, im, sd, cd)
        out.update(grad_re=a, grad_im=b, grad_sin_decay=gs, grad_cos_decay=gc)
    return out


def rf_iz(re_in, im_in, threshold, sin_decay, cos_decay, scale=64, re_state=0., im_state=0., grad_spike=None,
          tau_grad=1, scale_grad=1, graded=False):
    """neuron/rf_iz.py:331-520: resonator with Izhikevich reset, threshold spike on the imaginary part."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale
    sd, cd = quantize(sin_decay), quantize(cos_decay)
    re, im = res_fwd(re_in, im_in, sd, cd, re_state, im_state, s_scale, thr)
    spike = spike_fwd(im, thr, graded, 1)
    out = dict(real=re, imag=im, spike=spike)
    if grad_spike is not None:
        g_im = spike_bwd(im, thr, grad_spike, tau_grad * thr * 100, scale_grad * 0.1, graded)
        a, b, gs, gc = res_bwd(np.zeros_like(g_im), g_im, re, im, sd, cd)
        out.update(grad_re=a, grad_im=b, grad_sin_decay=gs, grad_cos_decay=gc, grad_imag_series=g_im)
    return out


def adrf_iz(re_in, im_in, threshold, threshold_step, sin_decay, cos_decay, threshold_decay, refractory_decay,
            scale=64, re_state=0., im_state=0., th_state=None, ref_state=0., grad_spike=None, tau_grad=1,
            scale_grad=1, graded=False):
    """neuron/adrf_iz.py:440-650: adaptive resonator, threshold spike on imag >= threshold + refractory."""
    w_scale, s_scale = scale, scale * 64
    thr = int(threshold * w_scale) / w_scale
    step = int(threshold_step * w_scale) / w_scale
    sd, cd = quantize(sin_decay), quantize(cos_decay)
    td, rd = quantize(threshold_decay), quantize(refractory_decay)
    re, im, th, ref = adres_fwd(re_in, im_in, sd, cd, rd, td, re_state, im_state, ref_state,
                                thr if th_state is None else th_state, step, thr, s_scale)
    thsum = th + ref
    spike = spike_fwd(im, thsum, graded, 1)
    out = dict(real=re, imag=im, threshold=th, refractory=ref, spike=spike)
    if grad_spike is not None:
        g_im = spike_bwd(im, thsum, grad_spike, tau_grad * thr * 100, scale_grad * 0.1, graded)
        a, b, gs, gc = res_bwd(np.zeros_like(g_im), g_im, re, im, sd, cd)
        out.update(grad_re=a, grad_im=b, grad_sin_decay=gs, grad_cos_decay=gc, grad_imag_series=g_im)
    return out
