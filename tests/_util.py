"""Comparison helpers shared by the parity tests.

Tolerances (stated once, used everywhere):

* spikes and quantised states: BIT-EXACT.  A state series ``s`` is quantised
  when ``s * w_scale`` is an integer; both sides are compared as int64 after
  that scaling.
* float quantities without cancellation (surrogate gradients, filter outputs
  of non-negative signals): ``|a - b| <= 1e-5 * max(|b|, 1e-2 * max|b|)``, i.e.
  1e-5 relative element-wise, the comparison scale floored at 1 % of the
  tensor's largest magnitude.
* gradients produced by a reverse scan, and parameter gradients, are sums of
  signed terms.  The two sides differ by a few ulp per term (``expf`` is not
  bit-identical between libm, SLEEF and CUDA), so an element that cancels to
  ~0 keeps the absolute error of its terms.  They are therefore held to 1e-5
  relative to the SUM OF THE MAGNITUDES of the terms each element adds up
  (``*_scale`` helpers below: the same recurrence run on absolute values),
  which is the plain relative error wherever nothing cancels:
  ``|a - b| <= 1e-5 * max(|b|, S)``.
"""

import glob
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
RTOL = 1e-5
FLOOR = 1e-2


def golden_cases(prefix):
    names = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + '*.npz')))
    assert names, f'no golden fixtures match {prefix}*'
    return names


def load_golden(name):
    with np.load(os.path.join(GOLDEN_DIR, name + '.npz'), allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


def to_np(a):
    if hasattr(a, 'detach'):
        a = a.detach().cpu().numpy()
    return np.asarray(a)


def assert_exact(a, b, what=''):
    a, b = to_np(a), to_np(b)
    assert a.shape == b.shape, f'{what}: shape {a.shape} vs {b.shape}'
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        i = tuple(bad[0])
        raise AssertionError(f'{what}: {len(bad)} of {a.size} elements differ; first at {i}: {a[i]!r} vs {b[i]!r}')


def assert_quantised_equal(a, b, w_scale, what=''):
    """Exact equality of integer states: compare round(x * w_scale) as int64 and
    require both to be integer valued."""
    a, b = to_np(a).astype(np.float64) * w_scale, to_np(b).astype(np.float64) * w_scale
    assert np.array_equal(a, np.round(a)), f'{what}: left side is not quantised'
    assert np.array_equal(b, np.round(b)), f'{what}: right side is not quantised'
    assert_exact(a.astype(np.int64), b.astype(np.int64), what)


# Reported, not asserted: how many elements of each sum-type comparison would also pass the plain
# element-wise criterion |a - b| <= 1e-5 * |b|.  what -> [elements, elements inside, smallest
# per-call fraction]; conftest prints the table at the end of a run.
LITERAL = {}


def record_literal(a, b, what, rtol=RTOL):
    inside = int(np.count_nonzero(np.abs(a - b) <= rtol * np.abs(b)))
    rec = LITERAL.setdefault(what, [0, 0, 1.0])
    rec[0] += a.size
    rec[1] += inside
    rec[2] = min(rec[2], inside / a.size)
    return inside / a.size


def assert_close(a, b, what='', rtol=RTOL, floor=FLOOR, scale=None):
    a, b = to_np(a).astype(np.float64), to_np(b).astype(np.float64)
    assert a.shape == b.shape, f'{what}: shape {a.shape} vs {b.shape}'
    if b.size == 0:
        return
    assert np.all(np.isfinite(a)), f'{what}: non-finite values'
    if scale is not None:
        record_literal(a, b, what, rtol)
    if scale is None:
        scale = np.maximum(np.abs(b), floor * np.max(np.abs(b)))
    else:
        scale = np.maximum(np.abs(b), np.broadcast_to(np.asarray(scale, dtype=np.float64), b.shape))
    err = np.abs(a - b)
    ok = err <= rtol * scale
    if not ok.all():
        i = tuple(np.argwhere(~ok)[0])
        raise AssertionError(
            f'{what}: {np.count_nonzero(~ok)} of {a.size} elements outside {rtol:g} relative; '
            f'first at {i}: {a[i]!r} vs {b[i]!r}; worst ratio {np.max(err / scale):.3g}')


# --------------------------------------------------------------------------
# magnitude scans: the recurrences of the backward passes run on |terms|
# --------------------------------------------------------------------------
def chan(p, ndim):
    """Parameter vector (1 or C entries) shaped to broadcast over [B, C, ..., T]."""
    p = np.asarray(to_np(p), dtype=np.float64).reshape(-1)
    if p.size == 1 or ndim < 3:
        return p.reshape(-1)[0]
    return p.reshape((1, -1) + (1,) * (ndim - 2))


def li_scale(go, decay):
    """S[t] = a * S[t+1] + |go[t]| with a = |1 - decay / 4096| (leaky-integrator backward)."""
    go = np.abs(to_np(go).astype(np.float64))
    a = np.abs(1.0 - chan(decay, go.ndim) / 4096.0)
    a = np.broadcast_to(a, go.shape[:-1] + (1,))[..., 0] if np.ndim(a) else a
    S = np.empty_like(go)
    acc = np.zeros(go.shape[:-1])
    for t in range(go.shape[-1] - 1, -1, -1):
        acc = a * acc + go[..., t]
        S[..., t] = acc
    return S


def res_scale(g_re, g_im, sin_decay, cos_decay):
    """Magnitude version of the reverse rotation scan (resonator backward)."""
    g_re = np.abs(to_np(g_re).astype(np.float64))
    g_im = np.abs(to_np(g_im).astype(np.float64))
    s = np.abs(chan(sin_decay, g_re.ndim)) / 4096.0
    c = np.abs(chan(cos_decay, g_re.ndim)) / 4096.0
    if np.ndim(s):
        s = np.broadcast_to(s, g_re.shape[:-1] + (1,))[..., 0]
        c = np.broadcast_to(c, g_re.shape[:-1] + (1,))[..., 0]
    S_re, S_im = np.empty_like(g_re), np.empty_like(g_im)
    a = np.zeros(g_re.shape[:-1])
    b = np.zeros(g_re.shape[:-1])
    for t in range(g_re.shape[-1] - 1, -1, -1):
        a, b = c * a + s * b + g_re[..., t], s * a + c * b + g_im[..., t]
        S_re[..., t], S_im[..., t] = a, b
    return S_re, S_im


def pgrad_scale(n, *product_pairs):
    """Sum of |g[t+1] * y[t]| over everything but the channel axis, for each
    (g, y) pair, added up; n = number of parameter entries."""
    total = None
    for g, y in product_pairs:
        g, y = to_np(g).astype(np.float64), to_np(y).astype(np.float64)
        prod = np.abs(g[..., 1:] * y[..., :-1])
        if n <= 1 or prod.ndim < 3:
            v = np.array([prod.sum()])
        else:
            v = prod.sum(axis=tuple(i for i in range(prod.ndim) if i != 1))
        total = v if total is None else total + v
    return total


def cspike_term_scale(re, im, threshold, grad_spike, tau_rho, scale_rho, graded):
    """Magnitudes of the two gradients of the complex spike (spike/complex.py:144-167)
    with its internal cancellation removed: the factor step_real = (1 + sign * (1 - e)) / 2
    loses all relative accuracy where e = 2 tau delta_real is small, so it is bounded by 1."""
    re, im, gs = (to_np(x).astype(np.float64) for x in (re, im, grad_spike))
    thr = to_np(threshold).astype(np.float64) if hasattr(threshold, 'shape') else float(threshold)
    if graded:
        delta_real = np.exp(-np.maximum(thr - re, 0) / tau_rho)
    else:
        delta_real = 0.5 / tau_rho * np.exp(-np.abs(re - thr) / tau_rho)
    delta_imag = 0.5 / tau_rho * np.exp(-np.abs(im) / tau_rho)
    return np.abs(gs) * scale_rho * delta_real * delta_imag, np.abs(gs) * scale_rho / tau_rho * delta_imag
