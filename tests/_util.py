"""Comparison helpers shared by the parity tests.

Tolerances (stated once, used everywhere):

* spikes and quantised states: BIT-EXACT.  A state series ``s`` is quantised
  when ``s * w_scale`` is an integer; both sides are compared as int64 after
  that scaling.
* float quantities (gradients, filter outputs): ``|a - b| <= 1e-5 * max(|b|,
  1e-2 * max|b|)``, i.e. 1e-5 relative element-wise with the comparison scale
  floored at 1 % of the tensor's largest magnitude.  The floor is needed
  because gradient scans are sums with cancellation: an element that cancels
  to ~0 carries the absolute rounding error of its O(max) terms.
* parameter gradients (sums over up to 10^9 products): 1e-5 relative to the
  larger of |b| and the sum of absolute values is not available from the
  reference, so they use ``|a - b| <= 1e-5 * max(|b|, 1e-2 * max|b|)`` too,
  per parameter vector.
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


def assert_close(a, b, what='', rtol=RTOL, floor=FLOOR):
    a, b = to_np(a).astype(np.float64), to_np(b).astype(np.float64)
    assert a.shape == b.shape, f'{what}: shape {a.shape} vs {b.shape}'
    if b.size == 0:
        return
    assert np.all(np.isfinite(a)), f'{what}: non-finite values'
    scale = np.maximum(np.abs(b), floor * np.max(np.abs(b)))
    err = np.abs(a - b)
    ok = err <= rtol * scale
    if not ok.all():
        i = tuple(np.argwhere(~ok)[0])
        raise AssertionError(
            f'{what}: {np.count_nonzero(~ok)} of {a.size} elements outside {rtol:g} relative; '
            f'first at {i}: {a[i]!r} vs {b[i]!r}; worst ratio {np.max(err / scale):.3g}')
