import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, 'lava-dl_b200'), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200); run with -m gpu')


@pytest.fixture(scope='session')
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip('no CUDA device')
    return torch.device('cuda:0')


def pytest_terminal_summary(terminalreporter):
    """Gradient comparisons are held to 1e-5 of the sum of term magnitudes (see _util.py); this table
    says how many of the compared elements also meet the plain |a - b| <= 1e-5 * |b|."""
    import _util
    if not _util.LITERAL:
        return
    tr = terminalreporter
    tr.write_line('')
    tr.write_line('elements inside the element-wise 1e-5 relative criterion (reported, not asserted):')
    for what, (n, inside, worst) in sorted(_util.LITERAL.items()):
        tr.write_line(f'  {what:45s} {inside / n:9.6f} of {n:>12d} elements; worst single comparison {worst:.6f}')
