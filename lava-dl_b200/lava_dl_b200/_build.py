"""In-tree build of the C-ABI library ``libslayer_b200.so`` for sm_100a.

The reference compiles its ``.cu`` files lazily with
``torch.utils.cpp_extension.load`` on first use
(``src/lava/lib/dl/slayer/neuron/dynamics/leaky_integrator.py:24-47``).  Here the
library is plain CUDA C++ without torch headers, built ahead of time with
``nvcc`` (cross-compiles without a GPU) and loaded with ``ctypes``.

Run as a script to build: ``python -m lava_dl_b200._build [--force]``.
"""

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(os.path.dirname(PKG_DIR), 'csrc')
INCLUDE_DIR = os.path.join(os.path.dirname(os.path.dirname(PKG_DIR)), 'include')
LIB_DIR = os.path.join(PKG_DIR, '_lib')
OBJ_DIR = os.path.join(LIB_DIR, 'obj')
LIB_PATH = os.path.join(LIB_DIR, 'libslayer_b200.so')

NVCC_FLAGS = [
    '-std=c++17', '-O3',
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-lineinfo',
    '-Xcompiler', '-fPIC',
]


def _nvcc():
    exe = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(exe):
        raise RuntimeError('nvcc not found; cannot build libslayer_b200.so')
    return exe


def sources():
    return sorted(
        os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith('.cu')
    )


def _deps():
    deps = [os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR)]
    deps.append(os.path.join(INCLUDE_DIR, 'slayer_b200.h'))
    deps.append(os.path.abspath(__file__))
    return deps


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > built for d in _deps())


def build(force=False, verbose=False, ptxas_verbose=False, defines=(), out=None):
    """Compile every ``.cu`` under ``csrc/`` and link the shared library.

    ``defines`` adds ``-D`` macros (pipeline-shape experiments), ``out`` writes
    the library somewhere else than the in-tree default.  Returns the path of
    the library.  Raises ``RuntimeError`` with the compiler output on failure.
    """
    lib_path = out or LIB_PATH
    obj_dir = OBJ_DIR if out is None else os.path.join(os.path.dirname(out), 'obj_' + os.path.basename(out))
    if out is None and not force and not is_stale():
        return LIB_PATH
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    flags = list(NVCC_FLAGS) + [f'-D{d}' for d in defines]
    if ptxas_verbose:
        flags += ['-Xptxas', '-v']

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + '.o')
        cmd = [nvcc] + flags + ['-I', INCLUDE_DIR, '-c', src, '-o', obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    objs = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for src, obj, r in ex.map(compile_one, sources()):
            if verbose or ptxas_verbose:
                sys.stderr.write(r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f'nvcc failed on {src}:\n{r.stdout}\n{r.stderr}')
            objs.append(obj)
    cmd = [nvcc, '-shared', '-o', lib_path] + objs + ['-cudart', 'static']
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f'link failed:\n{r.stdout}\n{r.stderr}')
    return lib_path


if __name__ == '__main__':
    print(build(force='--force' in sys.argv, verbose='-v' in sys.argv,
                ptxas_verbose='--ptxas' in sys.argv))
