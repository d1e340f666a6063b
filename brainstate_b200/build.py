"""Builds ``libbsx.so`` (the C-ABI CUDA library) in-tree with nvcc, for sm_100a only.

Run ``python -m brainstate_b200.build`` or call :func:`build_library`.  The
compiler works without a GPU.  Objects go to ``build/bsx`` under the repository
root; the shared library is written next to this file so that it travels with
the package.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_PKG, 'csrc')
INCLUDE = os.path.join(_ROOT, 'include')
LIB_PATH = os.path.join(_PKG, 'libbsx.so')

ARCH_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a']
NVCC_FLAGS = ['-O3', '-std=c++17', '-lineinfo', '-Xcompiler', '-fPIC', '--use_fast_math=false',
              '-Xptxas', '-v']


def _nvcc() -> str:
    for cand in (os.environ.get('NVCC'), shutil.which('nvcc'), '/usr/local/cuda/bin/nvcc'):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError('nvcc not found: libbsx.so cannot be built')


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith('.cu'))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    obj_dir = os.path.join(_ROOT, 'build', 'bsx')
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(('.cuh', '.h'))]
    headers += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith('.h')]
    flags = [f for f in NVCC_FLAGS if f != '--use_fast_math=false']
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + '.o')
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *ARCH_FLAGS, *flags, '-I', INCLUDE, '-I', CSRC, '-c', src, '-o', obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError('nvcc failed for %s:\n%s\n%s' % (src, r.stdout, r.stderr))
        return src, r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, log in ex.map(compile_one, jobs):
                with open(os.path.join(obj_dir, os.path.basename(src) + '.ptxas.log'), 'w') as f:
                    f.write(log)
                if verbose:
                    sys.stderr.write(log)
    if jobs or force or _stale(LIB_PATH, objs):
        cmd = [nvcc, *ARCH_FLAGS, '-shared', '-Xcompiler', '-fPIC', '-cudart', 'static', '-o', LIB_PATH, *objs]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError('link failed:\n%s\n%s' % (r.stdout, r.stderr))
    return LIB_PATH


if __name__ == '__main__':
    print(build_library(force='--force' in sys.argv, verbose='-v' in sys.argv))
