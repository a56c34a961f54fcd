"""Compile the CUDA sources into ``mmcv_b200/lib/libdcn_b200.so`` (sm_100a only).

``python -m mmcv_b200.build_ext [--force] [--verbose]``.  nvcc cross-compiles
without a GPU; the resulting library is loaded through ctypes by ``_lib.py``.
"""
import argparse
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, 'csrc')
LIB_DIR = os.path.join(PKG, 'lib')
LIB = os.path.join(LIB_DIR, 'libdcn_b200.so')
SOURCES = ['dcn_api.cu', 'dcn_simt.cu', 'dcn_tc.cu', 'dcn_static.cu', 'dcn_bwd.cu']
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')


def _deps():
    out = [os.path.join(ROOT, 'include', 'dcn_b200.h')]
    for f in sorted(os.listdir(CSRC)):
        if f.endswith(('.cu', '.cuh', '.h')):
            out.append(os.path.join(CSRC, f))
    return out


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(d) <= t for d in _deps())


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [NVCC, '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3',
           '-std=c++17', '-shared', '-Xcompiler', '-fPIC', '-cudart', 'static',
           '-I', os.path.join(ROOT, 'include'), '-I', CSRC]
    if verbose:
        cmd += ['-Xptxas', '-v']
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ['-o', LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError('nvcc failed building libdcn_b200.so')
    return LIB


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(a.force, a.verbose))
