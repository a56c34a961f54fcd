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
SOURCES = ['dcn_api.cu', 'dcn_simt.cu', 'dcn_tc.cu', 'dcn_tc2.cu', 'dcn_conv.cu', 'dcn_static.cu', 'dcn_bwd.cu', 'dcn_msda.cu']
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
EXTRA_FLAGS = os.environ.get('DCN_B200_NVCC_FLAGS', '').split()   # e.g. -DDCN_TC2_ABLATE for experiments


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


def _compile(src, obj, verbose):
    """One translation unit -> object file (skipped when the object is newer than every
    source and header)."""
    if os.path.exists(obj) and all(os.path.getmtime(d) <= os.path.getmtime(obj) for d in _deps()):
        return ''
    cmd = [NVCC, '-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3',
           '-std=c++17', '-Xcompiler', '-fPIC', '-I', os.path.join(ROOT, 'include'), '-I', CSRC]
    cmd += EXTRA_FLAGS
    if verbose:
        cmd += ['-Xptxas', '-v']
    cmd += ['-c', src, '-o', obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f'nvcc failed on {src}:\n{r.stdout}{r.stderr}')
    return r.stdout + r.stderr


def build(force=False, verbose=False):
    if not force and up_to_date():
        return LIB
    from concurrent.futures import ThreadPoolExecutor
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, 'obj')
    os.makedirs(obj_dir, exist_ok=True)
    objs = [os.path.join(obj_dir, s[:-3] + '.o') for s in SOURCES]
    if force:
        for o in objs:
            if os.path.exists(o):
                os.remove(o)
    # the translation units are independent: compile them side by side, then link
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        logs = list(pool.map(lambda so: _compile(os.path.join(CSRC, so[0]), so[1], verbose),
                             zip(SOURCES, objs)))
    if verbose:
        sys.stderr.write(''.join(logs))
    cmd = [NVCC, '-gencode', 'arch=compute_100a,code=sm_100a', '-shared', '-Xcompiler', '-fPIC',
           '-cudart', 'static'] + objs + ['-o', LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError('nvcc failed linking libdcn_b200.so')
    return LIB


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(a.force, a.verbose))
