"""Build recipe for the CPU checkers (test infrastructure, not product code).

Two artefacts, both git-ignored and both carried to a GPU machine as files:

* ``oracle/libdcn_oracle.so`` -- the plain-C restatement in ``dcn_oracle.c``
  (gcc, OpenMP).
* ``oracle/_ref/pywrap/`` -- the reference's three unchanged Python files of this path
  (the two operator wrappers and the extension loader they import), copied so that the GPU
  tests can run the reference's own wrappers on top of this library's extension module on a
  machine without the reference checkout.  git-ignored like the rest of ``oracle/_ref/``.
* ``oracle/_ref/dcn_ref_ext.so`` -- the UNMODIFIED reference CPU implementation,
  compiled from the reference checkout where it lies (four translation units of
  mmcv/ops/csrc/pytorch plus the two helper headers in mmcv/ops/csrc/common),
  behind the pybind front door in ``ref_binding.cpp``.  Built only when a
  reference checkout is present; no reference source is copied anywhere.

Run as ``python oracle/build_oracle.py [--ref-root DIR]``.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, 'libdcn_oracle.so')
REF_DIR = os.path.join(HERE, '_ref')
REF_NAME = 'dcn_ref_ext'
REF_SO = os.path.join(REF_DIR, REF_NAME + '.so')
# where the reference checkout lies: from the environment (no default location is assumed)
DEFAULT_REF_ROOT = os.environ.get('DCN_REFERENCE_ROOT', '')
WRAP_DIR = os.path.join(REF_DIR, 'pywrap')
# the reference's Python wrappers of this path (+ the loader they import), relative to its root
REF_WRAPPERS = ['mmcv/utils/ext_loader.py', 'mmcv/ops/modulated_deform_conv.py', 'mmcv/ops/deform_conv.py',
                'mmcv/ops/multi_scale_deform_attn.py']

# The reference's translation units for this path, relative to its root.
REF_UNITS = [
    ('loop_v2', 'mmcv/ops/csrc/pytorch/modulated_deform_conv.cpp'),
    ('cpu_v2', 'mmcv/ops/csrc/pytorch/cpu/modulated_deform_conv.cpp'),
    ('loop_v1', 'mmcv/ops/csrc/pytorch/deform_conv.cpp'),
    ('cpu_v1', 'mmcv/ops/csrc/pytorch/cpu/deform_conv.cpp'),
]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_port(force=False):
    src = os.path.join(HERE, 'dcn_oracle.c')
    if not force and _newer(PORT_SO, [src]):
        return PORT_SO
    cmd = ['gcc', '-O3', '-march=x86-64-v3', '-fopenmp', '-fPIC', '-shared',
           '-fno-fast-math', '-o', PORT_SO, src, '-lm']
    subprocess.check_call(cmd)
    return PORT_SO


def copy_wrappers(ref_root=DEFAULT_REF_ROOT):
    """Copies the reference's wrapper files into oracle/_ref/pywrap (same relative paths)."""
    import shutil
    if not ref_root or not os.path.isdir(ref_root):
        return WRAP_DIR if os.path.isdir(WRAP_DIR) else None
    for rel in REF_WRAPPERS:
        dst = os.path.join(WRAP_DIR, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(ref_root, rel), dst)
    return WRAP_DIR


def build_ref(ref_root=DEFAULT_REF_ROOT, force=False):
    """Compile the reference CPU path; returns the .so path or None."""
    if not ref_root or not os.path.isdir(ref_root):
        return REF_SO if os.path.exists(REF_SO) else None
    copy_wrappers(ref_root)
    binding = os.path.join(HERE, 'ref_binding.cpp')
    ref_sources = [os.path.join(ref_root, rel) for _, rel in REF_UNITS]
    if not force and _newer(REF_SO, [binding] + ref_sources):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    # Two pairs of reference files share a basename, and ninja wants distinct
    # object names: one-line units that include each file from where it lies.
    units = []
    for tag, rel in REF_UNITS:
        unit = os.path.join(REF_DIR, f'unit_{tag}.cpp')
        with open(unit, 'w') as f:
            f.write(f'#include "{os.path.join(ref_root, rel)}"\n')
        units.append(unit)
    from torch.utils.cpp_extension import load
    load(name=REF_NAME, sources=[binding] + units,
         extra_include_paths=[os.path.join(ref_root, 'mmcv/ops/csrc/common')],
         extra_cflags=['-O2'], build_directory=REF_DIR, verbose=False)
    return REF_SO if os.path.exists(REF_SO) else None


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--ref-root', default=DEFAULT_REF_ROOT)
    ap.add_argument('--force', action='store_true')
    a = ap.parse_args()
    print('port:', build_port(a.force))
    print('ref :', build_ref(a.ref_root, a.force))
    sys.exit(0)
