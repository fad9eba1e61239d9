"""Builds the sblocal_b200 shared library in-tree with nvcc for sm_100a.

    python -m fly_b200.build [--force] [--verbose]

The result, fly_b200/lib/libsblocal_b200.so, exports the C ABI declared in
include/sblocal_b200.h and links the CUDA runtime statically, so it loads
through ctypes without torch.  nvcc cross-compiles: no GPU is needed to build.
"""
import argparse
import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, 'csrc')
LIB_DIR = os.path.join(PKG, 'lib')
LIB_PATH = os.path.join(LIB_DIR, 'libsblocal_b200.so')
STAMP = os.path.join(LIB_DIR, 'libsblocal_b200.stamp')
SOURCES = ['sbl_api.cu', 'sbl_f32.cu', 'sbl_tc.cu', 'sbl_tc128.cu', 'sbl_tmap.cu', 'sbl_noalloc.cu']
NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-lineinfo', '-std=c++17',
              '-Xcompiler', '-fPIC']


def _nvcc():
    cand = os.environ.get('NVCC') or shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(cand):
        raise RuntimeError('nvcc not found: set NVCC or put /usr/local/cuda/bin on PATH')
    return cand


def _fingerprint():
    h = hashlib.sha256()
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))]
    files.append(os.path.join(ROOT, 'include', 'sblocal_b200.h'))
    for f in files:
        h.update(f.encode())
        with open(f, 'rb') as fh:
            h.update(fh.read())
    h.update(' '.join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current():
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as fh:
        return fh.read().strip() == _fingerprint()


def build(force=False, verbose=False):
    """Compiles every .cu under fly_b200/csrc into one shared library."""
    if not force and is_current():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIB_DIR, src.replace('.cu', '.o'))
        cmd = [_nvcc(), *NVCC_FLAGS, '-I', os.path.join(ROOT, 'include'), '-I', CSRC, '-c',
               os.path.join(CSRC, src), '-o', obj]
        if verbose:
            cmd.insert(1, '-Xptxas=-v')
            print(' '.join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            print(out)
        if pr.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}')
    # no -lcuda: the one driver entry point the library needs is looked up at run time (sbl_tmap.cu)
    link = [_nvcc(), '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', LIB_PATH, *objs,
            '-cudart', 'static']
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        print(res.stdout)
        raise RuntimeError('link failed')
    with open(STAMP, 'w') as fh:
        fh.write(_fingerprint())
    return LIB_PATH


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
