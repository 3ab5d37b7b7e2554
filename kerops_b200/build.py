"""Builds the C-ABI CUDA library in-tree: kerops_b200/csrc/libkdw.so (sm_100a only).

    python -m kerops_b200.build [--force] [--verbose]

Each .cu is compiled to an object with nvcc (in parallel) and linked with `nvcc -shared`.
The library links the CUDA runtime statically and needs only the driver at run time.
"""
import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'csrc')
INCLUDE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'include')
LIB = os.path.join(CSRC, 'libkdw.so')
SOURCES = ['kdw_host.cu', 'dwconv_fprop.cu', 'dwconv_fprop_mma.cu', 'dwconv_wgrad.cu', 'dwconv_wgrad_mma.cu', 'grad_allreduce.cu', 'dwconv_fprop_addstats.cu', 'dwconv_fprop_bnrelu.cu']
HEADERS = [os.path.join(CSRC, h) for h in (
    'kdw_common.cuh', 'mma_patch.cuh', 'fprop_core.cuh', 'wgrad_core.cuh', 'fprop_variants.inc', 'wgrad_variants.inc')] + [os.path.join(INCLUDE, 'kdw.h')]
NVCC_FLAGS = [
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-std=c++17', '-O3', '-lineinfo',
    '-Xcompiler', '-fPIC',
]


def find_nvcc():
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(nvcc):
        raise RuntimeError('nvcc not found: the CUDA library cannot be built on this machine')
    return nvcc


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def up_to_date():
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return _newer(LIB, deps)


def build(force=False, verbose=False):
    """Compile and link libkdw.so; returns its path."""
    if not force and up_to_date():
        return LIB
    nvcc = find_nvcc()
    extra = ['-Xptxas', '-v'] if verbose else []

    def compile_one(src):
        obj = os.path.join(CSRC, os.path.splitext(src)[0] + '.o')
        deps = [os.path.join(CSRC, src)] + HEADERS
        if not force and _newer(obj, deps):
            return obj, ''
        cmd = [nvcc] + NVCC_FLAGS + extra + ['-c', os.path.join(CSRC, src), '-o', obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f'nvcc failed on {src}:\n{r.stdout}\n{r.stderr}')
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        results = list(ex.map(compile_one, SOURCES))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [o for o, _ in results]
    tmp = LIB + '.tmp'
    cmd = [nvcc, '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', tmp] + objs
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f'link failed:\n{r.stdout}\n{r.stderr}')
    os.replace(tmp, LIB)
    return LIB


PROBES = {'issue_rate': [], 'tma_rows': ['-lcuda'], 'tcgen05_small_n': []}


def build_probes(force=False):
    """Compiles the stand-alone microbenchmarks of csrc/probes (not part of the library; run by hand on a GPU)."""
    nvcc = find_nvcc()
    pdir = os.path.join(CSRC, 'probes')

    def one(item):
        name, libs = item
        src, exe = os.path.join(pdir, name + '.cu'), os.path.join(pdir, name)
        if not force and _newer(exe, [src]):
            return exe
        r = subprocess.run([nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-o', exe, src] + libs,
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f'nvcc failed on probes/{name}.cu:\n{r.stdout}\n{r.stderr}')
        return exe

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(PROBES)) as ex:
        return list(ex.map(one, PROBES.items()))


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--force', action='store_true')
    ap.add_argument('--verbose', action='store_true')
    ap.add_argument('--probes', action='store_true', help='also build the microbenchmarks of csrc/probes')
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    if a.probes:
        print('\n'.join(build_probes(force=a.force)))
