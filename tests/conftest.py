import ctypes
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')


def _cuda_available():
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _cuda_available():
        return
    skip = pytest.mark.skip(reason='no CUDA device')
    for item in items:
        if 'gpu' in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope='session')
def kdw_lib():
    """The C-ABI library, built first when a compiler is present and the build is stale."""
    from kerops_b200 import _lib, build

    try:
        build.build()
    except RuntimeError:
        if not os.path.exists(_lib.LIB_PATH):
            raise
    return _lib.load()


@pytest.fixture(scope='session')
def kdw_emu(kdw_lib):
    """CPU emulation of the TMA kernels (tests/emu/kdw_emu.cu), compiled with nvcc on first use."""
    from kerops_b200 import build

    emu_dir = os.path.join(ROOT, 'tests', 'emu')
    so = os.path.join(emu_dir, 'libkdw_emu.so')
    src = os.path.join(emu_dir, 'kdw_emu.cu')
    deps = [src] + build.HEADERS
    if not os.path.exists(so) or any(os.path.getmtime(d) > os.path.getmtime(so) for d in deps):
        nvcc = build.find_nvcc()
        cmd = [nvcc, '-std=c++17', '-O2', '-Xcompiler', '-fPIC,-fno-strict-aliasing', '-shared', '-gencode',
               'arch=compute_100a,code=sm_100a', '-o', so, src, os.path.join(build.CSRC, 'kdw_host.o')]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError('building the kernel emulation failed:\n' + r.stderr)
    emu = ctypes.CDLL(so)
    i64, ci, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    emu.emu_fprop.argtypes = [ci, vp, vp, vp] + [i64] * 6 + [ci] * 5
    emu.emu_fprop.restype = ci
    emu.emu_wgrad.argtypes = [ci, vp, vp, vp] + [i64] * 6 + [ci] * 4
    emu.emu_wgrad.restype = ci
    emu.emu_schedule.argtypes = [i64] * 4 + [ci] * 6 + [vp, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    emu.emu_schedule.restype = ci
    emu.emu_fprop_addstats.argtypes = [ci, vp, vp, vp, vp, vp] + [i64] * 5 + [ci]
    emu.emu_fprop_addstats.restype = ci
    emu.emu_fprop_bnrelu.argtypes = [ci, vp, vp, vp, vp, vp] + [i64] * 5 + [ci]
    emu.emu_fprop_bnrelu.restype = ci
    return emu
