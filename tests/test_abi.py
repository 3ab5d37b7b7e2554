"""The C-ABI library loads on a machine without a GPU and exports every function include/kdw.h declares;
argument validation happens before any CUDA call."""
import os
import re

from kerops_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, 'include', 'kdw.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(kdw_[a-z0-9_]+)\s*\(', text)))


def test_every_declared_symbol_is_exported_and_bound(kdw_lib):
    names = _declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(kdw_lib, name), f'{name} is declared in kdw.h but not exported'
    assert sorted(_lib.SIGNATURES) == names, 'ctypes prototypes and kdw.h disagree'


def test_version_and_variant_tables(kdw_lib):
    assert kdw_lib.kdw_version() >= 100
    nf, nw = kdw_lib.kdw_fprop_variants(), kdw_lib.kdw_wgrad_variants()
    assert nf >= 1 and nw >= 1
    for v in range(1, nf + 1):
        assert kdw_lib.kdw_fprop_variant_channels(v) in (8, 16, 32, 64, 128)
    for v in range(1, nw + 1):
        assert kdw_lib.kdw_wgrad_variant_channels(v) in (8, 16, 32, 64, 128)
    assert kdw_lib.kdw_fprop_variant_channels(0) < 0
    assert kdw_lib.kdw_wgrad_variant_channels(nw + 1) < 0


def test_argument_errors_without_gpu(kdw_lib):
    # null pointers
    rc = kdw_lib.kdw_fprop_f16(None, None, None, 1, 8, 4, 4, 4, 512, 128, 32, 512, 128, 32, 0, 0, None)
    assert rc == -1 and b'null' in kdw_lib.kdw_last_error()
    # C not a power of two
    rc = kdw_lib.kdw_fprop_f16(16, 16, 16, 1, 24, 4, 4, 4, 1536, 384, 96, 1536, 384, 96, 0, 0, None)
    assert rc == -1
    # bad accumulate type
    rc = kdw_lib.kdw_fprop_f16(16, 16, 16, 1, 8, 4, 4, 4, 512, 128, 32, 512, 128, 32, 7, 0, None)
    assert rc == -1
    # plane range outside the tensor
    rc = kdw_lib.kdw_fprop_f16_range(16, 16, 16, 1, 8, 4, 4, 4, 512, 128, 32, 4, 512, 128, 32, 2, 6, 0, 0, 0, None)
    assert rc == -5
    # unknown variant
    rc = kdw_lib.kdw_fprop_f16(16, 16, 16, 1, 8, 4, 4, 4, 512, 128, 32, 512, 128, 32, 0, 999, None)
    assert rc == -4
    # wgrad: missing outputs
    rc = kdw_lib.kdw_wgrad_f16(16, 16, 16, 1 << 20, None, None, 1, 8, 4, 4, 4, 512, 128, 32, 512, 128, 32, 0, None)
    assert rc == -1
    assert kdw_lib.kdw_wgrad_workspace_bytes(1, 0, 4, 4, 4) < 0


def test_auto_variant_follows_the_shape(kdw_lib):
    """tune = 0: the benchmark shape gets the tiles measured fastest there (tensor-core kernels, numbered after the
    12 / 24 CUDA-core table variants); a depth that a deep tile would pad heavily gets a shallower tile; every
    choice is a variant whose channel slice divides C."""
    lib = kdw_lib
    assert [lib.kdw_fprop_auto_variant(C, 350, 128) for C in (8, 16, 32, 64, 128)] == [19, 20, 17, 13, 13]
    assert [lib.kdw_wgrad_auto_variant(C, 350, 128) for C in (8, 16, 32, 64, 128)] == [31, 32, 26, 25, 25]
    assert lib.kdw_fprop_auto_variant(32, 350, 40) != 17   # 32-deep tiles would compute 64 of 40 planes
    assert lib.kdw_wgrad_auto_variant(8, 48, 24) != 31     # 64-deep tiles would compute 64 of 24 planes
    assert lib.kdw_fprop_auto_variant(16, 350, 127) not in (20, 21)  # the paired-voxel tensor map needs an even D
    assert lib.kdw_wgrad_auto_variant(16, 350, 127) not in (32, 33)
    for C in (8, 16, 32, 64, 128, 256):
        for W, D in ((350, 128), (16, 8), (40, 40), (97, 61), (1, 1)):
            f, w = lib.kdw_fprop_auto_variant(C, W, D), lib.kdw_wgrad_auto_variant(C, W, D)
            assert 1 <= f <= lib.kdw_fprop_variants() and C % lib.kdw_fprop_variant_channels(f) == 0
            assert 1 <= w <= lib.kdw_wgrad_variants() and C % lib.kdw_wgrad_variant_channels(w) == 0
    assert lib.kdw_fprop_auto_variant(4, 16, 16) == 0 and lib.kdw_wgrad_auto_variant(24, 16, 16) == 0
