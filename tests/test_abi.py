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
