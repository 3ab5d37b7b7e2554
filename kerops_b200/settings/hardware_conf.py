"""Block-size budget constant kept for API compatibility (kerops/settings/hardware_conf.py:1-11).

The depthwise-conv path never used it in the reference either; the CUDA kernels here pick their
tiles from tables compiled into the extension.
"""
_state = {'l1_cache_bytes': 65536}


def get_l1_cache():
    return _state['l1_cache_bytes']


def set_l1_cache(new_cache):
    _state['l1_cache_bytes'] = int(new_cache)
