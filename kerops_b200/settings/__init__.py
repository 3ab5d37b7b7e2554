"""Keyword-default injection for operators (call-compatible with kerops.settings).

Mirrors the public names of kerops/settings/__init__.py:1-3 (including the reference's spelling
of ``CongiguratorError``) so user code written against kerops imports unchanged.
"""
from .hardware_conf import get_l1_cache, set_l1_cache
from .configure import ConfigurableArg, ConfiguredFunction, CongiguratorError, confexc, configure

__all__ = [
    'ConfigurableArg',
    'ConfiguredFunction',
    'CongiguratorError',
    'confexc',
    'configure',
    'get_l1_cache',
    'set_l1_cache',
]
