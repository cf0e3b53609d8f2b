"""ctypes face of the native host runtime (library "host", csrc/host_runtime.cpp): page pools,
the tables of what every live request holds, and the writer of a decode step's metadata."""
from __future__ import annotations

from ctypes import POINTER, c_int, c_longlong, c_void_p

from ..kernels import build

_P, _I, _LL = c_void_p, c_int, c_longlong
_SIGS = {
    "rllm_pool_new": (_P, [_I]), "rllm_pool_delete": (None, [_P]), "rllm_pool_alloc": (_I, [_P, _LL]),
    "rllm_pool_release": (_I, [_P, _I, _LL]), "rllm_pool_holder": (_LL, [_P, _I]), "rllm_pool_nobody": (_LL, []),
    "rllm_pool_num_free": (_I, [_P]), "rllm_pool_num_pages": (_I, [_P]), "rllm_pool_check": (_I, [_P]),
    "rllm_cache_new": (_P, [_I, POINTER(_I), POINTER(_I), _I, _I]), "rllm_cache_delete": (None, [_P]),
    "rllm_cache_pool": (_P, [_P, _I]), "rllm_cache_slots": (_P, [_P]), "rllm_cache_open": (_I, [_P, _LL]),
    "rllm_cache_reserve": (_I, [_P, _I, _I]), "rllm_cache_can_reserve": (_I, [_P, _I, _I]),
    "rllm_cache_commit": (_I, [_P, _I, _I]), "rllm_cache_trim": (_I, [_P, _I]), "rllm_cache_close": (_I, [_P, _I]),
    "rllm_cache_num_tokens": (_I, [_P, _I]), "rllm_cache_serial": (_LL, [_P, _I]), "rllm_cache_epoch": (_I, [_P, _I]),
    "rllm_cache_num_held": (_I, [_P, _I, _I]), "rllm_cache_pages": (_I, [_P, _I, _I, _P, _I]),
    "rllm_cache_check": (_I, [_P]), "rllm_rows_new": (_P, [_I, _I]), "rllm_rows_delete": (None, [_P]),
    "rllm_rows_forget": (None, [_P, _I]),
    "rllm_fill_decode": (_I, [_P, _P, _I, _P, _P, _I, _P, _P]),
}


class _Lib:
    """The loaded library with typed functions as attributes (built at first use)."""

    def __init__(self):
        cdll = build.load_library("host")
        for name, (res, args) in _SIGS.items():
            f = getattr(cdll, name)
            f.restype, f.argtypes = res, args
            setattr(self, name[len("rllm_"):], f)
        self.NOBODY = self.pool_nobody()


_lib = None


def lib() -> _Lib:
    global _lib
    if _lib is None:
        _lib = _Lib()
    return _lib
