"""ctypes binding of the C ABI declared in include/cllo_flash_gqa.h.

There is no fallback: if the compiled library is missing, importing a kernel entry point raises.
"""
import ctypes
import os

from .build import LIB_PATH

OK = 0
E_BAD_ARG = -1
E_UNSUPPORTED = -2
E_WORKSPACE = -3
E_CUDA = -4
E_DEVICE_TIMEOUT = -6
KV_BSHD = 0
KV_BHSD = 1
WS_COUNTERS_ZERO = 0x100

_lib = None

_vp, _i, _f, _sz, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_longlong

_SIGNATURES = {
    "cllo_version": (_i, []),
    "cllo_status_string": (ctypes.c_char_p, [_i]),
    "cllo_last_cuda_error": (_i, []),
    "cllo_device_status": (_i, [ctypes.POINTER(_i)]),
    "cllo_shutdown": (_i, []),
    "cllo_gqa_decode_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "cllo_gqa_decode_plan": (_i, [_i, _i, _i, _i, _i, _i, _i, ctypes.POINTER(_i)]),
    "cllo_gqa_decode_bf16": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "cllo_gqa_decode_rope_append_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _f, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i,
                                              _i, _i, _vp]),
    "cllo_gqa_combine_bf16": (_i, [_vp, _i, _vp, _ll, _i, _vp]),
    "cllo_gqa_exchange_combine_bf16": (_i, [_vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _i, ctypes.c_uint, _vp,
                                            _i, _i, _i, _i, _vp]),
    "cllo_gqa_decode_sharded_bf16": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _i,
                                          ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _i, ctypes.c_uint, _vp]),
    "cllo_gqa_shard_gather_bytes": (_sz, [_i, _i, _i, _i]),
    "cllo_gqa_shard_flag_bytes": (_sz, [_i]),
    "cllo_set_exchange_wait_limit": (_i, [_ll]),
    "cllo_gqa_prefill_fwd_bf16": (_i, [_vp, _vp, _vp, _f, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_gqa_prefill_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "cllo_gqa_prefill_fwd_ws_bf16": (_i, [_vp, _vp, _vp, _f, _i, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_gqa_bwd_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "cllo_gqa_bwd_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_rope_bf16": (_i, [_vp, _vp, _i, _i, _i, _f, _vp]),
    "cllo_swa_bwd_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_swa_prefill_fwd_bf16": (_i, [_vp, _vp, _vp, _f, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_mla_prefill_fwd_bf16": (_i, [_vp, _vp, _vp, _f, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_sgqa_prefill_fwd_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _f, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_gqa_decode_bf16_noalloc": (_i, [_vp, _vp, _vp, _f, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "cllo_gqa_decode_bf16_compat": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _i, _i]),
}


def load():
    """Load libcllo_flash_gqa.so (once) and attach argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "%s is missing: build it with `python -m cuda_llm_ops_b200.build` "
            "(there is no CPU or PyTorch fallback)" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def declared_symbols():
    return sorted(_SIGNATURES)


def check(status, what):
    if status == OK:
        return
    lib = load()
    msg = lib.cllo_status_string(status).decode()
    if status == E_CUDA:
        msg += " (cudaError %d)" % lib.cllo_last_cuda_error()
    raise RuntimeError("%s failed: %s [%d]" % (what, msg, status))
