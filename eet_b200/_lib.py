"""ctypes binding of libeet_b200.so - the only route from Python to the CUDA kernels.

There is no fallback: if the library is missing, cannot be loaded or does not export a symbol that
include/eet_b200.h declares, importing this module raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libeet_b200.so")

_c = ctypes
_vp, _i, _sz, _f = _c.c_void_p, _c.c_int, _c.c_size_t, _c.c_float

# name -> (restype, argtypes); must list every function of include/eet_b200.h
SIGNATURES = {
    "eet_abi_version": (_i, []),
    "eet_last_error": (_c.c_char_p, []),
    "eet_device_status": (_i, [_c.POINTER(_i)]),
    "eet_set_wait_limit": (_i, [_c.c_uint]),
    "eet_quantize_w8_workspace_bytes": (_sz, [_i, _i]),
    "eet_quantize_w8": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "eet_pack_w8": (_i, [_vp, _i, _i, _vp, _vp]),
    "eet_unpack_w8": (_i, [_vp, _i, _i, _vp, _vp]),
    "eet_repack_ref_w8": (_i, [_vp, _i, _i, _vp, _vp]),
    "eet_gemm_w8a16_workspace_bytes": (_sz, [_i, _i, _i]),
    "eet_gemm_w8a16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp, _sz, _vp]),
    "eet_gemm_w8a16_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp]),
    "eet_gemm_w8a16_accum": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "eet_gemm_w8a16_finalize": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "eet_rmsnorm_finalize": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "eet_rmsnorm_finalize_tp": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "eet_swiglu_finalize": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "eet_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "eet_swiglu": (_i, [_vp, _vp, _i, _i, _vp]),
    "eet_add_residual": (_i, [_vp, _vp, _sz, _vp]),
    "eet_qkv_split_store": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "eet_prefill_mha": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp]),
    "eet_decode_mha": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _i, _f, _i, _vp]),
    "eet_reorder_kv_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "eet_reorder_kv": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "eet_advance_steps": (_i, [_vp, _i, _i, _vp]),
    "eet_argmax_rows": (_i, [_vp, _vp, _i, _i, _sz, _vp]),
    "eet_lm_head_argmax": (_i, [_vp, _vp, _i, _i, _c.c_int64, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "eet_gather_rows": (_i, [_vp, _vp, _vp, _i, _i, _c.c_int64, _vp]),
}


class EETError(RuntimeError):
    """Raised when an entry point of libeet_b200.so reports a failure (the reference raises
    RuntimeError from check_cuda_error / TORCH_CHECK in the same situations)."""


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m eet_b200.build` (needs nvcc). "
            "There is no CPU or PyTorch fallback for this library.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != 0:
        raise EETError(lib.eet_last_error().decode())


def device_status() -> int:
    out = _i(0)
    check(lib.eet_device_status(ctypes.byref(out)))
    return out.value
