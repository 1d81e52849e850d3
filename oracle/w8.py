"""TEST INFRASTRUCTURE - not part of the product.

numpy restatement of the reference's int8 weight-only quantizer and weight packers, plus loaders for
the two checking libraries built by ``oracle/Makefile``:

* ``liboracle_w8.so``           - the C restatement in ``oracle/w8_oracle.c``
* ``_ref/libeet_ref_quant.so``  - the reference's own ``cutlass_preprocessors.cc`` compiled for the host

Only ``tests/``, the smoke check and the CPU-baseline legs of ``bench.py`` may import this module.

Parity pin: the numpy and C restatements are compared bit for bit with ``_ref`` (where the reference
checkout is present) and with the golden vectors under ``tests/golden/`` that were generated from it.

Reference code restated here (paths inside the reference project):
  3rdparty/cutlass_kernels/cutlass_preprocessors.cc:581-678  symmetric_quantize
  3rdparty/cutlass_kernels/cutlass_preprocessors.cc:497-534  preprocess_weights_for_mixed_gemm
  3rdparty/cutlass_kernels/fpA_intB_gemm_wrapper.cu:27-105   dtype rules of the torch entry point
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TILE = 64  # tile edge of the W8T64 layout, in output channels and in reduction indices


# --------------------------------------------------------------------------- numpy restatement
def symmetric_quantize_int8(weight: np.ndarray, variant: int = 0):
    """cutlass_preprocessors.cc:581-678 for INT8_WEIGHT_ONLY, without the packing step.

    weight: [K, N] float16 or float32, K = reduction dim.  Returns (q int8 [K, N], scales [N]) where the
    scales have the weight's dtype (fpA_intB_gemm_wrapper.cu:71).  variant 0 is the reference code
    (amax * 1/128, clip [-128, 127]); variant 1 is amax / 127 with clip [-127, 127].
    C round() (half away from zero, :646) is done in float64, which holds |x| + 0.5 exactly for every
    float32 quotient."""
    assert weight.ndim == 2 and weight.dtype in (np.float16, np.float32)
    w = weight.astype(np.float32)
    a = np.abs(w)
    amax = np.max(np.where(np.isnan(a), np.float32(0), a), axis=0).astype(np.float32)
    if variant == 0:
        s32 = (amax * np.float32(1.0 / 128.0)).astype(np.float32)
        lo = np.float64(-128.0)
    else:
        s32 = (amax / np.float32(127.0)).astype(np.float32)
        lo = np.float64(-127.0)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        r32 = (w / s32[None, :]).astype(np.float32)
        r = r32.astype(np.float64)
        r = np.where(np.isfinite(r), np.copysign(np.floor(np.abs(r) + 0.5), r), r)
    c = np.where(r < 127.0, r, 127.0)
    c = np.where(lo < c, c, lo)
    q = c.astype(np.int8)
    with np.errstate(over="ignore"):
        scales = s32.astype(weight.dtype)
    return q, scales


_REF_ROW_PERM = np.array([0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15])


def ref_pack_int8(q: np.ndarray) -> np.ndarray:
    """preprocess_weights_for_mixed_gemm for int8 on sm75-89 (cutlass_preprocessors.cc:497-534):
    row permutation (:137-195), transpose (:201-335), 2-column interleave in 64-row tiles (:432-495),
    +128 and byte 1<->2 swap per 32-bit word (:337-358).  Returns int8 [K, N] (opaque bytes)."""
    K, N = q.shape
    assert K % 64 == 0 and N % 64 == 0
    p = q.reshape(K // 16, 16, N)[:, _REF_ROW_PERM, :].reshape(K, N)
    t = np.ascontiguousarray(p.T)  # [N, K]
    v = t.reshape(N // 2, 2, K // 64, 64).transpose(0, 2, 1, 3).reshape(N // 2, 2 * K)
    u = (v.astype(np.int16) + 128).astype(np.uint8).reshape(-1, 4)[:, [0, 2, 1, 3]]
    return np.ascontiguousarray(u).reshape(K, N).view(np.int8)


def ref_unpack_int8(packed: np.ndarray) -> np.ndarray:
    """Inverse of ref_pack_int8."""
    K, N = packed.shape
    u = packed.view(np.uint8).reshape(-1, 4)[:, [0, 2, 1, 3]]
    v = (u.astype(np.int16) - 128).astype(np.int8).reshape(N // 2, K // 64, 2, 64)
    t = v.transpose(0, 2, 1, 3).reshape(N, K)
    p = np.ascontiguousarray(t.T)
    inv = np.argsort(_REF_ROW_PERM)
    return np.ascontiguousarray(p.reshape(K // 16, 16, N)[:, inv, :].reshape(K, N))


def b200_pack_int8(q: np.ndarray) -> np.ndarray:
    """W8T64: tiles of 64 channels x 64 reduction indices ordered [N/64][K/64]; inside a tile byte
    (n % 64) * 64 + (k % 64); each byte = q + 128.  Returned as int8 [K, N] (opaque bytes, same size
    as the reference's packed tensor)."""
    K, N = q.shape
    assert K % TILE == 0 and N % TILE == 0
    u = (q.astype(np.int16) + 128).astype(np.uint8)
    t = u.T.reshape(N // TILE, TILE, K // TILE, TILE).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(t).reshape(K, N).view(np.int8)


def b200_unpack_int8(packed: np.ndarray) -> np.ndarray:
    K, N = packed.shape
    u = packed.view(np.uint8).reshape(N // TILE, K // TILE, TILE, TILE).transpose(0, 2, 1, 3).reshape(N, K)
    return np.ascontiguousarray((u.astype(np.int16) - 128).astype(np.int8).T)


# --------------------------------------------------------------------------- checking libraries
def build(target: str = "all", quiet: bool = True) -> None:
    """Runs the Makefile beside this file ('oracle', 'ref' or 'all').  'ref' needs the reference checkout
    (the Makefile's REF variable) and is skipped silently by callers when it is absent."""
    subprocess.run(["make", "-C", HERE, target], check=True,
                   stdout=subprocess.DEVNULL if quiet else None, stderr=subprocess.DEVNULL if quiet else None)


_c_lib = None
_ref_lib = None


def c_oracle():
    """ctypes handle of liboracle_w8.so (built on demand)."""
    global _c_lib
    if _c_lib is None:
        path = os.path.join(HERE, "liboracle_w8.so")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(HERE, "w8_oracle.c")):
            build("oracle")
        lib = ctypes.CDLL(path)
        vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        lib.oracle_symmetric_quantize_int8.argtypes = [vp, ci, sz, sz, vp, vp, ci]
        lib.oracle_ref_pack_int8.argtypes = [vp, sz, sz, vp]
        lib.oracle_ref_unpack_int8.argtypes = [vp, sz, sz, vp]
        lib.oracle_b200_pack_int8.argtypes = [vp, sz, sz, vp]
        lib.oracle_b200_unpack_int8.argtypes = [vp, sz, sz, vp]
        _c_lib = lib
    return _c_lib


def ref_lib():
    """ctypes handle of _ref/libeet_ref_quant.so, or None when it has not been built (the reference
    checkout is only present on the authoring machine; the built library travels with the tree)."""
    global _ref_lib
    if _ref_lib is None:
        path = os.path.join(HERE, "_ref", "libeet_ref_quant.so")
        if not os.path.exists(path):
            return None
        lib = ctypes.CDLL(path)
        vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        lib.ref_symmetric_quantize_int8.argtypes = [vp, ci, sz, sz, vp, vp, vp]
        lib.ref_preprocess_weights_int8.argtypes = [vp, sz, sz, ci, vp]
        _ref_lib = lib
    return _ref_lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def c_symmetric_quantize_int8(weight: np.ndarray, variant: int = 0):
    weight = np.ascontiguousarray(weight)
    K, N = weight.shape
    q = np.empty((K, N), np.int8)
    scales = np.empty((N,), weight.dtype)
    rc = c_oracle().oracle_symmetric_quantize_int8(_ptr(weight), int(weight.dtype == np.float32), K, N,
                                                   _ptr(q), _ptr(scales), variant)
    assert rc == 0
    return q, scales


def c_ref_pack_int8(q: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q)
    out = np.empty_like(q)
    assert c_oracle().oracle_ref_pack_int8(_ptr(q), q.shape[0], q.shape[1], _ptr(out)) == 0
    return out


def c_b200_pack_int8(q: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q)
    out = np.empty_like(q)
    assert c_oracle().oracle_b200_pack_int8(_ptr(q), q.shape[0], q.shape[1], _ptr(out)) == 0
    return out


def c_b200_unpack_int8(p: np.ndarray) -> np.ndarray:
    p = np.ascontiguousarray(p)
    out = np.empty_like(p)
    assert c_oracle().oracle_b200_unpack_int8(_ptr(p), p.shape[0], p.shape[1], _ptr(out)) == 0
    return out


def ref_symmetric_quantize_int8(weight: np.ndarray):
    """The reference's symmetric_quantize itself (needs _ref).  Returns (unprocessed q [K,N], processed
    bytes in the reference's sm80 layout [K,N], scales [N])."""
    lib = ref_lib()
    assert lib is not None, "oracle/_ref has not been built"
    weight = np.ascontiguousarray(weight)
    K, N = weight.shape
    q = np.empty((K, N), np.int8)
    packed = np.empty((K, N), np.int8)
    scales = np.empty((N,), weight.dtype)
    rc = lib.ref_symmetric_quantize_int8(_ptr(weight), int(weight.dtype == np.float32), K, N, _ptr(q),
                                         _ptr(packed), _ptr(scales))
    assert rc == 0
    return q, packed, scales


def ref_preprocess_weights_int8(q: np.ndarray, arch: int = 80):
    lib = ref_lib()
    assert lib is not None, "oracle/_ref has not been built"
    q = np.ascontiguousarray(q)
    out = np.empty_like(q)
    rc = lib.ref_preprocess_weights_int8(_ptr(q), q.shape[0], q.shape[1], arch, _ptr(out))
    return rc, out
