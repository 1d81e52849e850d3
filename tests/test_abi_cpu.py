"""The C-ABI library loads without a GPU and exports exactly what include/eet_b200.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "eet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(eet_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from eet_b200 import _lib
    names = _declared()
    assert len(names) >= 15
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in include/eet_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    assert _lib.lib.eet_abi_version() == 4


def test_argument_validation_happens_before_any_cuda_call():
    from eet_b200 import _lib
    lib = _lib.lib
    # K not a multiple of 64 is refused on the host, with a message
    rc = lib.eet_gemm_w8a16(None, None, None, None, 1, 64, 100, None, 0, None, 0, None)
    assert rc != 0 and b"multiples of 64" in lib.eet_last_error()
    rc = lib.eet_quantize_w8(None, 0, 64, 64, None, None, None, 0, None, 0, None)
    assert rc != 0 and b"NULL" in lib.eet_last_error()
    rc = lib.eet_decode_mha(None, None, None, None, None, None, 1, 1, 128, 8, 1, None, None, None, 0, None, 1, 10000.0, 0,
                            None)
    assert rc != 0
    assert lib.eet_gemm_w8a16_workspace_bytes(16, 4096, 4096) == 16 * 4096 * 4
    assert lib.eet_gemm_w8a16_workspace_bytes(4096, 4096, 4096) == 128 * 4096 * 4
    assert lib.eet_quantize_w8_workspace_bytes(4096, 11008) == 11008 * 4
