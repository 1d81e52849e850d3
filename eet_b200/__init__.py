"""eet_b200 - the int8 weight-only (W8A16) inference path of NetEase-FuXi/EET, rebuilt for NVIDIA B200.

* ``eet_b200.EET``      - drop-in for the reference's pybind11 module ``EET`` on this path
* ``eet_b200.modeling`` - LLaMA / Baichuan model wrappers with the reference's schema and signatures
* ``eet_b200.tp``       - tensor parallelism over torch.distributed (NCCL)
* ``libeet_b200.so``    - the CUDA kernels behind a C ABI (include/eet_b200.h), built by ``eet_b200.build``

Importing ``eet_b200.EET`` loads the CUDA library and raises if it is missing: there is no fallback.
"""
import sys

__version__ = "0.1.0"


def install_as_EET():
    """Registers eet_b200.EET under the module name ``EET`` so that code written against the reference
    (``from EET import MetaDesc, LlamaMmha, ...``) imports this library instead."""
    from . import EET
    sys.modules["EET"] = EET
    return EET
