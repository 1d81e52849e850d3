"""CUDA quantizer / packer through the C ABI against the oracle: bit-exact."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import w8

pytestmark = pytest.mark.gpu

QUANT_FILES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "quant_*.npz")))


def _bits(t):
    return t.view(torch.int16 if t.dtype == torch.float16 else torch.int32)


@pytest.mark.parametrize("path", QUANT_FILES, ids=[os.path.basename(p) for p in QUANT_FILES])
def test_quantizer_matches_reference_golden(path):
    from eet_b200 import EET
    g = np.load(path)
    w = torch.from_numpy(g["w"])
    q, packed, scales = EET.quant_weights(w, torch.int8, True)
    assert not q.is_cuda and q.dtype == torch.int8 and tuple(q.shape) == tuple(w.shape)
    assert torch.equal(q, torch.from_numpy(g["q"]))
    assert torch.equal(_bits(scales), _bits(torch.from_numpy(g["scales"])))
    assert scales.dtype == w.dtype
    assert torch.equal(packed, torch.from_numpy(w8.b200_pack_int8(g["q"])))
    # the two-output form returns [packed, scales]
    p2, s2 = EET.quant_weights(w, torch.int8, False)
    assert torch.equal(p2, packed) and torch.equal(_bits(s2), _bits(scales))
    # reference-packed bytes convert to the same layout
    assert torch.equal(EET.repack_reference_weights(torch.from_numpy(g["ref_packed"])), packed)
    assert torch.equal(EET.unpack_weights(packed), q)
    assert torch.equal(EET.preprocess_weights(q), packed)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(64, 64), (4096, 4096), (4096, 11008), (11008, 4096)])
def test_quantizer_matches_oracle_at_config_sizes(dtype, shape):
    """configs[0]/[1] shapes: seeded W ~ N(0, 0.02^2); the C oracle runs these in well under a second."""
    from eet_b200 import EET
    if dtype == torch.float32 and shape[0] * shape[1] > 4096 * 4096:
        pytest.skip("fp32 input covered at 4096x4096")
    K, N = shape
    gen = torch.Generator().manual_seed(0)
    w = (torch.randn(N, K, generator=gen) * 0.02).to(dtype).t().contiguous()
    q, packed, scales = EET.quant_weights(w, torch.int8, True)
    qo, so = w8.c_symmetric_quantize_int8(w.numpy())
    assert torch.equal(q, torch.from_numpy(qo))
    assert torch.equal(_bits(scales), _bits(torch.from_numpy(so)))
    assert torch.equal(packed, torch.from_numpy(w8.c_b200_pack_int8(qo)))


def test_variant_127_and_three_d_input():
    from eet_b200 import EET
    gen = torch.Generator().manual_seed(4)
    w = (torch.randn(2, 128, 64, generator=gen) * 0.02).half()
    q, packed, scales = EET.quant_weights(w, torch.int8, True, variant=1)
    assert q.shape == (2, 128, 64) and scales.shape == (2, 64)
    for e in range(2):
        qo, so = w8.c_symmetric_quantize_int8(w[e].numpy(), variant=1)
        assert torch.equal(q[e], torch.from_numpy(qo))
        assert torch.equal(_bits(scales[e]), _bits(torch.from_numpy(so)))
    assert int(q.min()) >= -127


def test_cuda_input_stays_on_device_and_bad_shapes_raise():
    from eet_b200 import EET
    w = torch.randn(64, 128, device="cuda").half()
    packed, scales = EET.quant_weights(w, torch.int8)
    assert packed.is_cuda and scales.is_cuda
    with pytest.raises(RuntimeError, match="multiples of 64"):
        EET.quant_weights(torch.randn(60, 64).half(), torch.int8)
