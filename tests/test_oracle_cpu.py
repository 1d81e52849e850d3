"""The oracle against its pins: golden vectors generated from the reference, and (where the library
built from the reference checkout is present) the reference itself."""
import glob
import math
import json
import os

import numpy as np
import pytest
import torch

from oracle import ops, w8


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


QUANT_FILES = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "quant_*.npz")))


@pytest.mark.parametrize("path", QUANT_FILES, ids=[os.path.basename(p) for p in QUANT_FILES])
def test_quantizer_restatements_match_golden(path):
    g = np.load(path)
    w = g["w"]
    with np.errstate(all="ignore"):
        for impl in (w8.symmetric_quantize_int8, w8.c_symmetric_quantize_int8):
            q, s = impl(w)
            assert np.array_equal(q, g["q"]), impl.__name__
            assert np.array_equal(_bits(s), _bits(g["scales"])), impl.__name__
    assert len(QUANT_FILES) >= 5


@pytest.mark.parametrize("path", QUANT_FILES, ids=[os.path.basename(p) for p in QUANT_FILES])
def test_reference_packer_restatement_matches_golden(path):
    g = np.load(path)
    assert np.array_equal(w8.ref_pack_int8(g["q"]), g["ref_packed"])
    assert np.array_equal(w8.c_ref_pack_int8(g["q"]), g["ref_packed"])
    assert np.array_equal(w8.ref_unpack_int8(g["ref_packed"]), g["q"])


def test_edge_cases_of_the_golden_edges_file(golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_fp16_edges.npz"))
    q, s = g["q"], g["scales"]
    assert (q[:, 0] == 127).all() and s[0] == 0          # all-zero column
    assert q[3, 1] == 127 and q[5, 2] == -128             # +amax clips to 127, -amax is -128
    assert q[7, 7] == 127                                 # NaN element
    assert (q[:, 8] == 127).all() and np.isinf(s[8])      # inf column


def test_b200_layout_roundtrip_and_definition():
    rng = np.random.default_rng(1)
    q = rng.integers(-128, 128, size=(192, 320), dtype=np.int8)
    p = w8.b200_pack_int8(q)
    assert np.array_equal(w8.c_b200_pack_int8(q), p)
    assert np.array_equal(w8.b200_unpack_int8(p), q)
    assert np.array_equal(w8.c_b200_unpack_int8(p), q)
    flat = p.view(np.uint8).reshape(-1)
    for (k, n) in [(0, 0), (63, 63), (64, 1), (191, 319), (100, 200)]:
        off = ((n // 64) * (192 // 64) + k // 64) * 4096 + (n % 64) * 64 + k % 64
        assert flat[off] == int(q[k, n]) + 128


def test_variant_127():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((64, 64)) * 0.02).astype(np.float16)
    q, s = w8.symmetric_quantize_int8(w, variant=1)
    qc, sc = w8.c_symmetric_quantize_int8(w, variant=1)
    assert np.array_equal(q, qc) and np.array_equal(_bits(s), _bits(sc))
    assert q.min() >= -127 and q.max() == 127 or q.min() == -127
    amax = np.abs(w.astype(np.float32)).max(0)
    assert np.array_equal(_bits(s), _bits((amax / np.float32(127)).astype(np.float16)))


@pytest.mark.skipif(w8.ref_lib() is None, reason="oracle/_ref not built (needs the reference checkout)")
def test_restatements_match_the_compiled_reference():
    rng = np.random.default_rng(3)
    for dtype in (np.float16, np.float32):
        for K, N in [(64, 64), (256, 192), (512, 1024)]:
            w = (rng.standard_normal((K, N)) * rng.choice([0.02, 1.0, 30.0])).astype(dtype)
            w[:, 5] = 0
            qr, pr, sr = w8.ref_symmetric_quantize_int8(w)
            qc, sc = w8.c_symmetric_quantize_int8(w)
            assert np.array_equal(qc, qr) and np.array_equal(_bits(sc), _bits(sr))
            assert np.array_equal(w8.c_ref_pack_int8(qr), pr)
    rc, _ = w8.ref_preprocess_weights_int8(qr, arch=100)
    assert rc != 0  # the reference packer rejects sm_100 (cutlass_preprocessors.cc:113-127)


def test_alibi_restatement_matches_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "alibi.npz"))
    assert np.allclose(np.array(ops.alibi_slopes(40)), g["slopes_40"], rtol=0, atol=0)
    assert np.allclose(np.array(ops.alibi_slopes(32)), g["slopes_32"], rtol=0, atol=0)
    assert np.array_equal(ops.alibi_mask(40, 12).numpy(), g["mask_40x12"])
    assert np.array_equal(ops.alibi_mask(8, 33).half().numpy(), g["mask_8x33_fp16"])


def test_gemm_restatement_self_consistency():
    torch.manual_seed(0)
    K, N, M = 128, 192, 5
    w = (torch.randn(K, N) * 0.02).half().numpy()
    q, s = w8.symmetric_quantize_int8(w)
    q, s = torch.from_numpy(q), torch.from_numpy(s)
    x = torch.randn(M, K).half()
    y_exact = ops.gemm_w8a16(x, q, s, exact=True).double()
    y_ref = ops.gemm_w8a16_fp32(x, q, s)
    tol = 1e-2 * y_ref.abs().amax(1, keepdim=True)
    assert ((y_exact - y_ref).abs() <= tol).all()
    # one-hot activations deliver the dequantized weight rows exactly
    eye = torch.eye(K)[:7].half()
    y = ops.gemm_w8a16(eye, q, s, exact=True)
    assert torch.equal(y, (q[:7].float() * s.float()[None]).half())


def test_decode_attention_matches_prefill_last_row():
    """Two restatements of the same maths written from different reference kernels must agree."""
    torch.manual_seed(1)
    B, H, S, D = 2, 3, 9, 128
    q, k, v = (torch.randn(B, H, S, D).half() for _ in range(3))
    pad = torch.tensor([0, 2])
    full = ops.prefill_attention(q, k, v, pad)
    kc, vc = torch.zeros(B, H, 16, D).half(), torch.zeros(B, H, 16, D).half()
    kc[:, :, :S - 1], vc[:, :, :S - 1] = k[:, :, :S - 1], v[:, :, :S - 1]
    last = ops.decode_attention(q[:, :, -1], k[:, :, -1], v[:, :, -1], kc, vc, S, pad)
    assert torch.allclose(full[:, :, -1].float(), last.float(), atol=2e-3, rtol=2e-3)
    assert torch.equal(kc[:, :, S - 1], k[:, :, -1])


def test_convert_name_matches_reference(golden_dir):
    from eet_b200.modeling import convert_name
    names = json.load(open(os.path.join(golden_dir, "names.json")))
    for model, table in names.items():
        for src, dst in table.items():
            assert convert_name(src, model) == dst


# ---------------------------------------------------------------------------------------------------
# The attention restatements against an independent formulation.  oracle/ops.py is written from the
# reference's CUDA sources and nothing in the reference can run here to pin it; torch's
# scaled_dot_product_attention (fp32, additive mask) shares no code with it.  What this pins: the masking
# conventions (causal, left padding, which positions the ALiBi bias multiplies), the 1/sqrt(D) scale, the
# softmax and the P.V contraction.  What it cannot pin: the reference's rounding points (fp16 logits, fp16
# probabilities, the +1e-6 in the denominator), which only move the result inside the tolerance below.
# ---------------------------------------------------------------------------------------------------
def _sdpa(q, k, v, mask_add):
    import torch.nn.functional as F
    D = q.shape[-1]
    return F.scaled_dot_product_attention(q.float(), k.float(), v.float(), attn_mask=mask_add, scale=1.0 / math.sqrt(D))


@pytest.mark.parametrize("use_alibi", [False, True])
def test_prefill_attention_matches_sdpa_with_padding_and_alibi(use_alibi):
    from oracle import ops
    gen = torch.Generator().manual_seed(11)
    B, H, S, D = 3, 4, 37, 128
    q, k, v = (torch.randn(B, H, S, D, generator=gen).half() for _ in range(3))
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    neg = torch.tensor(float("-inf"))
    if use_alibi:
        alibi = ops.alibi_mask(H, S).half()
        got = ops.prefill_attention(q, k, v, None, alibi)
        slopes = torch.tensor(ops.alibi_slopes(H))
        mask = torch.where(j <= i, slopes[:, None, None] * j.float()[None], neg)[None]      # [1, H, S, S]
        want = _sdpa(q, k, v, mask.expand(B, H, S, S))
        rows = torch.ones(B, S, dtype=torch.bool)
    else:
        pad = torch.tensor([0, 5, 36])
        got = ops.prefill_attention(q, k, v, pad, None)
        ok = (j <= i)[None] & (j[None] >= pad.view(B, 1, 1))                                   # [B, S, S]
        rows = torch.arange(S)[None, :] >= pad[:, None]                                        # rows with any key
        mask = torch.where(ok, torch.tensor(0.0), neg)[:, None].expand(B, H, S, S).clone()
        mask[~rows[:, None, :, None].expand(B, H, S, S)] = 0.0                                 # keep SDPA finite there
        want = _sdpa(q, k, v, mask)
        # rows above the left padding are zeroed by the reference (gpt2_self_softmax.cu:24-30)
        assert (got[~rows[:, None, :].expand(B, H, S)] == 0).all()
    sel = rows[:, None, :].expand(B, H, S)
    err = (got.float() - want)[sel].abs()
    assert float(err.max()) <= 4e-3 + 1e-2 * float(want[sel].abs().max()), float(err.max())


@pytest.mark.parametrize("use_alibi", [False, True])
def test_decode_attention_matches_sdpa_with_padding_and_alibi(use_alibi):
    from oracle import ops
    gen = torch.Generator().manual_seed(12)
    B, H, D, T, step = 3, 4, 128, 48, 41
    kc = torch.randn(B, H, T, D, generator=gen).half()
    vc = torch.randn(B, H, T, D, generator=gen).half()
    q, kn, vn = (torch.randn(B, H, D, generator=gen).half() for _ in range(3))
    pad = None if use_alibi else torch.tensor([0, 7, 40])
    alibi = ops.alibi_mask(H, T).half()[:, step - 1, :step] if use_alibi else None
    got = ops.decode_attention(q, kn, vn, kc, vc, step, pad, alibi)
    assert torch.equal(kc[:, :, step - 1], kn) and torch.equal(vc[:, :, step - 1], vn)        # appended in place
    t = torch.arange(step)
    if use_alibi:
        slopes = torch.tensor(ops.alibi_slopes(H))
        mask = (slopes[:, None] * t.float()[None])[None, :, None, :].expand(B, H, 1, step)
    else:
        mask = torch.where(t[None] >= pad[:, None], torch.tensor(0.0), torch.tensor(float("-inf")))
        mask = mask[:, None, None, :].expand(B, H, 1, step)
    want = _sdpa(q[:, :, None], kc[:, :, :step], vc[:, :, :step], mask)[:, :, 0]
    err = (got.float() - want).abs()
    assert float(err.max()) <= 4e-3 + 1e-2 * float(want.abs().max()), float(err.max())
