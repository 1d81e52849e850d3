"""Decode and prefill attention through the C ABI against the oracle.

Tolerance: outputs are fp16 values of magnitude <= ~1 built from fp32 sums in a different order than the
oracle's, with logits rounded to fp16 on both sides: |err| <= 2e-3 + 2e-3*|ref| (about two fp16 ulps)."""
import pytest
import torch

from oracle import ops

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _decode(qkv, kc, vc, step, pad=None, alibi=None, slopes=None, rope=1, splits=0, step_dev=None):
    from eet_b200._lib import check, lib
    B, _, H, D = qkv.shape
    T = kc.shape[2]
    ctx = torch.empty(B, H * D, dtype=torch.float16, device="cuda")
    check(lib.eet_decode_mha(qkv.data_ptr(), None, None, kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(), B, H, D, T, step,
                             None if step_dev is None else step_dev.data_ptr(),
                             None if pad is None else pad.data_ptr(),
                             None if alibi is None else alibi.data_ptr(), 0 if alibi is None else alibi.shape[-1],
                             None if slopes is None else slopes.data_ptr(), rope, 10000.0, splits, _stream()))
    torch.cuda.synchronize()
    return ctx.cpu().view(B, H, D)


def _oracle_decode(qkv, k_hist, v_hist, step, pad, alibi_row, rope):
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    if rope:
        q, k = ops.rope_neox(q, step - 1), ops.rope_neox(k, step - 1)
    kc, vc = k_hist.clone(), v_hist.clone()
    ctx = ops.decode_attention(q, k, v, kc, vc, step, pad, alibi_row)
    return ctx, kc, vc


def _close(a, b):
    return torch.allclose(a.float(), b.float(), atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("step", [1, 2, 17, 128, 640, 1153])
@pytest.mark.parametrize("splits", [0, 1, 4, 8])
def test_decode_rope(step, splits):
    B, H, D, T = 2, 3, 128, 1160
    gen = torch.Generator().manual_seed(step)
    qkv = torch.randn(B, 3, H, D, generator=gen).half()
    kh = torch.randn(B, H, T, D, generator=gen).half()
    vh = torch.randn(B, H, T, D, generator=gen).half()
    ref, kc_ref, vc_ref = _oracle_decode(qkv, kh, vh, step, None, None, True)
    kc, vc = kh.cuda(), vh.cuda()
    got = _decode(qkv.cuda(), kc, vc, step, splits=splits)
    assert _close(got, ref)
    # the new K (rotated) and V were appended at step-1, nothing else moved
    assert _close(kc.cpu()[:, :, step - 1], kc_ref[:, :, step - 1])
    assert torch.equal(vc.cpu()[:, :, step - 1], vc_ref[:, :, step - 1])
    kc_host = kc.cpu()
    kc_host[:, :, step - 1] = kh[:, :, step - 1]
    assert torch.equal(kc_host, kh)


def test_decode_beyond_the_reference_4096_limit():
    B, H, D, T, step = 1, 2, 128, 5000, 4800
    gen = torch.Generator().manual_seed(1)
    qkv = torch.randn(B, 3, H, D, generator=gen).half()
    kh = torch.randn(B, H, T, D, generator=gen).half()
    vh = torch.randn(B, H, T, D, generator=gen).half()
    ref, _, _ = _oracle_decode(qkv, kh, vh, step, None, None, True)
    assert _close(_decode(qkv.cuda(), kh.cuda(), vh.cuda(), step), ref)


@pytest.mark.parametrize("pads", [[0, 17], [5, 0], [40, 39]])
def test_decode_left_padding(pads):
    B, H, D, T, step = 2, 4, 128, 64, 41
    gen = torch.Generator().manual_seed(3)
    qkv = torch.randn(B, 3, H, D, generator=gen).half()
    kh = torch.randn(B, H, T, D, generator=gen).half()
    vh = torch.randn(B, H, T, D, generator=gen).half()
    pad = torch.tensor(pads, dtype=torch.long)
    ref, _, _ = _oracle_decode(qkv, kh, vh, step, pad, None, True)
    got = _decode(qkv.cuda(), kh.cuda(), vh.cuda(), step, pad=pad.view(B, 1).cuda(), splits=2)
    assert _close(got, ref)


@pytest.mark.parametrize("step", [1, 33, 300])
def test_decode_alibi_tensor_and_slopes_forms_agree_with_oracle(step):
    B, H, D, T = 2, 8, 128, 320
    gen = torch.Generator().manual_seed(step)
    qkv = torch.randn(B, 3, H, D, generator=gen).half()
    kh = torch.randn(B, H, T, D, generator=gen).half()
    vh = torch.randn(B, H, T, D, generator=gen).half()
    mask = ops.alibi_mask(H, T).half()
    row = mask[:, step - 1, :step].contiguous()        # what the model passes: alibi_mask[:, -1:, :]
    ref, _, _ = _oracle_decode(qkv, kh, vh, step, None, row, False)
    got_t = _decode(qkv.cuda(), kh.cuda(), vh.cuda(), step, alibi=row.view(H, 1, step).cuda(), rope=0)
    slopes = torch.tensor(ops.alibi_slopes(H), dtype=torch.float32).cuda()
    got_s = _decode(qkv.cuda(), kh.cuda(), vh.cuda(), step, slopes=slopes, rope=0)
    assert _close(got_t, ref)
    assert torch.equal(got_t, got_s)


def test_decode_reads_step_from_device_memory():
    B, H, D, T, step = 2, 2, 128, 96, 50
    gen = torch.Generator().manual_seed(8)
    qkv = torch.randn(B, 3, H, D, generator=gen).half()
    kh = torch.randn(B, H, T, D, generator=gen).half()
    vh = torch.randn(B, H, T, D, generator=gen).half()
    ref, _, _ = _oracle_decode(qkv, kh, vh, step, None, None, True)
    from eet_b200._lib import check, lib
    dev = torch.tensor([step - 1, 7], dtype=torch.int32, device="cuda")
    check(lib.eet_advance_steps(dev.data_ptr(), 1, 1, _stream()))
    got = _decode(qkv.cuda(), kh.cuda(), vh.cuda(), 1, step_dev=dev)   # the host value is ignored
    assert _close(got, ref) and dev.tolist() == [step, 7]


@pytest.mark.parametrize("S", [1, 5, 16, 37, 130])
@pytest.mark.parametrize("mode", ["plain", "pad", "alibi"])
def test_prefill(S, mode):
    from eet_b200._lib import check, lib
    B, H, D, T = 2, 3, 128, 140
    gen = torch.Generator().manual_seed(S)
    q, k, v = (torch.randn(B, H, S, D, generator=gen).half() for _ in range(3))
    pad = torch.tensor([0, min(3, S - 1)], dtype=torch.long) if mode == "pad" else None
    alibi = ops.alibi_mask(H, T).half()[:, :S, :S].contiguous() if mode == "alibi" else None
    ref = ops.prefill_attention(q, k, v, pad, alibi)           # [B,H,S,D]
    kc = torch.zeros(B, H, T, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:, :, :S], vc[:, :, :S] = k.cuda(), v.cuda()
    ctx = torch.empty(B, S, H * D, dtype=torch.float16, device="cuda")
    qc = q.cuda()
    pad_c = None if pad is None else pad.cuda()
    alibi_c = None if alibi is None else alibi.cuda()
    check(lib.eet_prefill_mha(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(), B, S, H, D, T,
                              None if pad_c is None else pad_c.data_ptr(),
                              None if alibi_c is None else alibi_c.data_ptr(), S, _stream()))
    torch.cuda.synchronize()
    got = ctx.cpu().view(B, S, H, D).transpose(1, 2)
    # oracle and kernel both feed fp16 probabilities to P.V, but normalise at different points (the oracle
    # rounds p / sum, the blockwise kernel rounds exp(s - running max) and divides at the end)
    assert torch.allclose(got.float(), ref.float(), atol=4e-3, rtol=4e-3)


@pytest.mark.parametrize("case", [(200, [70, 130], "pad"), (512, [0, 0], "plain"), (300, [0, 0], "alibi"),
                                  (96, [0, 95], "pad"), (128, [0, 0], "plain"), (129, [1, 128], "pad"),
                                  (1024, [0, 0], "plain"), (1000, [0, 300], "pad"), (640, [0, 0], "alibi")])
def test_prefill_long_prompts(case):
    """Prompts of several query tiles (the tcgen05 kernel, 128 x 128 tiles, from 96 tokens on): left padding that
    swallows whole key blocks and whole query tiles (their rows must come out zero), prompts of exactly one tile
    and one token more, the configs[2] prompt length and the 1024 tokens of configs[4] (eight key blocks: both
    rings and both score buffers wrap several times), and ALiBi across tiles."""
    from eet_b200._lib import check, lib
    S, pads, mode = case
    B, H, D, T = 2, 2, 128, max(520, S + 8)
    gen = torch.Generator().manual_seed(S)
    q, k, v = (torch.randn(B, H, S, D, generator=gen).half() for _ in range(3))
    pad = torch.tensor(pads, dtype=torch.long) if mode == "pad" else None
    alibi = ops.alibi_mask(H, T).half()[:, :S, :S].contiguous() if mode == "alibi" else None
    ref = ops.prefill_attention(q, k, v, pad, alibi)
    kc = torch.zeros(B, H, T, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:, :, :S], vc[:, :, :S] = k.cuda(), v.cuda()
    ctx = torch.full((B, S, H * D), 7.0, dtype=torch.float16, device="cuda")
    qc = q.cuda()
    pad_c = None if pad is None else pad.cuda()
    alibi_c = None if alibi is None else alibi.cuda()
    check(lib.eet_prefill_mha(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(), B, S, H, D, T,
                              None if pad_c is None else pad_c.data_ptr(),
                              None if alibi_c is None else alibi_c.data_ptr(), S, _stream()))
    torch.cuda.synchronize()
    got = ctx.cpu().view(B, S, H, D).transpose(1, 2)
    assert torch.allclose(got.float(), ref.float(), atol=4e-3, rtol=4e-3)
    if mode == "pad":
        for b, p_len in enumerate(pads):
            if p_len:
                assert float(got[b, :, :p_len].abs().max()) == 0.0   # rows inside the padding are zeroed


def test_decode_finishes_projection_sums_itself():
    """qkv given as the fp32 sums of the projection GEMM + per-channel scales: same result as the fp16 form,
    and the sums are zero afterwards."""
    from eet_b200._lib import check, lib
    B, H, D, T, step = 2, 3, 128, 64, 33
    gen = torch.Generator().manual_seed(12)
    sums = torch.randn(B, 3 * H * D, generator=gen) * 300
    scale = (torch.rand(3 * H * D, generator=gen) * 4e-3 + 1e-3).half()
    qkv = (sums * scale.float()).half().view(B, 3, H, D)
    kh = torch.randn(B, H, T, D, generator=gen).half()
    vh = torch.randn(B, H, T, D, generator=gen).half()
    ref, kc_ref, _ = _oracle_decode(qkv, kh, vh, step, None, None, True)
    kc, vc, sums_c, scale_c = kh.cuda(), vh.cuda(), sums.cuda(), scale.cuda()
    ctx = torch.empty(B, H * D, dtype=torch.float16, device="cuda")
    check(lib.eet_decode_mha(None, sums_c.data_ptr(), scale_c.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(),
                             B, H, D, T, step, None, None, None, 0, None, 1, 10000.0, 4, _stream()))
    torch.cuda.synchronize()
    assert _close(ctx.cpu().view(B, H, D), ref)
    assert _close(kc.cpu()[:, :, step - 1], kc_ref[:, :, step - 1])
    assert float(sums_c.abs().max()) == 0
