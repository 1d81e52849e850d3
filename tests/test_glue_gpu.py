"""RMSNorm, gated SiLU, residual add, prefill QKV split + rotary + cache store, cache reordering."""
import pytest
import torch

from oracle import ops

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("n", [64, 256, 4096, 5120, 8192])
@pytest.mark.parametrize("M", [1, 7])
def test_rmsnorm(M, n):
    from eet_b200._lib import check, lib
    gen = torch.Generator().manual_seed(n + M)
    x = torch.randn(M, n, generator=gen).half()
    g = (1 + 0.1 * torch.randn(n, generator=gen)).half()
    y = torch.empty(M, n, dtype=torch.float16, device="cuda")
    xc, gc = x.cuda(), g.cuda()
    check(lib.eet_rmsnorm(xc.data_ptr(), gc.data_ptr(), y.data_ptr(), M, n, 1e-6, _stream()))
    ref = ops.rmsnorm(x, g, 1e-6)
    # fp32 sums in a different order: at most one fp16 ulp apart
    assert torch.allclose(y.cpu().float(), ref.float(), rtol=1e-3, atol=1e-3)
    assert (y.cpu() == ref).float().mean() > 0.98


def test_swiglu_bit_exact_and_residual():
    from eet_b200._lib import check, lib
    gen = torch.Generator().manual_seed(3)
    g = (torch.randn(5, 11008, generator=gen) * 2).half()
    u = torch.randn(5, 11008, generator=gen).half()
    gc, uc = g.cuda(), u.cuda()
    check(lib.eet_swiglu(gc.data_ptr(), uc.data_ptr(), 5, 11008, _stream()))
    ref = ops.gated_silu(g, u)
    diff = (gc.cpu().float() - ref.float()).abs()
    # expf on the device and on the host may differ by an ulp before the fp16 rounding
    assert (diff <= 2e-3 * ref.float().abs() + 1e-6).all()
    assert (gc.cpu() == ref).float().mean() > 0.97
    a, b = torch.randn(3, 4096, generator=gen).half(), torch.randn(3, 4096, generator=gen).half()
    ac, bc = a.cuda(), b.cuda()
    check(lib.eet_add_residual(ac.data_ptr(), bc.data_ptr(), a.numel(), _stream()))
    assert torch.equal(ac.cpu(), ops.add_residual(a, b))


@pytest.mark.parametrize("rope", [1, 0])
def test_qkv_split_store(rope):
    from eet_b200._lib import check, lib
    B, S, H, D, T = 2, 5, 3, 128, 9
    gen = torch.Generator().manual_seed(11)
    qkv = torch.randn(B, S, 3, H, D, generator=gen).half()
    qc = torch.empty(B, H, S, D, dtype=torch.float16, device="cuda")
    kc = torch.zeros(4, H, T, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    src = qkv.cuda()
    check(lib.eet_qkv_split_store(src.data_ptr(), qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, S, H, D, T, rope,
                                  10000.0, _stream()))
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    if rope:
        t = torch.arange(S).view(1, 1, S)
        q, k = ops.rope_neox(q, t), ops.rope_neox(k, t)
    assert torch.allclose(qc.cpu().float(), q.float(), atol=2e-3, rtol=2e-3)
    assert torch.allclose(kc[:B, :, :S].cpu().float(), k.float(), atol=2e-3, rtol=2e-3)
    assert torch.equal(vc[:B, :, :S].cpu(), v.contiguous())
    assert float(kc[:, :, S:].abs().max()) == 0 and float(kc[B:].abs().max()) == 0


def test_reorder_kv():
    from eet_b200._lib import check, lib
    B, H, D, T, step = 4, 2, 128, 12, 7
    gen = torch.Generator().manual_seed(5)
    k = torch.randn(B, H, T, D, generator=gen).half()
    v = torch.randn(B, H, T, D, generator=gen).half()
    idx = torch.tensor([2, 2, 0, 1])
    kc, vc, ic = k.cuda(), v.cuda(), idx.cuda()
    nbytes = lib.eet_reorder_kv_workspace_bytes(B, H, D, step)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    check(lib.eet_reorder_kv(kc.data_ptr(), vc.data_ptr(), ic.data_ptr(), B, H, D, T, step, ws.data_ptr(), nbytes,
                             _stream()))
    want_k, want_v = k.clone(), v.clone()
    want_k[:, :, :step] = k[idx][:, :, :step]
    want_v[:, :, :step] = v[idx][:, :, :step]
    assert torch.equal(kc.cpu(), want_k) and torch.equal(vc.cpu(), want_v)


def test_argmax_rows_and_gather_rows():
    """Greedy token choice and embedding lookup: equal to torch.argmax (first index on ties) / table[ids]."""
    from eet_b200 import EET
    gen = torch.Generator().manual_seed(41)
    logits = torch.randn(5, 32008, generator=gen).half().cuda()[:, :32003]   # rows 16-byte aligned, ragged length
    logits[1, 17] = logits[1, 30000] = 60000.0          # a tie: the smaller index wins
    logits[2, :] = -3.0                                  # all equal: index 0
    logits[3, 32002] = 50000.0                           # the maximum in the ragged tail (n % 8 != 0)
    got = EET.argmax_rows(logits)
    assert got.dtype == torch.int64 and got.tolist() == [int(logits[0].float().argmax()), 17, 0, 32002,
                                                         int(logits[4].float().argmax())]
    # strided rows, as lm_head(hidden)[:, -1, :] hands them over
    big = torch.randn(3, 4, 1000, generator=gen).half().cuda()
    view = big[:, -1, :]
    assert torch.equal(EET.argmax_rows(view), view.float().argmax(-1))
    odd = torch.randn(3, 1001, generator=gen).half().cuda()       # rows not 16-byte aligned: scalar path
    assert torch.equal(EET.argmax_rows(odd), odd.float().argmax(-1))
    table = torch.randn(50, 256, generator=gen).half().cuda()
    ids = torch.tensor([[3, 49], [0, 7]]).cuda()
    assert torch.equal(EET.gather_rows(table, ids), table[ids])
