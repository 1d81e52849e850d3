"""The bounded waits and range checks inside the kernels, exercised without faulting, trapping or hanging
anything: a wait is made to run out by simply not sending what it waits for, with the poll limit lowered
through eet_set_wait_limit so that the kernel gives up after microseconds; it then returns normally, the
host reads the status code, and the next ordinary call works."""
import ctypes

import pytest
import torch

from oracle import ops

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_tensor_parallel_inbox_wait_runs_out_and_reports_status_4():
    """eet_rmsnorm_finalize_tp as rank 0 of a world of 2 whose "peer" inbox is just another local buffer that
    nobody writes into: the poll of this rank's inbox can never succeed."""
    from eet_b200 import _lib
    from eet_b200._lib import check, lib
    M, n, world = 4, 4096, 2
    gen = torch.Generator().manual_seed(0)
    sums = torch.randn(M, n, generator=gen).cuda()
    sums_before = sums.clone()
    scale = (torch.rand(n, generator=gen) * 1e-2).half().cuda()
    res = torch.randn(M, n, generator=gen).half().cuda()
    gamma = torch.ones(n).half().cuda()
    h_out = torch.empty(M, n, dtype=torch.float16, device="cuda")
    xn = torch.empty_like(h_out)
    # an inbox: [2][8 source ranks][64 rows][n / 8][3] packets of 16 bytes {value, value, value, epoch}
    inbox = [torch.zeros(2 * 8 * 64 * (n // 8) * 3 * 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in inbox])
    epochs = torch.zeros(128, dtype=torch.int32, device="cuda")
    assert _lib.device_status() == 0
    check(lib.eet_set_wait_limit(2000))
    try:
        check(lib.eet_rmsnorm_finalize_tp(sums.data_ptr(), ptrs, world, 0, 0, epochs.data_ptr(), scale.data_ptr(),
                                          res.data_ptr(), h_out.data_ptr(), gamma.data_ptr(), xn.data_ptr(), M, n, 1e-6,
                                          _stream()))
        torch.cuda.synchronize()          # the kernel returned by itself
        assert _lib.device_status() == 4
        assert _lib.device_status() == 0   # reading clears it
        # the kernel kept its bookkeeping consistent: sums consumed, epoch advanced, pairs pushed to the "peer"
        assert float(sums.abs().max()) == 0 and int(epochs[0]) == 1
        pushed = inbox[1].view(2, 8, 64, n // 8, 3, 4)[0, 0, :M]    # inbox 0, source rank 0
        assert bool((pushed[..., 3] == 1).all())
        # the packets carry the partial sums themselves: {v0, v1, v2}, {v3, v4, v5}, {v6, v7, -}
        vals = pushed.view(torch.float32)
        got = torch.cat([vals[..., 0, :3], vals[..., 1, :3], vals[..., 2, :2]], -1).reshape(M, n)
        assert torch.equal(got, sums_before)
    finally:
        check(lib.eet_set_wait_limit(1 << 22))
    # an ordinary call afterwards is unaffected
    x = torch.randn(3, n, generator=gen).half()
    y = torch.empty(3, n, dtype=torch.float16, device="cuda")
    check(lib.eet_rmsnorm(x.cuda().data_ptr(), gamma.data_ptr(), y.data_ptr(), 3, n, 1e-6, _stream()))
    assert torch.allclose(y.cpu().float(), ops.rmsnorm(x, gamma.cpu(), 1e-6).float(), rtol=1e-3, atol=1e-3)
    assert _lib.device_status() == 0


def test_device_resident_step_outside_the_cache_is_refused_with_status_5():
    """A device-side step that a host check cannot see (CUDA-graph decode): beyond the cache length the kernel
    appends nothing, requests no tile, writes zeros as the context and records status 5."""
    from eet_b200 import _lib
    from eet_b200._lib import check, lib
    B, H, D, T = 2, 4, 128, 64
    gen = torch.Generator().manual_seed(1)
    qkv = torch.randn(B, 3, H, D, generator=gen).half().cuda()
    # the caches sit inside larger buffers whose margins must stay untouched
    pad = 4 * T * D
    kbuf = torch.full((pad + B * H * T * D + pad,), 7.0, dtype=torch.float16, device="cuda")
    vbuf = torch.full_like(kbuf, 7.0)
    k_before, v_before = kbuf.clone(), vbuf.clone()
    ctx = torch.full((B, H * D), 3.0, dtype=torch.float16, device="cuda")
    for bad in (T + 1, 0, -5, 1 << 20):
        step_dev = torch.tensor([bad], dtype=torch.int32, device="cuda")
        check(lib.eet_decode_mha(qkv.data_ptr(), None, None, kbuf.data_ptr() + 2 * pad, vbuf.data_ptr() + 2 * pad,
                                 ctx.data_ptr(), B, H, D, T, 1, step_dev.data_ptr(), None, None, 0, None, 1, 10000.0, 0,
                                 _stream()))
        torch.cuda.synchronize()
        assert _lib.device_status() == 5
        assert torch.equal(kbuf, k_before) and torch.equal(vbuf, v_before)
        assert float(ctx.float().abs().max()) == 0
        ctx.fill_(3.0)
    # the last valid step still works: appended at row T - 1
    step_dev = torch.tensor([T], dtype=torch.int32, device="cuda")
    check(lib.eet_decode_mha(qkv.data_ptr(), None, None, kbuf.data_ptr() + 2 * pad, vbuf.data_ptr() + 2 * pad,
                             ctx.data_ptr(), B, H, D, T, 1, step_dev.data_ptr(), None, None, 0, None, 0, 10000.0, 0,
                             _stream()))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    kc = kbuf[pad: pad + B * H * T * D].view(B, H, T, D)
    assert torch.equal(kc[:, :, T - 1].cpu(), qkv[:, 1].cpu())
    assert torch.equal(kbuf[:pad], k_before[:pad]) and torch.equal(kbuf[-pad:], k_before[-pad:])


def test_check_device_status_rezeroes_the_pooled_scratch():
    """EET.check_device_status after a kernel gave up: raises, and the pooled fp32 sum buffers are zero again."""
    from eet_b200 import EET, _lib
    from eet_b200._lib import check, lib
    buf = EET._pool.zeros("status_test_sums", 256, torch.float32, torch.device("cuda", 0))
    buf.fill_(5.0)
    # provoke status 5 (see above) - cheap and harmless
    B, H, D, T = 1, 1, 128, 8
    qkv = torch.zeros(B, 3, H, D, dtype=torch.float16, device="cuda")
    kc = torch.zeros(B, H, T, D, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    ctx = torch.zeros(B, H * D, dtype=torch.float16, device="cuda")
    step_dev = torch.tensor([T + 3], dtype=torch.int32, device="cuda")
    check(lib.eet_decode_mha(qkv.data_ptr(), None, None, kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(), B, H, D, T, 1,
                             step_dev.data_ptr(), None, None, 0, None, 1, 10000.0, 0, _stream()))
    with pytest.raises(EET.EETError, match="status 5"):
        EET.check_device_status()
    assert float(buf.abs().max()) == 0
    EET.check_device_status()   # clean again
    assert _lib.device_status() == 0


def test_lm_head_argmax_peer_wait_runs_out_and_still_answers():
    """eet_lm_head_argmax with a sharded vocabulary whose peer never sends its packet: the wait gives up (status
    4) and the kernel still writes this rank's own best index."""
    from eet_b200 import _lib
    from eet_b200._lib import check, lib
    M, n, world = 3, 512, 2
    gen = torch.Generator().manual_seed(3)
    sums = torch.randn(M, n, generator=gen).cuda()
    scale = torch.full((n,), 0.01).half().cuda()
    want = (sums.cpu() * scale.cpu().float()).half().float().argmax(1) + 1024   # of the fp16 logits, first on ties
    inbox = [torch.zeros(2 * 8 * 64 * 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in inbox])
    epochs = torch.zeros(64, dtype=torch.int32, device="cuda")
    out = torch.full((M,), -1, dtype=torch.int64, device="cuda")
    check(lib.eet_set_wait_limit(2000))
    try:
        check(lib.eet_lm_head_argmax(sums.data_ptr(), scale.data_ptr(), M, n, 1024, ptrs, world, 0, epochs.data_ptr(),
                                     out.data_ptr(), None, _stream()))
        torch.cuda.synchronize()
        assert _lib.device_status() == 4
    finally:
        check(lib.eet_set_wait_limit(1 << 22))
    assert torch.equal(out.cpu(), want) and float(sums.abs().max()) == 0 and int(epochs[0]) == 1
    # the packet for the peer went out: {logit bits, global index, epoch, -} in half 1 (epoch 1), source rank 0
    sent = inbox[1].view(2, 8, 64, 4)[1, 0, :M].cpu()
    assert torch.equal(sent[:, 1].long(), want) and bool((sent[:, 2] == 1).all())
