"""W8A16 GEMM through the C ABI against the oracle.

Tolerance (stated by the task): max |err| <= 1e-2 * ||row||_inf against an fp32 dequantize-then-matmul;
additionally the result must sit within a few fp16 ulps of the restatement that mirrors the reference's
rounding (fp16(q*scale) weights, fp32 accumulate, one fp16 rounding)."""
import numpy as np
import pytest
import torch

from oracle import ops, w8

pytestmark = pytest.mark.gpu


def _case(K, N, M, seed=0, wstd=0.02):
    gen = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=gen) * wstd).half().t().contiguous()
    x = torch.randn(M, K, generator=gen).half()
    qo, so = w8.c_symmetric_quantize_int8(w.numpy())
    return x, torch.from_numpy(qo), torch.from_numpy(so)


def _run(x, q, s, residual=None):
    from eet_b200 import EET
    packed = EET.preprocess_weights(q).cuda()
    y = EET.gemm_w8a16(x.cuda(), packed, s.cuda(), residual=None if residual is None else residual.cuda())
    torch.cuda.synchronize()
    from eet_b200 import _lib
    assert _lib.device_status() == 0
    return y.cpu()


def _check(y, x, q, s):
    ref = ops.gemm_w8a16_fp32(x, q, s)
    tol = 1e-2 * ref.abs().amax(1, keepdim=True)
    err = (y.double() - ref).abs()
    assert (err <= tol).all(), f"max err {err.max():.4g} vs tol {tol.min():.4g}"
    exact = ops.gemm_w8a16(x, q, s, exact=True).double()
    # both are fp16 roundings of nearly the same fp32 number
    assert ((y.double() - exact).abs() <= 2e-3 * ref.abs().amax(1, keepdim=True) + 1e-3).all()


@pytest.mark.parametrize("M", [1, 2, 3, 8, 9, 16])
@pytest.mark.parametrize("KN", [(64, 64), (128, 192), (256, 64), (1024, 320)])
def test_small_shapes(KN, M):
    x, q, s = _case(KN[0], KN[1], M, seed=M)
    _check(_run(x, q, s), x, q, s)


@pytest.mark.parametrize("M", [17, 33, 130])
def test_m_above_16(M):
    x, q, s = _case(256, 192, M, seed=5)
    _check(_run(x, q, s), x, q, s)


def test_config0_single_layer():
    """configs[0]: W[4096,4096] ~ N(0, 0.02^2), X[16,4096] ~ N(0,1)."""
    x, q, s = _case(4096, 4096, 16, seed=0)
    _check(_run(x, q, s), x, q, s)


@pytest.mark.parametrize("KN", [(4096, 11008), (11008, 4096), (4096, 12288)])
@pytest.mark.parametrize("M", [1, 8])
def test_llama7b_projection_shapes(KN, M):
    x, q, s = _case(KN[0], KN[1], M, seed=1)
    _check(_run(x, q, s), x, q, s)


def test_one_hot_rows_return_dequantized_weights_exactly():
    """Size-independent property used at full size: a one-hot activation row k must return
    fp16(q[k, :] * scale) bit for bit - it checks packing, tile addressing and the epilogue."""
    K, N = 4096, 11008
    gen = torch.Generator().manual_seed(2)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 1e-3 + 1e-4).half()
    rows = torch.tensor([0, 1, 63, 64, 1000, 2047, 2048, 4095, 17, 3000, 77, 4032, 511, 512, 2500, 3999])
    x = torch.zeros(16, K).half()
    x[torch.arange(16), rows] = 1.0
    y = _run(x, q, s)
    want = (q[rows].float() * s.float()[None]).half()
    assert torch.equal(y, want)


def test_linearity_and_residual_epilogue():
    x, q, s = _case(1024, 512, 8, seed=7)
    y1 = _run(x, q, s)
    y2 = _run((x * 2).half(), q, s)           # exact doubling in fp16 -> doubling of the result
    # (split-K partial sums meet in a different order from run to run: equal up to one fp16 ulp)
    assert torch.allclose(y2.float(), y1.float() * 2, rtol=2e-3, atol=1e-4)
    r = torch.randn(8, 512).half()
    yr = _run(x, q, s, residual=r)
    # fp16(product) + residual in fp16
    assert torch.allclose(yr.float(), (y1.float() + r.float()).half().float(), rtol=2e-3, atol=2e-3)


def test_repeated_calls_leave_scratch_clean():
    x, q, s = _case(4096, 4096, 4, seed=9)
    ys = [_run(x, q, s) for _ in range(3)]
    assert torch.equal(ys[0], ys[1]) or (ys[0].float() - ys[1].float()).abs().max() < 2e-3
    _check(ys[2], x, q, s)


def test_empty_and_invalid():
    from eet_b200 import EET, _lib
    x, q, s = _case(64, 64, 1)
    packed = EET.preprocess_weights(q).cuda()
    out = EET.gemm_w8a16(torch.empty(0, 64, device="cuda").half(), packed, s.cuda())
    assert out.shape == (0, 64)
    rc = _lib.lib.eet_gemm_w8a16(1, 1, 1, 1, 1, 64, 100, None, 0, None, 0, None)
    assert rc != 0


def test_accumulate_and_fused_finalize_kernels():
    """The decode-path split of the GEMM: sums from eet_gemm_w8a16_accum (two weights in one launch), finished
    by the generic finalize kernel, by the RMSNorm head and by the SwiGLU kernel - each against the oracle."""
    from eet_b200 import EET
    from eet_b200._lib import check, lib
    stream = torch.cuda.current_stream().cuda_stream
    M, K, N = 8, 512, 1024
    x, q1, s1 = _case(K, N, M, seed=21)
    _, q2, s2 = _case(K, N, M, seed=22)
    xc = x.cuda()
    p1, p2 = EET.preprocess_weights(q1).cuda(), EET.preprocess_weights(q2).cuda()
    s1c, s2c = s1.cuda(), s2.cuda()
    sums1 = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    sums2 = torch.zeros_like(sums1)
    EET.gemm_w8a16_accum(xc, p1, sums1, p2, sums2)
    want1 = x.double() @ q1.double()
    want2 = x.double() @ q2.double()
    assert torch.allclose(sums1.cpu().double(), want1, rtol=1e-5, atol=1e-2)
    assert torch.allclose(sums2.cpu().double(), want2, rtol=1e-5, atol=1e-2)
    # SwiGLU head: gate = fp16(sums1*s1), up = fp16(sums2*s2)
    act = torch.empty(M, N, dtype=torch.float16, device="cuda")
    g_ref, u_ref = (sums1.cpu() * s1.float()).half(), (sums2.cpu() * s2.float()).half()
    check(lib.eet_swiglu_finalize(sums1.data_ptr(), s1c.data_ptr(), sums2.data_ptr(), s2c.data_ptr(), act.data_ptr(),
                                  M, N, stream))
    ref = ops.gated_silu(g_ref, u_ref)
    assert torch.allclose(act.cpu().float(), ref.float(), rtol=2e-3, atol=1e-5)
    assert float(sums1.abs().max()) == 0 and float(sums2.abs().max()) == 0
    # RMSNorm head: h = fp16(sums*s) + residual, xn = rmsnorm(h)
    EET.gemm_w8a16_accum(xc, p1, sums1)
    res = torch.randn(M, N).half()
    gamma = (1 + 0.1 * torch.randn(N)).half()
    h_out = torch.empty(M, N, dtype=torch.float16, device="cuda")
    xn = torch.empty_like(h_out)
    resc, gc = res.cuda(), gamma.cuda()
    h_ref = ops.add_residual((sums1.cpu() * s1.float()).half(), res)
    check(lib.eet_rmsnorm_finalize(sums1.data_ptr(), s1c.data_ptr(), resc.data_ptr(), h_out.data_ptr(), gc.data_ptr(),
                                   xn.data_ptr(), M, N, 1e-6, stream))
    assert torch.equal(h_out.cpu(), h_ref)
    assert torch.allclose(xn.cpu().float(), ops.rmsnorm(h_ref, gamma, 1e-6).float(), rtol=1e-3, atol=1e-3)
    assert float(sums1.abs().max()) == 0
    # without sums it is a plain RMSNorm of `residual`
    check(lib.eet_rmsnorm_finalize(None, None, resc.data_ptr(), None, gc.data_ptr(), xn.data_ptr(), M, N, 1e-6, stream))
    assert torch.allclose(xn.cpu().float(), ops.rmsnorm(res, gamma, 1e-6).float(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("KN", [(5120, 15360), (5120, 13696), (13696, 5120), (8192, 24576), (8192, 22016), (22016, 8192)])
def test_baichuan13b_and_llama65b_projection_shapes(KN):
    """configs[3] / configs[4] layer shapes at full size: random activations against the fp32 oracle on the
    decode batch of those configs capped at 16 rows, plus a prefill-sized batch through the tensor-core path
    checked on sampled rows (the full fp32 product would take the CPU minutes)."""
    K, N = KN
    gen = torch.Generator().manual_seed(K + N)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 3e-4 + 1e-4).half()
    x = torch.randn(16, K, generator=gen).half()
    _check(_run(x, q, s), x, q, s)
    xl = torch.randn(384, K, generator=gen).half()
    y = _run(xl, q, s)
    rows = torch.tensor([0, 1, 63, 64, 127, 128, 255, 256, 300, 383])
    ref = ops.gemm_w8a16_fp32(xl[rows], q, s)
    assert ((y[rows].double() - ref).abs() <= 1e-2 * ref.abs().amax(1, keepdim=True)).all()


@pytest.mark.parametrize("M", [17, 32, 40, 64, 100, 128, 250, 256, 400, 512])
@pytest.mark.parametrize("KN", [(256, 128), (192, 256), (1024, 384), (4096, 4096)])
def test_stream_k_tensor_core_kernel(KN, M):
    """16 < M <= 512 goes to the stream-K tcgen05 kernel: token tiles of 32 / 64 / 128 with ragged tails,
    strips that end inside a CTA's range (small K) and ranges shorter than a strip (large K)."""
    x, q, s = _case(KN[0], KN[1], M, seed=M + KN[1])
    _check(_run(x, q, s), x, q, s)
    res = torch.randn(M, KN[1], generator=torch.Generator().manual_seed(1)).half()
    y = _run(x, q, s, residual=res)
    # (two runs may round differently in the last fp16 bit: the order of the fp32 atomic adds is not fixed)
    assert torch.allclose(y.float(), ops.add_residual(_run(x, q, s), res).float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M", [24, 64])
def test_stream_k_accumulate_two_weights_exact_sums(M):
    """eet_gemm_w8a16_accum above 16 rows, gate and up in one launch: integer-valued inputs make the fp32
    sums exact, so they must EQUAL the integer product whatever the order of the atomic adds."""
    from eet_b200 import EET
    K, N = 512, 640
    gen = torch.Generator().manual_seed(M)
    x = torch.randint(-4, 5, (M, K), generator=gen).half()
    q1 = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    q2 = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    sums1 = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    sums2 = torch.zeros_like(sums1)
    p1, p2 = EET.preprocess_weights(q1).cuda(), EET.preprocess_weights(q2).cuda()
    for rep in (1, 2):   # the second launch adds on top of the first
        EET.gemm_w8a16_accum(x.cuda(), p1, sums1, p2, sums2)
        assert torch.equal(sums1.cpu().double(), rep * (x.double() @ q1.double()))
        assert torch.equal(sums2.cpu().double(), rep * (x.double() @ q2.double()))
    from eet_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("KNM", [(512, 384, 600), (1024, 640, 1000), (256, 4096, 2048), (4096, 4096, 1024),
                                 (4096, 11008, 300), (4096, 11008, 512), (128, 14208, 512)])
def test_large_m_tensor_core_kernels(KNM):
    """M > 512: the 256 x 256 tile kernel when N is a multiple of 256 and there are enough tiles, else the
    128-channel x 256-token kernel; ragged last token tile, residual epilogue.  The two 4096 x 11008 cases are
    large enough for the stream-K kernel to choose its 256-token tiles (single accumulator buffer); 128 x 14208
    gives every CTA of that kernel three one-unit strips, i.e. a third accumulation that has to wait for the
    epilogue of the first."""
    K, N, M = KNM
    x, q, s = _case(K, N, M, seed=K + N + M)
    y = _run(x, q, s)
    rows = torch.tensor([r for r in (0, 1, 127, 128, 255, 256, 511, 512, M - 2, M - 1) if r < M])
    ref = ops.gemm_w8a16_fp32(x[rows], q, s)
    assert ((y[rows].double() - ref).abs() <= 1e-2 * ref.abs().amax(1, keepdim=True)).all()
    exact = ops.gemm_w8a16(x[rows], q, s, exact=True).double()
    assert ((y[rows].double() - exact).abs() <= 2e-3 * ref.abs().amax(1, keepdim=True) + 1e-3).all()
    res = torch.randn(M, N, generator=torch.Generator().manual_seed(2)).half()
    yr = _run(x, q, s, residual=res)
    # (M <= 512 sums with atomics: two runs may differ in the last fp16 bit)
    assert torch.allclose(yr[rows].float(), ops.add_residual(y[rows], res[rows]).float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M", [64, 256, 1024, 4096])
@pytest.mark.parametrize("KN", [(4096, 4096), (4096, 11008), (11008, 4096)])
def test_llama7b_projection_shapes_across_the_kernel_regimes(KN, M):
    """configs[1] at its large-M points: the three LLaMA-7B projection shapes at M = 64 and 256 (stream-K
    tcgen05 kernel), 1024 and 4096 (large-tile tcgen05 kernels; K = 11008 walks 172 k-blocks, so every
    shared-memory ring wraps dozens of times).  Sampled rows - every 256-token tile of the output is hit -
    against the fp64 dequantize-then-matmul on the CPU, and ALL elements against an fp32 matmul of the same
    dequantized weights run by torch on the GPU (a consistency check of the rows the CPU did not sample)."""
    K, N = KN
    gen = torch.Generator().manual_seed(K + N + M)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 3e-4 + 1e-4).half()
    x = torch.randn(M, K, generator=gen).half()
    y = _run(x, q, s)
    rows = sorted({r for t in range(0, M, 256) for r in (t, t + 127, t + 255) if r < M} | {1, M - 2, M - 1})
    rows = torch.tensor(rows[:: max(1, len(rows) // 24)] + [M - 1])
    ref = ops.gemm_w8a16_fp32(x[rows], q, s)
    tol = 1e-2 * ref.abs().amax(1, keepdim=True)
    assert ((y[rows].double() - ref).abs() <= tol).all()
    w = (q.cuda().float() * s.cuda().float()[None])
    full = x.cuda().float() @ w                       # fp32 (TF32 is off by default for matmul): checker only
    err = (y.cuda().float() - full).abs()
    assert bool((err <= 1e-2 * full.abs().amax(1, keepdim=True)).all()), float(err.max())
    res = torch.randn(M, N, generator=gen).half()
    yr = _run(x, q, s, residual=res)
    assert torch.allclose(yr[rows].float(), ops.add_residual(y[rows], res[rows]).float(), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("KNM", [(1088, 6144, 300), (832, 8192, 130), (2048, 2560, 700), (4096, 4096, 300), (4096, 4096, 512),
                                 (4096, 11008, 200), (11008, 4096, 700)])
def test_split_k_cluster_tiles(KNM):
    """Shapes with fewer 256 x 256 tiles than SMs (24 to 48 of them): the k-blocks of a tile are split over a
    cluster of 2, 3 or 4 CTAs whose partial accumulators meet through distributed shared memory.  Uneven k-splits
    (17 and 13 k-blocks), a ragged last token tile (blocks past M are neither sent nor reduced), with and without
    the residual.  Every element against an fp32 matmul of
    the dequantized weights run by torch on the GPU (checker only), sampled rows against the fp64 oracle."""
    K, N, M = KNM
    gen = torch.Generator().manual_seed(K + N + M)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 3e-4 + 1e-4).half()
    x = torch.randn(M, K, generator=gen).half()
    y = _run(x, q, s)
    rows = torch.tensor(sorted({0, 1, 31, 32, 63, 64, 95, 127, 128, 129, M // 2, M - 2, M - 1} & set(range(M))))
    ref = ops.gemm_w8a16_fp32(x[rows], q, s)
    assert ((y[rows].double() - ref).abs() <= 1e-2 * ref.abs().amax(1, keepdim=True)).all()
    exact = ops.gemm_w8a16(x[rows], q, s, exact=True).double()
    assert ((y[rows].double() - exact).abs() <= 2e-3 * ref.abs().amax(1, keepdim=True) + 1e-3).all()
    full = x.cuda().float() @ (q.cuda().float() * s.cuda().float()[None])
    err = (y.cuda().float() - full).abs()
    assert bool((err <= 1e-2 * full.abs().amax(1, keepdim=True)).all()), float(err.max())
    res = torch.randn(M, N, generator=gen).half()
    yr = _run(x, q, s, residual=res)
    # the partials are added in rank order: the residual run repeats the plain run bit for bit before the add
    assert torch.equal(yr, ops.add_residual(y, res))


@pytest.mark.parametrize("KNM", [(256, 4096, 2560), (192, 2560, 4000), (1088, 2816, 3400), (4096, 12288, 2304)])
def test_persistent_tiles_in_waves(KNM):
    """More 256 x 256 tiles than SMs, and no multiple of them: persistent CTAs take tiles i, i + G, ... and run
    two to four of them back to back on the same rings, barriers and tensor memory (short and odd k-loops of 4, 3
    and 17 k-blocks, a ragged last token tile, the fused QKV shape of LLaMA-7B); with and without the residual, and
    twice in a row (the kernel is deterministic).  Every element against an fp32 matmul of the dequantized weights
    run by torch on the GPU (checker only), sampled rows against the fp64 oracle."""
    K, N, M = KNM
    gen = torch.Generator().manual_seed(K + N + M)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 3e-4 + 1e-4).half()
    x = torch.randn(M, K, generator=gen).half()
    y = _run(x, q, s)
    rows = torch.tensor(sorted({0, 1, 255, 256, 257, 511, 1023, 1024, M // 2, M - 257, M - 2, M - 1} & set(range(M))))
    ref = ops.gemm_w8a16_fp32(x[rows], q, s)
    assert ((y[rows].double() - ref).abs() <= 1e-2 * ref.abs().amax(1, keepdim=True)).all()
    full = x.cuda().float() @ (q.cuda().float() * s.cuda().float()[None])
    err = (y.cuda().float() - full).abs()
    assert bool((err <= 1e-2 * full.abs().amax(1, keepdim=True)).all()), float(err.max())
    del full, err
    assert torch.equal(_run(x, q, s), y)
    res = torch.randn(M, N, generator=gen).half()
    yr = _run(x, q, s, residual=res)
    assert torch.equal(yr, ops.add_residual(y, res))


@pytest.mark.parametrize("KNM", [(256, 384, 8), (256, 384, 100), (1024, 640, 1000), (4096, 4096, 512), (256, 4096, 2560),
                                 (1088, 2816, 3400)])
def test_gated_activation_epilogue(KNM):
    """Epilogue 2: the GEMM is the up projection of a gated FFN and applies gated_silu(gate, .) to its own output,
    in every kernel regime (skinny and stream-K kernels through the finalize launch, the 128 x 256 and 256 x 256
    tensor-core kernels - persistent, cluster split, second launch for the last wave - in their epilogues), in
    place (the output buffer holds the gate values) and out of place.  Expected: the oracle's gated_silu
    (activation_kernel.cu:106-124) of the gate and of this library's plain GEMM output."""
    from eet_b200 import EET, _lib
    K, N, M = KNM
    gen = torch.Generator().manual_seed(K + N + M)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 3e-4 + 1e-4).half()
    x = torch.randn(M, K, generator=gen).half()
    gate = (torch.randn(M, N, generator=gen) * 2).half()
    packed = EET.preprocess_weights(q).cuda()
    xc, sc = x.cuda(), s.cuda()
    up = EET.gemm_w8a16(xc, packed, sc)
    want = ops.gated_silu(gate, up.cpu())
    got = EET.gemm_w8a16(xc, packed, sc, gate=gate.cuda())
    buf = gate.cuda().clone()
    got_inplace = EET.gemm_w8a16(xc, packed, sc, out=buf, gate=buf)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    # (the kernels that sum with atomics may round `up` differently in the last fp16 bit from run to run, and the
    # device's expf may differ from the host's in the last bit before its rounding to fp16)
    tol = dict(rtol=4e-3, atol=4e-3)
    assert torch.allclose(got.cpu().float(), want.float(), **tol)
    assert torch.allclose(got_inplace.cpu().float(), want.float(), **tol)
    assert got_inplace.data_ptr() == buf.data_ptr()
