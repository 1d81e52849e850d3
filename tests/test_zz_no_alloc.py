"""eet_gemm_w8a16_noalloc, the entry point for callers that may not allocate device memory (a server whose
HBM is one pre-reserved arena, a plugin in a foreign process, a decode loop that cannot afford cudaMalloc's
device-wide stall): through the C ABI, twice in a row, against the ordinary entry point.

Collected last on purpose (file name), so that a run stopping at the first failure has already run every
other test; it passes in a fresh process on its own as well."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(M, K, N, seed):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randint(-128, 128, (K, N), generator=gen, dtype=torch.int8)
    s = (torch.rand(N, generator=gen) * 1e-3 + 1e-4).half()
    x = torch.randn(M, K, generator=gen).half()
    r = torch.randn(M, N, generator=gen).half()
    return x, q, s, r


def test_noalloc_matches_the_scratch_taking_entry_point_twice_in_a_row():
    from eet_b200 import EET
    from eet_b200._lib import check, lib
    stream = torch.cuda.current_stream().cuda_stream
    for call, (M, K, N, with_res) in enumerate([(8, 1024, 2048, False), (16, 512, 4096, True)]):
        x, q, s, r = _inputs(M, K, N, seed=40 + call)
        packed = EET.preprocess_weights(q).cuda()
        xc, sc, rc = x.cuda(), s.cuda(), r.cuda()
        want = EET.gemm_w8a16(xc, packed, sc, residual=rc if with_res else None)
        got = torch.empty(M, N, dtype=torch.float16, device="cuda")
        mem_before = torch.cuda.memory_allocated()
        check(lib.eet_gemm_w8a16_noalloc(xc.data_ptr(), packed.data_ptr(), sc.data_ptr(), got.data_ptr(), M, N, K,
                                         rc.data_ptr() if with_res else None, int(with_res), stream))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == mem_before
        # same kernels, same arithmetic; split-K partial sums may meet in a different order: one fp16 ulp
        assert torch.allclose(got.float(), want.float(), rtol=2e-3, atol=2e-3)
        ref = x.double() @ (q.double() * s.double()[None]) + (r.double() if with_res else 0)
        assert ((got.cpu().double() - ref).abs() <= 1e-2 * ref.abs().amax(1, keepdim=True)).all()


def test_noalloc_rejects_what_does_not_fit():
    from eet_b200._lib import lib
    x = torch.zeros(32, 64, dtype=torch.float16, device="cuda")
    w = torch.zeros(64, 64, dtype=torch.int8, device="cuda")
    s = torch.zeros(64, dtype=torch.float16, device="cuda")
    c = torch.zeros(32, 64, dtype=torch.float16, device="cuda")
    rc = lib.eet_gemm_w8a16_noalloc(x.data_ptr(), w.data_ptr(), s.data_ptr(), c.data_ptr(), 32, 64, 64, None, 0, None)
    assert rc != 0 and b"exceeds 16" in lib.eet_last_error()
    rc = lib.eet_gemm_w8a16_noalloc(x.data_ptr(), w.data_ptr(), s.data_ptr(), c.data_ptr(), 16, 65536, 64, None, 0, None)
    assert rc != 0 and b"built-in scratch" in lib.eet_last_error()
