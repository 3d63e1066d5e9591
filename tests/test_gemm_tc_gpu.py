"""The tcgen05 tensor-core product alone, against a float64 product: tile
edges in M, N and K, every epilogue, and that a row does not depend on M."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P
from test_kernels_gpu import dev, rt

pytestmark = pytest.mark.gpu
DT = torch.bfloat16


@pytest.fixture(autouse=True)
def _no_timeouts():
    yield
    from kappai_b200.ops import kernels as Kn
    assert Kn.tc_status() == 0, "a bounded wait of the tcgen05 kernel gave up"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (65, 8, 8), (129, 130, 72), (300, 331, 120), (2048, 2048, 2048),
                                   (257, 6144, 2048), (130, 2048, 5632), (1000, 96, 200), (512, 1000, 4096),
                                   # few rows: short A boxes, and tiles of 64 columns while W has few rows
                                   (1, 200, 72), (8, 6144, 2048), (17, 2048, 5632), (64, 331, 120), (100, 20000, 256),
                                   # 17 to 128 rows, the products of a decode step: cut along K, clusters of 3 to 8 CTAs
                                   (64, 2048, 5632), (24, 6144, 2048), (128, 2048, 2048), (96, 3072, 2048), (33, 1024, 4608),
                                   (48, 2560, 10240), (17, 9216, 1024)])
def test_gemm_tc_against_plain(M, N, K):
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(60)
    a = rt(rng.standard_normal((M, K)), DT)
    w = rt(rng.standard_normal((N, K)) / math.sqrt(K), DT)
    b = rng.standard_normal(N).astype(np.float32)
    A, W = dev(a, DT), dev(w, DT)
    assert Kn.tc_ok(A, W)
    ref = P.linear(a, w, b.astype(np.float64))
    out = Kn.gemm_tc(A, W, torch.full((M, N), float("nan"), device="cuda"), dev(b))
    np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=2e-5, atol=3e-5 * math.sqrt(K))
    out16 = Kn.gemm_tc(A, W, torch.empty((M, N), dtype=DT, device="cuda"), dev(b))
    np.testing.assert_allclose(out16.cpu().double().numpy(), ref, rtol=1e-2, atol=2e-2)
    res = rng.standard_normal((M, N)).astype(np.float32)
    acc = dev(res).clone()
    Kn.gemm_tc(A, W, acc, None, accumulate=True)
    np.testing.assert_allclose(acc.cpu().double().numpy(), res + P.linear(a, w), rtol=2e-5, atol=3e-5 * math.sqrt(K))


@pytest.mark.parametrize("M", [17, 40, 64, 100, 128])
def test_gemm_tc_split_over_k(M):
    """17 to 128 rows: the product is cut along K, the CTAs of a tile (a cluster) add the parts in a fixed order.
    Every epilogue against the plain product; twice in a row gives the same bits (the order of the parts does not
    depend on who arrives when)."""
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(63)
    K, N, ff = 4096 + 64, 1000, 1024
    a = rt(rng.standard_normal((M, K)), DT)
    w = rt(rng.standard_normal((N, K)) / math.sqrt(K), DT)
    b = rng.standard_normal(N).astype(np.float32)
    A, W = dev(a, DT), dev(w, DT)
    ref = P.linear(a, w, b.astype(np.float64))
    out = Kn.gemm_tc(A, W, torch.full((M, N), float("nan"), device="cuda"), dev(b))
    np.testing.assert_allclose(out.cpu().double().numpy(), ref, rtol=2e-5, atol=3e-5 * math.sqrt(K))
    unsplit = Kn.gemm_tc(A, W, torch.full((M, N), float("nan"), device="cuda"), dev(b), split=False)
    assert not torch.equal(out, unsplit), "the split did not run (same bits as the unsplit product)"
    again = Kn.gemm_tc(A, W, torch.full((M, N), float("nan"), device="cuda"), dev(b))
    assert torch.equal(out, again)
    res = rng.standard_normal((M, N)).astype(np.float32)
    acc = dev(res).clone()
    Kn.gemm_tc(A, W, acc, None, accumulate=True)
    np.testing.assert_allclose(acc.cpu().double().numpy(), res + P.linear(a, w), rtol=2e-5, atol=3e-5 * math.sqrt(K))
    wgu = rt(rng.standard_normal((2 * ff, K)) * (2.0 / math.sqrt(K)), DT)
    gu = rt(P.linear(a, wgu), DT)
    act = Kn.gemm_tc(A, dev(wgu, DT), torch.empty((M, ff), dtype=DT, device="cuda"), None, swiglu=True)
    want = P.swiglu(gu[:, :ff], gu[:, ff:])
    assert np.all(np.abs(act.cpu().double().numpy() - want) <= 2e-2 * np.abs(want) + 2e-2)
    assert Kn.tc_status() == 0


def test_gemm_tc_rows_do_not_depend_on_m():
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(61)
    K, N = 520, 300
    a = dev(rt(rng.standard_normal((700, K)), DT), DT)
    w = dev(rt(rng.standard_normal((N, K)) / 20, DT), DT)
    full = Kn.gemm_tc(a, w, torch.empty((700, N), device="cuda"), split=False)
    for lo, hi in ((0, 65), (130, 400), (699, 700), (5, 133)):
        part = Kn.gemm_tc(a[lo:hi], w, torch.empty((hi - lo, N), device="cuda"), split=False)
        assert torch.equal(part, full[lo:hi]), (lo, hi)


@pytest.mark.parametrize("M,ff,K", [(128, 128, 64), (200, 100, 64), (2048, 5632, 2048), (70, 333, 96), (9, 5632, 2048),
                                    (64, 100, 64), (33, 15000, 128)])
def test_gemm_tc_swiglu(M, ff, K):
    from kappai_b200.ops import kernels as Kn
    rng = np.random.default_rng(62)
    a = rt(rng.standard_normal((M, K)), DT)
    w = rt(rng.standard_normal((2 * ff, K)) * (2.0 / math.sqrt(K)), DT)
    b = rng.standard_normal(2 * ff).astype(np.float32) * 0.1
    for bias in (b, None):
        gu = rt(P.linear(a, w, None if bias is None else bias.astype(np.float64)), DT)
        ref = P.swiglu(gu[:, :ff], gu[:, ff:])
        out = Kn.gemm_tc(dev(a, DT), dev(w, DT), torch.empty((M, ff), dtype=DT, device="cuda"),
                         None if bias is None else dev(bias), swiglu=True)
        got = out.cpu().double().numpy()
        assert np.all(np.abs(got - ref) <= 2e-2 * np.abs(ref) + 2e-2)


def test_linear_picks_the_tensor_core_kernel_for_many_rows():
    from kappai_b200.ops import kernels as Kn
    from kappai_b200.ops.linear import linear
    a = torch.randn((200, 256), device="cuda").to(DT)
    w = torch.randn((64, 256), device="cuda").to(DT)
    count = lambda: {k: Kn.LAUNCHES_BY.get(k, 0) for k in ("gemm_tc", "gemm_nt_simt", "gemm_stream", "gemm_skinny")}
    before = count()
    out = linear(a, w, out_dtype=torch.float32)
    after = count()
    assert after["gemm_tc"] == before["gemm_tc"] + 1 and all(after[k] == before[k] for k in after if k != "gemm_tc")
    ref = Kn.gemm_nt_simt(a, w, torch.empty((200, 64), device="cuda"))
    assert (out - ref).abs().max().item() < 1e-3
    # K % 8 != 0 is not for TMA: the general kernel takes it, and its result is right too
    odd = torch.randn((200, 100), device="cuda").to(DT)
    w_odd = torch.randn((64, 100), device="cuda").to(DT)
    before = count()
    out = linear(odd, w_odd, out_dtype=torch.float32)
    after = count()
    assert after["gemm_nt_simt"] == before["gemm_nt_simt"] + 1 and after["gemm_tc"] == before["gemm_tc"]
    assert (out - odd.float() @ w_odd.float().t()).abs().max().item() < 1e-2
    # few rows: the weight-streaming kernels
    before = count()
    linear(a[:8], w)
    after = count()
    assert after["gemm_stream"] + after["gemm_skinny"] == before["gemm_stream"] + before["gemm_skinny"] + 1
    assert Kn.tc_status() == 0
