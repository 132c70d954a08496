"""Each tensor-core primitive of the attention kernels, proven in isolation
against an FP32 matmul of the decoded operands (the reference validates its
primitives the same way: validate_e5m2_dout_mixed_mma_microgate_20260831.py:47-66).
Products of FP4/FP8 operands are exact in FP32; only the accumulation order
differs, hence rel-L2 <= 1e-5."""

import pytest
import torch

import fa4b_oracle as O
from fa4b import microgate

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-5


def _fp8(shape, seed, kind=torch.float8_e4m3fn):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g).to(kind)


@pytest.mark.parametrize("K", [64, 128])
def test_nvfp4_block_scaled(K):
    g = torch.Generator().manual_seed(K)
    a = O.nvfp4_quantize(torch.randn(128, K, generator=g).bfloat16())
    b = O.nvfp4_quantize((torch.randn(128, K, generator=g) * 3).bfloat16())
    want = (a.dequant() / a.global_scale) @ (b.dequant() / b.global_scale).t()
    got = microgate.run("nvfp4", K, a.codes.to(DEV), b.codes.to(DEV), a.pages().to(DEV), b.pages().to(DEV))
    assert O.rel_l2(want, got.cpu()) < TOL


def test_mxfp4_block_scaled():
    g = torch.Generator().manual_seed(5)
    a = O.mxfp4_quantize(torch.randn(128, 128, generator=g).bfloat16())
    b = O.mxfp4_quantize((torch.randn(128, 128, generator=g) * 5).bfloat16())
    # the tensor core applies 2^(e-127) to the codes; the oracle's decode also divides by 6 per operand
    want = (a.dequant() @ b.dequant().t()) * 36.0
    got = microgate.run("mxfp4", 128, a.codes.to(DEV), b.codes.to(DEV), a.pages().to(DEV), b.pages().to(DEV))
    assert O.rel_l2(want, got.cpu()) < TOL


@pytest.mark.parametrize("kind,K", [("e4m3_kk", 32), ("e4m3_kk", 64), ("e4m3_kk", 128), ("e4m3_kk_tma", 128),
                                    ("e4m3_kk_tma", 64), ("e4m3_e5m2_kk", 128)])
def test_fp8_k_major(kind, K):
    a = _fp8((128, K), 1)
    b = _fp8((128, K), 2, torch.float8_e5m2 if kind == "e4m3_e5m2_kk" else torch.float8_e4m3fn)
    want = a.float() @ b.float().t()
    got = microgate.run(kind, K, a.to(DEV), b.to(DEV))
    assert O.rel_l2(want, got.cpu()) < TOL


@pytest.mark.parametrize("K", [32, 128])
def test_fp8_mn_major_b(K):
    a, b = _fp8((128, K), 3), _fp8((K, 128), 4)  # b is [K, N]
    got = microgate.run("e4m3_k_mn", K, a.to(DEV), b.to(DEV))
    assert O.rel_l2(a.float() @ b.float(), got.cpu()) < TOL


@pytest.mark.parametrize("K", [32, 128])
def test_fp8_mn_major_both(K):
    a, b = _fp8((K, 128), 5), _fp8((K, 128), 6)  # a is [K, M], b is [K, N]
    got = microgate.run("e4m3_mn_mn", K, a.to(DEV), b.to(DEV))
    assert O.rel_l2(a.float().t() @ b.float(), got.cpu()) < TOL


@pytest.mark.parametrize("K", [32, 128])
def test_fp8_a_from_tmem(K):
    a, b = _fp8((128, K), 7), _fp8((K, 128), 8)
    got = microgate.run("e4m3_ts_mn", K, a.to(DEV), b.to(DEV))
    assert O.rel_l2(a.float() @ b.float(), got.cpu()) < TOL


def test_tensor_peak_reports_a_plausible_rate():
    """All-SM MMA-only run: FP8 dense should land between the cuBLAS bf16 rate and the nominal 4.5 PF/s,
    block-scaled FP4 above FP8."""
    from fa4b import microgate
    fp8 = microgate.tensor_peak("fp8", iters=4096)
    fp4 = microgate.tensor_peak("nvfp4", iters=4096)
    assert 1000.0 < fp8 < 5200.0, fp8
    assert fp8 < fp4 < 10400.0, (fp8, fp4)


def test_a_wait_that_runs_out_reports_timeout_and_leaves_the_context_usable():
    """The give-up path of the kernels' bounded waits (abort flag, status record, orderly return), made to run out on
    an unarmed barrier with a budget of a million cycles and nothing asynchronous in flight; then a normal launch."""
    from fa4b import _lib

    status = microgate.wait_selftest(1_000_000)
    assert status[0].item() == 1 and status[1].item() in (900, 901) and status[4:7].tolist() == [0, 0, 1]
    assert "site 90" in _lib.lib().fa4b_last_error().decode()
    with pytest.raises(TimeoutError):
        _lib.check(5, "fa4b_wait_selftest")
    a, b = _fp8((128, 64), 1), _fp8((128, 64), 2)
    got = microgate.run("e4m3_kk", 64, a.to(DEV), b.to(DEV))
    assert O.rel_l2(a.float() @ b.float().t(), got.cpu()) < TOL
