"""The many-row GEMM through the C ABI against the fp64 matmul of the dequantised operands (protocol of the
reference's engine/tests/test_gemm.py:25-110: residual in place, plain, C apart from D, bf16 == rounded fp32,
gate | up with the fused SiLU*mul epilogue)."""

import numpy as np
import pytest
import torch

from helpers import DEV, bf16_to_f32, dev, fp4_operand, rel_err, swizzled_dev, workspace
from oracle import nvfp4_oracle as O
from q27b200 import layouts
from q27b200.q27lib import call

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M", [1, 5, 128, 300, 2048])
@pytest.mark.parametrize("N,K", [(5120, 17408), (17408, 5120), (384, 5120), (128, 128)])
def test_gemm_fp4(M, N, K):
    rng = np.random.RandomState(M + N + K)
    a, asf, adq = fp4_operand(M, K, rng)
    b, bsf, bdq = fp4_operand(N, K, rng)
    ad, bd, asw, bsw = dev(a), dev(b), swizzled_dev(asf), swizzled_dev(bsf)
    alpha = 0.37
    prod = alpha * (torch.from_numpy(adq) @ torch.from_numpy(bdq).T).numpy()
    c = torch.randn(M, N, device=DEV)
    d = c.clone()
    call("q27t_gemm_fp4", M, N, K, ad, asw, bd, bsw, alpha, d, 1.0, d)  # residual in place
    assert rel_err(d.cpu().numpy(), prod + c.cpu().numpy().astype(np.float64)) < 1e-5
    d.fill_(float("nan"))
    call("q27t_gemm_fp4", M, N, K, ad, asw, bd, bsw, alpha, None, 0.0, d)
    assert rel_err(d.cpu().numpy(), prod) < 1e-5
    assert O.within_tolerance(d.cpu().numpy(), prod).all()
    d2 = torch.empty_like(d)
    call("q27t_gemm_fp4", M, N, K, ad, asw, bd, bsw, alpha, c, 0.5, d2)  # C apart from D
    assert rel_err(d2.cpu().numpy(), prod + 0.5 * c.cpu().numpy().astype(np.float64)) < 1e-5
    db = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    call("q27t_gemm_fp4_bf16", M, N, K, ad, asw, bd, bsw, alpha, db)
    assert torch.equal(db, d.bfloat16())
    if M <= 128:  # the weight-streaming kernel computes the same products in the same K order per tile
        ws = workspace()
        ds = torch.empty_like(d)
        call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, alpha, None, 0.0, ds, ws, ws.numel())
        assert rel_err(ds.cpu().numpy(), d.cpu().numpy()) < 5e-6


def test_gemm_fp4_empty():
    call("q27t_gemm_fp4", 0, 128, 128, None, None, None, None, 1.0, None, 0.0, None)


@pytest.mark.parametrize("M", [1, 77, 300, 2048])
@pytest.mark.parametrize("I,K", [(384, 5120), (17408, 5120)])
def test_gemm_fp4_glu_bf16(M, I, K):
    rng = np.random.RandomState(M + I)
    a, asf, adq = fp4_operand(M, K, rng)
    w, wsf, wdq = fp4_operand(2 * I, K, rng)  # gate rows, then up rows
    wi, wsfi = layouts.interleave_glu(w), layouts.interleave_glu(wsf)
    ad, asw, wid, wsw = dev(a), swizzled_dev(asf), dev(wi), swizzled_dev(wsfi)
    ag, au = 0.013, 0.021
    full = (torch.from_numpy(adq) @ torch.from_numpy(wdq).T).numpy()
    ref = O.silu_mul(ag * full[:, :I], au * full[:, I:])
    d = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    call("q27t_gemm_fp4_glu_bf16", M, I, K, ad, asw, wid, wsw, ag, au, d)
    out = bf16_to_f32(d)
    assert O.within_tolerance_bf16(out, ref).all()
    assert rel_err(out, ref) < 3e-3
    # the interleaved plain GEMM reproduces the row-major one column for column (the loader's path)
    gu = torch.empty(M, 2 * I, device=DEV)
    call("q27t_gemm_fp4", M, 2 * I, K, ad, asw, wid, wsw, 1.0, None, 0.0, gu)
    rows = layouts.glu_rows(I)
    assert rel_err(gu.cpu().numpy()[:, rows], full) < 1e-5
    if M <= 128:
        ws = workspace()
        ds = torch.zeros_like(d)
        call("q27t_skinny_fp4_glu_bf16", M, I, K, ad, asw, wid, wsw, ag, au, ds, ws, ws.numel())
        assert (ds != d).float().mean().item() < 1e-2 and rel_err(bf16_to_f32(ds), out) < 1e-3
