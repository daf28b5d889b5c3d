"""The many-row GEMM through the C ABI against the fp64 matmul of the dequantised operands (protocol of the
reference's engine/tests/test_gemm.py:25-110: residual in place, plain, C apart from D, bf16 == rounded fp32,
gate | up with the fused SiLU*mul epilogue)."""

import os

import numpy as np
import pytest
import torch

from helpers import DEV, bf16_to_f32, dev, fp4_operand, rel_err, swizzled_dev, workspace
from oracle import nvfp4_oracle as O
from q27b200 import layouts
from q27b200.q27lib import LIB_PATH, call, lib

pytestmark = pytest.mark.gpu


CASES = [(M, N, K) for N, K in [(5120, 17408), (17408, 5120), (384, 5120), (128, 128)] for M in [1, 5, 128, 300, 2048]]
CASES += [(M, N, K) for N, K in [(1024, 5120), (128, 5120), (34816, 5120)] for M in [300, 4096]]


@pytest.mark.parametrize("M,N,K", CASES)
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


def _nibbles(q):
    return torch.stack([q & 15, q >> 4], -1)


def _code_mismatch(q, q_ref):
    """Share of E2M1 codes that differ, the two zero codes taken as equal (its sign is unpinned in the reference)."""
    a, b = _nibbles(q), _nibbles(q_ref)
    a, b = torch.where(a == 8, torch.zeros_like(a), a), torch.where(b == 8, torch.zeros_like(b), b)
    return (a != b).float().mean().item()


@pytest.mark.parametrize("M", [1, 77, 300, 2048])
@pytest.mark.parametrize("I,K", [(384, 5120), (17408, 5120)])
def test_gemm_fp4_glu_nvfp4_out(M, I, K):
    """gate | up GEMM (interleaved weights) with silu(gate) * up quantised to NVFP4 in the epilogue, against the
    separate path (fp32 GEMM, then silu_mul_quant_fp4_glu) and against the CPU oracle. The fused epilogue uses the
    fast exponential and reciprocal and its own accumulation order, so a value on a rounding boundary may land in
    the next code: the reference's bounds apply (engine/tests/test_gemm.py:59-96: < 1e-3 of the scales, < 2e-3 of
    the codes)."""
    rng = np.random.RandomState(M + I + 1)
    a, asf, adq = fp4_operand(M, K, rng)
    w, wsf, wdq = fp4_operand(2 * I, K, rng)  # gate rows, then up rows
    wi, wsfi = layouts.interleave_glu(w), layouts.interleave_glu(wsf)
    ad, asw, wid, wsw = dev(a), swizzled_dev(asf), dev(wi), swizzled_dev(wsfi)
    ag, au, out_scale = 0.013, 0.021, 0.05
    sfb = lib().q27t_sf_bytes(M, I // 16)

    def out():
        return torch.zeros(M, I // 2, dtype=torch.uint8, device=DEV), torch.zeros(sfb, dtype=torch.uint8, device=DEV)

    # the separate path on this library's own kernels
    gui = torch.empty(M, 2 * I, device=DEV)
    call("q27t_gemm_fp4", M, 2 * I, K, ad, asw, wid, wsw, 1.0, None, 0.0, gui)
    q_ref, sf_ref = out()
    call("q27t_silu_mul_quant_fp4_glu", gui, M, I, ag, au, out_scale, q_ref, sf_ref)
    # fused
    q, sf = out()
    call("q27t_gemm_fp4_glu", M, I, K, ad, asw, wid, wsw, ag, au, out_scale, q, sf)
    sf_u, sf_ref_u = (layouts.unswizzle(t.cpu().numpy(), M, I // 16) for t in (sf, sf_ref))
    assert (sf_u != sf_ref_u).mean() < 1e-3
    assert _code_mismatch(q, q_ref) < 2e-3
    # rows past M inside the last scale atom stay untouched (zero here)
    touched = np.zeros(sfb, dtype=bool)
    touched[layouts.sf_index(M, I // 16).reshape(-1)] = True
    assert not sf.cpu().numpy()[~touched].any()
    # against the oracle: fp64 GEMM of the dequantised operands, SiLU*mul, then the activation quantiser
    full = (torch.from_numpy(adq) @ torch.from_numpy(wdq).T).numpy()
    h = O.silu_mul(ag * full[:, :I], au * full[:, I:]).astype(np.float32)
    codes, sfo = O.quant_act_codes(h, out_scale)
    assert (sf_u != sfo).mean() < 1e-3
    assert _code_mismatch(q, dev(codes)) < 2e-3


@pytest.mark.parametrize("M", [129, 300, 1000])
def test_many_row_kernels_agree_bit_for_bit(M, monkeypatch):
    """The many-row kernels (CTA pairs with staged whole-row stores, 128 x 256 tiles, 128 x 128 tiles and, where the
    optional single-GPU library is present and the token tiles pair up, clusters of four) run the
    same accumulation chain per output and the same roundings in their epilogues: identical bits for the fp32 output
    with and without a residual, the bf16 output and the SiLU*mul output (Q27B_MANY is read at every launch)."""
    N, K = 512, 1024
    rng = np.random.RandomState(M)
    a, asf, _ = fp4_operand(M, K, rng)
    b, bsf, _ = fp4_operand(N, K, rng)
    ad, bd, asw, bsw = dev(a), dev(b), swizzled_dev(asf), swizzled_dev(bsf)
    c = torch.randn(M, N, device=DEV)
    got = {}
    quad = os.path.exists(os.path.join(os.path.dirname(LIB_PATH), "libq27b200_quad.so")) and ((M + 255) // 256) % 2 == 0
    for kind in ("pairs", "wide", "narrow") + (("quad",) if quad else ()):
        monkeypatch.setenv("Q27B_MANY", kind)
        d = torch.full((M, N), float("nan"), device=DEV)
        call("q27t_gemm_fp4", M, N, K, ad, asw, bd, bsw, 0.37, None, 0.0, d)
        r = c.clone()
        call("q27t_gemm_fp4", M, N, K, ad, asw, bd, bsw, 0.37, r, 0.75, r)
        h = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        call("q27t_gemm_fp4_bf16", M, N, K, ad, asw, bd, bsw, 0.37, h)
        g = torch.zeros(M, N // 2, dtype=torch.bfloat16, device=DEV)
        call("q27t_gemm_fp4_glu_bf16", M, N // 2, K, ad, asw, bd, bsw, 0.013, 0.021, g)
        got[kind] = (d, r, h, g)
    for kind in [k for k in got if k != "pairs"]:
        for x, y, what in zip(got["pairs"], got[kind], ("fp32", "fp32 + residual", "bf16", "SiLU*mul")):
            assert torch.equal(x, y), f"{what}: pairs vs {kind} at M={M}"
