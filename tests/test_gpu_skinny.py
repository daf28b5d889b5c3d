"""The weight-streaming GEMM (1 <= M <= 128) through the C ABI against the fp64 matmul of the dequantised operands
(protocol of the reference's engine/tests/test_skinny.py:22-147: random code bytes, rel_err < 1e-5, run twice on
one workspace, rows bit-identical whatever M, shapes interleaved on a shared workspace, determinism)."""

import ctypes

import numpy as np
import pytest
import torch

from helpers import DEV, bf16_to_f32, dev, fp4_operand, rel_err, swizzled_dev, workspace
from oracle import nvfp4_oracle as O
from q27b200 import layouts
from q27b200.q27lib import call, lib

pytestmark = pytest.mark.gpu
WS = 48 << 20

_weights = {}


def weight(N, K):
    """One random weight operand per shape, kept on the device (codes, swizzled scales) and as fp32 values."""
    if (N, K) not in _weights:
        rng = np.random.RandomState(N + K)
        b, bsf, bdq = fp4_operand(N, K, rng)
        _weights[(N, K)] = (dev(b), swizzled_dev(bsf), bdq.astype(np.float32), b, bsf)
    return _weights[(N, K)]


def act(M, K, seed=0):
    rng = np.random.RandomState(1000 + M + seed)
    a, asf, adq = fp4_operand(M, K, rng)
    return dev(a), swizzled_dev(asf), adq


def expected(adq, bdq32, alpha):
    return alpha * (torch.from_numpy(adq) @ torch.from_numpy(bdq32).double().T).numpy()


SHAPES = [(5120, 5120), (5120, 17408), (17408, 5120), (34816, 5120), (128, 5120), (1024, 5120), (384, 448)]


@pytest.mark.parametrize("M", [1, 2, 3, 4, 8, 13, 16, 29, 32, 64, 77, 128])
@pytest.mark.parametrize("N,K", SHAPES)
def test_skinny_fp4(M, N, K):
    bd, bsw, bdq, _, _ = weight(N, K)
    ad, asw, adq = act(M, K)
    ws = workspace(WS)  # poisoned with NaN bit patterns: nothing may be read before it is written
    alpha = 0.37
    ref = expected(adq, bdq, alpha)
    c = torch.randn(M, N, device=DEV)
    d = c.clone()
    for _ in range(2):  # the second call runs on the workspace the first one left behind
        d.copy_(c)
        call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, alpha, d, 1.0, d, ws, WS)  # residual in place
        assert rel_err(d.cpu().numpy(), ref + c.cpu().numpy().astype(np.float64)) < 1e-5
    d.fill_(float("nan"))
    call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, alpha, None, 0.0, d, ws, WS)
    out = d.cpu().numpy()
    assert rel_err(out, ref) < 1e-5
    assert O.within_tolerance(out, ref).all()
    d2 = torch.empty_like(d)
    call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, alpha, c, 0.5, d2, ws, WS)  # C apart from D
    assert rel_err(d2.cpu().numpy(), ref + 0.5 * c.cpu().numpy().astype(np.float64)) < 1e-5
    # bf16 output is the fp32 output rounded to nearest even
    db = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    call("q27t_skinny_fp4_bf16", M, N, K, ad, asw, bd, bsw, alpha, db, ws, WS)
    assert torch.equal(db, d.bfloat16())


def test_skinny_lm_head_shape():
    """The widest projection of the model (248320 rows): 1940 tiles on one launch."""
    M, N, K = 3, 248320, 5120
    rng = np.random.RandomState(5)
    b, bsf, _ = fp4_operand(N, K, rng)
    ad, asw, adq = act(M, K)
    d = torch.full((M, N), float("nan"), device=DEV)
    ws = workspace(WS)
    call("q27t_skinny_fp4", M, N, K, ad, asw, dev(b), swizzled_dev(bsf), 1.0, None, 0.0, d, ws, WS)
    out = d.cpu().numpy()
    for r0 in (0, 100000, N - 4096):  # the oracle on three bands of 4096 rows (the full matrix is 5 GB in fp32)
        bdq = O.unpack_e2m1(b[r0:r0 + 4096]).astype(np.float64) * np.repeat(O.e4m3_decode(bsf[r0:r0 + 4096]).astype(np.float64), 16, -1)
        assert rel_err(out[:, r0:r0 + 4096], adq @ bdq.T) < 1e-5
    assert np.isfinite(out).all()


@pytest.mark.parametrize("residual", [False, True])
def test_rows_independent_of_m(residual):
    """A token's row is bit-identical whatever the number of tokens it is computed with (decode vs verify vs
    batched verify): the K split does not depend on M and the epilogue rounds explicitly. The reference states
    this for its M <= 64 path (engine/tests/test_skinny.py:59-117); here it holds for 1..128 across four kernel
    configurations and both ways of summing cut tiles."""
    N, K = 5120, 17408
    bd, bsw, _, _, _ = weight(N, K)
    ad, asw, _ = act(128, K)
    ws = workspace(WS)
    c = torch.randn(128, N, device=DEV) * 100
    outs = {}
    for M in (1, 2, 5, 8, 9, 16, 17, 29, 32, 33, 41, 64, 65, 100, 128):
        d = c[:M].clone() if residual else torch.empty(M, N, device=DEV)
        call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, 0.37, d if residual else None, 1.0 if residual else 0.0, d, ws, WS)
        outs[M] = d.cpu()
    for M, d in outs.items():
        assert torch.equal(d, outs[128][:M]), f"M={M}"


@pytest.mark.parametrize("glu", [False, True])
def test_rows_independent_of_m_on_a_wide_weight(glu):
    """gate | up (34816 x 5120) is not split along K; above 32 tokens the launcher hands it to the many-row tiles
    (tokens on the other side of the MMA). Rows must not change across that boundary either."""
    N, K = 34816, 5120
    bd, bsw, _, _, _ = weight(N, K)
    ad, asw, _ = act(128, K)
    ws = workspace(WS)
    outs = {}
    for M in (1, 16, 32, 33, 64, 65, 128):
        if glu:
            d = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
            call("q27t_skinny_fp4_glu_bf16", M, N // 2, K, ad, asw, bd, bsw, 0.013, 0.021, d, ws, WS)
        else:
            d = torch.empty(M, N, device=DEV)
            call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, 0.37, None, 0.0, d, ws, WS)
        outs[M] = d.cpu()
    for M, d in outs.items():
        assert torch.equal(d, outs[128][:M]), f"M={M}"


def test_shared_workspace_across_shapes():
    ws = workspace(WS)
    cases = []
    for N, K in [(17408, 5120), (5120, 17408), (1024, 5120), (34816, 5120)]:
        bd, bsw, bdq, _, _ = weight(N, K)
        ad, asw, adq = act(3, K)
        cases.append((N, K, ad, asw, bd, bsw, expected(adq, bdq, 1.0)))
    for _ in range(3):
        for N, K, ad, asw, bd, bsw, ref in cases:
            d = torch.empty(3, N, device=DEV)
            call("q27t_skinny_fp4", 3, N, K, ad, asw, bd, bsw, 1.0, None, 0.0, d, ws, WS)
            assert rel_err(d.cpu().numpy(), ref) < 1e-5


def test_deterministic():
    M, N, K = 1, 5120, 17408
    bd, bsw, _, _, _ = weight(N, K)
    ad, asw, _ = act(M, K)
    ws = workspace(WS)
    outs = []
    for _ in range(3):
        d = torch.empty(M, N, device=DEV)
        call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, 1.0, None, 0.0, d, ws, WS)
        outs.append(d.clone())
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def test_alpha_segments():
    """Fused projections: one alpha per block of output columns (AlphaSegments, engine/src/kernels.h:228-239)."""
    M, N, K = 4, 1024, 5120
    bd, bsw, bdq, _, _ = weight(N, K)
    ad, asw, adq = act(M, K)
    begin = (ctypes.c_int * 4)(0, 256, 640, 896)
    alpha = (ctypes.c_float * 4)(0.5, 0.25, 2.0, 0.125)
    ws = workspace(WS)
    d = torch.empty(M, N, device=DEV)
    call("q27t_skinny_fp4_segments", M, N, K, ad, asw, bd, bsw, 4, begin, alpha, None, 0.0, d, ws, WS)
    scale = np.repeat(np.array([0.5, 0.25, 2.0, 0.125]), [256, 384, 256, 128])
    assert rel_err(d.cpu().numpy(), expected(adq, bdq, 1.0) * scale[None, :]) < 1e-5


@pytest.mark.parametrize("M", [1, 7, 16, 50, 128])
@pytest.mark.parametrize("I,K", [(192, 512), (17408, 5120)])
def test_skinny_glu_bf16(M, I, K):
    """gate | up on interleaved weights with the SiLU*mul epilogue against silu(gate) * up of the fp64 GEMMs, and
    against the same epilogue applied to the plain fp32 GEMM of the interleaved weights."""
    rng = np.random.RandomState(I + M)
    w, wsf, wdq = fp4_operand(2 * I, K, rng)  # gate rows, then up rows
    wi, wsfi = layouts.interleave_glu(w), layouts.interleave_glu(wsf)
    ad, asw, adq = act(M, K)
    ag, au = 0.013, 0.021
    full = adq @ wdq.T
    ref = O.silu_mul(ag * full[:, :I], au * full[:, I:])
    ws = workspace(WS)
    wid, wsw = dev(wi), swizzled_dev(wsfi)
    d = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    call("q27t_skinny_fp4_glu_bf16", M, I, K, ad, asw, wid, wsw, ag, au, d, ws, WS)
    out = bf16_to_f32(d)
    assert O.within_tolerance_bf16(out, ref).all()  # 2e-3 |ref| + 1e-3 before the store, half a bf16 ulp from it
    assert rel_err(out, ref) < 3e-3
    # the same through the plain GEMM + host SiLU*mul on its fp32 output: equal up to the exponential's last ulps
    gu = torch.empty(M, 2 * I, device=DEV)
    call("q27t_skinny_fp4", M, 2 * I, K, ad, asw, wid, wsw, 1.0, None, 0.0, gu, ws, WS)
    rows = torch.from_numpy(layouts.glu_rows(I)).to(DEV)
    g, u = gu[:, rows[:I]] * np.float32(ag), gu[:, rows[I:]] * np.float32(au)
    host = (torch.nn.functional.silu(g) * u).bfloat16()
    assert (host != d).float().mean().item() < 2e-2
    assert rel_err(bf16_to_f32(host), out) < 1e-3


def test_workspace_too_small_and_bad_m():
    bd, bsw, _, _, _ = weight(1024, 5120)
    ad, asw, _ = act(4, 5120)
    d = torch.empty(4, 1024, device=DEV)
    ws = workspace(1024)
    with pytest.raises(RuntimeError, match="workspace too small"):
        call("q27t_skinny_fp4", 4, 1024, 5120, ad, asw, bd, bsw, 1.0, None, 0.0, d, ws, 1024)
    need = lib().q27b_skinny_workspace_bytes(4, 1024, 5120)
    assert 0 < need <= WS
    with pytest.raises(RuntimeError, match="M must be 1..128"):
        call("q27t_skinny_fp4", 0, 1024, 5120, ad, asw, bd, bsw, 1.0, None, 0.0, d, ws, 1024)


@pytest.mark.parametrize("M", [1, 7, 16, 40])
@pytest.mark.parametrize("N,K", [(1024, 5120), (5120, 2048)])
def test_skinny_fp4_scaled(M, N, K):
    """Per-output-channel weight scales and per-token activation scales: d[m][n] = acc * (wscale[n] * ascale[m])
    against the fp64 product of the dequantised operands (engine/tests/test_skinny.py:184-201 does the same for the
    reference's FP8 twin), and bit-identical to the unscaled call followed by that multiplication."""
    rng = np.random.RandomState(M + N)
    a, asf, adq = fp4_operand(M, K, rng)
    w, wsf, wdq = fp4_operand(N, K, rng)
    asc = (rng.rand(M) * 2 + 0.1).astype(np.float32)
    wsc = (rng.rand(N) * 0.01 + 1e-3).astype(np.float32)
    ad, asw, wd, wsw = dev(a), swizzled_dev(asf), dev(w), swizzled_dev(wsf)
    ws = workspace(WS)
    d = torch.full((M, N), float("nan"), device=DEV)
    call("q27t_skinny_fp4_scaled", M, N, K, ad, asw, dev(asc), wd, wsw, dev(wsc), d, ws, ws.numel())
    ref = (adq @ wdq.T) * wsc[None, :].astype(np.float64) * asc[:, None].astype(np.float64)
    assert rel_err(d.cpu().numpy(), ref) < 1e-5
    plain = torch.empty(M, N, device=DEV)
    call("q27t_skinny_fp4", M, N, K, ad, asw, wd, wsw, 1.0, None, 0.0, plain, ws, ws.numel())
    expect = plain.cpu().numpy() * (wsc[None, :] * asc[:, None])
    assert np.array_equal(d.cpu().numpy(), expect.astype(np.float32))
