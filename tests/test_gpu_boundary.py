"""The C++ face of the boundary (include/q27b200/kernels.h, the header the engine's model.cc would compile against)
driven from C++: the scaffolding library calls q27::quant_fp4, q27::skinny_fp4 with three AlphaSegments and
q27::gemm_fp4_glu, and the results must equal what the C ABI gives for the same buffers; a failed precondition must
arrive as std::runtime_error("check failed: ..."), the reference's convention (engine/src/check.h:6-13). Also the
naive device GEMM of the scaffolding library as an independent cross-check of both tensor-core kernels."""

import ctypes

import numpy as np
import pytest
import torch

from helpers import DEV, dev, fp4_operand, rel_err, swizzled_dev, workspace
from q27b200 import layouts
from q27b200.q27lib import call, lib, scaffold_lib

pytestmark = pytest.mark.gpu


def test_cxx_launchers_match_the_c_abi():
    M, K, N, I = 5, 5120, 7168, 256
    rng = np.random.RandomState(1)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(DEV)
    w, wsf, _ = fp4_operand(N, K, rng)
    gu, gusf, _ = fp4_operand(2 * I, K, rng)
    wd, wsw = dev(w), swizzled_dev(wsf)
    gud, gusw = dev(layouts.interleave_glu(gu)), swizzled_dev(layouts.interleave_glu(gusf))
    begin, alpha = (ctypes.c_int * 3)(0, 5120, 6144), (ctypes.c_float * 3)(0.5, 0.25, 2.0)
    s, ag, au, s_out = 0.01, 0.013, 0.021, 0.05
    ws = workspace()

    def buffers():
        return (torch.zeros(M, K // 2, dtype=torch.uint8, device=DEV), torch.zeros(lib().q27t_sf_bytes(M, K // 16), dtype=torch.uint8, device=DEV),
                torch.full((M, N), float("nan"), device=DEV), torch.zeros(M, I // 2, dtype=torch.uint8, device=DEV),
                torch.zeros(lib().q27t_sf_bytes(M, I // 16), dtype=torch.uint8, device=DEV))

    q1, sf1, d1, hq1, hsf1 = buffers()
    call("q27t_cxx_launchers", x, M, K, s, q1, sf1, N, wd, wsw, 3, begin, alpha, d1, ws, ws.numel(), I, gud, gusw, ag, au, s_out, hq1, hsf1)
    q2, sf2, d2, hq2, hsf2 = buffers()
    call("q27t_quant_fp4", x, M, K, s, q2, sf2)
    call("q27t_skinny_fp4_segments", M, N, K, q2, sf2, wd, wsw, 3, begin, alpha, None, 0.0, d2, ws, ws.numel())
    call("q27t_gemm_fp4_glu", M, I, K, q2, sf2, gud, gusw, ag, au, s_out, hq2, hsf2)
    for a, b in ((q1, q2), (sf1, sf2), (d1, d2), (hq1, hq2), (hsf1, hsf2)):
        assert torch.equal(a, b)
    assert torch.isfinite(d1).all()


def test_cxx_launchers_throw_on_a_failed_precondition():
    assert scaffold_lib().q27t_cxx_throws() == 1


@pytest.mark.parametrize("M,N,K", [(3, 256, 512), (130, 384, 448 + 64)])
def test_naive_device_gemm_agrees_with_the_tensor_core_kernels(M, N, K):
    rng = np.random.RandomState(M)
    a, asf, adq = fp4_operand(M, K, rng)
    b, bsf, bdq = fp4_operand(N, K, rng)
    ad, asw, bd, bsw = dev(a), swizzled_dev(asf), dev(b), swizzled_dev(bsf)
    naive = torch.empty(M, N, device=DEV)
    call("q27t_ref_gemm_fp4", M, N, K, ad, asw, bd, bsw, 0.37, naive)
    assert rel_err(naive.cpu().numpy(), 0.37 * (adq @ bdq.T)) < 1e-5
    d = torch.empty(M, N, device=DEV)
    if K % 128 == 0:
        call("q27t_gemm_fp4", M, N, K, ad, asw, bd, bsw, 0.37, None, 0.0, d)
        assert rel_err(d.cpu().numpy(), naive.cpu().numpy()) < 1e-5
    if M <= 128:
        ws = workspace()
        call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, 0.37, None, 0.0, d, ws, ws.numel())
        assert rel_err(d.cpu().numpy(), naive.cpu().numpy()) < 1e-5
