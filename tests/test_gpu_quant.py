"""Activation quantisers and the scale relayout on the GPU against the CPU oracle: codes and scale bytes bit for
bit (protocol of engine/tests/test_elementwise.py:46-58,85-90,118-130,161-170 in the reference, which compares
dequantised values with atol = 0; here the raw bytes are compared as well)."""

import numpy as np
import pytest
import torch

from helpers import DEV, dev
from oracle import nvfp4_oracle as O
from q27b200 import layouts
from q27b200.q27lib import call, lib

pytestmark = pytest.mark.gpu


def run_quant(x_t, M, K, s):
    q = torch.full((M, K // 2), 0xAA, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(lib().q27t_sf_bytes(M, K // 16), dtype=torch.uint8, device=DEV)
    call("q27t_quant_fp4_bf16" if x_t.dtype == torch.bfloat16 else "q27t_quant_fp4", x_t, M, K, float(s), q, sf)
    return q.cpu().numpy(), sf.cpu().numpy()


def check_against_oracle(x_f32, q, sf_buf, s):
    M, K = x_f32.shape
    codes, sfo = O.quant_act_codes(x_f32, s)
    sf = layouts.unswizzle(sf_buf, M, K // 16)
    assert np.array_equal(sf, sfo), "scale bytes differ"
    got, want = O.unpack_codes(q), O.unpack_codes(codes)
    assert np.array_equal(O.canonical_zero(got), O.canonical_zero(want)), "codes differ"
    # the sign of a zero is not pinned by the reference; report how often the raw nibbles agree too
    raw = float((got == want).mean())
    # dequantised values, in the reference's order of operations, equal its fake-quantised activations exactly
    gs = np.float32(1.0) / np.float32(s)
    deq = (O.decode_e2m1(got) * np.repeat(O.e4m3_decode(sf), 16, -1)).astype(np.float32) / gs
    assert np.array_equal(deq, O.quant_act_nvfp4(x_f32, s))
    # padding of the scale buffer is untouched
    mask = np.ones(sf_buf.size, dtype=bool)
    mask[layouts.sf_index(M, K // 16).ravel()] = False
    assert not sf_buf[mask].any()
    return raw


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,K", [(37, 5120), (1, 5120), (16, 5120), (128, 17408), (3, 64), (300, 1088 * 16)])
def test_quant_fp4_matches_oracle(M, K, dtype):
    rng = np.random.RandomState(M * 7 + K)
    x = (rng.standard_normal((M, K)) * np.logspace(-2, 1, M)[:, None]).astype(np.float32)
    x[min(3, M - 1), :16] = 0  # an all-zero block
    x[0, 16:32] = 3e4  # a block whose scale saturates at 448
    x[M - 1, 32:48] *= 1e-7  # a block whose scale rounds to zero
    xt = torch.from_numpy(x).to(dtype)
    s = 0.0123
    q, sf = run_quant(xt.to(DEV), M, K, s)
    raw = check_against_oracle(xt.float().numpy(), q, sf, s)
    assert raw == 1.0  # the hardware conversion keeps the sign of a negative zero, as the oracle models it


def test_quant_fp4_golden(golden):
    x, s = golden["act_x"], float(golden["act_scale"])
    M, K = x.shape  # K = 512
    q, sf = run_quant(dev(x), M, K, s)
    gs = np.float32(1.0) / np.float32(s)
    deq = (O.unpack_e2m1(q) * np.repeat(O.e4m3_decode(layouts.unswizzle(sf, M, K // 16)), 16, -1)).astype(np.float32) / gs
    assert np.array_equal(deq, golden["act_deq"])
    xb = torch.from_numpy(golden["act_x_bf16_bits"].view(np.int16)).view(torch.bfloat16)
    q, sf = run_quant(xb.to(DEV), M, K, s)
    deq = (O.unpack_e2m1(q) * np.repeat(O.e4m3_decode(layouts.unswizzle(sf, M, K // 16)), 16, -1)).astype(np.float32) / gs
    assert np.array_equal(deq, golden["act_deq_bf16"])


def test_quant_empty_is_noop():
    call("q27t_quant_fp4", None, 0, 5120, 1.0, None, None)


def test_swizzle_sf_roundtrip():
    rows, kb = 300, 1088
    src = np.random.RandomState(0).randint(0, 255, size=(rows, kb)).astype(np.uint8)
    dst = torch.zeros(lib().q27t_sf_bytes(rows, kb), dtype=torch.uint8, device=DEV)
    call("q27t_swizzle_sf", dev(src), rows, kb, dst)
    assert np.array_equal(layouts.unswizzle(dst.cpu().numpy(), rows, kb), src)
    assert np.array_equal(dst.cpu().numpy(), O.swizzle_sf(src))


def test_swizzle_sf_glu_halves():
    inter, kb = 192, 320
    sf = np.random.RandomState(1).randint(0, 255, size=(2 * inter, kb)).astype(np.uint8)  # gate rows then up rows
    want = O.swizzle_sf(O.interleave_glu(sf))
    dst = torch.zeros(want.size, dtype=torch.uint8, device=DEV)
    for h in range(2):
        call("q27t_swizzle_sf_glu", dev(sf[h * inter:(h + 1) * inter]), inter, kb, dst, h)
    assert np.array_equal(dst.cpu().numpy(), want)


def test_silu_mul_quant_fp4_variants_agree():
    """bf16 input == fp32 input on the same values; the interleaved (glu) form == the plain form on the
    de-interleaved, alpha-scaled values; all bit-equal (same arithmetic, engine/tests/test_elementwise.py:161-170
    and engine/tests/test_gemm.py:86-90 in the reference)."""
    T, I, s = 5, 17408, 0.02
    g = (torch.randn(T, I) * 4).bfloat16()
    u = (torch.randn(T, I) * 4).bfloat16()

    def out():
        return (torch.zeros(T, I // 2, dtype=torch.uint8, device=DEV),
                torch.zeros(lib().q27t_sf_bytes(T, I // 16), dtype=torch.uint8, device=DEV))

    q1, sf1 = out()
    q2, sf2 = out()
    call("q27t_silu_mul_quant_fp4_bf16", g.to(DEV), u.to(DEV), I, T, I, s, q1, sf1)
    call("q27t_silu_mul_quant_fp4", g.float().to(DEV), u.float().to(DEV), I, T, I, s, q2, sf2)
    assert torch.equal(q1, q2) and torch.equal(sf1, sf2)
    # interleaved input with alphas
    ag, au = 0.013, 0.021
    gu = torch.empty(T, 2 * I)
    rows = torch.from_numpy(layouts.glu_rows(I))
    gu[:, rows] = torch.cat([g.float(), u.float()], 1)
    q3, sf3 = out()
    call("q27t_silu_mul_quant_fp4_glu", gu.to(DEV), T, I, ag, au, s, q3, sf3)
    q4, sf4 = out()
    gs, us = (g.float() * np.float32(ag)).to(DEV), (u.float() * np.float32(au)).to(DEV)
    call("q27t_silu_mul_quant_fp4", gs, us, I, T, I, s, q4, sf4)
    assert torch.equal(q3, q4) and torch.equal(sf3, sf4)
    q5, sf5 = out()
    call("q27t_silu_mul_quant_fp4_glu_bf16", gu.bfloat16().to(DEV), T, I, ag, au, s, q5, sf5)
    assert torch.equal(q5, q3) and torch.equal(sf5, sf3)


def test_silu_mul_quant_fp4_against_oracle():
    """silu(g) * u then the block quantiser against the oracle: the device exponential differs from the host's by
    an ulp now and then, which can move a value across a rounding boundary, so a small mismatch rate is allowed
    (the bound the reference uses for its fused epilogue, engine/tests/test_gemm.py:92-96)."""
    T, I, s = 3, 17408, 0.02
    g = (torch.randn(T, I) * 4).numpy()
    u = torch.randn(T, I).numpy()
    q = torch.zeros(T, I // 2, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(lib().q27t_sf_bytes(T, I // 16), dtype=torch.uint8, device=DEV)
    call("q27t_silu_mul_quant_fp4", dev(g), dev(u), I, T, I, s, q, sf)
    h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32)) * u).astype(np.float32)
    codes, sfo = O.quant_act_codes(h, s)
    sf_got = layouts.unswizzle(sf.cpu().numpy(), T, I // 16)
    assert (sf_got != sfo).mean() < 1e-3
    assert (O.canonical_zero(O.unpack_codes(q.cpu().numpy())) != O.canonical_zero(O.unpack_codes(codes))).mean() < 2e-3


@pytest.mark.parametrize("n,k", [(96, 512), (300, 5120)])
def test_quant_fp4_weight_search_against_oracle(n, k):
    """The load-time weight quantiser (block scales searched for the smallest squared error) against the oracle:
    codes and scale bytes bit for bit, including all-zero blocks, an outlier block and tiny rows."""
    from q27b200 import weights

    g = torch.Generator().manual_seed(n + k)
    w = torch.randn(n, k, generator=g) * 0.02
    w[3, :16] = 0.0
    w[5, 16:32] *= 50.0
    w[9] *= 1e-3
    w = w.to(torch.bfloat16)
    codes, sf, gs = weights.quantize_weight_search(w.to(DEV))
    torch.cuda.synchronize()
    co, so = O.quant_weight_search(w.float().numpy(), gs)
    assert np.array_equal(layouts.unswizzle(sf.cpu().numpy(), n, k // 16), so)
    assert np.array_equal(codes.cpu().numpy(), co)
    # and it is what the GEMM kernels consume: dequantised error below the round-to-nearest quantiser's
    wq = O.dequant_nvfp4(co, so, gs)
    c_rtn, s_rtn, _ = O.quant_weight_rtn(w.float().numpy(), gs)
    assert ((wq - w.float().numpy()) ** 2).sum() < ((O.dequant_nvfp4(c_rtn, s_rtn, gs) - w.float().numpy()) ** 2).sum()


def test_quant_fp4_dynamic_against_oracle():
    """Per-token dynamic quantisation: row scales, codes and scale bytes bit for bit; rows of very different
    magnitude and an all-zero row (scale 1)."""
    M, K = 9, 5120
    rng = np.random.RandomState(5)
    x = (rng.standard_normal((M, K)) * np.logspace(-3, 2, M)[:, None]).astype(np.float32)
    x[4] = 0.0
    q = torch.zeros(M, K // 2, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(lib().q27t_sf_bytes(M, K // 16), dtype=torch.uint8, device=DEV)
    asc = torch.zeros(M, dtype=torch.float32, device=DEV)
    call("q27t_quant_fp4_dynamic", dev(x), M, K, q, sf, asc)
    codes, sfo, rs = O.quant_act_dynamic(x)
    assert np.array_equal(asc.cpu().numpy(), rs) and rs[4] == 1.0
    assert np.array_equal(layouts.unswizzle(sf.cpu().numpy(), M, K // 16), sfo)
    assert np.array_equal(q.cpu().numpy(), codes)
    # bf16 input: the same as the fp32 kernel on the widened values
    xb = torch.from_numpy(x).to(torch.bfloat16)
    q2, sf2, asc2 = torch.zeros_like(q), torch.zeros_like(sf), torch.zeros_like(asc)
    call("q27b_quant_fp4_dynamic_bf16", xb.to(DEV), M, K, q2, sf2, asc2, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    c3, s3, r3 = O.quant_act_dynamic(xb.float().numpy())
    assert np.array_equal(q2.cpu().numpy(), c3) and np.array_equal(asc2.cpu().numpy(), r3)
    assert np.array_equal(layouts.unswizzle(sf2.cpu().numpy(), M, K // 16), s3)


def test_quant_fp4_batch_equals_single_calls():
    """Several activations quantised by one launch (jobs in the launch parameters up to four, in device memory
    above) give the bytes of one call each."""
    import ctypes

    class Job(ctypes.Structure):  # q27b_quant_job
        _fields_ = [("x", ctypes.c_void_p), ("q", ctypes.c_void_p), ("sf", ctypes.c_void_p), ("M", ctypes.c_int),
                    ("K", ctypes.c_int), ("input_scale", ctypes.c_float), ("bf16", ctypes.c_int)]

    rng = np.random.RandomState(11)
    shapes = [(16, 5120, torch.bfloat16), (3, 17408, torch.float32), (128, 5120, torch.bfloat16), (1, 64, torch.float32),
              (7, 5120, torch.float32), (16, 17408, torch.bfloat16)]
    for n in (3, 6):
        xs, outs, want, jobs = [], [], [], (Job * n)()
        for i, (M, K, dt) in enumerate(shapes[:n]):
            x = torch.from_numpy((rng.standard_normal((M, K)) * (i + 1)).astype(np.float32)).to(dt).to(DEV)
            s = 0.01 * (i + 1)
            want.append(run_quant(x, M, K, s))
            q = torch.full((M, K // 2), 0xAA, dtype=torch.uint8, device=DEV)
            sf = torch.zeros(lib().q27t_sf_bytes(M, K // 16), dtype=torch.uint8, device=DEV)
            xs.append(x), outs.append((q, sf))
            jobs[i].x, jobs[i].q, jobs[i].sf = x.data_ptr(), q.data_ptr(), sf.data_ptr()
            jobs[i].M, jobs[i].K, jobs[i].input_scale, jobs[i].bf16 = M, K, s, int(dt == torch.bfloat16)
        table = None
        if n > 4:
            table = torch.frombuffer(bytearray(bytes(jobs)), dtype=torch.uint8).to(DEV)
        torch.cuda.synchronize()
        call("q27b_quant_fp4_batch", jobs, table, n, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        for (q, sf), (wq, wsf) in zip(outs, want):
            assert np.array_equal(q.cpu().numpy(), wq) and np.array_equal(sf.cpu().numpy(), wsf)
    with pytest.raises(RuntimeError, match="more than four jobs"):
        call("q27b_quant_fp4_batch", jobs, None, 6, 0)


@pytest.mark.parametrize("T", [1, 5, 16])
def test_rmsnorm_quant(T):
    """RMSNorm(1 + w) fused with the quantiser (protocol of engine/tests/test_elementwise.py:94-115): the fp32 result
    against the reference's definition within 1e-5, and - stronger - bit for bit against the fixed-order fp32
    restatement; the quantised copy exactly the quantisation of the fp32 result (codes and scale bytes)."""
    D = 5120
    rng = np.random.RandomState(T)
    x = (rng.standard_normal((T, D)) * 3).astype(np.float32)
    x[0, 64:80] = 0
    if T > 2:
        x[2] *= 1e-3
    w = torch.from_numpy((rng.standard_normal(D) * 0.1).astype(np.float32)).bfloat16()
    s = 0.0123
    out = torch.full((T, D), float("nan"), device=DEV)
    q = torch.full((T, D // 2), 0xAA, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(lib().q27t_sf_bytes(T, D // 16), dtype=torch.uint8, device=DEV)
    call("q27t_rmsnorm_quant", dev(x), w.to(DEV), T, 1e-6, out, 2, s, q, sf)
    y = out.cpu().numpy()
    ref = O.rms_norm(x, w.float().numpy(), 1e-6)
    assert (np.abs(y - ref) <= 1e-5 + 1e-5 * np.abs(ref)).all()
    y32, _ = O.rms_norm_fixed_order(x, w.float().numpy(), 1e-6)
    assert np.array_equal(y, y32)
    check_against_oracle(y, q.cpu().numpy(), sf.cpu().numpy(), s)
    # the plain form writes the same fp32 result and leaves q alone
    out2 = torch.empty_like(out)
    q2 = torch.full_like(q, 0x55)
    call("q27t_rmsnorm_quant", dev(x), w.to(DEV), T, 1e-6, out2, 0, s, q2, sf)
    assert torch.equal(out2, out) and (q2 == 0x55).all()


def test_rmsnorm_quant_golden_and_options():
    """On the golden vectors made by the reference's own functions; with the bf16 copy of the input and 1 / rms."""
    import os

    g = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_rmsnorm_golden.npz")))
    x, w, eps, s = g["x"], g["w"], float(g["eps"]), float(g["in_scale"])
    T, D = x.shape
    out = torch.empty(T, D, device=DEV)
    q = torch.zeros(T, D // 2, dtype=torch.uint8, device=DEV)
    sf = torch.zeros(lib().q27t_sf_bytes(T, D // 16), dtype=torch.uint8, device=DEV)
    cap = torch.zeros(T, D + 64, dtype=torch.bfloat16, device=DEV)
    rstd = torch.zeros(T, device=DEV)
    wd = torch.from_numpy(w).bfloat16().to(DEV)
    torch.cuda.synchronize()
    call("q27b_rmsnorm_quant_fp4", dev(x), wd, T, D, eps, out, s, q, sf, cap, D + 64, rstd, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    y = out.cpu().numpy()
    assert (np.abs(y - g["y"]) <= 1e-5 + 1e-5 * np.abs(g["y"])).all()
    gs = np.float32(1.0) / np.float32(s)
    deq = (O.unpack_e2m1(q.cpu().numpy()) * np.repeat(O.e4m3_decode(layouts.unswizzle(sf.cpu().numpy(), T, D // 16)), 16, -1)).astype(np.float32) / gs
    assert np.array_equal(deq, O.quant_act_nvfp4(y, s))
    assert (deq != g["y_quant"]).mean() < 1e-3  # the reference's fp32 result differs in the last bit here and there
    assert torch.equal(cap[:, :D].cpu(), torch.from_numpy(x).bfloat16()) and not cap[:, D:].any()
    _, r = O.rms_norm_fixed_order(x, w, eps)
    assert np.array_equal(rstd.cpu().numpy(), r)
    with pytest.raises(RuntimeError, match="multiple of 512"):
        call("q27b_rmsnorm_quant_fp4", dev(x), wd, T, 5000, eps, out, s, q, sf, None, 0, None, 0)
