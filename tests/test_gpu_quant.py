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
