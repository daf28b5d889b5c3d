"""Pins the CPU oracle: the reference's own known-answer tests (reference/tests/test_quant.py, restated as
literal vectors) and golden vectors recorded from the reference's Python modules (tests/golden)."""

import os

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


# ---- reference/tests/test_quant.py, restated -----------------------------------------------------------------


def test_unpack_low_nibble_first():
    packed = np.array([[0x21, 0xF8]], dtype=np.uint8)  # codes 1, 2 | 8 (-0), 15 (-6)
    out = O.unpack_e2m1(packed)
    assert out.tolist() == [[0.5, 1.0, -0.0, -6.0]]
    assert np.signbit(out[0, 2])


def test_round_e2m1_grid_and_ties():
    grid = O.E2M1_VALUES
    assert np.array_equal(O.round_e2m1(grid), grid)
    assert np.array_equal(O.round_e2m1(-grid), -grid)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    assert O.round_e2m1(ties).tolist() == [0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0]
    assert O.round_e2m1(np.array([0.26, 2.51, 7.0, -100.0], np.float32)).tolist() == [0.5, 3.0, 6.0, -6.0]


def test_quant_act_nvfp4_properties():
    x = (np.random.RandomState(0).standard_normal((4, 256)) * 3).astype(np.float32)
    q = O.quant_act_nvfp4(x, 0.01)
    assert np.allclose(O.quant_act_nvfp4(q, 0.01), q)  # idempotent
    blocks = np.abs(q.reshape(-1, 16))
    assert max(len(np.unique(b)) for b in blocks) <= 8
    rel = np.linalg.norm(x - q) / np.linalg.norm(x)
    assert rel < 0.15, rel


def test_e4m3_saturates():
    assert O.to_e4m3(np.array([1000.0, -1000.0], np.float32)).tolist() == [448.0, -448.0]


# ---- golden vectors recorded from the reference ---------------------------------------------------------------


def test_golden_round_e2m1(golden):
    assert np.array_equal(bits(O.round_e2m1(golden["e2m1_in"])), bits(golden["e2m1_out"]))


def test_golden_e4m3(golden):
    assert np.array_equal(bits(O.to_e4m3(golden["e4m3_in"])), bits(golden["e4m3_out"]))
    assert np.array_equal(O.e4m3_encode(golden["e4m3_in"]), golden["e4m3_code"])


def test_golden_unpack(golden):
    assert np.array_equal(bits(O.unpack_e2m1(golden["unpack_in"])), bits(golden["unpack_out"]))


def test_golden_quant_act(golden):
    deq = O.quant_act_nvfp4(golden["act_x"], golden["act_scale"])
    assert np.array_equal(bits(deq), bits(golden["act_deq"]))
    xb = O.bf16_bits_to_f32(golden["act_x_bf16_bits"])
    assert np.array_equal(bits(O.quant_act_nvfp4(xb, golden["act_scale"])), bits(golden["act_deq_bf16"]))


def test_quant_act_codes_roundtrip(golden):
    """Codes + scale bytes dequantise to the reference's fake-quantised values (its GPU test's protocol)."""
    x, s = golden["act_x"], golden["act_scale"]
    codes, sf = O.quant_act_codes(x, s)
    gs = np.float32(1.0) / np.float32(s)
    deq = (O.unpack_e2m1(codes) * np.repeat(O.e4m3_decode(sf), 16, -1)).astype(np.float32) / gs
    assert np.array_equal(deq, golden["act_deq"])  # (-0 == +0 here, as in the reference's comparison)
    assert (sf[3, 0] == 0) and not codes[3, :8].any()  # the all-zero block
    assert sf[5, 1] == 0x7E  # saturated block scale (448)


def test_golden_weight_quant(golden):
    codes, sf, g = O.quant_weight_rtn(golden["w"])
    assert g == golden["w_gscale"]
    assert np.array_equal(sf, golden["w_sf"])
    assert np.array_equal(codes, golden["w_codes"])
    assert np.array_equal(bits(O.dequant_nvfp4(codes, sf, g)), bits(golden["w_deq"]))


def test_golden_qlinear(golden):
    y = O.qlinear(golden["lin_x"], golden["w_codes"], golden["w_sf"], golden["w_gscale"], golden["lin_in_scale"])
    assert np.allclose(y, golden["lin_y_f64"], rtol=1e-12, atol=1e-14)
    # the reference's own fp32 evaluation agrees with the fp64 one far inside the acceptance tolerance
    assert O.within_tolerance(golden["lin_y_f32"], y, rel=1e-3, abs_=1e-5).all()


def test_golden_silu(golden):
    ref = golden["silu_out"]
    out = O.silu_mul(golden["silu_g"], golden["silu_u"])
    assert np.allclose(out, ref, rtol=2e-6, atol=1e-7)


# ---- the E4M3 cast the reference relies on (torch's), exhaustively --------------------------------------------


def test_e4m3_all_codes_roundtrip():
    codes = np.arange(256, dtype=np.uint8)
    vals = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    mine = O.e4m3_decode(codes)
    finite = np.isfinite(vals)
    assert np.array_equal(np.isnan(mine), np.isnan(vals))
    assert np.array_equal(bits(mine[finite]), bits(vals[finite]))
    assert np.array_equal(O.e4m3_encode(vals[finite]), codes[finite])


def test_e4m3_encode_random_vs_torch():
    rng = np.random.RandomState(1)
    x = np.concatenate([rng.standard_normal(200000) * 100, rng.standard_normal(200000) * 0.01,
                        rng.uniform(-2.0**-5, 2.0**-5, 100000)]).astype(np.float32)
    t = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x), t)


# ---- layouts -----------------------------------------------------------------------------------------------------


def test_sf_layout_roundtrip_and_atoms():
    rows, kb = 300, 1088
    src = np.random.RandomState(2).randint(0, 255, size=(rows, kb)).astype(np.uint8)
    buf = O.swizzle_sf(src)
    assert buf.size == O.sf_bytes(rows, kb) == 3 * 128 * 1088
    assert np.array_equal(O.unswizzle_sf(buf, rows, kb), src)
    # one 512-byte atom = 128 rows x 4 k-blocks: row r at line r % 32 (16 B), word r / 32, byte = k-block
    assert O.sf_offset(0, 0, kb) == 0 and O.sf_offset(33, 2, kb) == 1 * 16 + 1 * 4 + 2
    assert O.sf_offset(0, 4, kb) == 512 and O.sf_offset(128, 0, kb) == (kb // 4) * 512


def test_glu_interleave():
    inter = 192
    rows = O.glu_rows(inter)
    assert sorted(rows.tolist()) == list(range(2 * inter))
    assert rows[0] == 0 and rows[63] == 63 and rows[64] == 128 and rows[inter] == 64 and rows[inter + 64] == 192
    m = np.arange(2 * inter)[:, None] * np.ones((1, 3), dtype=np.int64)
    il = O.interleave_glu(m)
    assert il[64, 0] == inter and il[128, 0] == 64  # up row 0 sits after the first 64 gate rows


def test_bf16_round():
    x = np.random.RandomState(3).standard_normal(100000).astype(np.float32) * 37
    ref = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    assert np.array_equal(O.bf16_round(x), ref)


# ---- the searched weight quantiser (load-time) -----------------------------------------------------------------


@pytest.fixture(scope="module")
def search_golden():
    import os

    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_weight_search_golden.npz"))


def test_weight_search_matches_reference_pieces(search_golden):
    """Scale codes chosen by the oracle == the first-smallest of the reference's own block_error over the kernel's
    13 candidates; where they differ the two candidates' errors must be within rounding of each other (the
    reference's Python divides by the scale and sums in torch's order, the kernel multiplies by the reciprocal and
    keeps a running sum). Codes: equal to the reference's packer except on rounding boundaries of that same
    divide-versus-reciprocal difference."""
    g = search_golden
    codes, sf = O.quant_weight_search(g["w"], g["gscale"])
    differ = np.argwhere(sf != g["best"])
    assert len(differ) <= 0.001 * sf.size
    for r, b in differ:
        errs, cands = g["errs"][:, r, b], g["cands"][:, r, b]
        e_mine = errs[np.argmax(cands == sf[r, b])]
        assert abs(e_mine - errs.min()) <= 1e-5 * errs.min()
    same_scale = np.repeat(sf == g["best"], 16, axis=1)
    a, b = O.canonical_zero(O.unpack_codes(codes)), O.canonical_zero(O.unpack_codes(g["codes"]))
    assert (a != b)[same_scale].mean() < 1e-3
    assert (np.abs(O.decode_e2m1(a) - O.decode_e2m1(b))[same_scale].max()) <= 2.0  # a neighbouring code at most


def test_weight_search_properties(search_golden):
    g = search_golden
    w, gs = g["w"], g["gscale"]
    codes, sf = O.quant_weight_search(w, gs)
    c_rtn, sf_rtn, _ = O.quant_weight_rtn(w, gs)
    # never worse than round-to-nearest, block by block (the rounded code is among the candidates and wins ties)
    err = lambda c, s: ((O.dequant_nvfp4(c, s, gs) - w) ** 2).reshape(w.shape[0], -1, 16).sum(-1)
    assert (err(codes, sf) <= err(c_rtn, sf_rtn) * (1 + 1e-6)).all()
    assert err(codes, sf).sum() < 0.95 * err(c_rtn, sf_rtn).sum()
    # within the searched range, clamped
    d = sf.astype(np.int32) - sf_rtn.astype(np.int32)
    zero = np.abs(w).reshape(w.shape[0], -1, 16).max(-1) == 0
    assert (d[~zero] >= -4).all() and (d[~zero] <= 8).all() and (sf[~zero] >= 1).all() and (sf <= 126).all()
    assert (sf[zero] == sf_rtn[zero]).all() and (O.unpack_codes(codes).reshape(w.shape[0], -1, 16)[zero] & 7 == 0).all()
    # idempotent on its own output: a weight that is exactly representable is reproduced with zero error
    wq = O.dequant_nvfp4(codes, sf, gs).astype(np.float32)
    c2, s2 = O.quant_weight_search(wq, gs)
    assert np.array_equal(O.dequant_nvfp4(c2, s2, gs), O.dequant_nvfp4(codes, sf, gs))


def test_dynamic_per_token_quantiser_properties():
    """Row scale amax / (6 * 448) (1 for an all-zero row); a row quantises exactly as the static quantiser with
    that scale; scaling a row by a power of two scales its row scale and leaves codes and block scales alone."""
    rng = np.random.RandomState(3)
    x = (rng.standard_normal((6, 256)) * np.logspace(-2, 2, 6)[:, None]).astype(np.float32)
    x[2] = 0.0
    codes, sfs, rs = O.quant_act_dynamic(x)
    assert rs[2] == 1.0 and not codes[2].any() and not sfs[2].any()
    for m in (0, 3, 5):
        assert rs[m] == np.float32(np.abs(x[m]).max() / np.float32(6 * 448))
        c, s = O.quant_act_codes(x[m:m + 1], rs[m])
        assert np.array_equal(c[0], codes[m]) and np.array_equal(s[0], sfs[m])
        assert s.max() == 0x7E  # the largest block reaches the top of the E4M3 range: 448
    c2, s2, r2 = O.quant_act_dynamic(x * np.float32(8))
    assert np.array_equal(c2, codes) and np.array_equal(s2, sfs) and np.array_equal(r2[[0, 1, 3, 4, 5]], rs[[0, 1, 3, 4, 5]] * 8)


def test_rms_norm_against_the_references_function():
    """The oracle's RMSNorm and the fixed-order fp32 restatement of this repository's fused kernel against golden
    vectors made by the reference's own rms_norm and quant_act_nvfp4 (tests/golden/make_golden_rmsnorm.py), within the
    tolerance the reference's kernel test allows (engine/tests/test_elementwise.py:94-115: rtol = atol = 1e-5)."""
    g = dict(np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_rmsnorm_golden.npz")))
    x, w, eps, s = g["x"], g["w"], float(g["eps"]), float(g["in_scale"])
    y64 = O.rms_norm(x, w, eps)
    assert np.abs(y64 - g["y"]).max() < 2e-6
    y32, r = O.rms_norm_fixed_order(x, w, eps)
    assert y32.dtype == np.float32 and (np.abs(y32 - g["y"]) <= 1e-5 + 1e-5 * np.abs(g["y"])).all()
    assert np.allclose(r, 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(-1) + eps), rtol=1e-6)
    # the quantised copy is defined as the quantisation of the fp32 result
    assert np.array_equal(O.quant_act_nvfp4(g["y"], s), g["y_quant"])
    # an all-zero row stays zero (1 / sqrt(eps) is finite)
    z, rz = O.rms_norm_fixed_order(np.zeros((1, 512), np.float32), np.zeros(512, np.float32), 1e-6)
    assert not z.any() and np.isfinite(rz).all()
