"""CPU oracle for the NVFP4 weight-GEMM path: TEST INFRASTRUCTURE, not product code.

A plain numpy restatement of the reference's definition of the arithmetic. Only the tests, the smoke check and
the benchmark's CPU-baseline leg may import this module; the CUDA library never routes through it.

Parity status: PINNED. Every function below is checked (tests/test_oracle.py) against
  * the reference's own known-answer tests (reference/tests/test_quant.py: nibble order, grid fixed points, the
    seven tie cases, saturation, idempotence, E4M3 saturation), restated as literal vectors, and
  * golden vectors produced by importing the reference's Python modules (tests/golden/make_golden.py), and
  * torch's float8_e4m3fn cast over all fp32 midpoints and all 256 codes (the cast the reference relies on).

What each function follows (paths inside the reference project):
  unpack_e2m1        reference/qwen27b/quant.py:26-31
  round_e2m1         reference/qwen27b/quant.py:34-44   (== PTX cvt.rn.satfinite.e2m1x2.f32)
  to_e4m3            reference/qwen27b/quant.py:47-49   (torch float8_e4m3fn cast, saturating)
  dequant_nvfp4      reference/qwen27b/quant.py:52-55
  quant_act_nvfp4    reference/qwen27b/quant.py:58-67   (device twin: engine/src/kernels.cu:99-113)
  quant_weight_rtn   scripts/quantize_proj.py:77-81 (search = 0), :94-101 (pack), :176-180 (global scale)
  quant_weight_search engine/src/kernels.cu:167-206     (the load-time quantiser with a searched block scale; the
                     kernel cannot run where the golden vectors are made, so it is pinned through the pieces of its
                     Python twin, scripts/quantize_proj.py:70-97 block_error / pack, evaluated on the kernel's 13
                     candidates: tests/golden/make_golden_weight_search.py)
  qlinear            reference/qwen27b/quant.py:79-97   (matmul evaluated in fp64 as engine/tests/test_gemm.py:38)
  sf_offset/sf_bytes engine/src/kernels.h:192-199       (python twin engine/tests/test_elementwise.py:14-23)
  glu_row            engine/src/kernels.h:186           (python twin engine/tests/test_gemm.py:53-56)
  silu_mul           reference/qwen27b/model.py:182-185 (F.silu(gate) * up)
  rms_norm           reference/qwen27b/model.py:60-63   (zero-centred RMSNorm in fp32; golden vectors from the
                     reference's own function: tests/golden/make_golden_rmsnorm.py)
  rms_norm_fixed_order  the same quantity with the summation order and the separate IEEE operations of this
                     repository's fused kernel (one lane per 16 elements, a butterfly over 32 lanes, the warps in
                     order, IEEE sqrt and divisions), so that the kernel can be compared bit for bit; the reference's
                     kernel (engine/src/kernels.cu:211-262) uses an approximate rsqrt and its tests allow 1e-5
                     (engine/tests/test_elementwise.py:94-115), which is how rms_norm pins this function
"""

from __future__ import annotations

import numpy as np

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MIDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
FP4_BLOCK = 16
E4M3_MAX = np.float32(448.0)
E2M1_MAX = np.float32(6.0)

f32 = np.float32


# ----------------------------------------------------------------------------------------------- E2M1


def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """uint8 [..., n/2] -> uint8 codes [..., n]; the low nibble is the even column."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.uint8)
    out[..., 0::2] = packed & 0x0F
    out[..., 1::2] = packed >> 4
    return out


def pack_codes(codes: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def decode_e2m1(codes: np.ndarray) -> np.ndarray:
    """4-bit codes -> fp32 values; bit 3 is the sign, so code 8 is -0.0."""
    codes = np.asarray(codes)
    mag = E2M1_VALUES[codes & 0x7]
    return np.where(codes & 0x8, -mag, mag).astype(np.float32)


def unpack_e2m1(packed: np.ndarray) -> np.ndarray:
    return decode_e2m1(unpack_codes(packed))


def round_e2m1_index(x: np.ndarray) -> np.ndarray:
    """Magnitude index (0..7) of the nearest E2M1 value: ties go to the even index, saturating at 6."""
    a = np.minimum(np.abs(np.asarray(x, dtype=np.float32)), E2M1_MAX)
    # searchsorted(side="left") puts a value equal to a midpoint on its lower neighbour, as torch.bucketize.
    idx = np.searchsorted(E2M1_MIDS, a, side="left")
    tie = (a[..., None] == E2M1_MIDS).any(-1)
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    return idx.astype(np.int64)


def round_e2m1(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    return np.copysign(E2M1_VALUES[round_e2m1_index(x)], x).astype(np.float32)


def encode_e2m1(q: np.ndarray, signed_zero: bool = True) -> np.ndarray:
    """E2M1 grid values -> 4-bit codes. signed_zero=True keeps the sign bit of -0.0 (what the hardware
    conversion emits for small negatives); False maps every zero to code 0 (the reference's CPU packer)."""
    q = np.asarray(q, dtype=np.float32)
    mag = np.searchsorted(E2M1_VALUES, np.abs(q), side="left").astype(np.uint8)
    neg = np.signbit(q) if signed_zero else (q < 0)
    return (mag | (neg.astype(np.uint8) << 3)).astype(np.uint8)


def canonical_zero(codes: np.ndarray) -> np.ndarray:
    """Maps the -0 code (8) to +0 (0): the sign of a zero is not pinned by the reference."""
    codes = np.asarray(codes, dtype=np.uint8)
    return np.where(codes == 8, 0, codes).astype(np.uint8)


# ----------------------------------------------------------------------------------------------- E4M3


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    """float8_e4m3fn byte -> fp32 (0x7f / 0xff are NaN): e == 0 ? m/8 * 2^-6 : (1 + m/8) * 2^(e-7)."""
    code = np.asarray(code, dtype=np.uint8).astype(np.int64)
    e, m = (code >> 3) & 0xF, code & 0x7
    mag = np.where(e == 0, m / 8.0 * 2.0**-6, (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64)))
    mag = np.where((e == 15) & (m == 7), np.nan, mag)
    return np.where(code & 0x80, -mag, mag).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """fp32 -> float8_e4m3fn byte: clamp to +-448 (saturating), then round to nearest, ties to even mantissa."""
    x = np.asarray(x, dtype=np.float32)
    sign = np.signbit(x)
    a = np.minimum(np.abs(x).astype(np.float64), 448.0)
    # Spacing of the target grid at a: 2^-9 below 2^-6 (subnormals), else 2^(floor(log2 a) - 3).
    with np.errstate(divide="ignore"):
        ex = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    ex = np.maximum(ex, -6.0)
    ulp = np.exp2(ex - 3.0)
    q = np.rint(a / ulp) * ulp  # np.rint: ties to even (exact: a / ulp has at most 24 significant bits)
    q = np.minimum(q, 448.0)
    # encode q
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    normal = q >= 2.0**-6
    e_field = np.where(normal, e2 + 7, 0).astype(np.int64)
    m_field = np.where(normal, np.rint((q / np.exp2(e2) - 1.0) * 8.0), np.rint(q / 2.0**-9)).astype(np.int64)
    code = (e_field << 3) | m_field
    code = np.where(np.isnan(x), 0x7F, code)
    return (code | (sign.astype(np.int64) << 7)).astype(np.uint8)


def to_e4m3(x: np.ndarray) -> np.ndarray:
    return e4m3_decode(e4m3_encode(x))


# ----------------------------------------------------------------------------------------------- layouts


def sf_offset(row, kb, kblocks):
    """Byte offset of scale (row, k-block) in the swizzled layout: 512-byte atoms of 128 rows x 4 k-blocks."""
    row, kb = np.asarray(row, dtype=np.int64), np.asarray(kb, dtype=np.int64)
    katoms = (kblocks + 3) // 4
    return ((row // 128) * katoms + kb // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + (kb % 4)


def sf_bytes(rows: int, kblocks: int) -> int:
    return ((rows + 127) // 128) * 128 * ((kblocks + 3) // 4) * 4


def swizzle_sf(sf: np.ndarray, row_map=None, out: np.ndarray | None = None, total_rows: int | None = None):
    """Row-major scale bytes [rows][kblocks] -> swizzled buffer (padding bytes are zero)."""
    sf = np.asarray(sf, dtype=np.uint8)
    rows, kblocks = sf.shape
    r = np.arange(rows) if row_map is None else np.asarray(row_map)
    if out is None:
        out = np.zeros(sf_bytes(total_rows if total_rows is not None else rows, kblocks), dtype=np.uint8)
    out[sf_offset(r[:, None], np.arange(kblocks)[None, :], kblocks)] = sf
    return out


def unswizzle_sf(buf: np.ndarray, rows: int, kblocks: int) -> np.ndarray:
    buf = np.asarray(buf, dtype=np.uint8)
    return buf[sf_offset(np.arange(rows)[:, None], np.arange(kblocks)[None, :], kblocks)]


def glu_row(r, half: int):
    """Row of gate (half 0) / up (half 1) row r in the interleaved gate | up matrix (blocks of 64 rows)."""
    r = np.asarray(r, dtype=np.int64)
    return (r // 64) * 128 + half * 64 + r % 64


def glu_rows(inter: int) -> np.ndarray:
    """Interleaved positions of gate rows 0..I-1 followed by up rows 0..I-1."""
    r = np.arange(inter)
    return np.concatenate([glu_row(r, 0), glu_row(r, 1)])


def interleave_glu(rows_major: np.ndarray) -> np.ndarray:
    """[2I][...] laid out gate rows then up rows -> the interleaved order."""
    out = np.empty_like(rows_major)
    out[glu_rows(rows_major.shape[0] // 2)] = rows_major
    return out


# ----------------------------------------------------------------------------------------------- quantisers


def quant_act_nvfp4_parts(x: np.ndarray, input_scale: float):
    """Activation quantiser [..., k] (k % 16 == 0). Returns (q values fp32 [..., k], scale bytes [..., k/16],
    dequantised fp32 [..., k]) with the reference's fp32 operation order:
    gs = 1 / input_scale; sf = e4m3(gs * amax / 6); inv = sf != 0 ? gs / sf : 0; q = rne_e2m1(x * inv)."""
    x = np.asarray(x, dtype=np.float32)
    shape = x.shape
    xb = x.reshape(shape[:-1] + (-1, FP4_BLOCK))
    gs = f32(1.0) / f32(input_scale)
    amax = np.abs(xb).max(-1, keepdims=True)
    sf_code = e4m3_encode((gs * amax).astype(np.float32) / E2M1_MAX)
    sf = e4m3_decode(sf_code)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(sf != 0, (gs / sf).astype(np.float32), f32(0.0)).astype(np.float32)
    q = round_e2m1((xb * inv).astype(np.float32))
    deq = ((q * sf).astype(np.float32) / gs).astype(np.float32)
    return q.reshape(shape), sf_code[..., 0], deq.reshape(shape)


def quant_act_nvfp4(x: np.ndarray, input_scale: float) -> np.ndarray:
    """Fake-quantised activations (fp32), exactly the reference's quant_act_nvfp4."""
    return quant_act_nvfp4_parts(x, input_scale)[2]


def quant_act_codes(x: np.ndarray, input_scale: float):
    """What the device quantiser must emit for x [M][K]: packed codes [M][K/2] (sign of zero kept as the
    hardware conversion does) and row-major scale bytes [M][K/16]."""
    q, sf_code, _ = quant_act_nvfp4_parts(x, input_scale)
    return pack_codes(encode_e2m1(q, signed_zero=True)), sf_code


def quant_act_dynamic(x: np.ndarray):
    """Per-token dynamic quantisation (the draft model's rule, engine/src/draft.cu:70-111): row scale
    amax(row) / (6 * 448), 1 for an all-zero row, then the activation quantiser with that scale per row. Returns
    (packed codes [M][K/2], scale bytes [M][K/16], row scales [M] fp32)."""
    x = np.asarray(x, dtype=np.float32)
    amax = np.abs(x).max(-1)
    rs = np.where(amax > 0, (amax / f32(E2M1_MAX * E4M3_MAX)).astype(np.float32), f32(1.0)).astype(np.float32)
    codes = np.empty((x.shape[0], x.shape[1] // 2), dtype=np.uint8)
    sfs = np.empty((x.shape[0], x.shape[1] // FP4_BLOCK), dtype=np.uint8)
    for m in range(x.shape[0]):
        codes[m], sfs[m] = (t[0] for t in quant_act_codes(x[m:m + 1], rs[m]))
    return codes, sfs, rs


def weight_global_scale(w: np.ndarray) -> np.float32:
    """weight_scale_2 = amax(W) / (6 * 448)."""
    return f32(np.abs(np.asarray(w, dtype=np.float32)).max() / (E2M1_MAX * E4M3_MAX))


def quant_weight_rtn(w: np.ndarray, gscale: float | None = None):
    """Round-to-nearest NVFP4 weight quantiser. Returns (packed codes [N][K/2], scale bytes [N][K/16], scale_2).
    sf = e4m3(amax_block / 6 / scale_2); q = rne_e2m1(w / (sf * scale_2)) (divisor 1 where the scale is 0);
    zeros are packed as code 0 whatever their sign."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    gscale = weight_global_scale(w) if gscale is None else f32(gscale)
    wb = w.reshape(n, k // FP4_BLOCK, FP4_BLOCK)
    sf_code = e4m3_encode((np.abs(wb).max(-1) / E2M1_MAX).astype(np.float32) / gscale)
    sf = e4m3_decode(sf_code)
    s = np.repeat((sf * gscale).astype(np.float32), FP4_BLOCK, axis=1)
    q = round_e2m1((w / np.where(s > 0, s, f32(1.0))).astype(np.float32))
    return pack_codes(encode_e2m1(q, signed_zero=False)), sf_code, gscale


# Offsets of the E4M3 codes the searched weight quantiser tries around the code of amax / 6, in its order
# (engine/src/kernels.cu:187-188): the rounded code first, so that it stays on a tie, 4 below, 8 above.
WEIGHT_SEARCH_OFFSETS = (0, -1, -2, -3, -4, 1, 2, 3, 4, 5, 6, 7, 8)


def quant_weight_search(w: np.ndarray, gscale: float):
    """The load-time weight quantiser with a per-block scale search (quant_fp4_weight_kernel,
    engine/src/kernels.cu:167-206; the same search as scripts/quantize_proj.py:77-97 with a wider range): for every
    16-element block the E4M3 scale code c in {c0, c0-1..c0-4, c0+1..c0+8} (clamped to 1..126, c0 = code of
    amax / 6 / gscale) with the smallest squared error sum((v - e2m1(v / s) * s)^2), s = e4m3(c) * gscale, the first
    of equals winning; an all-zero block keeps c0. Every operation is a separate fp32 operation, the error summed
    in element order. Returns (packed codes [N][K/2] with the sign of zero as the hardware conversion leaves it,
    scale codes [N][K/16])."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    g = f32(gscale)
    wb = w.reshape(n, k // FP4_BLOCK, FP4_BLOCK)
    amax = np.abs(wb).max(-1)
    c0 = e4m3_encode(((amax / E2M1_MAX).astype(np.float32) / g).astype(np.float32)).astype(np.int32)
    best = c0.copy()
    best_err = np.full(c0.shape, np.inf, dtype=np.float32)
    for d in WEIGHT_SEARCH_OFFSETS:
        c = np.clip(c0 + d, 1, 126)
        s = (e4m3_decode(c.astype(np.uint8)) * g).astype(np.float32)[..., None]
        inv = (f32(1.0) / s).astype(np.float32)
        q = round_e2m1((wb * inv).astype(np.float32))
        diff = (wb - (q * s).astype(np.float32)).astype(np.float32)
        sq = (diff * diff).astype(np.float32)
        err = np.zeros(c0.shape, dtype=np.float32)
        for j in range(0, FP4_BLOCK, 2):  # the kernel adds a^2 + b^2 of one byte, then that to the running sum
            err = (err + (sq[..., j] + sq[..., j + 1]).astype(np.float32)).astype(np.float32)
        better = (err < best_err) & (amax > 0)
        best = np.where(better, c, best)
        best_err = np.where(better, err, best_err)
    sf = e4m3_decode(best.astype(np.uint8))
    sg = (sf * g).astype(np.float32)
    inv = np.where(sf != 0, (f32(1.0) / np.where(sg != 0, sg, f32(1.0))).astype(np.float32), f32(0.0))[..., None]
    q = round_e2m1((wb * inv).astype(np.float32)).reshape(n, k)
    return pack_codes(encode_e2m1(q, signed_zero=True)), best.astype(np.uint8)


def dequant_nvfp4(codes: np.ndarray, sf_code: np.ndarray, scale_2: float) -> np.ndarray:
    """W = e2m1(code) * e4m3(scale) * scale_2, in fp32 and in that order."""
    w = unpack_e2m1(codes)
    s = np.repeat(e4m3_decode(sf_code), FP4_BLOCK, axis=-1)
    return ((w * s).astype(np.float32) * f32(scale_2)).astype(np.float32)


# ----------------------------------------------------------------------------------------------- GEMM


def gemm_codes(a_codes, a_sf, b_codes, b_sf, alpha=1.0) -> np.ndarray:
    """alpha * A . B^T in fp64 from raw NVFP4 operands (codes [rows][K/2], row-major scale bytes), the form the
    reference's GPU tests use for their expected value (engine/tests/test_gemm.py:17-22,38)."""
    a = unpack_e2m1(a_codes).astype(np.float64) * np.repeat(e4m3_decode(a_sf).astype(np.float64), 16, -1)
    b = unpack_e2m1(b_codes).astype(np.float64) * np.repeat(e4m3_decode(b_sf).astype(np.float64), 16, -1)
    return float(alpha) * (a @ b.T)


def qlinear(x, w_codes, w_sf, scale_2, input_scale, dtype=np.float64) -> np.ndarray:
    """y = quant_act(x) @ dequant(W)^T: the reference's QLinear("nvfp4", act_quant=True)."""
    xq = quant_act_nvfp4(x, input_scale).astype(dtype)
    w = dequant_nvfp4(w_codes, w_sf, scale_2).astype(dtype)
    return xq @ w.T


def silu_mul(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate = np.asarray(gate, dtype=np.float64)
    return gate / (1.0 + np.exp(-gate)) * np.asarray(up, dtype=np.float64)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """x / rms(x) * (1 + w) over the last axis, evaluated in fp64 (the reference evaluates it in fp32)."""
    x64 = np.asarray(x, dtype=np.float64)
    r = 1.0 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + eps)
    return x64 * r * (1.0 + np.asarray(w, dtype=np.float64))


def rms_norm_fixed_order(x: np.ndarray, w: np.ndarray, eps: float):
    """fp32 [T][D] (D a multiple of 512), w fp32 [D] -> (fp32 [T][D], 1 / rms [T]) with every operation a separate
    fp32 operation in the order of the fused kernel."""
    x = np.asarray(x, dtype=np.float32)
    w = np.asarray(w, dtype=np.float32)
    T, D = x.shape
    assert D % 512 == 0
    lanes = x.reshape(T, D // 16, 16)
    ss = np.zeros((T, D // 16), dtype=np.float32)
    for j in range(16):  # each lane: its 16 squares in order
        ss = (ss + (lanes[:, :, j] * lanes[:, :, j]).astype(np.float32)).astype(np.float32)
    ss = ss.reshape(T, D // 512, 32)
    lane = np.arange(32)
    for o in (16, 8, 4, 2, 1):  # butterfly over the 32 lanes of a warp
        ss = (ss + ss[:, :, lane ^ o]).astype(np.float32)
    total = np.zeros(T, dtype=np.float32)
    for i in range(D // 512):  # the warps' sums in order
        total = (total + ss[:, i, 0]).astype(np.float32)
    r = (f32(1.0) / np.sqrt(((total / f32(D)).astype(np.float32) + f32(eps)).astype(np.float32)).astype(np.float32)).astype(np.float32)
    y = ((x * r[:, None]).astype(np.float32) * (f32(1.0) + w).astype(np.float32)[None, :]).astype(np.float32)
    return y, r


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest bf16 (ties to even), returned as fp32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def within_tolerance(out, ref, rel=2e-3, abs_=1e-3):
    """|out - ref| <= rel * |ref| + abs_ elementwise (the benchmark's acceptance rule for the fp32-accumulated
    result)."""
    out, ref = np.asarray(out, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return np.abs(out - ref) <= rel * np.abs(ref) + abs_


def bf16_half_ulp(x):
    """Half the spacing of bf16 (8 significant bits) at |x|: the most a round-to-nearest store can move a value."""
    a = np.maximum(np.abs(np.asarray(x, dtype=np.float64)), 2.0**-126)
    return np.exp2(np.floor(np.log2(a)) - 8)


def within_tolerance_bf16(out, ref, rel=2e-3, abs_=1e-3):
    """The acceptance rule for a result that was stored as bf16: the fp32-accumulated value may be off by
    rel * |ref| + abs_, and rounding it to bf16 (unit roundoff 2^-8, more than rel) moves it by at most half a
    bf16 ulp of a value that large."""
    out, ref = np.asarray(out, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    slack = rel * np.abs(ref) + abs_
    return np.abs(out - ref) <= slack + bf16_half_ulp(np.abs(ref) + slack)
