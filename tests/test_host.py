"""CPU-only checks of the host side: the C-ABI library loads and exports every declared symbol, the work split of
the weight-streaming GEMM covers every unit exactly once, the layout helpers and the load-time quantiser agree
with the oracle, and precondition failures come back as error codes with a message (no GPU needed)."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from q27b200 import configs, layouts, shard, weights
from q27b200.q27lib import SIGNATURES, TEST_SIGNATURES, call, last_error, lib, scaffold_lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(header="capi.h"):
    text = open(os.path.join(ROOT, "include", "q27b200", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q27[bt]?_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 35
    l = lib()
    for n in names:
        assert hasattr(l, n), f"{n} is declared in capi.h but not exported"
        assert n in SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(SIGNATURES) == names  # and nothing is bound that the header does not declare
    # the scaffolding of the test suite lives in a library of its own, which the product library does not export
    scaffolding = declared_functions("testing.h")
    assert sorted(TEST_SIGNATURES) == scaffolding
    for n in scaffolding:
        assert hasattr(scaffold_lib(), n) and not hasattr(l, n), n


def test_sf_layout_matches_oracle():
    l = lib()
    for rows, kb in [(1, 320), (37, 320), (128, 4), (300, 1088), (5120, 1088)]:
        assert l.q27b_sf_bytes(rows, kb) == O.sf_bytes(rows, kb) == layouts.sf_bytes(rows, kb)
    rng = np.random.RandomState(0)
    for _ in range(200):
        kb = int(rng.randint(1, 2000))
        r, k = int(rng.randint(0, 40000)), int(rng.randint(0, kb))
        assert l.q27b_sf_offset(r, k, kb) == int(O.sf_offset(r, k, kb))
    assert np.array_equal(layouts.sf_index(300, 1088), O.sf_offset(np.arange(300)[:, None], np.arange(1088)[None, :], 1088))
    for r in (0, 63, 64, 100, 17407):
        for h in (0, 1):
            assert l.q27b_glu_row(r, h) == int(O.glu_row(r, h))
    assert np.array_equal(layouts.glu_rows(384), O.glu_rows(384))


def plan(N, K, slots):
    l = scaffold_lib()
    grid, units, split = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int()
    seg = (ctypes.c_int * (4 * 2048))()
    l.q27b_skinny_plan(N, K, slots, -1, None, 0, ctypes.byref(grid), ctypes.byref(units), ctypes.byref(split))
    pieces = []
    for g in range(grid.value):
        n = l.q27b_skinny_plan(N, K, slots, g, seg, 2048, None, None, None)
        assert 1 <= n <= 2048
        pieces.append([tuple(seg[4 * i:4 * i + 4]) for i in range(n)])
    return grid.value, units.value, split.value, pieces


@pytest.mark.parametrize("N,K", [(5120, 5120), (1024, 5120), (34816, 5120), (5120, 17408), (128, 5120), (128, 64),
                                 (384, 512), (248320, 5120), (640, 5120), (4352, 5120), (128, 65536)])
@pytest.mark.parametrize("slots", [296, 148, 7])
def test_skinny_plan_covers_every_unit_once(N, K, slots):
    grid, units, split, pieces = plan(N, K, slots)
    tiles, chunks = N // 128, (K + 255) // 256
    assert units == tiles * chunks and 1 <= grid <= min(slots, units)
    cover = np.zeros((tiles, chunks), dtype=np.int32)
    slot_of = {}
    sizes = []
    l = scaffold_lib()
    for g, segs in enumerate(pieces):
        sizes.append(sum(c1 - c0 for _, c0, c1, _ in segs))
        for t, c0, c1, slot in segs:
            assert 0 <= c0 < c1 <= chunks
            cover[t, c0:c1] += 1
            whole = c0 == 0 and c1 == chunks
            assert (slot == -1) == whole
            if not whole:
                assert slot >= 0 and slot not in slot_of  # every partial tile has a slot of its own
                slot_of[slot] = (t, c0)
        if split == 0:  # ranges: a cut tile at the end of the range is worked on first, the rest in ascending order
            order = [t * chunks + c0 for t, c0, _, _ in segs]
            if len(segs) > 1 and order[0] == max(order):
                assert order[1:] == sorted(order[1:])
            else:
                assert order == sorted(order)
            assert len([1 for seg in segs if seg[3] >= 0]) <= 2  # at most two partial tiles per CTA
    assert (cover == 1).all()
    if split == 0:
        assert max(sizes) - min(sizes) <= 1  # every CTA streams the same number of bytes (+- one unit)
    # the lookup used when a cut tile is summed lists exactly that tile's partial tiles, in ascending K order
    buf = (ctypes.c_int * 2048)()
    for t in sorted({0, tiles // 2, tiles - 1}):
        n = l.q27b_skinny_tile_parts(N, K, slots, t, buf, 2048)
        parts = [slot_of[buf[i]] for i in range(n)] if n > 1 else []
        assert all(pt == t for pt, _ in parts) and [c for _, c in parts] == sorted(c for _, c in parts)
        assert n == max(1, sum(1 for pt, _ in slot_of.values() if pt == t))
    need = max(slot_of) + 1 if slot_of else 0
    assert need <= 2 * slots  # partial tiles fit the workspace bound stated in the header


def test_skinny_plan_choices():
    """The cost model's picks for the benchmark shapes on a 148-SM device (two CTA slots per SM)."""
    assert plan(34816, 5120, 296)[2] == 1      # gate | up: one whole tile per CTA, nothing is cut
    assert plan(5120, 5120, 296)[2] == 7       # q / o: seven aligned K-parts per tile
    assert plan(5120, 17408, 148)[2] == 0      # down at many tokens: contiguous ranges
    assert plan(248320, 5120, 296)[2] == 0     # lm_head: contiguous ranges (no wave quantisation)


def group_plan(shapes, slots, rotate=0, whole=0):
    n = len(shapes)
    Ns, Ks = (ctypes.c_int * n)(*[s[0] for s in shapes]), (ctypes.c_int * n)(*[s[1] for s in shapes])
    ctas, nslots, counters = ctypes.c_int(), ctypes.c_int64(), ctypes.c_int()
    l = scaffold_lib()
    count = l.q27b_skinny_group_plan(n, Ns, Ks, slots, whole, rotate, None, 0, ctypes.byref(ctas), ctypes.byref(nslots), ctypes.byref(counters))
    buf = (ctypes.c_int * (9 * count))()
    assert l.q27b_skinny_group_plan(n, Ns, Ks, slots, whole, rotate, buf, count, None, None, None) == count
    pieces = [tuple(buf[9 * i:9 * i + 9]) for i in range(count)]
    return ctas.value, nslots.value, counters.value, pieces


LAYER_SHAPES = [(7168, 5120), (5120, 5120), (34816, 5120), (5120, 17408)]  # q|k|v stacked, o, gate|up, down


@pytest.mark.parametrize("shapes,slots", [(LAYER_SHAPES, 296), (LAYER_SHAPES * 3, 296), ([(384, 448), (128, 5120), (248320, 5120)], 296),
                                          (LAYER_SHAPES, 7), ([(1024, 5120)], 264)])
def test_group_schedule_keeps_each_problems_own_split(shapes, slots):
    """The grouped launch deals the pieces of all problems to the CTAs, but every problem is cut exactly as its
    stand-alone launch cuts it (same pieces, and the pieces of a cut tile in consecutive slots in ascending K order):
    that is what makes the grouped results bit-identical to per-GEMM calls."""
    ctas, nslots, counters, pieces = group_plan(shapes, slots)
    assert 1 <= ctas <= slots
    by_problem = {}
    loads = np.zeros(ctas, dtype=np.int64)
    last_key = {}
    for cta, prob, tile, c0, c1, slot, nparts, slot0, sums in pieces:
        assert 0 <= cta < ctas
        by_problem.setdefault(prob, []).append((tile, c0, c1, slot, nparts, slot0, sums))
        loads[cta] += c1 - c0
        # a CTA walks its pieces of cut tiles first, then its whole tiles, each in problem order
        assert last_key.get(cta, (-1, -1, -1, -1)) < (int(nparts == 1), prob, tile, c0)
        last_key[cta] = (int(nparts == 1), prob, tile, c0)
    used_slots = set()
    cut_tiles = 0
    for prob, (N, K) in enumerate(shapes):
        _, _, _, alone = plan(N, K, slots)
        want = sorted((t, c0, c1) for segs in alone for t, c0, c1, _ in segs)
        got = sorted(by_problem[prob])
        assert [g[:3] for g in got] == want  # the same pieces as the stand-alone launch
        chunks = (K + 255) // 256
        tiles = {}
        for t, c0, c1, slot, nparts, slot0, sums in got:
            tiles.setdefault(t, []).append((c0, c1, slot, nparts, slot0, sums))
        for t, parts in tiles.items():
            assert all(p[3] == len(parts) for p in parts)
            assert parts[0][0] == 0 and parts[-1][1] == chunks and all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            # exactly one piece of a cut tile is marked: its CTA sums the tile (dealt round the pieces by tile index)
            assert [p[5] for p in parts] == [int(len(parts) > 1 and k == t % len(parts)) for k in range(len(parts))]
            if len(parts) == 1:
                assert parts[0][2] == -1
            else:
                cut_tiles += 1
                assert [p[2] for p in parts] == list(range(parts[0][4], parts[0][4] + len(parts)))  # ascending K = ascending slot
                for p in parts:
                    assert p[2] not in used_slots
                    used_slots.add(p[2])
    assert used_slots == set(range(nslots)) and counters == cut_tiles
    total = sum(N // 128 * ((K + 255) // 256) for N, K in shapes)
    assert loads.sum() == total
    biggest = max(p[4] - p[3] for p in pieces)
    assert loads.max() - loads.min() <= biggest  # longest-first dealing: no CTA is more than one piece ahead
    # the experimental order: the same pieces on the same CTAs, each CTA's list rotated to a start of its own
    _, _, _, rotated = group_plan(shapes, slots, rotate=1)
    assert sorted(rotated) == sorted(pieces)
    per_cta = {}
    for p in pieces:
        per_cta.setdefault(p[0], []).append(p)
    rot_cta = {}
    for p in rotated:
        rot_cta.setdefault(p[0], []).append(p)
    for g, lst in per_cta.items():
        k = g % len(lst)
        assert rot_cta[g] == lst[k:] + lst[:k]


def test_group_schedule_balance_on_a_layer():
    """One layer of the model on 296 CTA slots: every CTA streams 34 +- 2 of the 10080 stages."""
    ctas, _, _, pieces = group_plan(LAYER_SHAPES, 296)
    loads = np.zeros(ctas, dtype=np.int64)
    for cta, _, _, c0, c1, *_ in pieces:
        loads[cta] += c1 - c0
    assert ctas == 296 and loads.sum() == 10080 and loads.max() <= 36 and loads.min() >= 32


def test_weight_quantiser_matches_oracle(golden):
    w = torch.from_numpy(golden["w"])
    codes, sf, g = weights.quantize_weight_rtn(w)
    assert np.array_equal(codes.numpy(), golden["w_codes"]) and np.array_equal(sf.numpy(), golden["w_sf"])
    assert np.float32(g) == golden["w_gscale"]
    w2 = configs.make_w(384, 1024, 5)
    w2[7, 32:48] = 0
    c2, s2, g2 = weights.quantize_weight_rtn(w2, rows_per_step=100)
    co, so, go = O.quant_weight_rtn(w2.numpy())
    assert np.array_equal(c2.numpy(), co) and np.array_equal(s2.numpy(), so) and np.float32(g2) == go
    assert np.array_equal(weights.swizzle_scales(s2).numpy(), O.swizzle_sf(so))
    assert np.array_equal(weights.interleave_gate_up(c2).numpy(), O.interleave_glu(co))


def test_config_byte_counts():
    c = configs.CONFIGS
    assert c[0].algorithmic_bytes() == 14_766_080 and c[1].algorithmic_bytes() == 100_990_976
    assert c[2].algorithmic_bytes() == 55_902_208 and c[4].algorithmic_bytes() == 284_819_456
    assert c[4].flops() == 1_460_288_880_640
    assert configs.layer_weight_bytes() * 64 == 11_890_851_840
    assert configs.sweep_algorithmic_bytes(1) == 11_900_813_312 and configs.sweep_algorithmic_bytes(128) == 13_165_920_256


def test_configs_are_seeded():
    a, b = configs.make_x(configs.CONFIGS[1]), configs.make_x(configs.CONFIGS[1])
    assert torch.equal(a, b) and a.dtype == torch.bfloat16 and tuple(a.shape) == (16, 5120)
    w = configs.make_w(256, 512, 1001)
    assert torch.equal(w[128:], configs.make_w(256, 512, 1001, rows=slice(128, 256)))
    assert abs(float(w.std()) - 0.02) < 1e-3


# ---- precondition failures come back as -1 + message before any CUDA work ------------------------------------


def expect_error(fragment, name, *args):
    with pytest.raises(RuntimeError) as e:
        call(name, *args)
    assert fragment in str(e.value), str(e.value)
    assert fragment in last_error()


def test_argument_errors_without_a_gpu():
    expect_error("multiple of 64", "q27b_quant_fp4", 16, 1, 100, 1.0, 16, 16, None)
    expect_error("null pointer", "q27b_quant_fp4", None, 1, 128, 1.0, 16, 16, None)
    expect_error("aligned", "q27b_quant_fp4", 4, 1, 128, 1.0, 16, 16, None)
    expect_error("positive", "q27b_quant_fp4", 16, 1, 128, 0.0, 16, 16, None)
    zero, one = (ctypes.c_int * 1)(0), (ctypes.c_float * 1)(1.0)
    expect_error("M must be 1..128", "q27b_skinny_fp4", 129, 128, 256, 16, 16, 16, 16, 1, zero, one, None, 0.0, 16, 16, 1 << 20, None)
    expect_error("multiple of 128", "q27b_skinny_fp4", 1, 100, 256, 16, 16, 16, 16, 1, zero, one, None, 0.0, 16, 16, 1 << 20, None)
    expect_error("multiple of 64", "q27b_skinny_fp4", 1, 128, 100, 16, 16, 16, 16, 1, zero, one, None, 0.0, 16, 16, 1 << 20, None)
    expect_error("null pointer", "q27b_skinny_fp4", 1, 128, 256, None, 16, 16, 16, 1, zero, one, None, 0.0, 16, 16, 1 << 20, None)
    expect_error("16-byte aligned", "q27b_skinny_fp4", 1, 128, 256, 8, 16, 16, 16, 1, zero, one, None, 0.0, 16, 16, 1 << 20, None)
    expect_error("alpha segments", "q27b_skinny_fp4", 1, 128, 256, 16, 16, 16, 16, 5, zero, one, None, 0.0, 16, 16, 1 << 20, None)
    expect_error("multiple of 128", "q27b_gemm_fp4", 5, 128, 192, 16, 16, 16, 16, 1.0, None, 0.0, 16, None)
    expect_error("multiple of 64", "q27b_gemm_fp4_glu_bf16", 5, 100, 256, 16, 16, 16, 16, 1.0, 1.0, 16, None)
    # M == 0 is a no-op for the many-row GEMM and the quantisers, as in the reference
    call("q27b_gemm_fp4", 0, 128, 256, None, None, None, None, 1.0, None, 0.0, None, None)
    call("q27b_quant_fp4", None, 0, 128, 1.0, None, None, None)


# ---- N-sharding across ranks ---------------------------------------------------------------------------------


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_rows(world):
    for n_rows, glu in [(5120, False), (1024, False), (34816, True)]:
        spans = [shard.shard_rows(n_rows, world, r, glu) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n_rows
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0
        for a0, a1 in spans:
            assert a0 % 128 == 0 and (a1 - a0) % 128 == 0 and a1 > a0
    assert shard.shard_rows(34816, 8, 3, True) == (3 * 4352, 4 * 4352)
    # output columns owned by a rank: for gate | up every 128 interleaved rows give 64 outputs
    assert shard.output_columns(34816, 8, 3, True) == (3 * 2176, 4 * 2176)
    assert shard.output_columns(5120, 8, 7, False) == (7 * 640, 8 * 640)


def test_gathered_layout_to_row_major():
    world, M, n_out = 4, 3, 8
    full = np.arange(M * n_out).reshape(M, n_out)
    per = n_out // world
    gathered = np.stack([full[:, r * per:(r + 1) * per] for r in range(world)])  # what all_gather yields
    assert np.array_equal(shard.gathered_to_row_major(torch.from_numpy(gathered)).numpy(), full)


def test_group_schedule_whole_tiles():
    """Whole-tile mode: every tile is one piece, nothing is cut, no slots or counters; eight layers fill 296 CTAs
    evenly, one layer does not (its down-projection tiles are 68 stages long)."""
    ctas, nslots, counters, pieces = group_plan(LAYER_SHAPES * 8, 296, whole=1)
    assert nslots == 0 and counters == 0 and len(pieces) == 8 * 408
    assert all(p[5] == -1 and p[6] == 1 and p[8] == 0 and p[3] == 0 for p in pieces)
    chunks = {i: (K + 255) // 256 for i, (N, K) in enumerate(LAYER_SHAPES * 8)}
    assert all(p[4] == chunks[p[1]] for p in pieces)
    loads = np.zeros(ctas, dtype=np.int64)
    for p in pieces:
        loads[p[0]] += p[4] - p[3]
    assert loads.sum() == 8 * 10080 and loads.max() <= 1.07 * loads.mean()  # (a piece is 20 or 68 stages: 272 +- 16)
    ctas, _, _, pieces = group_plan(LAYER_SHAPES, 296, whole=1)
    loads = np.zeros(ctas, dtype=np.int64)
    for p in pieces:
        loads[p[0]] += p[4] - p[3]
    assert loads.max() == 68 and loads.max() > 1.9 * loads.sum() / 296
    # tiles of 256 weight rows on one CTA per SM (33..128 tokens): half as many pieces of the same lengths
    ctas, nslots, counters, pieces = group_plan(LAYER_SHAPES * 8, 148, whole=2)
    assert ctas == 148 and nslots == 0 and counters == 0 and len(pieces) == 8 * 204
    assert sorted(p[2] for p in pieces if p[1] == 2) == list(range(34816 // 256))
    loads = np.zeros(ctas, dtype=np.int64)
    for p in pieces:
        assert p[3] == 0 and p[4] == chunks[p[1]]
        loads[p[0]] += p[4]
    assert loads.sum() == 8 * 5040 and loads.max() <= 1.07 * loads.mean()
