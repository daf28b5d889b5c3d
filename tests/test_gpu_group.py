"""The grouped weight-streaming GEMM (q27b_skinny_fp4_group): a list of skinny GEMMs run as one persistent launch
must reproduce, BIT FOR BIT, the results of the per-GEMM entry points called one by one - for a whole layer of the
model (q|k|v stacked with three alpha segments, o with a residual, gate | up with the SiLU*mul epilogue, down in
bf16) at every token count of the decode sweep, on a workspace left behind by the previous launch, for several layers
in one launch, and for small odd shapes."""

import ctypes

import numpy as np
import pytest
import torch

from helpers import DEV, dev, fp4_operand, rel_err, swizzled_dev, workspace
from q27b200.group import EPI_BF16, EPI_F32, EPI_GLU_BF16, Fp4Group, GroupProblem
from q27b200.q27lib import call

pytestmark = pytest.mark.gpu
WS = 48 << 20

_ops = {}


def operand(rows, K, seed):
    if (rows, K, seed) not in _ops:
        c, sf, dq = fp4_operand(rows, K, np.random.RandomState(seed))
        _ops[(rows, K, seed)] = (dev(c), swizzled_dev(sf), dq)
    return _ops[(rows, K, seed)]


def problem(N, K, epi, a, a_sf, w, w_sf, d, alphas=(1.0,), begins=(0,), alpha_up=1.0, c=None):
    p = GroupProblem()
    p.N, p.K, p.epilogue, p.alpha_count = N, K, epi, len(alphas)
    for i, (b, al) in enumerate(zip(begins, alphas)):
        p.alpha_begin[i], p.alpha[i] = b, al
    p.alpha_up, p.beta = alpha_up, 1.0 if c is not None else 0.0
    p.a, p.a_sf, p.w, p.w_sf = a.data_ptr(), a_sf.data_ptr(), w.data_ptr(), w_sf.data_ptr()
    p.c = c.data_ptr() if c is not None else None
    p.d = d.data_ptr()
    return p


QKV_BEGIN, QKV_ALPHA = (0, 5120, 6144), (0.37, 0.11, 0.23)


def layer_by_single_calls(M, ws, res):
    """The four projections of one layer through the per-GEMM entry points; returns their outputs."""
    a5, a5sf, _ = operand(128, 5120, 11)
    a17, a17sf, _ = operand(128, 17408, 12)
    out = {}
    w, wsf, _ = operand(7168, 5120, 21)
    out["qkv"] = torch.empty(M, 7168, device=DEV)
    call("q27t_skinny_fp4_segments", M, 7168, 5120, a5, a5sf, w, wsf, 3, (ctypes.c_int * 3)(*QKV_BEGIN),
         (ctypes.c_float * 3)(*QKV_ALPHA), None, 0.0, out["qkv"], ws, ws.numel())
    w, wsf, _ = operand(5120, 5120, 22)
    out["o"] = torch.empty(M, 5120, device=DEV)
    call("q27t_skinny_fp4", M, 5120, 5120, a5, a5sf, w, wsf, 0.5, res[:M], 1.0, out["o"], ws, ws.numel())
    w, wsf, _ = operand(34816, 5120, 23)
    out["gate_up"] = torch.empty(M, 17408, dtype=torch.bfloat16, device=DEV)
    call("q27t_skinny_fp4_glu_bf16", M, 17408, 5120, a5, a5sf, w, wsf, 0.013, 0.021, out["gate_up"], ws, ws.numel())
    w, wsf, _ = operand(5120, 17408, 24)
    out["down"] = torch.empty(M, 5120, dtype=torch.bfloat16, device=DEV)
    call("q27t_skinny_fp4_bf16", M, 5120, 17408, a17, a17sf, w, wsf, 0.7, out["down"], ws, ws.numel())
    return out


def layer_problems(M, res, outs):
    a5, a5sf, _ = operand(128, 5120, 11)
    a17, a17sf, _ = operand(128, 17408, 12)
    ps = []
    w, wsf, _ = operand(7168, 5120, 21)
    ps.append(problem(7168, 5120, EPI_F32, a5, a5sf, w, wsf, outs["qkv"], QKV_ALPHA, QKV_BEGIN))
    w, wsf, _ = operand(5120, 5120, 22)
    ps.append(problem(5120, 5120, EPI_F32, a5, a5sf, w, wsf, outs["o"], (0.5,), c=res))
    w, wsf, _ = operand(34816, 5120, 23)
    ps.append(problem(34816, 5120, EPI_GLU_BF16, a5, a5sf, w, wsf, outs["gate_up"], (0.013,), alpha_up=0.021))
    w, wsf, _ = operand(5120, 17408, 24)
    ps.append(problem(5120, 17408, EPI_BF16, a17, a17sf, w, wsf, outs["down"], (0.7,)))
    return ps


def fresh_outputs(M):
    return {"qkv": torch.full((M, 7168), float("nan"), device=DEV), "o": torch.full((M, 5120), float("nan"), device=DEV),
            "gate_up": torch.zeros(M, 17408, dtype=torch.bfloat16, device=DEV),
            "down": torch.zeros(M, 5120, dtype=torch.bfloat16, device=DEV)}


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32, 64, 128])
def test_group_of_a_layer_equals_single_calls(M):
    res = torch.randn(128, 5120, device=DEV)
    want = layer_by_single_calls(M, workspace(WS), res)
    # sanity of the reference side against the fp64 product (one projection; the others have tests of their own)
    _, _, adq = operand(128, 5120, 11)
    _, _, wdq = operand(5120, 5120, 22)
    assert rel_err(want["o"].cpu().numpy(), 0.5 * (adq[:M] @ wdq.T) + res[:M].cpu().numpy().astype(np.float64)) < 1e-5
    got = fresh_outputs(M)
    grp = Fp4Group(M, layer_problems(M, res[:M].contiguous(), got))
    assert grp.ctas == 2 * torch.cuda.get_device_properties(0).multi_processor_count and grp.counters == 136
    grp.ws[grp.partials_offset:] = 0xFF  # partial tiles poisoned with NaN bit patterns
    for _ in range(2):  # the second launch runs on the counters and partial tiles the first one left behind
        for t in got.values():
            t.fill_(float("nan")) if t.dtype == torch.float32 else t.zero_()
        grp.run_sync()
        for name in want:
            assert torch.equal(got[name], want[name]), f"{name} differs at M={M}"


def test_group_of_three_layers_in_place_residual():
    """Several layers in one launch (the same weights, separate outputs), o with its residual in place."""
    M = 16
    res = torch.randn(128, 5120, device=DEV)
    want = layer_by_single_calls(M, workspace(WS), res)
    probs, outs = [], []
    for _ in range(3):
        got = fresh_outputs(M)
        got["o"] = res[:M].clone()
        ps = layer_problems(M, got["o"], got)  # c aliases d
        probs += ps
        outs.append(got)
    grp = Fp4Group(M, probs)
    grp.run_sync()
    for got in outs:
        for name in want:
            assert torch.equal(got[name], want[name]), name


@pytest.mark.parametrize("M", [3, 16, 77])
def test_group_of_small_and_odd_shapes(M):
    """K not a multiple of 256, a single tile, a tile count below the CTA count, and the contiguous-range split of a
    very wide weight in one group."""
    shapes = [(384, 448), (128, 5120), (1024, 5120), (128, 64), (44032, 5120)]
    ws = workspace(WS)
    probs, got, want = [], [], []
    for i, (N, K) in enumerate(shapes):
        a, asf, _ = operand(128, K, 100 + i)
        w, wsf, _ = operand(N, K, 200 + i)
        d = torch.empty(M, N, device=DEV)
        call("q27t_skinny_fp4", M, N, K, a, asf, w, wsf, 0.37, None, 0.0, d, ws, ws.numel())
        want.append(d)
        g = torch.full((M, N), float("nan"), device=DEV)
        got.append(g)
        probs.append(problem(N, K, EPI_F32, a, asf, w, wsf, g, (0.37,)))
    grp = Fp4Group(M, probs)
    for _ in range(2):
        grp.run_sync()
        for (N, K), g, w_ in zip(shapes, got, want):
            assert torch.equal(g, w_), (N, K)


def test_group_rejects_bad_arguments():
    a, asf, _ = operand(128, 5120, 11)
    w, wsf, _ = operand(5120, 5120, 22)
    d = torch.empty(4, 5120, device=DEV)
    with pytest.raises(RuntimeError, match="M must be 1..128"):
        Fp4Group(129, [problem(5120, 5120, EPI_F32, a, asf, w, wsf, d)])
    with pytest.raises(RuntimeError, match="multiple of 128"):
        Fp4Group(4, [problem(5000, 5120, EPI_F32, a, asf, w, wsf, d)])
    with pytest.raises(RuntimeError, match="residual needs the fp32 epilogue"):
        Fp4Group(4, [problem(5120, 5120, EPI_BF16, a, asf, w, wsf, d, c=d)])
    grp = Fp4Group(4, [problem(5120, 5120, EPI_F32, a, asf, w, wsf, d)])
    small = torch.zeros(64, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="workspace too small"):
        call("q27t_skinny_fp4_group", grp.table_host, grp.table_dev, small, small.numel())


@pytest.mark.parametrize("M,tokens_on_n", [(1, False), (16, False), (32, False), (33, False), (64, False), (64, True), (100, False), (128, False), (128, True)])
def test_group_of_whole_tiles_equals_the_many_row_gemm(M, tokens_on_n):
    """Whole-tile mode (no K split): every output is one accumulation chain over all of K, exactly what the many-row
    GEMM computes - bit for bit, for every epilogue; a stacked weight with three alphas equals the many-row GEMM of
    each part with its own alpha. Two layers in one launch. From 33 tokens the group is planned on tiles of 256 weight
    rows with the tokens on the MMA's M side (another kernel, the same bits) unless the caller keeps the few-token roles."""
    res = torch.randn(128, 5120, device=DEV)
    a5, a5sf, _ = operand(128, 5120, 11)
    a17, a17sf, _ = operand(128, 17408, 12)
    want = {}
    w, wsf, _ = operand(7168, 5120, 21)
    want["qkv"] = torch.empty(M, 7168, device=DEV)
    for (b, e), al in zip(((0, 5120), (5120, 6144), (6144, 7168)), QKV_ALPHA):
        part = torch.empty(M, e - b, device=DEV)
        # rows b..e of the stacked weight: codes and scale atoms of whole 128-row tiles
        call("q27t_gemm_fp4", M, e - b, 5120, a5, a5sf, w[b:e], wsf[b // 128 * (5120 // 64) * 512:], al, None, 0.0, part)
        want["qkv"][:, b:e] = part
    w, wsf, _ = operand(5120, 5120, 22)
    want["o"] = torch.empty(M, 5120, device=DEV)
    call("q27t_gemm_fp4", M, 5120, 5120, a5, a5sf, w, wsf, 0.5, res[:M].contiguous(), 1.0, want["o"])
    w, wsf, _ = operand(34816, 5120, 23)
    want["gate_up"] = torch.empty(M, 17408, dtype=torch.bfloat16, device=DEV)
    call("q27t_gemm_fp4_glu_bf16", M, 17408, 5120, a5, a5sf, w, wsf, 0.013, 0.021, want["gate_up"])
    w, wsf, _ = operand(5120, 17408, 24)
    want["down"] = torch.empty(M, 5120, dtype=torch.bfloat16, device=DEV)
    call("q27t_gemm_fp4_bf16", M, 5120, 17408, a17, a17sf, w, wsf, 0.7, want["down"])
    outs = [fresh_outputs(M) for _ in range(2)]
    probs = []
    for got in outs:
        probs += layer_problems(M, res[:M].contiguous(), got)
    grp = Fp4Group(M, probs, whole_tiles=True, tokens_on_n=tokens_on_n)
    wide = M > 32 and not tokens_on_n
    assert grp.tokens_tile == (256 if wide else 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128)
    assert grp.slots == 0 and grp.counters == 0 and grp.pieces == 2 * (204 if wide else 408) and grp.ctas <= (148 if wide else 296)
    grp.run_sync()
    for got in outs:
        for name in want:
            assert torch.equal(got[name], want[name]), f"{name} differs at M={M}"


@pytest.mark.parametrize("M", [33, 77, 128])
def test_whole_tile_group_on_256_row_tiles_of_small_and_odd_shapes(M):
    """The 256-row form (33..128 tokens, whole tiles): a reduction length that ends inside a stage (K = 384: the last
    stage holds two of four MMA steps), a single tile, fewer tiles than CTAs, one tile per CTA and more, every epilogue -
    against the many-row GEMM, bit for bit, twice (the second launch finds the first one's state). A weight whose rows
    are not a multiple of 256 sends the whole group back to 128-row tiles."""
    shapes = [(256, 384, EPI_F32), (512, 5120, EPI_BF16), (256, 128, EPI_F32), (148 * 256, 256, EPI_BF16), (1024, 1024, EPI_GLU_BF16),
              (6400, 640, EPI_F32)]
    probs, got, want, keep = [], [], [], []
    res = torch.randn(M, 6400, device=DEV)
    for i, (N, K, epi) in enumerate(shapes):
        a, asf, _ = operand(128, K, 300 + i)
        w, wsf, _ = operand(N, K, 400 + i)
        if epi == EPI_GLU_BF16:
            d = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
            call("q27t_gemm_fp4_glu_bf16", M, N // 2, K, a, asf, w, wsf, 0.013, 0.021, d)
            g = torch.zeros_like(d)
            probs.append(problem(N, K, epi, a, asf, w, wsf, g, (0.013,), alpha_up=0.021))
        elif epi == EPI_BF16:
            d = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            call("q27t_gemm_fp4_bf16", M, N, K, a, asf, w, wsf, 0.37, d)
            g = torch.zeros_like(d)
            probs.append(problem(N, K, epi, a, asf, w, wsf, g, (0.37,)))
        else:
            c = res[:, :N].contiguous() if N == 6400 else None
            keep.append(c)  # (the problem record holds its address)
            d = torch.empty(M, N, device=DEV)
            call("q27t_gemm_fp4", M, N, K, a, asf, w, wsf, 0.37, c, 0.5 if c is not None else 0.0, d)
            g = torch.full((M, N), float("nan"), device=DEV)
            p = problem(N, K, epi, a, asf, w, wsf, g, (0.37,), c=c)
            p.beta = 0.5 if c is not None else 0.0
            probs.append(p)
        got.append(g)
        want.append(d)
    grp = Fp4Group(M, probs, whole_tiles=True)
    assert grp.tokens_tile == 256 and grp.ctas <= 148 and grp.slots == 0
    for _ in range(2):
        grp.run_sync()
        for s, g, w_ in zip(shapes, got, want):
            assert torch.equal(g, w_), s
    a, asf, _ = operand(128, 256, 1)
    w, wsf, _ = operand(384, 256, 2)
    odd = Fp4Group(M, probs + [problem(384, 256, EPI_F32, a, asf, w, wsf, torch.empty(M, 384, device=DEV))], whole_tiles=True)
    assert odd.tokens_tile in (64, 128)


@pytest.mark.parametrize("M", [1, 5, 16, 32])
def test_fused_gather_stores_on_one_gpu(M):
    """The stores of the fused gather without a second GPU: the "peers" are two more buffers in this GPU's memory, so
    every output must appear three times, identical to a launch without peers - for the fp32 (+ residual), bf16 and
    SiLU*mul epilogues, whole tiles (up to 16 tokens these leave through the token-major staging tile) and cut tiles -
    and the launch must raise this GPU's word once in each peer's signal block."""
    from q27b200.peer import GroupPeers

    shapes = [(256, 384, EPI_F32), (640, 5120, EPI_BF16), (1024, 1024, EPI_GLU_BF16), (5120, 5120, EPI_F32)]
    res = torch.randn(M, 5120, device=DEV)
    for whole in (True, False):
        sizes = [M * (N // 2 if epi == EPI_GLU_BF16 else N) * (4 if epi == EPI_F32 else 2) for N, K, epi in shapes]
        offs = np.concatenate([[0], np.cumsum([(sz + 255) // 256 * 256 for sz in sizes])])
        region = torch.zeros(3, int(offs[-1]), dtype=torch.uint8, device=DEV)  # [local, "peer" 0, "peer" 1]
        plain = torch.zeros(int(offs[-1]), dtype=torch.uint8, device=DEV)
        signals = torch.zeros(3, 64, dtype=torch.int32, device=DEV)

        def problems(base):
            ps = []
            for i, (N, K, epi) in enumerate(shapes):
                a, asf, _ = operand(128, K, 500 + i)
                w, wsf, _ = operand(N, K, 600 + i)
                d = base[int(offs[i]):int(offs[i]) + sizes[i]]
                c = res if N == 5120 and epi == EPI_F32 else None
                al = (0.013,) if epi == EPI_GLU_BF16 else (0.37,)
                ps.append(problem(N, K, epi, a, asf, w, wsf, d, al, alpha_up=0.021, c=c))
            return ps

        Fp4Group(M, problems(plain), whole_tiles=whole, tokens_on_n=True).run_sync()
        grp = Fp4Group(M, problems(region[0]), whole_tiles=whole, tokens_on_n=True)
        peers = GroupPeers()
        peers.n_peers, peers.my_slot, peers.signals = 2, 3, signals[0].data_ptr()
        for j in range(2):
            peers.out_delta[j] = region[j + 1].data_ptr() - region[0].data_ptr()
            peers.peer_signals[j] = signals[j + 1].data_ptr()
        for launch in (1, 2):
            region.zero_()
            grp.launch_gather(peers)
            torch.cuda.synchronize()
            for j in range(3):
                assert torch.equal(region[j], plain), f"copy {j} differs (M={M}, whole={whole})"
            assert signals[1:, 3].tolist() == [launch, launch] and int(signals[0, 9]) == 0
    from q27b200.q27lib import device_status

    assert device_status() == 0
