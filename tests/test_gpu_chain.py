"""Chains of kernels as an engine runs them: launched back to back with programmatic dependent launch, captured
into a CUDA graph and replayed, with weights rotating between copies. Every other GPU test goes through the
synchronous one-kernel wrappers; these check that nothing is lost when kernels overlap their neighbours:
results must equal, bit for bit, the same steps run one kernel at a time with the device synchronised in between.
Also the launch-time switches (Q27_NO_PDL, Q27_SKINNY_EXT_REDUCE_M) and the contract on weights written shortly
before a GEMM."""

import os

import numpy as np
import pytest
import torch

from helpers import DEV, dev, fp4_operand, rel_err, swizzled_dev, workspace
from oracle import nvfp4_oracle as O
from q27b200 import configs, weights
from q27b200.group import Fp4Group, problem_of
from q27b200.linear import ActQuant, Fp4Linear
from q27b200.q27lib import call, device_status, lib

pytestmark = pytest.mark.gpu


def small_layer(copies=2):
    """A narrow layer with the model's structure (q|k|v stacked, o, gate | up, down) in `copies` distinct copies."""
    H, I, KV = 1024, 2560, 256
    ws = torch.zeros(48 << 20, dtype=torch.uint8, device=DEV)
    protos = {}
    for pi, (name, N, K, glu) in enumerate((("q", H, H, False), ("k", KV, H, False), ("v", KV, H, False), ("o", H, H, False),
                                            ("gate_up", 2 * I, H, True), ("down", H, I, False))):
        w = configs.make_w(N, K, 4000 + pi).to(DEV)
        codes, sfb, g = weights.quantize_weight_rtn(w)
        if glu:
            codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
        protos[name] = (codes.contiguous(), weights.swizzle_scales(sfb), g, N // 2 if glu else N, K, glu)
    layers = []
    for _ in range(copies):
        l = {n: Fp4Linear(c.clone(), s.clone(), g, 1.0, out, K, glu, ws) for n, (c, s, g, out, K, glu) in protos.items()}
        l["qkv"] = Fp4Linear.fused([l.pop("q"), l.pop("k"), l.pop("v")])
        layers.append(l)
    return layers, H, I


@pytest.mark.parametrize("M", [1, 16, 48])
def test_graph_replayed_pdl_chain_equals_synchronous_run(M):
    layers, H, I = small_layer()
    g = torch.Generator().manual_seed(M)
    xh = torch.randn(M, H, generator=g).bfloat16().to(DEV)
    xd = torch.randn(M, I, generator=g).bfloat16().to(DEV)
    s_h, s_d = configs.input_scale_of(xh), configs.input_scale_of(xd)
    act_h, act_d = ActQuant(128, H), ActQuant(128, I)
    for l in layers:
        for name, lin in l.items():
            lin.set_in_scale(s_d if name == "down" else s_h)
    names = ("qkv", "o", "gate_up", "down")

    def fresh():
        return [{n: torch.zeros(M, l[n].out, dtype=torch.bfloat16, device=DEV) for n in names} for l in layers]

    def step(l, outs, sync):
        for n in names:
            q, sf = (act_d.quantize(xd, s_d) if n == "down" else act_h.quantize(xh, s_h))
            if sync:
                torch.cuda.synchronize()
            l[n].gemm(M, q, sf, outs[n])
            if sync:
                torch.cuda.synchronize()

    want = fresh()
    os.environ["Q27_NO_PDL"] = "1"
    try:
        for l, o in zip(layers, want):
            step(l, o, True)
    finally:
        del os.environ["Q27_NO_PDL"]
    assert device_status() == 0
    # eager, back to back, programmatic dependent launch on
    got = fresh()
    for _ in range(3):
        for l, o in zip(layers, got):
            step(l, o, False)
    torch.cuda.synchronize()
    for w_, g_ in zip(want, got):
        for n in names:
            assert torch.equal(w_[n], g_[n]), f"eager chain: {n}"
    # the same steps captured once and replayed
    got = fresh()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for l, o in zip(layers, got):
                step(l, o, False)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        for o in got:
            for t in o.values():
                t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for w_, g_ in zip(want, got):
            for n in names:
                assert torch.equal(w_[n], g_[n]), f"graph replay: {n}"
    assert device_status() == 0


def test_graph_replayed_group_equals_synchronous_run():
    """The grouped launch inside a graph, behind the batched quantiser that produces its activations."""
    import ctypes

    M = 16
    layers, H, I = small_layer()
    g = torch.Generator().manual_seed(7)
    xh = torch.randn(M, H, generator=g).bfloat16().to(DEV)
    xd = torch.randn(M, I, generator=g).bfloat16().to(DEV)
    s_h, s_d = configs.input_scale_of(xh), configs.input_scale_of(xd)
    act_h, act_d = ActQuant(128, H), ActQuant(128, I)
    names = ("qkv", "o", "gate_up", "down")
    want = [{n: torch.zeros(M, l[n].out, dtype=torch.bfloat16, device=DEV) for n in names} for l in layers]
    got = [{n: torch.zeros(M, l[n].out, dtype=torch.bfloat16, device=DEV) for n in names} for l in layers]
    probs = []
    for l, w_, g_ in zip(layers, want, got):
        for n in names:
            l[n].set_in_scale(s_d if n == "down" else s_h)
            q, sf = (act_d.quantize(xd, s_d) if n == "down" else act_h.quantize(xh, s_h))
            torch.cuda.synchronize()
            l[n].gemm(M, q, sf, w_[n])
            torch.cuda.synchronize()
            probs.append(problem_of(l[n], q, sf, g_[n]))
    grp = Fp4Group(M, probs)

    class Job(ctypes.Structure):  # q27b_quant_job
        _fields_ = [("x", ctypes.c_void_p), ("q", ctypes.c_void_p), ("sf", ctypes.c_void_p), ("M", ctypes.c_int),
                    ("K", ctypes.c_int), ("input_scale", ctypes.c_float), ("bf16", ctypes.c_int)]

    jobs = (Job * 2)()
    for j, (x, a, s) in zip(jobs, ((xh, act_h, s_h), (xd, act_d, s_d))):
        j.x, j.q, j.sf, j.M, j.K, j.input_scale, j.bf16 = x.data_ptr(), a.q.data_ptr(), a.sf.data_ptr(), M, x.shape[1], s, 1

    def step():
        call("q27b_quant_fp4_batch", jobs, None, 2, torch.cuda.current_stream().cuda_stream)
        grp.launch()

    step()  # eager once (function attributes), then captured
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step()
            step()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        act_h.q.fill_(0x77), act_d.q.fill_(0x77)  # the replay must re-quantise before the group reads
        for o in got:
            for t in o.values():
                t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for w_, g_ in zip(want, got):
            for n in names:
                assert torch.equal(w_[n], g_[n]), n
    assert device_status() == 0


def test_weights_written_shortly_before_the_gemm():
    """The GEMM fetches its first weight tiles before it waits for the preceding kernel. The contract this rests
    on: weights are not written by the kernel DIRECTLY before the GEMM. One kernel in between is enough, because
    every kernel of the library releases its successor only after its own wait: here the weight operand is rewritten
    on the same stream (a copy, and - harder - this library's own quantiser producing it), then the activation is
    quantised, then the GEMM runs, several times over with changing weights."""
    M, N, K = 8, 5120, 5120
    rng = np.random.RandomState(2)
    ws = workspace()
    a32 = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(DEV)
    aq = ActQuant(128, K)
    wq = torch.zeros(N, K // 2, dtype=torch.uint8, device=DEV)
    wsf = torch.zeros(lib().q27t_sf_bytes(N, K // 16), dtype=torch.uint8, device=DEV)
    srcs = [torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32) * (i + 1)).to(DEV) for i in range(3)]
    s_a, s_w = 0.002, 0.003
    stream = torch.cuda.current_stream().cuda_stream
    want = []
    for src in srcs:  # one kernel at a time
        call("q27t_quant_fp4", src, N, K, s_w * (1 + len(want)), wq, wsf)
        q, sf = aq.quantize(a32, s_a)
        d = torch.empty(M, N, device=DEV)
        call("q27t_skinny_fp4", M, N, K, q, sf, wq, wsf, 1.0, None, 0.0, d, ws, ws.numel())
        want.append(d.clone())
    assert not torch.equal(want[0], want[1])
    for rounds in range(2):
        got = []
        for i, src in enumerate(srcs):  # back to back on one stream, programmatic dependent launch on
            call("q27b_quant_fp4", src, N, K, s_w * (1 + i), wq, wsf, stream)   # produces the weight operand
            q, sf = aq.quantize(a32, s_a)                                        # one kernel in between
            d = torch.empty(M, N, device=DEV)
            call("q27b_skinny_fp4", M, N, K, q, sf, wq, wsf, 1, np.zeros(1, np.int32), np.ones(1, np.float32), None, 0.0, d,
                 ws, ws.numel(), stream)
            got.append(d)
        torch.cuda.synchronize()
        for w_, g_ in zip(want, got):
            assert torch.equal(w_, g_)
    # directly before the GEMM the caller switches programmatic launch off for that launch
    os.environ["Q27_NO_PDL"] = "1"
    try:
        got = []
        q, sf = aq.quantize(a32, s_a)
        for i, src in enumerate(srcs):
            call("q27b_quant_fp4", src, N, K, s_w * (1 + i), wq, wsf, stream)
            d = torch.empty(M, N, device=DEV)
            call("q27b_skinny_fp4", M, N, K, q, sf, wq, wsf, 1, np.zeros(1, np.int32), np.ones(1, np.float32), None, 0.0, d,
                 ws, ws.numel(), stream)
            got.append(d)
        torch.cuda.synchronize()
    finally:
        del os.environ["Q27_NO_PDL"]
    for w_, g_ in zip(want, got):
        assert torch.equal(w_, g_)
    assert device_status() == 0


def test_ext_reduce_switch_keeps_the_bits():
    """Q27_SKINNY_EXT_REDUCE_M moves the token count above which cut tiles are summed by the fix-up kernel; both
    ways add the parts in ascending K order, so the results do not change."""
    M, N, K = 6, 5120, 5120
    rng = np.random.RandomState(9)
    a, asf, adq = fp4_operand(M, K, rng)
    b, bsf, bdq = fp4_operand(N, K, rng)
    ad, asw, bd, bsw = dev(a), swizzled_dev(asf), dev(b), swizzled_dev(bsf)
    ws = workspace()
    outs = []
    for m in (None, "0", "16"):
        if m is not None:
            os.environ["Q27_SKINNY_EXT_REDUCE_M"] = m
        try:
            d = torch.empty(M, N, device=DEV)
            call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, 0.5, None, 0.0, d, ws, ws.numel())
            outs.append(d)
        finally:
            os.environ.pop("Q27_SKINNY_EXT_REDUCE_M", None)
    assert rel_err(outs[0].cpu().numpy(), 0.5 * (adq @ bdq.T)) < 1e-5
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_dispatch_switches(capsys):
    """Q27_NO_SKINNY sends few tokens to the many-row kernel as well; Q27_SKINNY_CHECK runs both and stays silent
    when they agree (they compute the same products in the same order per tile)."""
    layers, H, I = small_layer(1)
    lin = layers[0]["o"]
    x = torch.randn(5, H, generator=torch.Generator().manual_seed(3)).bfloat16().to(DEV)
    lin.set_in_scale(configs.input_scale_of(x))
    y = lin(x)
    for name in ("Q27_NO_SKINNY", "Q27_SKINNY_CHECK"):
        os.environ[name] = "1"
        try:
            y2 = lin(x)
        finally:
            del os.environ[name]
        torch.cuda.synchronize()
        assert rel_err(y2.float().cpu().numpy(), y.float().cpu().numpy()) < 2e-3
    assert "differ" not in capsys.readouterr().err
    assert device_status() == 0
