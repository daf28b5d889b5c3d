"""Several GPUs of one node (skipped where fewer than two are visible): the gather fused into the grouped launch.
Two ranks each hold half of the weight rows of a small layer; the grouped launch of every rank stores its block of the
outputs into its own memory and, through peer-mapped pointers, into the other rank's; after the wait kernel both ranks
must hold exactly what an NCCL all-gather of the per-GEMM results gives, step after step on alternating buffers."""

import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import ctypes, os, sys
    import torch, torch.distributed as dist
    root = sys.argv[1]
    sys.path[:0] = [root, os.path.join(root, "qwen3-27b-5090_b200")]
    from q27b200 import configs, shard, weights
    from q27b200.group import Fp4Group, problem_of
    from q27b200.linear import ActQuant, Fp4Linear
    from q27b200.peer import PeerRegion
    from q27b200.q27lib import call, device_status
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    M, H, I = 16, 1024, 2560
    shapes = (("qkv", 1536, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False))
    lins = {}
    for pi, (name, N, K, glu) in enumerate(shapes):
        w = configs.make_w(N, K, 5000 + pi).cuda()
        codes, sfb, g = weights.quantize_weight_rtn(w)
        if glu:
            codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
        shard.check_even_shards(N, world)
        b, e = shard.shard_rows(N, world, rank, glu)
        lins[name] = Fp4Linear(codes[b:e].contiguous(), weights.swizzle_scales(sfb[b:e]), g, 1.0, (e - b) // 2 if glu else e - b, K, glu)
    gen = torch.Generator().manual_seed(1)
    xh = torch.randn(M, H, generator=gen).bfloat16().cuda()
    xd = torch.randn(M, I, generator=gen).bfloat16().cuda()
    acts = {"h": ActQuant(128, H), "d": ActQuant(128, I)}
    scales = {"h": configs.input_scale_of(xh), "d": configs.input_scale_of(xd)}
    widths = [lins[n].out for n, *_ in shapes]
    block = M * sum(widths)
    region = PeerRegion(2 * world * block * 2)
    pay = region.payload()[:2 * world * block * 2].view(torch.bfloat16).view(2, world, block)
    peers = region.peers()
    slots = (ctypes.c_int * (world - 1))(*region.peer_slots())
    stream = torch.cuda.current_stream().cuda_stream
    # default plan (cut tiles summed in the kernel: same bits as the weight-streaming launches) and whole tiles (same
    # bits as the many-row GEMM; at 16 tokens finished tiles leave through the token-major staging tile)
    for whole in (False, True):
        groups, outs = [], []
        for b in range(2):
            o, off, probs = {}, 0, []
            for (n, *_), wd in zip(shapes, widths):
                o[n] = pay[b][rank][off:off + M * wd].view(M, wd)
                off += M * wd
            for n, N, K, glu in shapes:
                k = "d" if n == "down" else "h"
                lins[n].set_in_scale(scales[k])
                probs.append(problem_of(lins[n], acts[k].q, acts[k].sf, o[n]))
            groups.append(Fp4Group(M, probs, whole_tiles=whole, tokens_on_n=True))
            outs.append(o)
        # reference: per-GEMM launches, then an NCCL all-gather
        want = torch.zeros(block, dtype=torch.bfloat16, device="cuda")
        off = 0
        os.environ["Q27_NO_SKINNY"] = "1" if whole else "0"
        for (n, N, K, glu), wd in zip(shapes, widths):
            k = "d" if n == "down" else "h"
            q, sf = acts[k].quantize(xd if k == "d" else xh, scales[k])
            lins[n].gemm(M, q, sf, want[off:off + M * wd].view(M, wd))
            off += M * wd
        os.environ["Q27_NO_SKINNY"] = "0"
        want_all = torch.empty(world, block, dtype=torch.bfloat16, device="cuda")
        dist.all_gather_into_tensor(want_all.view(-1), want)
        torch.cuda.synchronize()
        for step in range(6):
            b = step & 1
            pay[b].zero_()           # (both ranks clear the buffer the step before last used ...
            torch.cuda.synchronize()
            dist.barrier()           #  ... before either writes into the other's copy of it)
            acts["h"].quantize(xh, scales["h"]); acts["d"].quantize(xd, scales["d"])
            groups[b].launch_gather(peers)
            call("q27b_group_gather_wait", region.ptrs[rank], world - 1, slots, stream)
            torch.cuda.synchronize()
            assert torch.equal(pay[b], want_all), f"rank {rank} step {step} whole={whole}: gathered outputs differ"
    assert device_status() == 0
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_fused_gather_equals_nccl_all_gather(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=600)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out[-3000:]}"
        assert f"rank {rank} ok" in out
