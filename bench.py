"""Benchmark of the NVFP4 weight-GEMM path.

One "step" is one pass of the hot path over one batch: quantise the bf16 activation to NVFP4, then the
weight-streaming GEMM with its fused epilogue. At one GPU the workload is the speculative-verify gate | up
projection (x bf16 [16, 5120], W NVFP4 [34816, 5120], SiLU*mul -> bf16 [16, 17408]); with N > 1 GPUs the weight
rows are sharded N ways (every rank computes its block of output columns, no reduction) and one NCCL all-gather
of the bf16 output is timed separately.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 0|1|2|3|4]
                    [--m M] [--layers L] [--separate-qkv] [--no-graph] [--no-cpu]

Prints one JSON line (rank 0). `value` = algorithmic bytes of the step / device time with everything resident in
HBM and the weights rotating through more than L2-size of distinct copies (the steps are replayed from a CUDA
graph unless --no-graph); `e2e` = the same step through the host API with the activation coming from pinned host
memory and the result copied back to pinned host memory every step, copies inside the timed region. `--impl
reference` times the CPU restatement of the reference's own path (fake-quantise, fp32 matmul against the
dequantised weight, SiLU*mul) on the host cores instead.

--config 0 / 2 / 4 run the other single-GEMM configurations (decode GEMV, batched verify down-projection, prefill
chunk: reported in TFLOP/s against the tensor roof). --config 3 is the whole-model decode weight sweep: 64 layers
(--layers) x {q|k|v stacked, o, gate_up, down} at M = 1 ... 128 (--m for one M), every projection in its own
device memory; its line carries the GB/s of every M under "sweep".
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [ROOT, os.path.join(ROOT, "qwen3-27b-5090_b200")]

import numpy as np  # noqa: E402
import torch  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the GEMM kernel on the benchmark workload, from the
# ncu capture summarised in profiles/ (None where no capture has been taken).
NCU_TRAFFIC_BYTES = {1: 104_100_000}  # profiles/umma_gemm_kernel_cfg1_verify_gate_up.md


_json_out = None


def emit(text: str) -> None:
    out = _json_out if _json_out is not None else sys.stdout
    out.write(text + "\n")
    out.flush()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json: copy bandwidth)"
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
            time.sleep(0.3)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.1)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])), (mx := max(mx, float(f[1])))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def build_layers(cfg, rank, world, nbuf_min_bytes):
    """The rank's shard of the configuration's weight, quantised on the GPU, in `nbuf` distinct device copies
    (identical contents; distinct memory so that no step finds its weights in L2)."""
    from q27b200 import configs, shard, weights
    from q27b200.linear import Fp4Linear

    x = configs.make_x(cfg)
    in_scale = configs.input_scale_of(x)
    w = configs.make_w(cfg.N, cfg.K, 1000 + cfg.index, cfg.w_std).cuda()
    codes, sfb, g = weights.quantize_weight_rtn(w)
    del w
    if cfg.glu:
        codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
    b, e = shard.shard_rows(cfg.N, world, rank, cfg.glu)
    codes, sfs = codes[b:e].contiguous(), weights.swizzle_scales(sfb[b:e])
    n_out = (e - b) // 2 if cfg.glu else e - b
    per = codes.numel() + sfs.numel()
    nbuf = max(2, -(-nbuf_min_bytes // per))
    ws = torch.zeros(48 << 20, dtype=torch.uint8, device="cuda")  # zeroed once, as the contract asks
    layers = [Fp4Linear(codes if i == 0 else codes.clone(), sfs if i == 0 else sfs.clone(), g, in_scale, n_out, cfg.K,
                        cfg.glu, ws) for i in range(nbuf)]
    return x, in_scale, layers, n_out


def sync_all(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms, world):
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def timed(fn, steps, warmup, world, graph=False, after=None, before=None, graph_cap=None):
    """`steps` calls of fn(i) bracketed by a barrier + synchronize, timed with CUDA events on the current stream
    (the stream every launch of the library goes to); max over ranks, in ms. graph=True: the steps are captured
    once into a CUDA graph and the timed region is its replay, so that the host's launch cost (two ctypes calls
    and two tensor-map encodings per step from Python) does not sit between the kernels - the way the reference
    engine runs its decode step (engine/src/model.cc:1388-1461) and times its GEMMs (engine/src/capi.cc:57-92)."""
    for i in range(warmup):
        fn(i)
    sync_all(world)
    run = None
    if graph:
        # the graph holds `per` steps and is replayed steps / per times (per = steps unless a cap is given: a step
        # of hundreds of launches makes a graph of all the steps needlessly large)
        per = steps
        if graph_cap:
            per = max(d for d in range(1, min(graph_cap, steps) + 1) if steps % d == 0)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            if before:
                before()
            with torch.cuda.graph(g, stream=side):
                for i in range(per):
                    fn(warmup + i)
                if after:
                    after()  # other streams the steps used rejoin the captured stream
        torch.cuda.current_stream().wait_stream(side)
        g.replay()  # once untimed
        sync_all(world)

        def run():
            for _ in range(steps // per):
                g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if run:
        run()
    else:
        for i in range(steps):
            fn(warmup + i)
    if after and not run:
        after()  # make the timed stream wait for work the steps put on another stream
    e1.record()
    sync_all(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


def cpu_reference(cfg, steps, warmup, frac_rows=4):
    """The reference's CPU path (fake-quantise the activation, fp32 matmul against the once-dequantised weight,
    SiLU*mul) restated by the oracle, on a bounded sample: the first 1/frac_rows of the output channels. Returns
    (GB/s of algorithmic bytes, seconds per step, cores, description)."""
    from oracle import nvfp4_oracle as O
    from q27b200 import configs

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x = configs.make_x(cfg).float().numpy()
    s = configs.input_scale_of(configs.make_x(cfg))
    n_out = cfg.n_out // frac_rows // 64 * 64
    w_full = configs.make_w(cfg.N, cfg.K, 1000 + cfg.index, cfg.w_std)
    rows = np.concatenate([np.arange(n_out), cfg.N // 2 + np.arange(n_out)]) if cfg.glu else np.arange(n_out)
    g = O.weight_global_scale(w_full.numpy())
    codes, sfb, _ = O.quant_weight_rtn(w_full.numpy()[rows], g)
    del w_full
    wdq = torch.from_numpy(O.dequant_nvfp4(codes, sfb, g))  # dequantised once, outside the timed loop

    def step():
        xq = torch.from_numpy(O.quant_act_nvfp4(x, s))
        y = xq @ wdq.T  # fp32, all host threads
        if cfg.glu:
            y = torch.nn.functional.silu(y[:, :n_out]) * y[:, n_out:]
        return y.to(torch.bfloat16)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    n_rows = len(rows)
    sample_bytes = n_rows * cfg.K // 2 + n_rows * cfg.K // 16 + 2 * cfg.M * cfg.K + 2 * cfg.M * n_out
    desc = (f"{cfg.name}: output channels 0..{n_out - 1} of {cfg.n_out} ({n_rows} of {cfg.N} weight rows), "
            f"{steps} steps; weight dequantised once outside the timed loop")
    return sample_bytes / dt / 1e9, dt, cores, desc


def sweep_main(args, rank, world, local_rank):
    """Configuration 3: the whole-model decode weight sweep. 64 layers x {q, k, v, o, gate_up, down}, every
    projection in its own device memory (11.9 GB in total, far beyond L2; the contents of one quantised layer are
    repeated), N-sharded over the ranks; per layer the kernels a model step would launch: quantise the hidden
    state, q / k / v on it, quantise, o, quantise, gate | up with SiLU*mul, quantise, down. One "step" = the sweep
    at one M; timed as a CUDA-graph replay; value = algorithmic bytes of the sweep / time."""
    from q27b200 import configs, shard, weights
    from q27b200.linear import ActQuant, Fp4Linear
    from q27b200.q27lib import device_status

    layers_n = args.layers
    ws = torch.zeros(48 << 20, dtype=torch.uint8, device="cuda")
    protos = {}
    for pi, (name, N, K, glu) in enumerate(configs.LAYER_PROJECTIONS):
        w = configs.make_w(N, K, 1000 + pi, 0.02).cuda()
        codes, sfb, g = weights.quantize_weight_rtn(w)
        del w
        if glu:
            codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
        b, e = shard.shard_rows(N, world, rank, glu)
        protos[name] = (codes[b:e].contiguous(), weights.swizzle_scales(sfb[b:e]), g, (e - b) // 2 if glu else e - b, K, glu)
    model = []
    for _ in range(layers_n):
        layer = {}
        for name, (codes, sfs, g, n_out, K, glu) in protos.items():
            layer[name] = Fp4Linear(codes.clone(), sfs.clone(), g, 1.0, n_out, K, glu, ws)
        if args.fuse_qkv:
            layer["qkv"] = Fp4Linear.fused([layer.pop("q"), layer.pop("k"), layer.pop("v")])
        model.append(layer)
    del protos
    results = {}
    ms_list = list(configs.SWEEP_M) if args.m == 0 else [args.m]
    for M in ms_list:
        gx = torch.Generator().manual_seed(3)
        xh = torch.randn(M, configs.HIDDEN, generator=gx).to(torch.bfloat16).cuda()
        xo = torch.randn(M, configs.HIDDEN, generator=gx).to(torch.bfloat16).cuda()
        xd = torch.randn(M, configs.INTER, generator=gx).to(torch.bfloat16).cuda()
        s_h, s_o, s_d = (configs.input_scale_of(t) for t in (xh, xo, xd))
        act_h, act_d = ActQuant(max(M, 128), configs.HIDDEN), ActQuant(max(M, 128), configs.INTER)
        outs = {name: torch.empty(M, model[0][name].out, dtype=torch.bfloat16, device="cuda") for name in model[0]}
        for layer in model:
            for name, lin in layer.items():
                lin.set_in_scale(s_d if name == "down" else s_o if name == "o" else s_h)

        def sweep(_i):
            for layer in model:
                q, sf = act_h.quantize(xh, s_h)
                for name in (("qkv",) if args.fuse_qkv else ("q", "k", "v")):
                    layer[name].gemm(M, q, sf, outs[name])
                q, sf = act_h.quantize(xo, s_o)
                layer["o"].gemm(M, q, sf, outs["o"])
                q, sf = act_h.quantize(xh, s_h)
                layer["gate_up"].gemm(M, q, sf, outs["gate_up"])
                q, sf = act_d.quantize(xd, s_d)
                layer["down"].gemm(M, q, sf, outs["down"])

        ms = timed(sweep, args.steps, min(args.warmup, 3), world, not args.no_graph, graph_cap=10)
        per_sweep_s = ms / args.steps / 1e3
        nbytes = configs.sweep_algorithmic_bytes(M, layers_n)
        results[M] = {"gbs": nbytes / per_sweep_s / 1e9, "ms_per_sweep": per_sweep_s * 1e3}
    assert device_status() == 0, "a bounded wait inside a kernel ran out"
    if rank != 0:
        return
    peak, peak_src = peaks()
    head = 16 if 16 in results else ms_list[0]
    r = results[head]
    emit(json.dumps({
        "metric": "nvfp4_gemm_hbm_gbs", "value": r["gbs"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": min(args.warmup, 3), "ms_per_step": r["ms_per_sweep"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e2m1, ue4m3 scale per 16, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"cfg3 decode weight sweep, {layers_n} layers x (q,k,v,o,gate_up,down), M={head}",
                   "l2": "every projection of every layer in its own device memory (11.9 GB at 64 layers)",
                   "step": ("per layer: quant, q|k|v (one stacked weight), quant, o, quant, gate_up(SiLU*mul), quant, down; "
                            "8 launches") if args.fuse_qkv else
                           "per layer: quant, q, k, v, quant, o, quant, gate_up(SiLU*mul), quant, down; 10 launches",
                   "timing": "CUDA-graph replay" if not args.no_graph else "eager launches",
                   "sharding": f"N-sharded {world} way(s)"},
        "roofline": {"bound": "hbm", "achieved": r["gbs"] / world, "peak": peak, "unit": "GB/s", "frac": r["gbs"] / world / peak,
                     "traffic": None, "peak_source": peak_src, "kernel": "umma_gemm_kernel (weight streaming), whole sweep"},
        "gpu_launches": args.steps * layers_n * (8 if args.fuse_qkv else 10),
        "sweep": {str(m): v for m, v in results.items()}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=1, choices=[0, 1, 2, 3, 4])
    ap.add_argument("--m", type=int, default=0, help="configuration 3: the M to sweep at (0: all of 1..128)")
    ap.add_argument("--layers", type=int, default=64, help="configuration 3: layers in the sweep")
    ap.add_argument("--separate-qkv", dest="fuse_qkv", action="store_false",
                    help="configuration 3: q, k and v as three launches instead of one stacked weight with three "
                         "alpha segments (the engine stacks projections that share an input, engine/src/weights.cc:254-267)")
    ap.add_argument("--cpu-steps", type=int, default=20)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from q27b200 import configs

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    # stdout carries the one JSON line and nothing else: libraries that print to file descriptor 1 on their own
    # (NCCL's version banner) are sent to stderr, the line goes out through a private copy of the descriptor
    global _json_out
    sys.stdout.flush()
    _json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.config == 3:
        assert args.impl == "ours", "the CPU arm times single GEMM configurations"
        torch.cuda.set_device(local_rank)
        if world > 1:
            torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        sweep_main(args, rank, world, local_rank)
        if world > 1:
            torch.distributed.destroy_process_group()
        return
    cfg = configs.CONFIGS[args.config]
    metric = "nvfp4_gemm_tflops" if cfg.M > 128 else "nvfp4_gemm_hbm_gbs"
    unit = "TFLOP/s" if cfg.M > 128 else "GB/s"

    if args.impl == "reference":
        if rank != 0:
            return
        gbs, dt, cores, desc = cpu_reference(cfg, max(1, min(args.steps, 50)), min(args.warmup, 3))
        val = gbs if unit == "GB/s" else cfg.flops() / cfg.algorithmic_bytes() * gbs / 1e3
        emit(json.dumps({
            "impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus,
            "steps": max(1, min(args.steps, 50)), "warmup": min(args.warmup, 3), "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (host matmul of fake-quantised operands)",
            "data": "synthetic", "config": {"workload": cfg.name, "sample": desc},
            "cpu_baseline": {"value": val, "unit": unit, "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from q27b200 import shard
    from q27b200.linear import ActQuant
    from q27b200.q27lib import device_status

    x, in_scale, layers, n_local = build_layers(cfg, rank, world, 4 * L2_BYTES // 1 if world == 1 else 3 * L2_BYTES)
    nbuf, M = len(layers), cfg.M
    xd = x.cuda()
    outs = [torch.empty(M, n_local, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    act = ActQuant(max(M, 128), cfg.K)
    for l in layers:
        l._act = act  # one activation scratch for every copy, as one engine would have

    def step(i):  # device-resident step: quantise + GEMM (+ fix-up)
        layers[i % nbuf](xd, out=outs[i & 1])

    q, sf = act.quantize(xd, in_scale)

    def gemm_only(i):
        layers[i % nbuf].gemm(M, q, sf, outs[i & 1])

    # host-facing step: pinned host activation in, result back to pinned host memory
    xh = x.pin_memory()
    yh = [torch.empty(M, n_local, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    xdev = [torch.empty_like(xd) for _ in range(2)]
    up_stream, down_stream = torch.cuda.Stream(), torch.cuda.Stream()
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]

    def step_e2e_sync(i):  # latency form: the caller waits for every result before the next step
        xdev[0].copy_(xh, non_blocking=True)
        layers[i % nbuf](xdev[0], out=outs[0])
        yh[0].copy_(outs[0], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    fresh = [0]  # steps whose buffers nothing has used yet (the first two of a graph capture)

    def step_e2e(i):
        # throughput form: every step copies its input in, computes, and copies its result out; the two copies run
        # on streams of their own so that they overlap the neighbouring steps' kernels (two buffers of everything);
        # nothing waits on the host
        b = i & 1
        main = torch.cuda.current_stream()
        first = fresh[0] > 0
        if first:
            if fresh[0] == 2:  # the copy streams branch off the stream the steps are issued (or captured) on
                fork = torch.cuda.Event()
                fork.record(main)
                up_stream.wait_event(fork)
                down_stream.wait_event(fork)
            fresh[0] -= 1
        else:
            up_stream.wait_event(computed[b])  # step i - 2 has consumed this input buffer
        with torch.cuda.stream(up_stream):
            xdev[b].copy_(xh, non_blocking=True)
            uploaded[b].record(up_stream)
        main.wait_event(uploaded[b])
        if not first:
            main.wait_event(copied[b])  # the result buffer of step i - 2 has been read out
        layers[i % nbuf](xdev[b], out=outs[b])
        computed[b].record(main)
        down_stream.wait_event(computed[b])
        with torch.cuda.stream(down_stream):
            yh[b].copy_(outs[b], non_blocking=True)
            copied[b].record(down_stream)

    gathered = torch.empty(world, M, n_local, dtype=torch.bfloat16, device="cuda") if world > 1 else None

    def step_gather(i):
        step(i)
        torch.distributed.all_gather_into_tensor(gathered, outs[i & 1])

    graph = not args.no_graph
    with ClockSampler(local_rank) as clk:
        ms = timed(step, args.steps, args.warmup, world, graph)
        if graph:  # keep the GPU busy long enough for the clock sampler to see it under load
            for _ in range(20):
                timed(step, args.steps, 0, world, False)
    ms_gemm = timed(gemm_only, args.steps, args.warmup, world, graph)
    ms_eager = timed(step, args.steps, args.warmup, world, False)

    def e2e_join():  # the timed region ends when the last results have reached the host buffers
        for ev in copied:
            torch.cuda.current_stream().wait_event(ev)

    fresh[0] = 2
    ms_e2e_eager = timed(step_e2e, args.steps, args.warmup, world, after=e2e_join)
    ms_e2e = ms_e2e_eager
    if graph:  # the same steps, copies included, replayed from one CUDA graph: the host's launch cost drops out
        fresh[0] = 2
        ms_e2e = timed(step_e2e, args.steps, args.warmup, world, graph=True, after=e2e_join, before=lambda: fresh.__setitem__(0, 2))
    ms_e2e_sync = timed(step_e2e_sync, args.steps, args.warmup, world)
    ms_gather = timed(step_gather, args.steps, args.warmup, world) if world > 1 else None
    assert device_status() == 0, "a bounded wait inside a kernel ran out"
    clocks = clk.summary()

    if rank != 0:
        torch.distributed.destroy_process_group()
        return

    total_bytes = cfg.algorithmic_bytes()  # whole job: all ranks' weight shards + activation in + output
    flops = cfg.flops()
    per_step_s, gemm_s, e2e_s = ms / args.steps / 1e3, ms_gemm / args.steps / 1e3, ms_e2e / args.steps / 1e3

    def val(seconds):
        return total_bytes / seconds / 1e9 if unit == "GB/s" else flops / seconds / 1e12

    peak, peak_src = peaks()
    # per-GPU roofline of the dominant kernel: the rank's share of the weight bytes + the whole activation + its
    # output block, over the average duration of one GEMM launch (launch gap included)
    n_rows_local = layers[0].rows()
    launch_bytes = n_rows_local * cfg.K // 2 + n_rows_local * cfg.K // 16 + 2 * M * cfg.K + 2 * M * n_local
    if M <= 128:
        achieved = launch_bytes / gemm_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(cfg.index) if world == 1 else None, "algorithmic_bytes": launch_bytes,
                "kernel": "umma_gemm_kernel (weight streaming)", "us_per_launch": gemm_s * 1e6, "peak_source": peak_src}
    else:
        # No FP4 figure is measured on this pool: the denominator is 4 x the measured dense bf16 cuBLAS burst
        # (block-scaled FP4 runs at 4 x the bf16 rate; nominal dense FP4 is 9000 TFLOP/s).
        pk = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
        tpeak = 4.0 * float(pk.get("bf16_tflops", 1590.0))
        tpeak_sustained = 4.0 * float(pk.get("bf16_tflops_sustained", 1400.0))
        launch_flops = 2 * M * n_rows_local * cfg.K
        achieved = launch_flops / gemm_s / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": tpeak, "unit": "TFLOP/s", "frac": achieved / tpeak,
                "traffic": None, "algorithmic_flops": launch_flops, "kernel": "umma_gemm_kernel (many rows)",
                "us_per_launch": gemm_s * 1e6,
                # the timed region is a long run of back-to-back GEMMs under the power cap: the sustained cuBLAS
                # figure (seconds-long loop, clocks settled) is the like-for-like denominator; the burst one is kept
                # as `peak`
                "peak_sustained": tpeak_sustained, "frac_of_sustained": achieved / tpeak_sustained,
                "peak_source": "4 x bf16_tflops of MEASURED_PEAKS.json (no measured FP4 peak; nominal dense FP4 9000)"
                if pk else "4 x fallback bf16 1590 (no measured FP4 peak; nominal dense FP4 9000)"}
    line = {
        "metric": metric, "value": val(per_step_s), "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x e2m1, ue4m3 scale per 16, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": cfg.name, "M": M, "N": cfg.N, "K": cfg.K, "epilogue": "silu*mul->bf16" if cfg.glu else "bf16",
                   "sharding": f"N-sharded {world} way(s), no reduction", "l2": f"weights rotate through {nbuf} distinct copies "
                   f"({nbuf * layers[0].weight_bytes() / 2**20:.0f} MiB per GPU > 126 MiB L2)",
                   "step": "quant_fp4_bf16 + skinny_fp4_glu_bf16" if M <= 128 else "quant_fp4_bf16 + gemm_fp4_glu_bf16",
                   "timing": "CUDA-graph replay of the timed steps" if graph else "eager launches", "eager_ms_per_step": ms_eager / args.steps},
        "e2e": {"value": val(e2e_s), "unit": unit, "h2d_bytes_per_step": x.numel() * 2, "d2h_bytes_per_step": M * n_local * 2,
                "ms_per_step": ms_e2e / args.steps, "ms_per_step_host_waits_each_result": ms_e2e_sync / args.steps,
                "ms_per_step_eager_launches": ms_e2e_eager / args.steps,
                "how": "per step: pinned host activation -> device, quantise + GEMM through Fp4Linear, result -> pinned "
                       "host; the two copies on streams of their own, overlapping the neighbouring steps; " +
                       ("the steps with their copies replayed from one CUDA graph" if graph else "eager launches")},
        "gpu_launches": args.steps * 2,  # quantiser + GEMM
        "roofline": roof,
        "clocks": clocks,
    }
    if ms_gather is not None:
        line["with_allgather"] = {"value": val(ms_gather / args.steps / 1e3), "unit": unit, "ms_per_step": ms_gather / args.steps}
    if world == 1 and not args.no_cpu:
        gbs, dt, cores, desc = cpu_reference(cfg, args.cpu_steps, 2)
        line["cpu_baseline"] = {"value": gbs if unit == "GB/s" else flops / total_bytes * gbs / 1e3, "unit": unit, "cores": cores,
                                "kind": "port", "sample": desc, "ms_per_step_sample": dt * 1e3}
    emit(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
