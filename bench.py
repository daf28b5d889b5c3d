"""Benchmark of the NVFP4 weight-GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--only sweep,cfg0,cfg1,cfg2,cfg4] [--m M] [--layers L] [--group-layers G] [--no-cpu]

Prints ONE JSON line (rank 0). The headline is the configuration the bandwidth target is stated on: the whole-model
decode weight sweep (64 layers x {q|k|v stacked, o, gate|up with SiLU*mul, down}, every projection in its own device
memory, 11.9 GB in all) at M = 16 tokens. One "step" is one sweep: per group of G layers one launch that quantises
the layers' bf16 activations to NVFP4 and one launch of the grouped weight-streaming GEMM over all their projections
(G = 64 by default: the whole sweep is one persistent launch). `value` = algorithmic bytes of a sweep / device time,
inputs resident in HBM, exactly K steps replayed from a CUDA graph and timed with CUDA events. The same line carries

  "sweep":   GB/s and fraction of the measured HBM peak for every M in 1..128 (same mode as the headline),
  "modes":   the M = 16 sweep run per GEMM (one launch per projection, chained with programmatic dependent launch,
             the way the reference's engine runs a decode step) and in groups of 1, 8 and 64 layers,
  "configs": the single-GEMM configurations cfg0 (decode GEMV), cfg1 (verify gate|up), cfg2 (batched verify down)
             and cfg4 (prefill, tensor-bound), each with its roofline and clocks,
  "e2e":     the headline sweep driven from HOST buffers: activations copied from pinned host memory and the last
             layer's outputs copied back every step, copies inside the timed region,
  "verified": after every timed region the outputs left by the LAST timed step are compared bit for bit with the
             same step run one kernel at a time (device synchronised in between, programmatic launch off).

With N > 1 GPUs the weight rows are sharded N ways (no reduction anywhere) and every step ends with every rank
holding every rank's outputs: by default the grouped launch stores its outputs into all peers' memory from its
epilogue (plain peer stores overlapping the weight stream, then a wait for the peers' signals; --gather nccl: one NCCL
all-gather after the launch instead). Either way the gather is inside the timed graph and inside `value`; the figures
without it and with the other way are reported beside it.

--impl reference times the CPU restatement of the reference's own path (fake-quantise, fp32 matmul against the
once-dequantised weight, SiLU*mul) on the host cores for the same workload, on a bounded sample of it.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import math
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
FALLBACK_BF16_TFLOPS = 1590.0
DTYPE = "nvfp4 (e2m1 x e2m1, ue4m3 scale per 16, fp32 accumulate)"
MIN_REGION_MS = 60.0  # sub-configurations are replayed until their timed region is at least this long

_json_out = None


def emit(text: str) -> None:
    out = _json_out if _json_out is not None else sys.stdout
    out.write(text + "\n")
    out.flush()


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0,
            "source": "fallback (6.65 TB/s, 1.59 PFLOP/s: earlier measurements on this pool)"}


def ncu_traffic():
    """dram bytes per launch from the ncu captures summarised under profiles/ (a record of those captures, keyed by
    configuration; null where none was taken). Not measured by this run."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    return json.load(open(path)) if os.path.exists(path) else {}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "10",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.thread.start()
            time.sleep(0.3)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.05)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        rows, mx, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                rows.append((float(f[0]), float(f[2])))
                mx = max(mx, float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # "under load" = the samples in the upper half of the power readings seen (the sampler also sees idle time)
        power = sorted(p for _, p in rows)
        busy = [c for c, p in rows if p >= power[len(power) // 2]]
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(rows),
                "power_w_max": power[-1]}


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


def timed(fn, steps, warmup, world, graph=True, graph_cap=None, busy_ms=0.0):
    """Exactly `steps` calls of fn(i), bracketed by a barrier + synchronize, timed with CUDA events on the current
    stream (the stream every launch of the library goes to); max over ranks, in ms. graph=True: `per` steps are
    captured once into a CUDA graph and the timed region is steps / per replays of it, so that the host's launch cost
    (ctypes calls and tensor-map encodings from Python) does not sit between the kernels - the way the reference engine
    runs its decode step (engine/src/model.cc:1388-1461) and times its GEMMs (engine/src/capi.cc:57-92). busy_ms: the
    graph is replayed untimed for about that long first (a clock sampler then sees the GPU under this load)."""
    for i in range(warmup):
        fn(i)
    sync_all(world)
    run = None
    if graph:
        per = steps
        if graph_cap:
            per = max(d for d in range(1, min(graph_cap, steps) + 1) if steps % d == 0)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(per):
                    fn(warmup + i)
        torch.cuda.current_stream().wait_stream(side)
        g.replay()  # once untimed
        sync_all(world)
        if busy_ms > 0:
            # the number of untimed replays is agreed between the ranks (their steps may contain a gather: every rank must
            # run the same number of them)
            t0 = time.perf_counter()
            g.replay()
            torch.cuda.synchronize()
            one = max_over_ranks((time.perf_counter() - t0) * 1e3, world)
            for _ in range(int(min(2000, max(1, busy_ms / max(one, 1e-3))))):
                g.replay()
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
    e1.record()
    sync_all(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


class serial_launches:
    """Context: programmatic dependent launch off, for the one-kernel-at-a-time runs the timed results are checked
    against (the caller synchronises the device between the launches)."""

    def __enter__(self):
        self.old = os.environ.get("Q27_NO_PDL")
        os.environ["Q27_NO_PDL"] = "1"

    def __exit__(self, *a):
        if self.old is None:
            os.environ.pop("Q27_NO_PDL", None)
        else:
            os.environ["Q27_NO_PDL"] = self.old


# ------------------------------------------------------------------------------------------- the decode weight sweep


class QuantJob(ctypes.Structure):  # q27b_quant_job (include/q27b200/capi.h)
    _fields_ = [("x", ctypes.c_void_p), ("q", ctypes.c_void_p), ("sf", ctypes.c_void_p), ("M", ctypes.c_int),
                ("K", ctypes.c_int), ("input_scale", ctypes.c_float), ("bf16", ctypes.c_int)]


def build_model(layers_n, rank, world):
    """The rank's shard of every projection of every layer: contents of one quantised layer repeated, every copy in
    device memory of its own (so that no launch finds its weights in L2)."""
    from q27b200 import configs, shard, weights
    from q27b200.linear import Fp4Linear

    ws = torch.zeros(48 << 20, dtype=torch.uint8, device="cuda")  # per-GEMM workspace, zeroed once
    protos = {}
    for pi, (name, N, K, glu) in enumerate(configs.LAYER_PROJECTIONS):
        w = configs.make_w(N, K, 1000 + pi, 0.02).cuda()
        codes, sfb, g = weights.quantize_weight_rtn(w)
        del w
        if glu:
            codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
        shard.check_even_shards(N, world)
        b, e = shard.shard_rows(N, world, rank, glu)
        protos[name] = (codes[b:e].contiguous(), weights.swizzle_scales(sfb[b:e]), g, (e - b) // 2 if glu else e - b, K, glu)
    model = []
    for _ in range(layers_n):
        layer = {name: Fp4Linear(c.clone(), s.clone(), g, 1.0, n_out, K, glu, ws) for name, (c, s, g, n_out, K, glu) in protos.items()}
        # q, k and v read the same activation: one stacked weight with one alpha per part, as the engine stacks
        # projections that share an input (engine/src/weights.cc:254-267)
        layer["qkv"] = Fp4Linear.fused([layer.pop("q"), layer.pop("k"), layer.pop("v")])
        model.append({n: layer[n] for n in ("qkv", "o", "gate_up", "down")})
    return model


class Sweep:
    """One token count of the sweep: inputs, per-layer quantised activations and outputs, and the launch sequences.

    gather (several GPUs): "fused" - the grouped launch stores every output into all peers' memory as well (plain
    peer stores from its epilogue, overlapping the weight stream) and a one-warp kernel behind it waits for the peers'
    signals; "nccl" - one NCCL all-gather of all outputs after the launches. Either way the step ends with every rank
    holding every rank's block of the outputs, rank-major ([rank][layer][M x columns of the rank]). With the fused
    gather the outputs alternate between two buffers from step to step: a rank may start its next step while a peer
    still reads the previous one's."""

    NAMES = ("qkv", "o", "gate_up", "down")

    def __init__(self, model, M, world, gather="nccl"):
        from q27b200 import configs
        from q27b200.linear import ActQuant

        self.model, self.M, self.world, self.L = model, M, world, len(model)
        self.rank = torch.distributed.get_rank() if world > 1 else 0
        self.fused = world > 1 and gather == "fused"
        gx = torch.Generator().manual_seed(3)
        self.x_host = {"h": torch.randn(M, configs.HIDDEN, generator=gx).to(torch.bfloat16).pin_memory(),
                       "o": torch.randn(M, configs.HIDDEN, generator=gx).to(torch.bfloat16).pin_memory(),
                       "d": torch.randn(M, configs.INTER, generator=gx).to(torch.bfloat16).pin_memory()}
        self.x = {k: v.cuda() for k, v in self.x_host.items()}
        self.scale = {k: configs.input_scale_of(v) for k, v in self.x.items()}
        self.src = {"qkv": "h", "o": "o", "gate_up": "h", "down": "d"}  # which activation a projection reads
        # every layer has quantised activations of its own (a model's layers see different values), and its own outputs
        self.act = [{k: ActQuant(max(M, 128), v.shape[1]) for k, v in self.x.items()} for _ in range(self.L)]
        widths = [model[0][n].out for n in self.NAMES]
        self.width = sum(widths)
        block = self.L * M * self.width  # bf16 elements one rank contributes
        if self.fused:
            from q27b200.peer import PeerRegion

            self.region = PeerRegion(2 * world * block * 2)
            pay = self.region.payload()[:2 * world * block * 2].view(torch.bfloat16).view(2, world, block)
            self.gathered = [pay[0], pay[1]]
            self.out_all = [pay[b][self.rank].view(self.L, M * self.width) for b in range(2)]
            self.peers = self.region.peers()
            self.wait_slots = (ctypes.c_int * (world - 1))(*self.region.peer_slots())
        else:
            self.out_all = [torch.zeros(self.L, M * self.width, dtype=torch.bfloat16, device="cuda")]
            self.gathered = [torch.empty(world, block, dtype=torch.bfloat16, device="cuda")] if world > 1 else [None]
        self.outs = []
        for oa in self.out_all:
            per_layer = []
            for l in range(self.L):
                o, off = {}, 0
                for n, wd in zip(self.NAMES, widths):
                    o[n] = oa[l, off:off + M * wd].view(M, wd)
                    off += M * wd
                per_layer.append(o)
            self.outs.append(per_layer)
        for layer in model:
            for n, lin in layer.items():
                lin.set_in_scale(self.scale[self.src[n]])
        self.last_b = 0
        self._groups = {}
        self._jobs = {}

    # -- launch sequences --------------------------------------------------------------------------------------------

    def _quant_jobs(self, l0, l1):
        key = (l0, l1)
        if key not in self._jobs:
            n = 3 * (l1 - l0)
            jobs = (QuantJob * n)()
            i = 0
            for l in range(l0, l1):
                for k in ("h", "o", "d"):
                    a, j = self.act[l][k], jobs[i]
                    j.x, j.q, j.sf, j.M, j.K = self.x[k].data_ptr(), a.q.data_ptr(), a.sf.data_ptr(), self.M, self.x[k].shape[1]
                    j.input_scale, j.bf16 = self.scale[k], 1
                    i += 1
            table = torch.frombuffer(bytearray(bytes(jobs)), dtype=torch.uint8).cuda() if n > 4 else None
            self._jobs[key] = (jobs, table, n)
        return self._jobs[key]

    def quantise(self, l0, l1):
        from q27b200.q27lib import call

        jobs, table, n = self._quant_jobs(l0, l1)
        call("q27b_quant_fp4_batch", jobs, table, n, torch.cuda.current_stream().cuda_stream)

    def whole_tiles(self, layers):
        """Groups of several layers run without the K split (whole tiles fill the GPU evenly by themselves); a single
        layer keeps the split of the stand-alone launches."""
        return layers >= 8

    def group(self, l0, l1, b=0):
        from q27b200.group import Fp4Group, problem_of

        key = (l0, l1, b)
        if key not in self._groups:
            probs = []
            for l in range(l0, l1):
                for n in self.NAMES:
                    a = self.act[l][self.src[n]]
                    probs.append(problem_of(self.model[l][n], a.q, a.sf, self.outs[b][l][n]))
            self._groups[key] = Fp4Group(self.M, probs, whole_tiles=self.whole_tiles(l1 - l0), tokens_on_n=self.fused)  # (256-row tiles have no fused gather)
        return self._groups[key]

    def drop_groups(self):
        self._groups.clear()

    def step_grouped(self, G, i=0, gather=True):
        from q27b200.q27lib import call

        b = self.last_b = i % len(self.out_all)
        launches = 0
        for l0 in range(0, self.L, G):
            l1 = min(l0 + G, self.L)
            self.quantise(l0, l1)
            if self.fused and gather:
                self.group(l0, l1, b).launch_gather(self.peers)
            else:
                self.group(l0, l1, b).launch()
            launches += 1
        if self.fused and gather:  # one wait per launch: each launch raises this rank's word in every peer once
            for _ in range(launches):
                call("q27b_group_gather_wait", self.region.ptrs[self.rank], self.world - 1, self.wait_slots,
                     torch.cuda.current_stream().cuda_stream)
        elif gather:
            self.gather(b)

    def step_per_gemm(self, i=0):
        b = self.last_b = i % len(self.out_all)
        for l in range(self.L):
            self.quantise(l, l + 1)
            for n in self.NAMES:
                a = self.act[l][self.src[n]]
                self.model[l][n].gemm(self.M, a.q, a.sf, self.outs[b][l][n])
        self.gather(b)

    def gather(self, b=0):
        if self.world > 1:  # the one collective of the path: every rank's block of output columns, all layers at once
            assert not self.fused, "the NCCL gather writes into a buffer of its own"
            torch.distributed.all_gather_into_tensor(self.gathered[b].view(-1), self.out_all[b].view(-1))

    def launches_per_step(self, G):
        # per GEMM: the quantiser, four GEMMs and, above 8 tokens, the fix-up kernel of the three weights that are cut along K
        n = self.L * (1 + len(self.NAMES) + (3 if self.M > 8 else 0)) if G == 0 else 2 * math.ceil(self.L / G)
        if self.world > 1:
            n += math.ceil(self.L / max(G, 1)) if self.fused else 1  # the wait kernels / the collective
        return n

    # -- checking ----------------------------------------------------------------------------------------------------

    def _many_row(self, lin, a, out):
        """One projection through the many-row GEMM entry points (no K split): per alpha segment of a stacked weight."""
        from q27b200.q27lib import call

        s, K, M = torch.cuda.current_stream().cuda_stream, lin.inp, self.M
        if lin.glu:
            call("q27b_gemm_fp4_glu_bf16", M, lin.out, K, a.q, a.sf, lin.w, lin.sf, lin.alpha, lin.alpha, out, s)
            return
        begins = [lin._zero[i] for i in range(lin._nseg)] + [lin.rows()]
        for i in range(lin._nseg):
            b, e = begins[i], begins[i + 1]
            part = out if lin._nseg == 1 else torch.empty(M, e - b, dtype=out.dtype, device=out.device)
            call("q27b_gemm_fp4_bf16", M, e - b, K, a.q, a.sf, lin.w[b:e], lin.sf[b // 128 * (K // 64) * 512:], lin._alpha[i], part, s)
            if lin._nseg > 1:
                out[:, b:e] = part

    def verify(self, G, gathered=True):
        """The outputs the last timed step left behind, against the same step run one kernel at a time through the
        per-GEMM entry points: the weight-streaming launch, or - for groups planned without the K split, whose sums
        run over all of K in one chain - the many-row GEMM. On several GPUs every rank also checks the other ranks'
        blocks it received against an all-gather of those one-kernel-at-a-time results."""
        b = self.last_b
        got = self.out_all[b].clone()
        got_all = self.gathered[b].clone() if (self.world > 1 and gathered) else None
        want = torch.zeros_like(got)
        wouts, widths = [], [self.model[0][n].out for n in self.NAMES]
        for l in range(self.L):
            o, off = {}, 0
            for n, wd in zip(self.NAMES, widths):
                o[n] = want[l, off:off + self.M * wd].view(self.M, wd)
                off += self.M * wd
            wouts.append(o)
        whole = G > 0 and self.whole_tiles(min(G, self.L))
        with serial_launches():
            for l in range(self.L):
                for n in self.NAMES:
                    a = self.act[l][self.src[n]]
                    k = self.src[n]
                    a.quantize(self.x[k], self.scale[k])
                    torch.cuda.synchronize()
                    if whole:
                        self._many_row(self.model[l][n], a, wouts[l][n])
                    else:
                        self.model[l][n].gemm(self.M, a.q, a.sf, wouts[l][n])
                    torch.cuda.synchronize()
        ok = bool(torch.equal(got, want)) and bool(torch.isfinite(got.float()).all()) and bool(got.any())
        if self.world > 1:
            if got_all is not None:
                ref_all = torch.empty_like(got_all)
                torch.distributed.all_gather_into_tensor(ref_all.view(-1), want.view(-1))
                ok = ok and bool(torch.equal(got_all, ref_all))
            flag = torch.tensor([int(ok)], device="cuda")
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
            ok = bool(flag.item())
        return ok


def run_sweep(args, model, rank, world, local_rank, peaks):
    from q27b200 import configs
    from q27b200.q27lib import device_status

    L = len(model)
    G = min(args.group_layers, L)
    ms_list = list(configs.SWEEP_M) if args.m == 0 else [args.m]
    head_m = 16 if 16 in ms_list else ms_list[0]
    gather, gather_note = args.gather_mode, args.gather_note
    cap = 4 if world > 1 else 5  # steps per captured graph (even on several GPUs: the output buffers alternate)
    sweep, modes, verified, head = {}, {}, True, None

    # the reference's own bench counts the weight and scale bytes only (engine/tests/test_skinny.py:175): reported beside
    weight_bytes = configs.sweep_algorithmic_bytes(0, L)

    def rate(nbytes, ms):
        per = ms / args.steps
        return {"gbs": nbytes / per / 1e6, "ms_per_sweep": per, "frac": nbytes / per / 1e6 / world / peaks["hbm_gbs"],
                "weights_only_gbs": weight_bytes / per / 1e6}

    for M in ms_list:
        sw = Sweep(model, M, world, gather)
        nbytes = configs.sweep_algorithmic_bytes(M, L)
        mode = f"grouped, {G} layer(s) per launch" + (", whole tiles" if sw.whole_tiles(G) else "")
        if world > 1:
            mode += ", gather fused into the epilogue (peer stores)" if sw.fused else ", NCCL all-gather"
        if M == head_m:
            with ClockSampler(local_rank) as clk:  # covers the warm-up steps, the capture and the K timed steps
                ms = timed(lambda i: sw.step_grouped(G, i), args.steps, args.warmup, world, graph_cap=cap)
            clocks = clk.summary()
        else:
            ms = timed(lambda i: sw.step_grouped(G, i), args.steps, args.warmup, world, graph_cap=cap)
        ok = sw.verify(G)
        verified = verified and ok
        sweep[str(M)] = dict(rate(nbytes, ms), mode=mode, verified=ok)
        if M > 16 and world == 1:
            # many tokens: the per-GEMM form is timed as well and the faster of the two is reported, by name
            sw.drop_groups()
            ms2 = timed(lambda i: sw.step_per_gemm(i), args.steps, args.warmup, world, graph_cap=cap)
            ok2 = sw.verify(0)
            verified = verified and ok2
            sweep[str(M)]["grouped_gbs"] = sweep[str(M)]["gbs"]
            sweep[str(M)]["per_gemm_gbs"] = rate(nbytes, ms2)["gbs"]
            if ms2 < ms:
                sweep[str(M)].update(dict(rate(nbytes, ms2), mode="per GEMM (one launch per projection, programmatic dependent launch)",
                                          verified=ok2))
        if M > 32 and world > 1 and sw.fused:
            # many tokens on several GPUs: the outputs are large and the fused gather has to keep the tokens on the MMA's N
            # side (small peer stores); the other way - 256-row tiles and one NCCL all-gather per sweep - is timed as well
            # and the faster of the two is reported, by name
            sw2 = Sweep(model, M, world, "nccl")
            ms2 = timed(lambda i: sw2.step_grouped(G, i), args.steps, args.warmup, world, graph_cap=cap)
            ok2 = sw2.verify(G)
            verified = verified and ok2
            sweep[str(M)]["fused_gather_gbs"] = sweep[str(M)]["gbs"]
            sweep[str(M)]["nccl_gather_gbs"] = rate(nbytes, ms2)["gbs"]
            if ms2 < ms:
                sweep[str(M)].update(dict(rate(nbytes, ms2), mode=f"grouped, {G} layer(s) per launch, whole tiles of 256 rows, NCCL all-gather",
                                          verified=ok2))
            del sw2
        log(f"sweep M={M}: {sweep[str(M)]}")
        if M == head_m:
            head = dict(sweep[str(M)], clocks=clocks, bytes=nbytes)
            modes[f"group_{G}_layer{'s' if G > 1 else ''}"] = dict(rate(nbytes, ms), launches_per_sweep=sw.launches_per_step(G), verified=ok)
            if world == 1:  # the same sweep in the other launch forms
                for name, g in (("per_gemm", 0), ("group_1_layer", 1), ("group_4_layers", 4), ("group_8_layers", 8), ("group_64_layers", 64)):
                    if g > L or (g == G):
                        continue
                    sw.drop_groups()
                    fn = (lambda i: sw.step_per_gemm(i)) if g == 0 else (lambda i, g=g: sw.step_grouped(g, i))
                    ms_mode = timed(fn, args.steps, args.warmup, world, graph_cap=cap)
                    okm = sw.verify(g)
                    verified = verified and okm
                    modes[name] = dict(rate(nbytes, ms_mode), launches_per_sweep=sw.launches_per_step(g), verified=okm)
                    log(f"mode {name}: {modes[name]}")
            else:  # the cost of the gather: the same steps without it, and with the other way of gathering
                ms_ng = timed(lambda i: sw.step_grouped(G, i, gather=False), args.steps, args.warmup, world, graph_cap=cap)
                head["without_gather"] = rate(nbytes, ms_ng)
                log(f"without gather: {head['without_gather']}")
                other = "nccl" if sw.fused else None
                if other:
                    sw2 = Sweep(model, M, world, other)
                    ms_o = timed(lambda i: sw2.step_grouped(G, i), args.steps, args.warmup, world, graph_cap=cap)
                    oko = sw2.verify(G)
                    verified = verified and oko
                    head["with_nccl_all_gather"] = dict(rate(nbytes, ms_o), verified=oko)
                    log(f"with NCCL all-gather: {head['with_nccl_all_gather']}")
                    del sw2
            # the same K steps after 0.4 s of uninterrupted replays: streaming at this rate runs into the board's power cap
            # (sw_power_cap, SM clock down to 1.5-1.7 GHz), which a long-running decode loop would see
            with ClockSampler(local_rank) as clk:
                ms_sus = timed(lambda i: sw.step_grouped(G, i), args.steps, args.warmup, world, graph_cap=cap, busy_ms=400.0)
            head["sustained"] = dict(rate(nbytes, ms_sus), clocks=clk.summary(),
                                     how="the K timed steps directly after 0.4 s of back-to-back replays of the same graph")
            # end to end from host buffers: activations in from pinned host memory, the last layer's outputs back out
            y_host = [torch.empty(M * sw.width, dtype=torch.bfloat16).pin_memory() for _ in range(len(sw.out_all))]

            def last_layer(bb):  # the last layer's outputs as the step leaves them (on several GPUs: rank 0's block)
                return sw.gathered[bb][0][-M * sw.width:] if world > 1 else sw.out_all[bb][L - 1]

            def step_e2e(i):
                for k in ("h", "o", "d"):
                    sw.x[k].copy_(sw.x_host[k], non_blocking=True)
                sw.step_grouped(G, i)
                y_host[sw.last_b].copy_(last_layer(sw.last_b), non_blocking=True)

            ms_e2e = timed(step_e2e, args.steps, args.warmup, world, graph_cap=cap)
            oke = sw.verify(G) and bool(torch.equal(y_host[sw.last_b].cuda(), last_layer(sw.last_b)))
            verified = verified and oke
            head["e2e"] = {"value": rate(nbytes, ms_e2e)["gbs"], "unit": "GB/s",
                           "h2d_bytes_per_step": sum(v.numel() * 2 for v in sw.x_host.values()),
                           "d2h_bytes_per_step": y_host[0].numel() * 2, "ms_per_step": ms_e2e / args.steps, "verified": oke,
                           "how": "per step: the three bf16 activations pinned host -> device, the sweep (quantisers + grouped "
                                  "GEMM" + (" + gather" if world > 1 else "") + "), the last layer's outputs device -> pinned "
                                  "host; all on the launching stream, replayed from a CUDA graph"}
            head["launches"] = sw.launches_per_step(G)
        del sw
        torch.cuda.empty_cache()
    assert device_status() == 0, "a bounded wait inside a kernel ran out"
    return {"head_m": head_m, "G": G, "sweep": sweep, "modes": modes, "verified": verified, "head": head, "gather": gather,
            "gather_note": gather_note}


# ------------------------------------------------------------------------------------------- single-GEMM configurations


def total_bytes_of(cfg):
    return cfg.algorithmic_bytes()


def many_row_kernel_name(M, fused_gather):
    """Which many-row kernel the library picks for the prefill shape (its rule: csrc/umma_gemm.cu run_many)."""
    from q27b200.q27lib import lib

    forced = os.environ.get("Q27B_MANY", "")
    quad = lib().q27b_quad_available() and not fused_gather and forced == "quad" and M > 128 and ((M + 255) // 256) % 2 == 0
    if quad:
        return "quad_gemm_kernel (many rows, clusters of four CTAs sharing the weight tile; optional single-GPU library)"
    return "umma_gemm2_kernel (many rows, CTA pairs)" if forced in ("", "pairs", "quad") else f"umma_gemm_kernel ({forced} tiles)"


def run_single(cfg, args, rank, world, local_rank, peaks):
    """One of cfg0 / cfg1 / cfg2 / cfg4: step = quantise the bf16 activation + the GEMM with its epilogue, weights
    rotating through more than L2-size of distinct copies, replayed from a CUDA graph until the region is long enough."""
    from q27b200 import configs, shard, weights
    from q27b200.linear import ActQuant, Fp4Linear
    from q27b200.q27lib import device_status

    x = configs.make_x(cfg)
    in_scale = configs.input_scale_of(x)
    w = configs.make_w(cfg.N, cfg.K, 1000 + cfg.index, cfg.w_std).cuda()
    codes, sfb, g = weights.quantize_weight_rtn(w)
    del w
    if cfg.glu:
        codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
    shard.check_even_shards(cfg.N, world)
    b, e = shard.shard_rows(cfg.N, world, rank, cfg.glu)
    codes, sfs = codes[b:e].contiguous(), weights.swizzle_scales(sfb[b:e])
    n_local = (e - b) // 2 if cfg.glu else e - b
    nbuf = max(2, -(-4 * L2_BYTES // (codes.numel() + sfs.numel())))
    ws = torch.zeros(48 << 20, dtype=torch.uint8, device="cuda")
    layers = [Fp4Linear(codes if i == 0 else codes.clone(), sfs if i == 0 else sfs.clone(), g, in_scale, n_local, cfg.K, cfg.glu, ws)
              for i in range(nbuf)]
    M = cfg.M
    xd = x.cuda()
    act = ActQuant(max(M, 128), cfg.K)
    fused = world > 1 and args.gather_mode == "fused" and cfg.glu and M > 128 and (e - b) % 256 == 0
    if fused:
        # outputs in peer-mapped memory, two buffers used alternately; the GEMM's epilogue stores into the peers' copies too
        from q27b200.peer import PeerRegion
        from q27b200.q27lib import call

        region = PeerRegion(2 * world * M * n_local * 2)
        pay = region.payload()[:2 * world * M * n_local * 2].view(torch.bfloat16).view(2, world, M, n_local)
        outs, gath = [pay[0][rank], pay[1][rank]], [pay[0], pay[1]]
        peers, wait_slots = region.peers(), (ctypes.c_int * (world - 1))(*region.peer_slots())
    else:
        outs = [torch.zeros(M, n_local, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        gath = [torch.empty(world, M, n_local, dtype=torch.bfloat16, device="cuda") for _ in range(2)] if world > 1 else None

    def step(i, gather=True):
        q, sf = act.quantize(xd, in_scale)
        lin, s_ = layers[i % nbuf], torch.cuda.current_stream().cuda_stream
        if fused and gather:
            call("q27b_gemm_fp4_glu_bf16_gather", M, lin.out, cfg.K, q, sf, lin.w, lin.sf, lin.alpha, lin.alpha, outs[i & 1],
                 ctypes.byref(peers), s_)
            call("q27b_group_gather_wait", region.ptrs[rank], world - 1, wait_slots, s_)
        else:
            lin.gemm(M, q, sf, outs[i & 1])
            if world > 1 and gather:
                torch.distributed.all_gather_into_tensor(gath[i & 1].view(-1), outs[i & 1].view(-1))

    q0, sf0 = act.quantize(xd, in_scale)

    def gemm_only(i):
        layers[i % nbuf].gemm(M, q0, sf0, outs[i & 1])

    total_bytes, flops = cfg.algorithmic_bytes(), cfg.flops()
    # how many steps make a region of MIN_REGION_MS: from a short graph-replayed run
    est = timed(step, 40, 5, world, graph_cap=40) / 40
    per = int(min(200, max(10, MIN_REGION_MS / max(est, 1e-4) / 4))) // 2 * 2  # (even: the output buffers alternate)
    steps = per * max(1, math.ceil(MIN_REGION_MS / max(est, 1e-4) / per))
    with ClockSampler(local_rank) as clk:
        ms = timed(step, steps, args.warmup, world, graph_cap=per)
    clocks = clk.summary()
    last = args.warmup + per - 1  # the last step of the replayed graph
    got = outs[last & 1].clone()
    want = torch.zeros_like(got)
    with serial_launches():
        q, sf = act.quantize(xd, in_scale)
        torch.cuda.synchronize()
        layers[last % nbuf].gemm(M, q, sf, want)
        torch.cuda.synchronize()
    ok = bool(torch.equal(got, want)) and bool(got.any())
    extra = {}
    if world > 1:
        ref_all = torch.empty(world, M, n_local, dtype=torch.bfloat16, device="cuda")
        torch.distributed.all_gather_into_tensor(ref_all.view(-1), want.view(-1))
        ok = ok and bool(torch.equal(gath[last & 1], ref_all))  # every rank holds every rank's block
        flag = torch.tensor([int(ok)], device="cuda")
        torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
        ok = bool(flag.item())
        ms_ng = timed(lambda i: step(i, gather=False), steps, args.warmup, world, graph_cap=per)
        extra["without_gather"] = {"value": flops / (ms_ng / steps / 1e3) / 1e12 if M > 128 else cfg.algorithmic_bytes() / (ms_ng / steps / 1e3) / 1e9,
                                   "ms_per_step": ms_ng / steps}
        if fused:  # the same step with one NCCL all-gather after the GEMM instead
            g2 = torch.empty(world, M, n_local, dtype=torch.bfloat16, device="cuda")

            def step_nccl(i):
                q, sf = act.quantize(xd, in_scale)
                layers[i % nbuf].gemm(M, q, sf, outs[i & 1])
                torch.distributed.all_gather_into_tensor(g2.view(-1), outs[i & 1].view(-1))

            ms_nc = timed(step_nccl, steps, args.warmup, world, graph_cap=per)
            extra["with_nccl_all_gather"] = {"value": flops / (ms_nc / steps / 1e3) / 1e12 if M > 128 else cfg.algorithmic_bytes() / (ms_nc / steps / 1e3) / 1e9,
                                             "ms_per_step": ms_nc / steps}
    ms_gemm = timed(gemm_only, steps, args.warmup, world, graph_cap=per)
    grouped = None
    if world == 1 and M <= 128 and MIN_REGION_MS >= 20.0:
        # The same GEMM on all the rotating weight copies as ONE grouped launch (behind one quantiser launch): what the
        # shape streams at once the launch boundaries are out of the way. One launch = nbuf GEMMs; reported per GEMM.
        from q27b200.group import Fp4Group, problem_of

        g_outs = [torch.zeros(M, n_local, dtype=torch.bfloat16, device="cuda") for _ in range(nbuf)]
        best = None
        for whole in (True, False):
            grp = Fp4Group(M, [problem_of(l, act.q, act.sf, o) for l, o in zip(layers, g_outs)], whole_tiles=whole)

            def step_grouped(i, grp=grp):
                act.quantize(xd, in_scale)
                grp.launch()

            reps = max(4, int(MIN_REGION_MS / max(est * nbuf, 1e-3)) // 4 * 4)
            ms_g = timed(step_grouped, reps, 3, world, graph_cap=4)
            want_g = torch.zeros_like(g_outs[0])
            with serial_launches():
                q, sf = act.quantize(xd, in_scale)
                torch.cuda.synchronize()
                if whole:  # (no K split: the many-row GEMM's bits)
                    layers[0]._dispatch(M, q, sf, want_g, None, False, layers[0].rows(), cfg.K, torch.cuda.current_stream().cuda_stream)
                else:
                    layers[0].gemm(M, q, sf, want_g)
                torch.cuda.synchronize()
            ok_g = all(bool(torch.equal(o, want_g)) for o in g_outs)
            ok = ok and ok_g
            per_gemm_s = ms_g / reps / nbuf / 1e3
            r = {"value": total_bytes_of(cfg) / per_gemm_s / 1e9, "unit": "GB/s", "us_per_gemm": per_gemm_s * 1e6,
                 "frac": total_bytes_of(cfg) / per_gemm_s / 1e9 / peaks["hbm_gbs"], "gemms_per_launch": nbuf,
                 "plan": "whole tiles" if whole else "the stand-alone launch's K split", "imbalance": grp.imbalance, "verified": ok_g}
            if best is None or r["value"] > best["value"]:
                best = r
            del grp
        grouped = best
    assert device_status() == 0, "a bounded wait inside a kernel ran out"
    per_step_s, gemm_s = ms / steps / 1e3, ms_gemm / steps / 1e3
    tensor_bound = M > 128
    n_rows_local = e - b
    launch_bytes = n_rows_local * cfg.K // 2 + n_rows_local * cfg.K // 16 + 2 * M * cfg.K + 2 * M * n_local
    if not tensor_bound:
        achieved = launch_bytes / gemm_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "traffic": ncu_traffic().get(f"cfg{cfg.index}") if world == 1 else None,
                "traffic_source": "ncu capture recorded in profiles/ncu_traffic.json (not measured by this run)",
                "algorithmic_bytes": launch_bytes, "kernel": "umma_gemm_kernel (weight streaming)", "us_per_launch": gemm_s * 1e6,
                "peak_source": peaks["source"] + ": copy bandwidth"}
        value, unit, metric = total_bytes / per_step_s / 1e9, "GB/s", "nvfp4_gemm_hbm_gbs"
    else:
        # No FP4 figure is measured on this pool: the denominator is 4 x the measured dense bf16 cuBLAS burst
        # (block-scaled FP4 runs at 4 x the bf16 rate; nominal dense FP4 is 9000 TFLOP/s).
        tpeak = 4.0 * peaks["bf16_tflops"]
        launch_flops = 2 * M * n_rows_local * cfg.K
        achieved = launch_flops / gemm_s / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": tpeak, "unit": "TFLOP/s", "frac": achieved / tpeak,
                "traffic": ncu_traffic().get(f"cfg{cfg.index}") if world == 1 else None, "algorithmic_flops": launch_flops, "kernel": many_row_kernel_name(M, fused),
                "us_per_launch": gemm_s * 1e6, "peak_sustained": 4.0 * peaks["bf16_tflops_sustained"],
                "frac_of_sustained": achieved / (4.0 * peaks["bf16_tflops_sustained"]),
                "peak_source": "4 x bf16_tflops (burst) of " + peaks["source"] + "; no FP4 peak is measured on this pool, nominal dense FP4 is 9000"}
        value, unit, metric = flops / per_step_s / 1e12, "TFLOP/s", "nvfp4_gemm_tflops"
    res = {"workload": cfg.name, "metric": metric, "value": value, "unit": unit, "ms_per_step": ms / steps, "steps": steps,
           "timed_region_ms": ms, "step": "quant_fp4_bf16 + " + ("skinny_fp4" if M <= 128 else "gemm_fp4") + ("_glu_bf16" if cfg.glu else "_bf16")
           + ("" if world == 1 else " with the gather fused into its epilogue (peer stores) + wait for the peers" if fused
              else " + all-gather (NCCL, in the graph)"),
           "l2": f"weights rotate through {nbuf} distinct copies ({nbuf * layers[0].weight_bytes() / 2**20:.0f} MiB per GPU > 126 MiB L2)",
           "roofline": roof, "clocks": clocks, "verified": ok}
    res.update(extra)
    if grouped:
        res["grouped_over_the_weight_copies"] = grouped
    log(f"{cfg.name}: {value:.1f} {unit}, GEMM {gemm_s * 1e6:.2f} us, frac {roof['frac']:.3f}, verified {ok}"
        + (f"; grouped {grouped['value']:.0f} GB/s ({grouped['frac']:.2f}, {grouped['plan']})" if grouped else ""))
    del layers, codes, sfs
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------- the CPU arm


def cpu_sweep_sample(M, steps, warmup, frac_rows=8):
    """The reference's CPU path (fake-quantise the activation, fp32 matmul against the once-dequantised weight,
    SiLU*mul; reference/qwen27b/quant.py:79-97 restated by the oracle) on a bounded sample of the sweep: ONE layer, the
    first 1/frac_rows of the output channels of each of its four projections, M tokens; all host threads. Returns
    (GB/s of the sample's algorithmic bytes, seconds per step, cores, description)."""
    from oracle import nvfp4_oracle as O
    from q27b200 import configs

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gx = torch.Generator().manual_seed(3)
    xs = {"h": torch.randn(M, configs.HIDDEN, generator=gx).to(torch.bfloat16).float().numpy(),
          "o": torch.randn(M, configs.HIDDEN, generator=gx).to(torch.bfloat16).float().numpy(),
          "d": torch.randn(M, configs.INTER, generator=gx).to(torch.bfloat16).float().numpy()}
    scales = {k: float(np.abs(v).max() / np.float32(6.0 * 448.0)) for k, v in xs.items()}
    parts, nbytes = [], 0
    for pi, (name, N, K, glu) in enumerate(configs.LAYER_PROJECTIONS):
        w = configs.make_w(N, K, 1000 + pi, 0.02).numpy()
        g = O.weight_global_scale(w)
        n_out = (N // 2 if glu else N) // frac_rows // 64 * 64
        rows = np.concatenate([np.arange(n_out), N // 2 + np.arange(n_out)]) if glu else np.arange(n_out)
        codes, sfb, _ = O.quant_weight_rtn(w[rows], g)
        del w
        wdq = torch.from_numpy(O.dequant_nvfp4(codes, sfb, g))  # dequantised once, outside the timed loop
        src = "d" if name == "down" else "o" if name == "o" else "h"
        parts.append((src, wdq, glu, n_out))
        nbytes += len(rows) * K // 2 + len(rows) * K // 16 + 2 * M * K + 2 * M * n_out

    def step():
        xq = {k: torch.from_numpy(O.quant_act_nvfp4(v, scales[k])) for k, v in xs.items()}
        outs = []
        for src, wdq, glu, n_out in parts:
            y = xq[src] @ wdq.T  # fp32, all host threads
            if glu:
                y = torch.nn.functional.silu(y[:, :n_out]) * y[:, n_out:]
            outs.append(y.to(torch.bfloat16))
        return outs

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    desc = (f"one layer of the sweep at M={M}: the first 1/{frac_rows} of the output channels of q, k, v, o, gate|up and down "
            f"({nbytes / 1e6:.1f} MB of the layer's {configs.sweep_algorithmic_bytes(M, 1) / 1e6:.1f} MB), {steps} steps; the whole "
            "sweep is 64 such layers, so GB/s carries over; weights dequantised once outside the timed loop")
    return nbytes / dt / 1e9, dt, cores, desc


def pick_gather(requested, world):
    """How every rank gets every rank's outputs on several GPUs: "fused" (peer stores from the epilogues) needs
    peer-mapped memory, set up through torch's symmetric memory; where that is not available on a box every rank falls
    back to the NCCL all-gather together (and the line says so)."""
    if world == 1:
        return "none", None
    if requested != "fused":
        return requested, None
    try:
        from q27b200.peer import PeerRegion
        probe = PeerRegion(4096)
        okp, why = (len(probe.ptrs) == world), "unexpected pointer table"
        del probe
    except Exception as e:  # noqa: BLE001
        okp, why = False, f"{type(e).__name__}: {e}"
    flag = torch.tensor([int(okp)], device="cuda")
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    if bool(flag.item()):
        return "fused", None
    note = "peer-mapped memory could not be set up (" + (why if not okp else "on another rank") + "): NCCL all-gather instead"
    log(note)
    return "nccl", note


def workload_name(layers, M):
    return f"cfg3 decode weight sweep, {layers} layers x (q|k|v, o, gate_up, down), M={M}"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=25)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="", help="comma-separated subset of sweep,cfg0,cfg1,cfg2,cfg4 (default: all that apply)")
    ap.add_argument("--m", type=int, default=0, help="the sweep at this token count only (0: all of 1..128)")
    ap.add_argument("--layers", type=int, default=64, help="layers in the sweep")
    ap.add_argument("--group-layers", type=int, default=64, help="layers per grouped launch in the headline mode")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="several GPUs: how every rank gets every rank's outputs at the end of a step of the sweep")
    ap.add_argument("--cpu-steps", type=int, default=20)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--region-ms", type=float, default=MIN_REGION_MS,
                    help="single-GEMM configurations are replayed until their timed region is this long (profiling runs: a few ms)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    globals()["MIN_REGION_MS"] = args.region_ms

    from q27b200 import configs

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    # stdout carries the one JSON line and nothing else: libraries that print to file descriptor 1 on their own
    # (NCCL's version banner) are sent to stderr, the line goes out through a private copy of the descriptor
    global _json_out
    sys.stdout.flush()
    _json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    head_m = args.m or 16

    if args.impl == "reference":
        if rank != 0:
            return
        gbs, dt, cores, desc = cpu_sweep_sample(head_m, max(1, args.steps), args.warmup)
        emit(json.dumps({
            "impl": "reference", "metric": "nvfp4_gemm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": max(1, args.steps), "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (host matmul of fake-quantised operands)", "data": "synthetic",
            "config": {"workload": workload_name(args.layers, head_m)},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    args.gather_mode, args.gather_note = pick_gather(args.gather, world)
    only = [s for s in args.only.split(",") if s]
    want = lambda name: not only or name in only  # noqa: E731

    t_start = time.perf_counter()
    line = {"metric": "nvfp4_gemm_hbm_gbs", "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic"}
    verified = True
    if want("sweep"):
        model = build_model(args.layers, rank, world)
        log(f"model built in {time.perf_counter() - t_start:.1f} s")
        r = run_sweep(args, model, rank, world, local_rank, peaks)
        del model
        torch.cuda.empty_cache()
        h, G = r["head"], r["G"]
        verified = verified and r["verified"]
        line.update({
            "value": h["gbs"], "ms_per_step": h["ms_per_sweep"],
            "config": {"workload": workload_name(args.layers, r["head_m"]),
                       "l2": f"every projection of every layer in its own device memory ({configs.layer_weight_bytes() * args.layers / 1e9:.1f} GB), far beyond the 126 MB L2",
                       "step": f"per group of {G} layer(s): one launch quantising the layers' bf16 activations (q27b_quant_fp4_batch), "
                               f"one grouped weight-streaming GEMM over their projections (q27b_skinny_fp4_group"
                               + (", planned without the K split: whole tiles)" if G >= 8 else ")")
                               + ("" if world == 1 else "; its epilogue stores every output into all peers' memory as well, a "
                                  "one-warp kernel behind it waits for the peers' signals (inside the timed graph)" if r["gather"] == "fused"
                                  else "; then one NCCL all-gather of all outputs, inside the timed graph"),
                       "timing": "CUDA-graph replay, CUDA events on the launching stream",
                       "sharding": f"weight rows N-sharded {world} way(s), no reduction"},
            "roofline": {"bound": "hbm", "achieved": h["gbs"] / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": h["gbs"] / world / peaks["hbm_gbs"], "traffic": ncu_traffic().get("cfg3_group") if world == 1 else None,
                         "traffic_source": "ncu capture recorded in profiles/ncu_traffic.json (not measured by this run)",
                         "algorithmic_bytes": h["bytes"] // world, "kernel": "skinny_group_kernel (grouped weight streaming), whole sweep, per GPU",
                         "us_per_launch": h["ms_per_sweep"] * 1e3 / math.ceil(args.layers / G),
                         "peak_source": peaks["source"] + ": copy bandwidth"},
            "clocks": h["clocks"], "sustained": h["sustained"], "e2e": h["e2e"], "gpu_launches": args.steps * h["launches"],
            **{k: h[k] for k in ("without_gather", "with_nccl_all_gather") if k in h},
            **({"gather_note": r["gather_note"]} if r["gather_note"] else {}),
            "sweep": r["sweep"], "modes": r["modes"]})
    subs = {}
    for idx in (0, 1, 2, 4):
        if not want(f"cfg{idx}"):
            continue
        if world > 1 and idx != 4:
            continue  # only the sweep and the prefill GEMM are sharded
        subs[f"cfg{idx}"] = run_single(configs.CONFIGS[idx], args, rank, world, local_rank, peaks)
        verified = verified and subs[f"cfg{idx}"]["verified"]
    line["configs"] = subs
    line["verified"] = verified
    if "value" not in line and subs:  # a run restricted to single configurations: the first one is the headline
        first = next(iter(subs.values()))
        line.update({"metric": first["metric"], "unit": first["unit"], "value": first["value"], "ms_per_step": first["ms_per_step"],
                     "steps": first["steps"], "config": {"workload": first["workload"], "step": first["step"], "l2": first["l2"]},
                     "roofline": first["roofline"], "clocks": first["clocks"], "gpu_launches": first["steps"] * 2})
    if rank == 0 and world == 1 and not args.no_cpu:
        gbs, dt, cores, desc = cpu_sweep_sample(head_m, args.cpu_steps, 2)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc, "ms_per_step_sample": dt * 1e3}
    line["bench_wall_s"] = time.perf_counter() - t_start
    if world > 1:
        torch.distributed.barrier()
    assert verified, "a timed region left outputs that differ from the one-kernel-at-a-time run"
    if rank == 0:
        emit(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
