"""The N > 1 path on CPU: two gloo ranks each take their block of weight rows (shard.shard_rows), compute their
block of output columns with the CPU oracle standing in for the GPU kernels, and all-gather through
shard.all_gather_output; every rank must end up with the unsharded result, for a plain projection and for the
interleaved gate | up with the SiLU*mul epilogue. (The collective, the shard arithmetic and the gathered layout
are the product code under test; the arithmetic is the oracle's.)"""

import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import os, sys
    import numpy as np, torch, torch.distributed as dist
    root = sys.argv[1]
    sys.path[:0] = [root, os.path.join(root, "qwen3-27b-5090_b200")]
    from oracle import nvfp4_oracle as O
    from q27b200 import layouts, shard
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.RandomState(7)  # the same operands on every rank
    M, K = 5, 256
    x = rng.randn(M, K).astype(np.float32)
    s = float(np.abs(x).max() / (6 * 448))
    for n_rows, glu in ((512, False), (768, True)):
        w = (rng.randn(n_rows, K) * 0.02).astype(np.float32)
        codes, sfb, g = O.quant_weight_rtn(w)
        full = O.qlinear(x, codes, sfb, g, s)
        if glu:
            want = O.silu_mul(full[:, :n_rows // 2], full[:, n_rows // 2:])
            codes, sfb = layouts.interleave_glu(codes), layouts.interleave_glu(sfb)
        else:
            want = full
        b, e = shard.shard_rows(n_rows, world, rank, glu)
        local = O.qlinear(x, codes[b:e], sfb[b:e], g, s)  # this rank's weight rows only
        if glu:  # 128 interleaved rows = gate and up of the same 64 outputs
            idx = layouts.glu_rows((e - b) // 2)
            local = O.silu_mul(local[:, idx[:(e - b) // 2]], local[:, idx[(e - b) // 2:]])
        c0, c1 = shard.output_columns(n_rows, world, rank, glu)
        assert local.shape[1] == c1 - c0
        got = shard.all_gather_output(torch.from_numpy(np.ascontiguousarray(local, dtype=np.float32))).numpy()
        assert got.shape == want.shape, (got.shape, want.shape)
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6), np.abs(got - want).max()
        assert np.array_equal(got[:, c0:c1], local.astype(np.float32))
    # unequal contributions never reach the collective: the host check raises on every rank first
    try:
        shard.check_even_shards(640, 2)  # 5 tiles of 128 rows on 2 ranks
        raise SystemExit("uneven shards were accepted")
    except ValueError:
        pass
    shard.check_even_shards(512, 2)
    ragged = torch.zeros(M, 128 + 128 * rank)
    try:
        shard.all_gather_output(ragged)
        raise SystemExit("a ragged gather was attempted")
    except ValueError:
        pass
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_ranks_reproduce_the_unsharded_output(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=240)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out}"
        assert f"rank {rank} ok" in out
