"""Generates tests/golden/nvfp4_golden.npz by running the reference's own Python code on seeded inputs.

Run once, in a container that has the reference checked out (its path is the first argument):

    python tests/golden/make_golden.py /path/to/reference

It imports reference/qwen27b/quant.py (activation quantiser, dequantiser, E2M1 / E4M3 rounding, QLinear) and
scripts/quantize_proj.py (round-to-nearest weight quantiser, packer) unmodified and stores inputs and outputs.
The test-suite only reads the .npz; it never needs the reference tree.
"""

import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "reference"))
    sys.path.insert(0, os.path.join(ref_root, "scripts"))
    from qwen27b import quant as rq  # noqa: E402

    # quantize_proj.py parses arguments only under __main__; importing it is side-effect free.
    import quantize_proj as qp  # noqa: E402

    rng = np.random.RandomState(20240607)
    out = {}

    # --- E2M1 rounding on a dense sweep incl. every midpoint, +-0, saturation
    sweep = np.concatenate([
        np.linspace(-8, 8, 2049, dtype=np.float32),
        np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0], np.float32),
        np.nextafter(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32), np.float32(10)),
        np.nextafter(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32), np.float32(-10)),
        np.array([0.0, -0.0, 1e-30, -1e-30, 100.0, -100.0, 7.0], np.float32),
    ])
    out["e2m1_in"] = sweep
    out["e2m1_out"] = rq.round_e2m1(torch.from_numpy(sweep)).numpy()

    # --- E4M3 cast: every code's value, every midpoint between neighbours, the neighbours of those, saturation
    codes = np.arange(256, dtype=np.uint8)
    vals = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    pos = np.sort(vals[np.isfinite(vals) & (vals >= 0)]).astype(np.float32)
    mids = ((pos[1:].astype(np.float64) + pos[:-1]) / 2).astype(np.float32)
    e4 = np.concatenate([pos, mids, np.nextafter(mids, np.float32(1e9)), np.nextafter(mids, np.float32(-1e9)),
                         np.array([448.0, 449.0, 463.9, 464.0, 500.0, 1000.0, 1e-9, 2.0**-10, 2.0**-9], np.float32)])
    e4 = np.concatenate([e4, -e4])
    out["e4m3_in"] = e4
    out["e4m3_out"] = rq.to_e4m3(torch.from_numpy(e4)).numpy()
    out["e4m3_code"] = torch.from_numpy(e4).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()

    # --- activation quantiser: row magnitudes 1e-2..1e1, an all-zero block, a saturating block, tiny values
    m, k = 37, 512
    x = (rng.standard_normal((m, k)) * np.logspace(-2, 1, m)[:, None]).astype(np.float32)
    x[3, :16] = 0.0
    x[5, 16:32] = 1e4  # block scale saturates at 448
    x[7, 32:48] *= 1e-6  # scale rounds to zero / subnormal
    s = np.float32(0.0123)
    out["act_x"], out["act_scale"] = x, s
    out["act_deq"] = rq.quant_act_nvfp4(torch.from_numpy(x), torch.tensor(s)).numpy()
    xb = torch.from_numpy(x.astype(np.float32)).to(torch.bfloat16)
    out["act_x_bf16_bits"] = xb.view(torch.int16).numpy().view(np.uint16)
    out["act_deq_bf16"] = rq.quant_act_nvfp4(xb, torch.tensor(s)).numpy()

    # --- weight quantiser (search = 0) + packer + dequantiser
    n, k = 256, 512
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    w[11, :16] = 0.0
    wt = torch.from_numpy(w)
    gscale = wt.abs().amax() / (rq.E2M1_MAX * rq.E4M3_MAX)
    sf = qp.quant_rtn(wt, gscale, None, 0)
    wq, wsf = qp.pack(wt, sf, gscale)
    out["w"], out["w_gscale"] = w, np.float32(gscale.item())
    out["w_codes"], out["w_sf"] = wq.numpy(), wsf.view(torch.uint8).numpy()
    wdq = rq.dequant_nvfp4(wq, wsf, gscale)
    out["w_deq"] = wdq.numpy()

    # --- unpack on raw random bytes (includes the -0 code)
    raw = rng.randint(0, 256, size=(4, 64)).astype(np.uint8)
    out["unpack_in"], out["unpack_out"] = raw, rq.unpack_e2m1(torch.from_numpy(raw)).numpy()

    # --- QLinear on the above (fp32 as the reference evaluates it, and fp64 as its GPU tests do)
    xs = (rng.standard_normal((9, k))).astype(np.float32)
    in_scale = np.float32(np.abs(xs).max() / (6 * 448))
    lin = rq.QLinear("nvfp4", wdq, torch.tensor(in_scale), act_quant=True)
    out["lin_x"], out["lin_in_scale"] = xs, in_scale
    out["lin_y_f32"] = lin(torch.from_numpy(xs)).numpy()
    xq = rq.quant_act_nvfp4(torch.from_numpy(xs), torch.tensor(in_scale))
    out["lin_y_f64"] = (xq.double() @ wdq.double().T).numpy()

    # --- silu(gate) * up as the reference model's MLP evaluates it
    g = (rng.standard_normal((5, 64)) * 4).astype(np.float32)
    u = rng.standard_normal((5, 64)).astype(np.float32)
    out["silu_g"], out["silu_u"] = g, u
    out["silu_out"] = (torch.nn.functional.silu(torch.from_numpy(g)) * torch.from_numpy(u)).numpy()

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nvfp4_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
