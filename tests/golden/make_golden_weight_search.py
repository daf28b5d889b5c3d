"""Generates tests/golden/nvfp4_weight_search_golden.npz: the searched weight quantiser evaluated with the
reference's own Python functions.

    python tests/golden/make_golden_weight_search.py /path/to/reference

The reference's load-time quantiser is a CUDA kernel (engine/src/kernels.cu:167-206), which cannot run where this
file is made; its Python twin (scripts/quantize_proj.py: block_error, choose_scales) searches a narrower range of
scale codes. So the golden vectors are built from the twin's pieces on the kernel's candidate set: for every block
the squared error of each of the kernel's 13 candidate codes from quantize_proj.block_error, the first smallest
one chosen as the kernel does, and the codes packed by quantize_proj.pack. The division by the scale and torch's
summation order differ from the kernel's reciprocal and running sum in the last bit, so a block whose two best
candidates are within rounding of each other may legitimately choose the other one; the test allows exactly that.
"""

import os
import sys

import numpy as np
import torch

OFFSETS = (0, -1, -2, -3, -4, 1, 2, 3, 4, 5, 6, 7, 8)  # engine/src/kernels.cu:187-188


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "reference"))
    sys.path.insert(0, os.path.join(ref_root, "scripts"))
    import quantize_proj as qp  # noqa: E402

    g = torch.Generator().manual_seed(77)
    n, k = 96, 512
    w = (torch.randn(n, k, generator=g) * 0.02)
    w[3, :16] = 0.0                       # an all-zero block keeps the rounded code
    w[5, 16:32] *= 50.0                   # an outlier block
    w[7, 32:48] = w[7, 32:48].abs() * 0   # another zero block
    w[9] *= 1e-3                          # small rows: codes near the bottom of the range
    w = w.to(torch.bfloat16).float()      # the kernel reads bf16 weights
    gscale = w.abs().max() / (6.0 * 448.0)
    wb = w.view(n, k // 16, 16)
    hd = torch.ones(k // 16, 16)
    sf0 = qp.to_e4m3(wb.abs().amax(-1) / qp.E2M1_MAX / gscale)
    c0 = sf0.to(torch.float8_e4m3fn).view(torch.uint8).to(torch.int16)
    errs = []
    cands = []
    for d in OFFSETS:
        c = (c0 + d).clamp(1, 126)
        sf = qp.e4m3_from_code(c)
        errs.append(qp.block_error(wb, sf, gscale, hd))
        cands.append(c)
    errs, cands = torch.stack(errs), torch.stack(cands)       # [13, n, nb]
    pick = errs.argmin(0)                                      # the first of equal minima, as the kernel's strict <
    best = torch.gather(cands, 0, pick[None])[0]
    best = torch.where(sf0 > 0, best, c0)
    sf = qp.e4m3_from_code(best)
    sf = torch.where(sf0 > 0, sf, sf0)
    codes, sf8 = qp.pack(w, sf, gscale)
    out = {"w": w.numpy(), "gscale": np.float32(gscale), "errs": errs.numpy(), "cands": cands.numpy().astype(np.int16),
           "best": best.numpy().astype(np.uint8), "codes": codes.numpy(), "sf": sf8.view(torch.uint8).numpy()}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nvfp4_weight_search_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
