"""Generates tests/golden/nvfp4_rmsnorm_golden.npz: the reference's zero-centred RMSNorm (reference/qwen27b/model.py:
rms_norm) and the NVFP4 quantisation of its result (reference/qwen27b/quant.py: quant_act_nvfp4) on seeded inputs
of the model's hidden size, evaluated by the reference's own functions.

    python tests/golden/make_golden_rmsnorm.py /path/to/reference
"""

import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "reference"))
    from qwen27b.model import rms_norm  # noqa: E402
    from qwen27b.quant import quant_act_nvfp4  # noqa: E402

    g = torch.Generator().manual_seed(2024)
    T, D = 5, 5120
    x = torch.randn(T, D, generator=g) * 3  # the reference's fixture (engine/tests/test_elementwise.py:96-97)
    x[1] *= 1e-2
    x[2, 64:80] = 0.0
    w = (torch.randn(D, generator=g) * 0.1).bfloat16()
    eps, s = 1e-6, 0.0123
    y = rms_norm(x, w, eps)
    q = quant_act_nvfp4(y, torch.tensor(s))
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nvfp4_rmsnorm_golden.npz")
    np.savez_compressed(out, x=x.numpy(), w=w.float().numpy(), eps=np.float32(eps), in_scale=np.float32(s), y=y.numpy(),
                        y_quant=q.numpy())
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden_rmsnorm.py /path/to/reference")
    main(sys.argv[1])
