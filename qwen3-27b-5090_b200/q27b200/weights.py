"""Load-time side of the path, in torch (runs on CPU or on the GPU that will hold the weights): the round-to-nearest
NVFP4 weight quantiser, the scale relayout and the gate | up interleave that turn an [N][K] matrix into the
buffers the kernels read.

The recipe is the reference's (scripts/quantize_proj.py:77-81 with search = 0, :94-101, :176-180):
    scale_2 = amax(W) / (6 * 448)
    sf      = e4m3(amax_block / 6 / scale_2)                (one per 16 K-elements)
    code    = rne_e2m1(w / (sf * scale_2))                  (divisor 1 where the scale is 0; zeros as code 0)
and the layouts are those of the engine's loader (engine/src/weights.cc:177-185,218-234: scales swizzled into
512-byte atoms, gate and up rows interleaved in blocks of 64).
"""

import numpy as np
import torch

from . import layouts

E2M1_MIDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def round_e2m1_index(x: torch.Tensor) -> torch.Tensor:
    """Magnitude index 0..7 of the nearest E2M1 value, ties to the even index, saturating."""
    a = x.abs().clamp(max=6.0)
    mids = torch.tensor(E2M1_MIDS, dtype=torch.float32, device=x.device)
    idx = torch.bucketize(a, mids)  # a value equal to a midpoint lands on the lower neighbour
    tie = (a.unsqueeze(-1) == mids).any(-1)
    return torch.where(tie & (idx % 2 == 1), idx + 1, idx)


def quantize_weight_rtn(w: torch.Tensor, scale_2: float | None = None, rows_per_step: int = 4096):
    """fp32 [N][K] -> (codes uint8 [N][K/2], scale bytes uint8 [N][K/16] row-major, scale_2 float)."""
    assert w.dtype == torch.float32 and w.dim() == 2 and w.shape[1] % 16 == 0
    n, k = w.shape
    dev = w.device
    # Divisors are tensors on purpose: torch turns a division by a Python scalar into a multiplication by its
    # reciprocal on CUDA, which is not the IEEE quotient the recipe (and its CPU evaluation) means.
    six, full_range, one = (torch.tensor(v, dtype=torch.float32, device=dev) for v in (6.0, 6.0 * 448.0, 1.0))
    g = torch.tensor(scale_2, dtype=torch.float32, device=dev) if scale_2 is not None else torch.div(w.abs().amax(), full_range)
    codes = torch.empty(n, k // 2, dtype=torch.uint8, device=dev)
    sfb = torch.empty(n, k // 16, dtype=torch.uint8, device=dev)
    for r in range(0, n, rows_per_step):
        wb = w[r:r + rows_per_step].reshape(-1, k // 16, 16)
        sf8 = torch.div(torch.div(wb.abs().amax(-1), six), g).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
        s = (sf8.float() * g).unsqueeze(-1)
        v = torch.div(wb, torch.where(s > 0, s, one.expand_as(s)))
        idx = round_e2m1_index(v)
        # the sign bit is set only for non-zero results (a zero is stored as code 0 whatever its sign)
        c = (idx | (((v < 0) & (idx > 0)).to(torch.int64) << 3)).to(torch.uint8).reshape(-1, k)
        codes[r:r + rows_per_step] = c[:, 0::2] | (c[:, 1::2] << 4)
        sfb[r:r + rows_per_step] = sf8.view(torch.uint8)
    return codes, sfb, float(g)


def swizzle_scales(sf_rowmajor: torch.Tensor) -> torch.Tensor:
    """Row-major scale bytes [rows][kblocks] -> swizzled buffer (on the tensor's device; padding is zero)."""
    rows, kb = sf_rowmajor.shape
    out = torch.zeros(layouts.sf_bytes(rows, kb), dtype=torch.uint8, device=sf_rowmajor.device)
    idx = torch.from_numpy(layouts.sf_index(rows, kb)).to(sf_rowmajor.device)
    out[idx.flatten()] = sf_rowmajor.flatten()
    return out


def interleave_gate_up(t: torch.Tensor) -> torch.Tensor:
    """[2I][...] gate rows then up rows -> blocks of 64 gate rows followed by the 64 up rows of the same outputs."""
    return layouts.interleave_glu(t)


def quantize_weight_search(w: torch.Tensor, scale_2: float | None = None):
    """bf16 [N][K] on the GPU -> (codes uint8 [N][K/2], SWIZZLED scale buffer, scale_2 float) through the library's
    load-time quantiser (q27b_quant_fp4_weight: every block's scale searched for the smallest squared error, the
    engine's way of making an NVFP4 copy of a bf16 weight at load, engine/src/weights.cc:560-570)."""
    from .q27lib import call

    assert w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[1] % 64 == 0 and w.is_contiguous()
    n, k = w.shape
    if scale_2 is None:
        scale_2 = float(torch.div(w.float().abs().amax(), torch.tensor(6.0 * 448.0, device=w.device)))
    codes = torch.empty(n, k // 2, dtype=torch.uint8, device=w.device)
    sf = torch.zeros(layouts.sf_bytes(n, k // 16), dtype=torch.uint8, device=w.device)
    call("q27b_quant_fp4_weight", w, n, k, float(scale_2), codes, sf, torch.cuda.current_stream().cuda_stream)
    return codes, sf, float(scale_2)
