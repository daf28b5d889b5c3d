"""Shared helpers of the GPU tests: random NVFP4 operands in the reference's fixture style
(engine/tests/test_gemm.py:17-22: uniform random code bytes, scales U(0.25, 2.25) rounded to E4M3), device
buffers through torch, and the fp64 expected value from the CPU oracle."""

import numpy as np
import torch

from oracle import nvfp4_oracle as O
from q27b200 import layouts
from q27b200.q27lib import call, lib

DEV = "cuda"


def rel_err(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def fp4_operand(rows, K, rng, scale_lo=0.25, scale_hi=2.25):
    """codes [rows][K/2] u8, scale bytes [rows][K/16] u8, dequantised fp64 [rows][K]."""
    codes = rng.randint(0, 256, size=(rows, K // 2)).astype(np.uint8)
    sf = O.e4m3_encode((rng.rand(rows, K // 16) * (scale_hi - scale_lo) + scale_lo).astype(np.float32))
    deq = O.unpack_e2m1(codes).astype(np.float64) * np.repeat(O.e4m3_decode(sf).astype(np.float64), 16, -1)
    return codes, sf, deq


def dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV)


def swizzled_dev(sf):
    """Row-major scale bytes -> device buffer in the swizzled layout, through the library's own kernel."""
    rows, kb = sf.shape
    buf = torch.zeros(lib().q27t_sf_bytes(rows, kb), dtype=torch.uint8, device=DEV)
    call("q27t_swizzle_sf", dev(sf), rows, kb, buf)
    return buf


COUNTER_BYTES = 16384


def workspace(nbytes=48 << 20, poison=True):
    """A workspace as the caller must provide it: the arrival counters at its head zeroed once, the rest
    arbitrary (poisoned with NaN bit patterns here: a partial tile read before it is written shows up)."""
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    if poison:
        ws.fill_(0xFF)
    ws[:min(COUNTER_BYTES, nbytes)] = 0
    return ws


def bf16_to_f32(t):
    return t.float().cpu().numpy()
