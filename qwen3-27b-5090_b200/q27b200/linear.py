"""Host-side mirror of the engine's NVFP4 linear layer for this path: the weight record the reference keeps per
projection (LinearFp4 {w, sf, w_scale2, in_scale, out, in, alpha}, engine/src/weights.h:25-31) and the dispatch
of Model::gemm_q / Model::mlp (engine/src/model.cc:869-888,1054-1096): quantise the activation, then the
weight-streaming GEMM for few rows and the many-row GEMM otherwise. Every launch goes through the C ABI on
torch's current stream; torch only owns the device memory.
"""

from __future__ import annotations

import ctypes
import os
import sys

import torch

from . import layouts, weights
from .q27lib import call, lib

SKINNY_MAX_M = 128  # rows up to which the weight-streaming kernel is used (the reference: 64)
# The reference shares one 32 MiB workspace (engine/src/model.h:462), enough here for every shape of the model up to
# 64 tokens (19.4 MiB); 65 .. 128 tokens need up to 38.8 MiB (q27b_skinny_workspace_bytes gives the exact figure).
WORKSPACE_BYTES = 40 << 20


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class ActQuant:
    """Device scratch for one quantised activation [max_rows][K] (codes + swizzled scales), reused across calls."""

    def __init__(self, max_rows: int, K: int, device="cuda"):
        self.K = K
        self.q = torch.empty(max_rows, K // 2, dtype=torch.uint8, device=device)
        # zero once: rows past M inside the last 128-row atom are never valid but are copied along
        self.sf = torch.zeros(layouts.sf_bytes(max_rows, K // 16), dtype=torch.uint8, device=device)

    def quantize(self, x: torch.Tensor, input_scale: float):
        M, K = x.shape
        assert K == self.K and x.is_contiguous() and M <= self.q.shape[0]
        name = {torch.bfloat16: "q27b_quant_fp4_bf16", torch.float32: "q27b_quant_fp4"}[x.dtype]
        call(name, x, M, K, float(input_scale), self.q, self.sf, _stream())
        return self.q, self.sf


class Fp4Linear:
    """y = alpha * quant(x) . W^T for one NVFP4 projection; `glu=True` holds gate | up interleaved and produces
    silu(gate) * up. Weights live on the device; nothing is allocated per call when `out` is passed."""

    def __init__(self, codes, sf_swizzled, w_scale2: float, in_scale: float, out_features: int, in_features: int,
                 glu: bool = False, workspace: torch.Tensor | None = None):
        self.w, self.sf = codes, sf_swizzled
        self.w_scale2, self.in_scale = float(w_scale2), float(in_scale)
        self.out, self.inp, self.glu = out_features, in_features, glu
        self.alpha = self.in_scale * self.w_scale2  # engine/src/weights.cc:286
        # gate | up: the two halves may carry tensor scales of their own (a checkpoint's gate_proj and up_proj); the
        # SiLU*mul epilogue applies them (engine/src/weights.cc:302-310)
        self.w_scale2_gate = self.w_scale2_up = self.w_scale2
        self.alpha_gate = self.alpha_up = self.alpha
        dev = codes.device
        # zeroed once: the head of the workspace holds arrival counters that the kernels leave at zero
        self.ws = workspace if workspace is not None else torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=dev)
        self._act: ActQuant | None = None
        self._set_segments([0], [self.alpha])

    def _set_segments(self, begins, alphas):
        # output-channel segments with their own alpha (AlphaSegments, engine/src/kernels.h:228-239): at most four
        assert 1 <= len(begins) == len(alphas) <= 4 and begins[0] == 0
        self._nseg = len(begins)
        self._zero = (ctypes.c_int * self._nseg)(*begins)
        self._alpha = (ctypes.c_float * self._nseg)(*alphas)

    def set_in_scale(self, in_scale: float):
        """A new activation tensor scale: alpha = in_scale * w_scale2 per segment."""
        self.in_scale = float(in_scale)
        self.alpha = self.in_scale * self.w_scale2
        self.alpha_gate, self.alpha_up = self.in_scale * self.w_scale2_gate, self.in_scale * self.w_scale2_up
        for i, g in enumerate(getattr(self, "_w_scales", [self.w_scale2])):
            self._alpha[i] = self.in_scale * g

    @classmethod
    def fused(cls, parts: "list[Fp4Linear]"):
        """Projections that read the same activation, stacked along the output dimension into one weight with one
        alpha per part (the engine's fuse4, engine/src/weights.cc:254-267): one launch instead of len(parts). Each
        part's rows are a multiple of 128, so the swizzled scale buffers concatenate as they are."""
        assert 2 <= len(parts) <= 4 and all(not p.glu and p.inp == parts[0].inp and p.rows() % 128 == 0 for p in parts)
        codes = torch.cat([p.w for p in parts]).contiguous()
        sfs = torch.cat([p.sf for p in parts]).contiguous()
        f = cls(codes, sfs, parts[0].w_scale2, parts[0].in_scale, codes.shape[0], parts[0].inp, False, parts[0].ws)
        begins, row = [], 0
        for p in parts:
            begins.append(row)
            row += p.rows()
        f._w_scales = [p.w_scale2 for p in parts]
        f._set_segments(begins, [f.in_scale * g for g in f._w_scales])
        return f

    @classmethod
    def from_float(cls, w: torch.Tensor, in_scale: float, glu: bool = False, device="cuda", workspace=None):
        """Quantises an fp32 [N][K] weight (for glu: gate rows then up rows, one tensor scale over both) on
        `device` and lays it out for the kernels."""
        w = w.to(device=device, dtype=torch.float32)
        codes, sfb, g = weights.quantize_weight_rtn(w)
        if glu:
            codes, sfb = weights.interleave_gate_up(codes), weights.interleave_gate_up(sfb)
        n, k = w.shape
        return cls(codes.contiguous(), weights.swizzle_scales(sfb), g, in_scale, n // 2 if glu else n, k, glu, workspace)

    def rows(self) -> int:
        return self.w.shape[0]

    def weight_bytes(self) -> int:
        return self.w.numel() + self.sf.numel()

    def _scratch(self, M: int) -> ActQuant:
        if self._act is None or self._act.q.shape[0] < M:
            self._act = ActQuant(max(M, 128), self.inp, self.w.device)
        return self._act

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, out_dtype=torch.bfloat16,
                 residual: torch.Tensor | None = None) -> torch.Tensor:
        """x: bf16 or fp32 [M][K] on the device. Returns [M][out] (bf16 by default; fp32 allows a residual:
        out = alpha * x . W^T + residual, which may be `out` itself)."""
        M = x.shape[0]
        if out is None:
            out = torch.empty(M, self.out, dtype=out_dtype, device=x.device)
        if M == 0:
            return out
        q, sf = self._scratch(M).quantize(x, self.in_scale)
        self.gemm(M, q, sf, out, residual)
        return out

    def gemm(self, M, q, sf, out, residual=None):
        """The dispatch of Model::gemm_q (engine/src/model.cc:869-888) with its two debugging switches, read at every
        call like the reference's: Q27_NO_SKINNY=1 sends every token count to the many-row kernel; Q27_SKINNY_CHECK=1
        runs the many-row kernel beside the weight-streaming one and reports a relative difference above 1e-4 on
        stderr (engine/src/model.cc:773-805). The check synchronises; it is a debugging aid, not a product path."""
        N, K, s = self.rows(), self.inp, _stream()
        skinny = M <= SKINNY_MAX_M and os.environ.get("Q27_NO_SKINNY", "0") in ("", "0")
        if skinny and os.environ.get("Q27_SKINNY_CHECK", "0") not in ("", "0") and self._nseg == 1 and residual is None and N % 128 == 0 and K % 128 == 0:
            self._dispatch(M, q, sf, out, residual, True, N, K, s)
            other = torch.empty_like(out)
            self._dispatch(M, q, sf, other, residual, False, N, K, s)
            a, b = out.float(), other.float()
            rel = float((a - b).norm() / b.norm().clamp_min(1e-30))
            if rel > 1e-4:
                print(f"Q27_SKINNY_CHECK: M={M} N={N} K={K}: weight-streaming vs many-row GEMM differ by {rel:.3e}", file=sys.stderr)
            return
        self._dispatch(M, q, sf, out, residual, skinny, N, K, s)

    def _dispatch(self, M, q, sf, out, residual, skinny, N, K, s):
        if self.glu:
            assert out.dtype == torch.bfloat16 and residual is None
            if skinny:
                call("q27b_skinny_fp4_glu_bf16", M, self.out, K, q, sf, self.w, self.sf, self.alpha_gate, self.alpha_up, out,
                     self.ws, self.ws.numel(), s)
            else:
                call("q27b_gemm_fp4_glu_bf16", M, self.out, K, q, sf, self.w, self.sf, self.alpha_gate, self.alpha_up, out, s)
        elif out.dtype == torch.bfloat16:
            assert residual is None
            if skinny:
                call("q27b_skinny_fp4_bf16", M, N, K, q, sf, self.w, self.sf, self._nseg, self._zero, self._alpha, out, self.ws,
                     self.ws.numel(), s)
            else:
                assert self._nseg == 1, "the many-row GEMM takes one alpha"
                call("q27b_gemm_fp4_bf16", M, N, K, q, sf, self.w, self.sf, self.alpha, out, s)
        else:
            beta = 1.0 if residual is not None else 0.0
            if skinny:
                call("q27b_skinny_fp4", M, N, K, q, sf, self.w, self.sf, self._nseg, self._zero, self._alpha, residual, beta, out,
                     self.ws, self.ws.numel(), s)
            else:
                assert self._nseg == 1, "the many-row GEMM takes one alpha"
                call("q27b_gemm_fp4", M, N, K, q, sf, self.w, self.sf, self.alpha, residual, beta, out, s)


class Fp4Mlp:
    """The NVFP4 MLP of one layer, down(silu(gate(x)) * up(x)) (+ residual), as Model::mlp runs it
    (engine/src/model.cc:1054-1096): `gate_up` holds gate | up interleaved, `down` consumes NVFP4 activations
    quantised with its own in_scale.

    * many rows (M > 128): one gate | up GEMM whose epilogue writes silu(gate) * up as NVFP4 codes and scales
      (gemm_fp4_glu), then the down GEMM on them: the [M][I] intermediate never exists in bf16 or fp32;
    * few rows: the weight-streaming GEMM to fp32 [M][2 I], the SiLU*mul quantiser, the weight-streaming down GEMM.
    """

    def __init__(self, gate_up: Fp4Linear, down: Fp4Linear, alpha_gate: float | None = None, alpha_up: float | None = None):
        assert gate_up.glu and not down.glu and gate_up.out == down.inp
        self.gate_up, self.down = gate_up, down
        self.alpha_gate = gate_up.alpha_gate if alpha_gate is None else float(alpha_gate)
        self.alpha_up = gate_up.alpha_up if alpha_up is None else float(alpha_up)
        self._one = (ctypes.c_float * 1)(1.0)
        self._zero = (ctypes.c_int * 1)(0)
        self._rows = 0

    def _buffers(self, M: int):
        if self._rows < M:
            dev, inter = self.gate_up.w.device, self.gate_up.out
            self._rows = max(M, 128)
            self._x = ActQuant(self._rows, self.gate_up.inp, dev)
            self._h = ActQuant(self._rows, inter, dev)
            self._gu = torch.empty(min(self._rows, SKINNY_MAX_M), 2 * inter, dtype=torch.float32, device=dev)
        return self._x, self._h, self._gu

    def __call__(self, x: torch.Tensor, residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """x: bf16 / fp32 [M][hidden]; returns fp32 [M][hidden] = down(...) (+ residual, which may be `out`)."""
        M = x.shape[0]
        gu, dn, s = self.gate_up, self.down, _stream()
        if out is None:
            out = torch.empty(M, dn.rows(), dtype=torch.float32, device=x.device)
        if M == 0:
            return out
        xq, hq, gbuf = self._buffers(M)
        q, sf = xq.quantize(x, gu.in_scale)
        if M > SKINNY_MAX_M:
            call("q27b_gemm_fp4_glu", M, gu.out, gu.inp, q, sf, gu.w, gu.sf, self.alpha_gate, self.alpha_up, dn.in_scale,
                 hq.q, hq.sf, s)
        else:
            call("q27b_skinny_fp4", M, gu.rows(), gu.inp, q, sf, gu.w, gu.sf, 1, self._zero, self._one, None, 0.0, gbuf,
                 gu.ws, gu.ws.numel(), s)
            call("q27b_silu_mul_quant_fp4_glu", gbuf, M, gu.out, self.alpha_gate, self.alpha_up, dn.in_scale, hq.q, hq.sf, s)
        dn.gemm(M, hq.q, hq.sf, out, residual)
        return out
