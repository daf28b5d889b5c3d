"""Host side of the grouped weight-streaming GEMM (q27b_skinny_group_build / q27b_skinny_fp4_group): a list of skinny
GEMMs - the projections of one or several layers at one token count - planned once and then run as ONE persistent
launch in which every CTA streams its share of all the weight tiles back to back. The reference launches one kernel
per projection from Model::gemm_q (engine/src/model.cc:869-888); this is the same work with the launch boundaries
taken out, bit-identical to calling the projections one by one.
"""

from __future__ import annotations

import ctypes
import struct

import torch

from .q27lib import call

EPI_F32, EPI_BF16, EPI_GLU_BF16 = 0, 1, 2
WHOLE_TILES = 1  # Q27B_GROUP_WHOLE_TILES
TOKENS_ON_N = 2  # Q27B_GROUP_TOKENS_ON_N


class GroupProblem(ctypes.Structure):
    """Mirror of q27b_group_problem (include/q27b200/capi.h)."""

    _fields_ = [("N", ctypes.c_int), ("K", ctypes.c_int), ("epilogue", ctypes.c_int), ("alpha_count", ctypes.c_int),
                ("alpha_begin", ctypes.c_int * 4), ("alpha", ctypes.c_float * 4), ("alpha_up", ctypes.c_float),
                ("beta", ctypes.c_float), ("a", ctypes.c_void_p), ("a_sf", ctypes.c_void_p), ("w", ctypes.c_void_p),
                ("w_sf", ctypes.c_void_p), ("c", ctypes.c_void_p), ("d", ctypes.c_void_p)]


def problem_of(lin, q: torch.Tensor, sf: torch.Tensor, out: torch.Tensor, residual: torch.Tensor | None = None) -> GroupProblem:
    """The problem `lin.gemm(M, q, sf, out, residual)` would run, for an Fp4Linear `lin`."""
    p = GroupProblem()
    p.N, p.K = lin.rows(), lin.inp
    if lin.glu:
        assert out.dtype == torch.bfloat16 and residual is None
        p.epilogue = EPI_GLU_BF16
    else:
        p.epilogue = EPI_BF16 if out.dtype == torch.bfloat16 else EPI_F32
        assert p.epilogue == EPI_F32 or residual is None
    p.alpha_count = lin._nseg
    for i in range(lin._nseg):
        p.alpha_begin[i], p.alpha[i] = lin._zero[i], lin._alpha[i]
    if lin.glu:
        p.alpha[0] = lin.alpha_gate
    p.alpha_up = lin.alpha_up
    p.beta = 1.0 if residual is not None else 0.0
    p.a, p.a_sf, p.w, p.w_sf = q.data_ptr(), sf.data_ptr(), lin.w.data_ptr(), lin.sf.data_ptr()
    p.c = residual.data_ptr() if residual is not None else None
    p.d = out.data_ptr()
    return p


class Fp4Group:
    """A planned group: the table on the host and on the device, and its workspace. `problems` is a list of
    GroupProblem; the tensors they point to must stay alive (and in place) as long as the group is used."""

    def __init__(self, M: int, problems: list[GroupProblem], device="cuda", workspace: torch.Tensor | None = None,
                 whole_tiles: bool = False, tokens_on_n: bool = False):
        """whole_tiles: no tile is cut along K (for groups of several layers: fastest, and bit-identical to the
        many-row GEMM instead of to the weight-streaming launch). With whole tiles and 33..128 tokens the group is
        planned on tiles of 256 weight rows with the tokens on the MMA's M side (`self.tokens_tile == 256`) unless
        tokens_on_n is set, which the fused gather needs; the results are the same bits either way."""
        self.M, self.n = M, len(problems)
        flags = (WHOLE_TILES if whole_tiles else 0) | (TOKENS_ON_N if tokens_on_n else 0)
        arr = (GroupProblem * self.n)(*problems)
        tb, wb = ctypes.c_size_t(), ctypes.c_size_t()
        call("q27b_skinny_group_build", M, self.n, arr, flags, None, 0, ctypes.byref(tb), ctypes.byref(wb))
        self.table_host = (ctypes.c_uint8 * tb.value)()
        call("q27b_skinny_group_build", M, self.n, arr, flags, self.table_host, tb.value, ctypes.byref(tb), ctypes.byref(wb))
        self.table_bytes, self.ws_bytes = tb.value, max(wb.value, 256)
        # header of the table (GroupHeader, csrc/skinny_group.inl): what was planned
        (_, _, self.tokens_tile, _, self.ctas, self.pieces, self.counters, self.sms, self.slots) = struct.unpack_from("<I7iq", self.table_host)
        self.partials_offset = (self.counters * 4 + 255) // 256 * 256  # arrival counters first, then the partial tiles
        self.imbalance = struct.unpack_from("<i", self.table_host, 4 + 7 * 4 + 7 * 8)[0] / 1000.0  # busiest CTA over the mean
        host = torch.frombuffer(self.table_host, dtype=torch.uint8)
        self.table_dev = host.to(device)  # torch's device allocations are at least 256-byte aligned
        if workspace is None:
            workspace = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=device)  # zeroed once
        assert workspace.numel() >= self.ws_bytes
        self.ws = workspace

    def launch(self):
        call("q27b_skinny_fp4_group", self.table_host, self.table_dev, self.ws, self.ws.numel(),
             torch.cuda.current_stream().cuda_stream)

    def launch_gather(self, peers):
        """The launch with the gather fused into its epilogue: every output is also stored into the peers' memory
        (`peers`: a peer.GroupPeers; all outputs of the group must lie in the payload of one peer.PeerRegion)."""
        call("q27b_skinny_fp4_group_gather", self.table_host, self.table_dev, self.ws, self.ws.numel(), ctypes.byref(peers),
             torch.cuda.current_stream().cuda_stream)

    def run_sync(self):
        """Through the synchronous test wrapper (synchronises, checks the device status)."""
        call("q27t_skinny_fp4_group", self.table_host, self.table_dev, self.ws, self.ws.numel())
