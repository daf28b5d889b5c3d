"""The workspace-free variant of the weight-streaming GEMM (q27b_skinny_fp4_static).

Who needs it: callers that are not allowed to allocate device memory at the point where they run the GEMM and have
no buffer of their own to lend as a workspace - an inference process that fixed its whole memory plan at start-up,
a plug-in loaded into such a process. Its scratch is an array
inside the library image (7.8 MiB per GPU), which limits it to M <= 16.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already run everything else.
It checks, on two calls in a row (the second call finds the array as the first one left it), that the result is
bit-identical to the ordinary entry point, for shapes whose tiles are and are not cut between CTAs, with and without
a residual, and that sizes beyond the limit are rejected with a clear message.
"""

import numpy as np
import pytest
import torch

from helpers import DEV, dev, fp4_operand, rel_err, swizzled_dev, workspace
from q27b200.q27lib import call

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(1, 5120, 5120), (16, 34816, 5120), (7, 5120, 17408), (3, 128, 5120)])
def test_static_scratch_matches_workspace_entry_point(M, N, K):
    rng = np.random.RandomState(M + N + K)
    a, asf, adq = fp4_operand(M, K, rng)
    b, bsf, bdq = fp4_operand(N, K, rng)
    ad, bd, asw, bsw = dev(a), dev(b), swizzled_dev(asf), swizzled_dev(bsf)
    ws = workspace()
    alpha = 0.37
    want = torch.empty(M, N, device=DEV)
    call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, alpha, None, 0.0, want, ws, ws.numel())
    assert rel_err(want.cpu().numpy(), alpha * (adq @ bdq.T)) < 1e-5
    c = torch.randn(M, N, device=DEV)
    want_res = c.clone()
    call("q27t_skinny_fp4", M, N, K, ad, asw, bd, bsw, alpha, want_res, 1.0, want_res, ws, ws.numel())
    got = torch.empty(M, N, device=DEV)
    got_res = torch.empty(M, N, device=DEV)
    call("q27t_skinny_fp4_static", M, N, K, ad, asw, bd, bsw, alpha, None, 0.0, got)  # (first use on this device)
    torch.equal(got, want)  # (torch's comparison takes its scratch from the caching allocator once, before the reading)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(2):  # the second call runs on the scratch array exactly as the first one left it
        got.fill_(float("nan"))
        call("q27t_skinny_fp4_static", M, N, K, ad, asw, bd, bsw, alpha, None, 0.0, got)
        assert torch.equal(got, want)  # same kernel, same split: the tolerance is zero
        got_res.copy_(c)
        call("q27t_skinny_fp4_static", M, N, K, ad, asw, bd, bsw, alpha, got_res, 1.0, got_res)
        assert torch.equal(got_res, want_res)
    # what the entry point is for: the calls took no device memory (every tensor above existed before them)
    assert torch.cuda.mem_get_info()[0] == free_before


def test_static_scratch_rejects_sizes_beyond_its_limit():
    M, N, K = 17, 128, 256
    t = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    out = torch.zeros(M, N, device=DEV)
    with pytest.raises(RuntimeError, match=r"M must be 1\.\.16"):
        call("q27t_skinny_fp4_static", M, N, K, t, t, t, t, 1.0, None, 0.0, out)
