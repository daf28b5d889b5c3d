"""The device status word: every wait inside the kernels is bounded, and a wait that runs out is reported to the host
instead of hanging the GPU. The self-test below makes a wait run out on purpose in the only safe way: a barrier
nothing arrives at, a budget of one millisecond, a kernel that then ends normally."""

import numpy as np
import pytest
import torch

from helpers import DEV, dev, fp4_operand, rel_err, swizzled_dev, workspace
from q27b200.q27lib import call

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports():
    """The kernels' waits are bounded: a wait that cannot succeed (a barrier nothing arrives at, budget 1 ms) ends by
    itself, the kernel returns normally, the status word names the reason, reading it clears it, and the device
    goes on working (no fault, no hang, no lost context)."""
    from q27b200.q27lib import device_status

    assert device_status() == 0
    call("q27b_probe_wait_timeout", 1000, torch.cuda.current_stream().cuda_stream)
    assert device_status() == 6  # kStatusProbeTimeout
    assert device_status() == 0  # cleared by the read
    rng = np.random.RandomState(1)
    a, asf, adq = fp4_operand(2, 1024, rng)
    w, wsf, wdq = fp4_operand(256, 1024, rng)
    d = torch.empty(2, 256, device=DEV)
    ws = workspace()
    call("q27t_skinny_fp4", 2, 256, 1024, dev(a), swizzled_dev(asf), dev(w), swizzled_dev(wsf), 1.0, None, 0.0, d, ws, ws.numel())
    assert rel_err(d.cpu().numpy(), adq @ wdq.T) < 1e-5 and device_status() == 0
