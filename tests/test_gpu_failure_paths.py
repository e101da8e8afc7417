"""The kernels' time-out paths, exercised without any fault: a diagnostic option makes the producers inside a kernel
stay silent (phase-A units do not report, code loads are not issued), a short wait limit makes the consumers give up,
and the test checks that the launch returned, that the status word says what happened, and that the next ordinary
call is correct again.  No trap, no bad address, no endless loop is involved; the GPU context stays usable."""
from __future__ import annotations

import pytest
import torch

from ade_b200 import _lib, kernels, synth

pytestmark = pytest.mark.gpu
DEV = "cuda"
LIMIT = 400_000          # clock cycles, about 0.2 ms


@pytest.fixture
def silent_producers():
    _lib.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, LIMIT)
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 1)
    try:
        yield
    finally:
        _lib.set_option(_lib.OPT_DROP_SIGNALS, 0)
        _lib.set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 0)


@pytest.mark.parametrize("T,fused", [(4, True), (16, True), (40, False), (128, False)])
def test_factored_wait_for_h_expires_and_recovers(T, fused, silent_producers):
    M, N, r = 512, 1024, 256
    p4 = kernels.pack_int4(synth.random_packed(M, N, r, 5), device=DEV)
    W = synth.base_weight(M, N, 6).to(DEV)
    x = synth.activations(T, N, 7).to(DEV)
    yd = None if fused else torch.nn.functional.linear(x, W)
    call = lambda: kernels.factored_forward(x, p4, weight=W if fused else None, y_dense=yd)
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 0)
    good = call()
    torch.cuda.synchronize()
    assert kernels.factored_status(DEV, T, r) == 0
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 1)
    call()                                                  # nobody reports h: every CTA's wait runs out
    torch.cuda.synchronize()                                # ... and the launch still ends
    assert kernels.factored_status(DEV, T, r) == 1
    with pytest.raises(_lib.AdeKernelError):
        kernels.check_factored_status(DEV)
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 0)
    kernels.reset_factored_scratch(DEV)
    again = call()
    torch.cuda.synchronize()
    assert kernels.factored_status(DEV, T, r) == 0 and torch.equal(again, good)


@pytest.mark.parametrize("r,codes,expanded", [(256, {1, 2, 3, 4, 5, 8, 9}, False), (640, {1, 2, 3, 4, 5, 8, 9}, False),
                                              (1152, {1, 3}, False), (256, {1, 3, 9}, True), (640, {1, 3, 9}, True)])
def test_reconstruction_waits_expire_and_recover(r, codes, expanded, silent_producers):
    """Both configurations of the strip-resident kernel (with packed and with expanded operands) and the general
    kernel: without code loads the first waiting role records its ADE_DEV_TIMEOUT_* code, every role runs to its
    end, tensor memory is released."""
    M, N = 384, 512
    p4 = kernels.pack_int4(synth.random_packed(M, N, r, 8), device=DEV)
    W = synth.base_weight(M, N, 9).to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 0)
    x8 = kernels.expand_codes(p4) if expanded else None
    good = kernels.recon_int4(p4, W, status=status, expanded=x8)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 1)
    kernels.recon_int4(p4, W, status=status, expanded=x8)
    torch.cuda.synchronize()
    code = int(status.item())
    assert code in codes, _lib.DEVICE_STATUS.get(code, code)
    _lib.set_option(_lib.OPT_DROP_SIGNALS, 0)
    status.zero_()
    again = kernels.recon_int4(p4, W, status=status, expanded=x8)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(again, good)
