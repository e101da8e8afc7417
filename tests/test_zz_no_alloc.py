"""The scratch-free entry point `ade_b200_factored_static` against `ade_b200_factored`.

Some callers may not allocate device memory when they call the kernel (they run inside someone else's
memory plan, or cannot afford cudaMalloc's implicit synchronisation) and have no buffer to lend; for them
the library keeps h = V^T x in a fixed array of its own.  Both entry points launch the same kernel, so
their outputs must be identical; the test calls the new one twice in a row because the array keeps the
first call's contents.  This file is collected last on purpose.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from ade_b200 import _lib, kernels, synth

pytestmark = pytest.mark.gpu


def _static_status(lib, stream, clear=0):
    """The sticky status word of the built-in array, fetched into a device int by the accessor."""
    word = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    assert lib.ade_b200_factored_static_status(word.data_ptr(), clear, stream) == 0
    torch.cuda.synchronize()
    return int(word.item())


def test_static_scratch_entry_matches_the_regular_one():
    dev = "cuda"
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    # the last case is wide enough for the sliced phase A above 16 tokens (four slices of d_i in both entries)
    for (M, N, r, T) in [(256, 384, 256, 5), (512, 256, 512, 40), (300, 4096, 256, 40)]:
        p4 = kernels.pack_int4(synth.random_packed(M, N, r, seed=M + T), device=dev)
        W = synth.base_weight(M, N, 11).to(dev)
        x = synth.activations(T, N, 12).to(dev)
        ref = kernels.factored_forward(x, p4, weight=W)                      # regular entry, caller's scratch
        d = kernels._cdelta(p4)
        for _ in range(2):                                                    # second call sees the first one's leftovers
            out = torch.full((T, M), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = lib.ade_b200_factored_static(ctypes.byref(d), x.data_ptr(), None, W.data_ptr(), out.data_ptr(), T, stream)
            assert rc == 0, _lib.ERRORS.get(rc, rc)
            torch.cuda.synchronize()
            assert torch.equal(out, ref)
            assert _static_status(lib, stream) == 0                            # no wait for h expired
        # the reference's calling convention (y_dense supplied) through the same entry
        yd = torch.nn.functional.linear(x, W)
        ref2 = kernels.decode_forward_packed(x, yd, p4)
        out2 = torch.empty_like(ref2)
        assert lib.ade_b200_factored_static(ctypes.byref(d), x.data_ptr(), yd.data_ptr(), None, out2.data_ptr(), T, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(out2, ref2)
    # T = 128 at r = 512: h fills the array, no room is left for partial sums, so this entry computes h unsliced while
    # the regular entry (with its recommended scratch) slices it four ways.  Other summation order: compared with
    # the oracle's tolerance against the regular entry instead of bit for bit.
    from oracle import oracle as O
    M, N, r, T = 384, 4096, 512, 128
    p4 = kernels.pack_int4(synth.random_packed(M, N, r, seed=77), device=dev)
    W = synth.base_weight(M, N, 13).to(dev)
    x = synth.activations(T, N, 14).to(dev)
    yd = torch.nn.functional.linear(x, W)
    ref3 = kernels.decode_forward_packed(x, yd, p4)
    out3 = torch.empty_like(ref3)
    assert lib.ade_b200_factored_static(ctypes.byref(kernels._cdelta(p4)), x.data_ptr(), yd.data_ptr(), None,
                                        out3.data_ptr(), T, stream) == 0
    torch.cuda.synchronize()
    err, cos = O.parity(out3.float().cpu().numpy(), ref3.float().cpu().numpy())
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)
    assert _static_status(lib, stream, clear=1) == 0
    # T * r beyond the built-in buffer is refused before any launch
    p4 = kernels.pack_int4(synth.random_packed(128, 128, 2048, seed=3), device=dev)
    x = synth.activations(128, 128, 4).to(dev)
    W = synth.base_weight(128, 128, 5).to(dev)
    out = torch.empty(128, 128, dtype=torch.bfloat16, device=dev)
    assert lib.ade_b200_factored_static(ctypes.byref(kernels._cdelta(p4)), x.data_ptr(), None, W.data_ptr(),
                                        out.data_ptr(), 128, stream) == -4
