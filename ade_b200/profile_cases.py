"""Small, fixed workloads for profiling one kernel at a time.

    python -m ade_b200.profile_cases recon [M N r]        # default 11008 4096 512 (Llama-2-7B gate_proj delta)
    python -m ade_b200.profile_cases factored [T M N r]   # default 16 4096 4096 256 (q_proj delta)

Each case launches its kernel a handful of times on seeded random packed fields (no SVD) and holds
well under 1 GB on the device, so that a profiler capture of two or three launches ends in a minute.
"""
from __future__ import annotations

import sys

import torch

from . import kernels, synth


def main(argv):
    what = argv[0] if argv else "recon"
    dev = "cuda"
    if what == "recon":
        M, N, r = (int(a) for a in argv[1:4]) if len(argv) >= 4 else (11008, 4096, 512)
        p4 = kernels.pack_int4(synth.random_packed(M, N, r, 1), device=dev)
        W = synth.base_weight(M, N, 5).to(dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        for _ in range(4):
            kernels.recon_int4(p4, W, status=status)
        torch.cuda.synchronize()
        print(f"recon {M}x{N} r={r}: 4 launches, device status {int(status.item())}")
    elif what == "factored":
        T, M, N, r = (int(a) for a in argv[1:5]) if len(argv) >= 5 else (16, 4096, 4096, 256)
        p4 = kernels.pack_int4(synth.random_packed(M, N, r, 1), device=dev)
        W = synth.base_weight(M, N, 5).to(dev)
        x = synth.activations(T, N, 6).to(dev)
        for _ in range(4):
            kernels.factored_forward(x, p4, weight=W)
        torch.cuda.synchronize()
        print(f"factored T={T} {M}x{N} r={r}: 4 launches, status {kernels.factored_status(dev, T, r)}")
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main(sys.argv[1:])
