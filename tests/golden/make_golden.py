"""Generate the golden fixtures under tests/golden/ from the reference's own Python code.

Run where the reference checkout is available (it is imported, never copied):

    python tests/golden/make_golden.py --reference /path/to/ADE

For each small seeded case the script builds a synthetic delta the way the benchmark
configurations describe it (low-rank A.B plus noise, truncated SVD), compresses it with the
reference's ``quantization.compress_module`` and records, next to the inputs, what the
reference computes from them:

* ``reconstruct_delta``                      (quantization.py, float32 delta of eq. 7)
* per-group INT32 ``prod``                   (obtained from ``reconstruct_delta`` itself by calling
                                              it on one group with unit scales: the float32 result
                                              is then the integer product, exactly)
* ``dequantize_rowwise`` / ``dequantize_colwise``
* ``kernels.pack_int4``                      (reference stored form uq, vq, R, C)
* ``serving.ADEKernelLinear`` CPU fallback   (use_decode=False, use_recon=False; float16 output)
* ``adaptation.FoldInLinear`` in float32     (the reference's PyTorch factored application)
* ``quantize_rowwise`` / ``quantize_colwise`` on a stored float32 matrix, and the Sylvester
  rotation, to pin the format producer.

16-bit tensors are stored as bit patterns (uint16).  The fixtures are tiny (a few hundred KB).
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, M, N, r, T): every dimension the kernels tile on appears at least once ragged in T
CASES = [
    ("a_128x128_r128_t3", 128, 128, 128, 3),
    ("b_256x128_r256_t16", 256, 128, 256, 16),
    ("c_128x256_r384_t17", 128, 256, 384, 17),     # non power-of-two rank: random orthogonal H
    ("d_256x256_r128_t1", 256, 256, 128, 1),
]


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.uint16).numpy().copy()


def synth(M, N, r, T, seed):
    g = torch.Generator().manual_seed(seed)
    W_b = (torch.randn(M, N, generator=g) * 0.02).to(torch.bfloat16)
    A = torch.randn(M, 64, generator=g) * 0.004
    B = torch.randn(64, N, generator=g) * 0.004
    E = torch.randn(M, N, generator=g) * 1e-4
    dW = A @ B + E
    U, S, V = torch.svd(dW.float())
    x = torch.randn(T, N, generator=g).to(torch.bfloat16)
    return W_b, U[:, :r].contiguous(), S[:r].contiguous(), V[:, :r].contiguous(), x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory that holds src/)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    import adaptation
    import kernels
    import quantization
    import serving

    torch.manual_seed(0)
    G = 128
    for i, (name, M, N, r, T) in enumerate(CASES):
        W_b, U, S, V, x = synth(M, N, min(r, min(M, N)), T, 1000 + i)
        if r > min(M, N):        # rank above the matrix size: pad the factors with tiny directions
            pad = r - U.shape[1]
            gpad = torch.Generator().manual_seed(5000 + i)
            U = torch.cat([U, torch.randn(M, pad, generator=gpad) * 1e-3], 1)
            V = torch.cat([V, torch.randn(N, pad, generator=gpad) * 1e-3], 1)
            S = torch.cat([S, torch.full((pad,), 1e-6)])
        gen = torch.Generator().manual_seed(0)
        packed = quantization.compress_module(U, S, V, 4, G, gen)
        out = {"M": M, "N": N, "r": r, "T": T, "G": G}
        out["U_codes"] = packed["U_codes"].numpy()
        out["Vt_codes"] = packed["Vt_codes"].numpy()
        for k in ("U_scale", "U_zero", "Vt_scale", "Vt_zero"):
            assert packed[k].dtype == torch.bfloat16
            out[k] = bits(packed[k])
        out["W_b"] = bits(W_b)
        out["x"] = bits(x)

        # reference float32 reconstruction (quantization.py:288-317)
        out["ref_delta"] = quantization.reconstruct_delta(packed, G).numpy()
        # per-group integer products through the reference function itself
        ng = r // G
        prods = []
        for g in range(ng):
            one = {
                "U_codes": packed["U_codes"][:, g * G:(g + 1) * G].contiguous(),
                "U_scale": torch.ones(M, 1, dtype=torch.bfloat16),
                "U_zero": packed["U_zero"][:, g:g + 1].contiguous(),
                "Vt_codes": packed["Vt_codes"][g * G:(g + 1) * G, :].contiguous(),
                "Vt_scale": torch.ones(1, N, dtype=torch.bfloat16),
                "Vt_zero": packed["Vt_zero"][g:g + 1, :].contiguous(),
            }
            pf = quantization.reconstruct_delta(one, G)
            pi = pf.to(torch.int32)
            assert torch.equal(pi.float(), pf)
            prods.append(pi.numpy())
        out["ref_prod"] = np.stack(prods)
        out["ref_Uh"] = quantization.dequantize_rowwise(packed["U_codes"], packed["U_scale"], packed["U_zero"], G).numpy()
        out["ref_Vh"] = quantization.dequantize_colwise(packed["Vt_codes"], packed["Vt_scale"], packed["Vt_zero"], G).numpy()
        # reference stored form (kernels.py:164-188)
        p4 = kernels.pack_int4(packed, G)
        out["ref_uq"] = p4["uq"].numpy()
        out["ref_vq"] = p4["vq"].numpy()
        out["ref_R"] = p4["R"].numpy()
        out["ref_C"] = p4["C"].numpy()
        # reference module, CPU fallback (serving.py:84-112), float16 in / out
        lin = serving.ADEKernelLinear(W_b.float(), packed, G, use_decode=False, use_recon=False)
        with torch.no_grad():
            out["ref_y_fallback_fp16"] = lin(x.float()).float().numpy()
        # reference PyTorch factored application in float32 (adaptation.py:201-242)
        fold = adaptation.FoldInLinear(W_b.float(), packed, G, param_dtype=torch.float32)
        with torch.no_grad():
            out["ref_y_factored_fp32"] = fold(x.float()).float().numpy()
        np.savez_compressed(os.path.join(HERE, f"case_{name}.npz"), **out)
        print(name, {k: (v.shape if hasattr(v, "shape") else v) for k, v in out.items() if k.startswith("ref_")})

    # ---- format producer pins: quantize_rowwise / quantize_colwise / rotation
    g = torch.Generator().manual_seed(77)
    Xr = torch.randn(64, 256, generator=g) * 0.05
    Xr[3, :128] = 0.0                       # an all-zero group
    Xr[5, 128:] = Xr[5, 128:].abs() + 0.01  # an all-positive group (zero-point pinned to 0)
    Xr[7, :128] = -Xr[7, :128].abs() - 0.01  # an all-negative group (zero-point pinned to 15)
    Xc = Xr.t().contiguous()
    qc, qs, qz = quantization.quantize_rowwise(Xr, 4, G)
    cc, cs, cz = quantization.quantize_colwise(Xc, 4, G)
    np.savez_compressed(
        os.path.join(HERE, "quantizer.npz"),
        Xr=Xr.numpy(), row_codes=qc.numpy(), row_scale=bits(qs), row_zero=bits(qz),
        Xc=Xc.numpy(), col_codes=cc.numpy(), col_scale=bits(cs), col_zero=bits(cz),
        H256=quantization.rotation_matrix(256).numpy(),
    )
    print("quantizer", qc.shape, cc.shape)


if __name__ == "__main__":
    main()
