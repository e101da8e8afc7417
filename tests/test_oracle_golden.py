"""Pin the CPU oracle against what the reference's own Python code produced (tests/golden)."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def test_group_products_exact(case):
    p, G = case["packed"], case["G"]
    ref = case["ref_prod"]
    assert np.array_equal(O.group_products_np(p, G), ref)
    for g in range(case["r"] // G):
        assert np.array_equal(O.group_product(p, g, G), ref[g])
    # a row window of the C oracle matches the same rows
    assert np.array_equal(O.group_product(p, 0, G, rows=(32, 96)), ref[0][32:96])


def test_reconstruct_delta_bit_exact(case):
    p, G = case["packed"], case["G"]
    ref = case["ref_delta"]
    assert np.array_equal(O.reconstruct_delta_np(p, G).view(np.uint32), ref.view(np.uint32))
    delta, merged = O.reconstruct(p, G, base_bits=case["W_b"])
    assert np.array_equal(delta.view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(merged, O.f32_to_bf16(O.bf16_to_f32(case["W_b"]) + ref))
    d2, m2 = O.reconstruct(p, G, rows=(16, 80), base_bits=case["W_b"])
    assert np.array_equal(d2, ref[16:80]) and np.array_equal(m2, merged[16:80])


def test_dequantize_exact(case):
    p, G = case["packed"], case["G"]
    Uh, Vh = O.dequantize_np(p, G)
    assert np.array_equal(Uh, case["ref_Uh"]) and np.array_equal(Vh, case["ref_Vh"])
    Uh, Vh = O.dequantize(p, G)
    assert np.array_equal(Uh, case["ref_Uh"]) and np.array_equal(Vh, case["ref_Vh"])


def test_reference_stored_form(case):
    p, G = case["packed"], case["G"]
    assert np.array_equal(O.pack_nibbles_ref_np(p["U_codes"]), case["ref_uq"])
    assert np.array_equal(O.pack_nibbles_ref(p["U_codes"]), case["ref_uq"])
    assert np.array_equal(O.pack_nibbles_ref_np(np.ascontiguousarray(p["Vt_codes"].T)), case["ref_vq"])
    R, C = O.ref_tables_np(p, G)
    assert np.array_equal(R, case["ref_R"]) and np.array_equal(C, case["ref_C"])


def test_kernel_identity_matches_products(case):
    """<U-mu, V-nu> = <U,V> - mu colsum - nu rowsum + G mu nu  (src/kernels.py:16-22), in integers."""
    p, G = case["packed"], case["G"]
    M, N, r = case["M"], case["N"], case["r"]
    mu, nu = O.zero_points(p)
    for g in range(r // G):
        U = p["U_codes"][:, g * G:(g + 1) * G].astype(np.int64)
        V = p["Vt_codes"][g * G:(g + 1) * G].astype(np.int64)
        raw = U @ V
        ident = raw - mu[:, g:g + 1] * V.sum(0)[None, :] - nu[g:g + 1, :] * U.sum(1)[:, None] + G * mu[:, g:g + 1] * nu[g:g + 1, :]
        assert np.array_equal(ident, case["ref_prod"][g].astype(np.int64))


def test_factored_oracle_matches_reference_factored(case):
    p, G = case["packed"], case["G"]
    ref = case["ref_y_factored_fp32"]                     # FoldInLinear in float32
    y = O.factored_apply(case["x"], case["W_b"], p, G)
    y_np = O.factored_apply_np(case["x"], case["W_b"], p, G)
    assert np.abs(y - y_np).max() <= 1e-9 * max(1.0, np.abs(y_np).max())
    err, cos = O.parity(y, ref)
    assert err <= 2e-5 and cos >= 1 - 1e-9, (err, cos)


def test_recon_oracle_matches_reference_fallback(case):
    p, G = case["packed"], case["G"]
    ref = case["ref_y_fallback_fp16"]                     # ADEKernelLinear CPU fallback, float16
    y = O.recon_apply_np(case["x"], case["W_b"], p, G)
    err, cos = O.parity(y, ref)
    # the reference rounds x, W' and y to float16, the oracle W' to bfloat16: both inside the
    # stated tolerance (max normalised error <= 1e-2, cosine >= 0.9999)
    assert err <= 1e-2 and cos >= 0.9999, (err, cos)
    # and the two applications agree with each other
    err2, cos2 = O.parity(O.factored_apply_np(case["x"], case["W_b"], p, G), y)
    assert err2 <= 1e-2 and cos2 >= 0.9999, (err2, cos2)


def test_bf16_roundtrip():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(4096).astype(np.float32)
    b = O.f32_to_bf16(x)
    assert np.array_equal(O.f32_to_bf16(O.bf16_to_f32(b)), b)
    import torch

    assert np.array_equal(torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy(), b)
