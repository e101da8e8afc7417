"""CPU-side checks of the host logic: stored form, format producer, file format, C ABI exports."""
from __future__ import annotations

import ctypes
import os
import re

import numpy as np
import pytest
import torch

from ade_b200 import _lib, kernels, packed_io, quantization, synth
from conftest import GOLDEN, ROOT
from oracle import oracle as O


def _torch_packed(case):
    p = {}
    for k, v in case["packed"].items():
        t = torch.from_numpy(v.copy())
        p[k] = t.view(torch.bfloat16) if v.dtype == np.uint16 else t
    return p


def test_pack_roundtrip_and_layout(case):
    p = _torch_packed(case)
    p4 = kernels.pack_int4(p)
    M, N, r = case["M"], case["N"], case["r"]
    assert p4["uq"].shape == (M, r // 2) and p4["vq"].shape == (N, r // 2) and p4["vt"].shape == (r, N // 2)
    assert torch.equal(kernels.unpack_nibbles(p4["uq"]), p["U_codes"])
    assert torch.equal(kernels.unpack_nibbles(p4["vq"]), p["Vt_codes"].t())
    assert torch.equal(kernels.unpack_nibbles(p4["vt"]), p["Vt_codes"])
    mu, nu = O.zero_points(case["packed"])
    assert np.array_equal(p4["uz"].numpy().astype(np.int32), mu) and np.array_equal(p4["vz"].numpy().astype(np.int32), nu)
    assert np.array_equal(p4["us"].view(torch.uint16).numpy(), case["U_scale"])
    assert np.array_equal(p4["vs"].view(torch.uint16).numpy(), case["Vt_scale"])
    # same codes as the reference's own stored form, nibble for nibble: word w of the reference holds
    # code k in bits 4(k%8); ours holds the same 8 codes in the order 0 2 4 6 1 3 5 7
    ref_words = case["ref_uq"].view(np.uint32)
    ours = p4["uq"].numpy().view(np.uint32)
    nib = lambda w, i: (w >> np.uint32(4 * i)) & np.uint32(15)
    for i, k in enumerate((0, 2, 4, 6, 1, 3, 5, 7)):
        assert np.array_equal(nib(ours, i), nib(ref_words, k))


def test_quantizer_matches_reference():
    z = np.load(os.path.join(GOLDEN, "quantizer.npz"))
    c, s, zp = quantization.quantize_rowwise(torch.from_numpy(z["Xr"]), 4, 128)
    assert np.array_equal(c.numpy(), z["row_codes"])
    assert np.array_equal(s.view(torch.uint16).numpy(), z["row_scale"])
    assert np.array_equal(zp.view(torch.uint16).numpy(), z["row_zero"])
    c, s, zp = quantization.quantize_colwise(torch.from_numpy(z["Xc"]), 4, 128)
    assert np.array_equal(c.numpy(), z["col_codes"])
    assert np.array_equal(s.view(torch.uint16).numpy(), z["col_scale"])
    assert np.array_equal(zp.view(torch.uint16).numpy(), z["col_zero"])
    assert np.array_equal(quantization.rotation_matrix(256).numpy(), z["H256"])
    H = quantization.rotation_matrix(384, torch.Generator().manual_seed(3))
    assert torch.allclose(H @ H.T, torch.eye(384), atol=1e-4)


def test_compress_module_reconstructs():
    W_b, packed = synth.synthetic_module(128, 256, 128, config=9, module=1)
    p = O.packed_from_torch(packed)
    dW = synth.delta_weight(128, 256, synth.seed_for(9, 1, 1)).numpy()
    rec = O.reconstruct_delta_np(p)
    assert np.linalg.norm(rec - dW) / np.linalg.norm(dW) < 0.2
    z = bf = O.bf16_to_f32(p["U_zero"])
    assert z.min() >= 0 and z.max() <= 15 and np.array_equal(z, np.round(bf))
    assert p["U_codes"].max() <= 15 and p["Vt_codes"].max() <= 15


def test_packed_file_roundtrip(tmp_path):
    _, a = synth.synthetic_module(128, 128, 128, config=9, module=2)
    b = synth.random_packed(128, 256, 256, seed=5)
    path = str(tmp_path / "delta.pt")
    packed_io.save_packed(path, {"model.layers.0.self_attn.q_proj": a, "model.layers.0.mlp.up_proj": b},
                          {"bits": 4, "group_size": 128})
    per, meta = packed_io.load_packed(path)
    assert meta["format"] == "ade_packed_v1" and meta["group_size"] == 128
    assert set(per) == {"model.layers.0.self_attn.q_proj", "model.layers.0.mlp.up_proj"}
    for k in packed_io.PACKED_FIELDS:
        assert torch.equal(per["model.layers.0.mlp.up_proj"][k], b[k])
    torch.save({"__meta__": {"format": "other"}}, path)
    with pytest.raises(ValueError):
        packed_io.load_packed(path)
    torch.save({"__meta__": {"format": "ade_packed_v1"}, "m.U_codes": a["U_codes"]}, path)
    with pytest.raises(ValueError):
        packed_io.load_packed(path)


def test_rank_draw_fits_budget():
    shapes = [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]
    ranks = synth.draw_ranks(shapes * 4, seed=2)
    assert all(r % 128 == 0 and 128 <= r <= 1024 for r in ranks)
    cost = sum(quantization.group_cost_bits(a, b) * (r // 128) for (a, b), r in zip(shapes * 4, ranks))
    assert cost <= sum(a * b for a, b in shapes * 4)           # alpha * 16 bits = 1 bit per weight


def test_library_exports_every_declared_symbol():
    """The C-ABI library loads on a machine without a GPU and exports what include/ade_b200.h declares."""
    header = open(os.path.join(ROOT, "include", "ade_b200.h")).read()
    declared = set(re.findall(r"\b(ade_b200_\w+)\s*\(", header))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.ade_b200_version() >= 1
    assert lib.ade_b200_factored_scratch_bytes(16, 256) >= 16 * 256 * 2 + 12
    assert lib.ade_b200_factored_sync_offset(16, 256) == lib.ade_b200_factored_scratch_bytes(16, 256) - 256
    assert lib.ade_b200_factored_scratch_bytes(0, 256) == 0


def test_torch_binding_loads_and_registers_its_operators():
    """The thin torch binding (libade_b200_torch.so) loads without a GPU and registers the two hot entry points."""
    ops = _lib.ops()
    assert str(ops.factored.default._schema).startswith("ade_b200::factored(Tensor x, Tensor? weight, Tensor? y_dense, Tensor uq")
    assert "Tensor? dbg_acc, Tensor? status, Tensor? u8, Tensor? v8) -> Tensor" in str(ops.recon.default._schema)
    assert str(ops.expand.default._schema).endswith("-> (Tensor, Tensor)")
    with pytest.raises((RuntimeError, NotImplementedError)):           # CPU tensors: no CPU kernel is registered
        ops.recon(torch.zeros(128, 128, dtype=torch.bfloat16), *[torch.zeros(1, dtype=torch.uint8)] * 7, 128, 128, 128, None, None)


def test_status_tables_follow_the_header():
    """The Python tables of return codes and device status codes name exactly what the header defines."""
    header = open(os.path.join(ROOT, "include", "ade_b200.h")).read()
    dev = {int(v): k for k, v in re.findall(r"#define (ADE_DEV_TIMEOUT_\w+) (\d+)", header)}
    assert set(dev) == set(_lib.DEVICE_STATUS) and all(_lib.DEVICE_STATUS[c].startswith(n + ":") for c, n in dev.items())
    err = {int(v): k for k, v in re.findall(r"#define (ADE_ERR_\w+) \((-\d+)\)", header)}
    assert set(err) == set(_lib.ERRORS) and all(_lib.ERRORS[c].startswith(n + ":") for c, n in err.items())
    opts = dict(re.findall(r"#define (ADE_OPT_\w+) (\d+)", header))
    assert (int(opts["ADE_OPT_WAIT_LIMIT_CYCLES"]), int(opts["ADE_OPT_COOPERATIVE_LAUNCH"]), int(opts["ADE_OPT_DROP_SIGNALS"])) == (
        _lib.OPT_WAIT_LIMIT_CYCLES, _lib.OPT_COOPERATIVE_LAUNCH, _lib.OPT_DROP_SIGNALS)
    lib = _lib.load()
    assert lib.ade_b200_set_option(99, 1) == -2 and lib.ade_b200_set_option(_lib.OPT_WAIT_LIMIT_CYCLES, -5) == -2
    assert lib.ade_b200_set_option(_lib.OPT_WAIT_LIMIT_CYCLES, 0) == 0          # back to the default


def test_packed_file_is_validated_and_mapped(tmp_path):
    """The reader checks every module's shapes against each other, the writer refuses inconsistent modules and leaves
    no partial file behind."""
    good = synth.random_packed(128, 256, 256, seed=6)
    path = str(tmp_path / "d.pt")
    packed_io.save_packed(path, {"model.layers.0.mlp.gate_proj": good}, {"bits": 4, "group_size": 128})
    f = packed_io.PackedDeltaFile(path)
    assert len(f) == 1 and "model.layers.0.mlp.gate_proj" in f and f.dims["model.layers.0.mlp.gate_proj"] == (128, 256, 256)
    assert torch.equal(f.module("model.layers.0.mlp.gate_proj")["Vt_codes"], good["Vt_codes"])
    bad = dict(good, U_scale=good["U_scale"][:, :1])
    with pytest.raises(ValueError):
        packed_io.save_packed(str(tmp_path / "bad.pt"), {"m": bad}, {})
    assert sorted(os.listdir(tmp_path)) == ["d.pt"]
    torch.save({"__meta__": {"format": "ade_packed_v1"}, **{f"m.{k}": v for k, v in bad.items()}}, path)
    with pytest.raises(ValueError):
        packed_io.PackedDeltaFile(path)


def test_argument_errors_before_any_launch():
    """Bad arguments are rejected by status code before anything touches a device."""
    lib = _lib.load()
    assert lib.ade_b200_recon(None, None, None, None, None, None) == -1
    d = _lib.AdeDelta(16, 16, 16, 16, 16, 16, 16, 128, 100, 128)          # N not a multiple of 128
    assert lib.ade_b200_recon(ctypes.byref(d), 16, 32, None, None, None) == -2
    d = _lib.AdeDelta(16, 16, 16, 16, 16, 16, 16, 128, 128, 96)           # rank not a multiple of 128
    assert lib.ade_b200_factored(ctypes.byref(d), 16, 16, None, 16, 16, 1 << 20, 4, None) == -2
    d = _lib.AdeDelta(8, 16, 16, 16, 16, 16, 16, 128, 128, 128)           # misaligned pointer
    assert lib.ade_b200_recon(ctypes.byref(d), 16, 32, None, None, None) == -3
    d = _lib.AdeDelta(16, 16, 16, 16, 16, 16, 16, 128, 128, 128)
    assert lib.ade_b200_factored(ctypes.byref(d), 16, 16, 16, 16, 16, 1 << 20, 4, None) == -1    # both base terms
    assert lib.ade_b200_factored(ctypes.byref(d), 16, 16, None, 16, 16, 1 << 20, 129, None) == -2  # T too large
    assert lib.ade_b200_factored(ctypes.byref(d), 16, 16, None, 16, 16, 64, 4, None) == -4        # scratch too small
    # expanded operands of the reconstruction: both arrays are required and 16-byte aligned; the delta is checked first
    assert lib.ade_b200_expand_codes(ctypes.byref(d), None, 32, None) == -1
    assert lib.ade_b200_expand_codes(ctypes.byref(d), 16, 40, None) == -3
    assert lib.ade_b200_recon_expanded(ctypes.byref(d), None, None, 16, 32, None, None, None) == -1
    assert lib.ade_b200_recon_expanded(ctypes.byref(d), 24, 32, 16, 32, None, None, None) == -3
    assert lib.ade_b200_recon_expanded(None, 16, 32, 16, 32, None, None, None) == -1
    assert lib.ade_b200_set_option(99, 0) == -2 and lib.ade_b200_set_option(_lib.OPT_ATTN_SINGLE_PASS, 1) == 0
    with pytest.raises(ValueError):
        kernels.pack_int4({"U_codes": torch.zeros(8, 96, dtype=torch.uint8), "Vt_codes": torch.zeros(96, 8, dtype=torch.uint8)})


def test_serving_module_rejects_fallback_flags():
    from ade_b200.serving import ADEKernelLinear

    _, packed = synth.synthetic_module(128, 128, 128, config=9, module=3)
    with pytest.raises(ValueError):
        ADEKernelLinear(torch.zeros(128, 128), packed, use_decode=False)
    m = ADEKernelLinear(torch.zeros(128, 128), packed)
    assert (m.out_features, m.in_features) == (128, 128) and m.weight.dtype == torch.bfloat16
    assert set(k for k, _ in m.named_buffers()) == {"weight", *(f"p4_{k}" for k in kernels.STORED_KEYS)}
