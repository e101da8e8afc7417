"""Benchmark of the delta-application hot path on synthetic inputs of the named shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ade|reference] [--skip-model] [--case NAME ...]

Headline workload (the step that is timed K times): the reconstructed application of the Llama-2-7B MLP
deltas -- gate / up (11008 x 4096) and down (4096 x 11008), rank 512, groups of 128, X = 2048 x d_i bfloat16.
One step is one pass of that path over the three modules: the reconstruction kernel (W' = W_b + U^V^^T, tcgen05
INT8 contraction) followed by x W'^T, per module.  With N > 1 every rank runs the same step on its own seeded
delta (replicas, no collective): weak scaling.

The printed JSON line carries, next to the device-resident throughput (`value`):
  e2e            the same metric through the module API with host buffers (copies inside the timed region);
  roofline       of the reconstruction kernel, timed with CUDA events inside the timed steps;
  factored       the factored kernel's own roofline: q_proj (config 0: 4096 x 4096, r = 256) at T = 1 and 16,
                 gate / down (r = 512) at T = 1, each call replayed from a CUDA graph over rotated instances;
  decode         config 2: random-init Llama-2-7B architecture (32 layers, 224 delta modules, ranks drawn for
                 alpha = 1/16), batch 1, 64-token prompt, 128 greedy tokens, decode step replayed from a CUDA graph;
  prefill_decode_13b   config 3: Llama-2-13B architecture (40 layers, 280 delta modules), batch 8, 512-token prompts run
                 as one reconstructed-path prefill (T = 4096), then 64 greedy steps on the factored path (T = 8);
  gpu_reference  the reference's own Blackwell route for this step restated in torch (torch._int_mm per group,
                 float32 rescale, base add, F.linear: src/quantization.py:303-316, src/serving.py:84-92), timed
                 on the same three modules;
  int8_peak_measured   torch._int_mm 8192^3;
  cpu_baseline   the reference's CPU arithmetic (oracle port) on the host cores, bounded sample;
  and with N > 1: sharded_recon (config 4b: the 280 modules of a 13B-shaped delta split over the ranks, fixed total
  work, plus the optional NCCL gather timed apart) and multi_delta_decode (config 4a: one 7B model + delta per GPU,
  batch-4 greedy decode, tokens/s summed).

`--impl reference` times the reference's CPU implementation of the same path (its PyTorch arithmetic restated
in oracle/, all host threads) on a bounded sample of the workload.  `--case recon|factored ...` runs one small
fixed workload of a single kernel and exits (what the profiler captures summarised under profiles/ were taken on).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODULES = [("gate_proj", 11008, 4096), ("up_proj", 11008, 4096), ("down_proj", 4096, 11008)]
RANK, TOKENS = 512, 2048
METRIC, UNIT = "recon_apply_int8_tops", "TOP/s"
# identical in both arms: it names the workload, not the implementation
CONFIG = {
    "workload": "llama2-7b MLP deltas, reconstructed path (gate/up 11008x4096, down 4096x11008, r=512, X 2048xd_i)",
    "step": "per module: W' = W_b + U^V^^T (INT8 contraction per group of 128 ranks, float32 rescale), then x W'^T; 3 modules",
    "ops_counted": "2*M*N*r of the delta contraction per module",
    "l2": "inputs larger than L2: 553 MB of weights and codes touched per step, no flush needed",
}


def delta_ops(M, N, r):
    """INT8 operations of the delta contraction of one module (2 M N r)."""
    return 2.0 * M * N * r


def recon_bytes(M, N, r):
    """Algorithmic bytes of one reconstruction launch: read W_b, write W' (bf16), read both code
    arrays once (4 bits per code), bf16 scales and 4-bit zero-points per (row, group)."""
    ng = r // 128
    return 4.0 * M * N + (M + N) * r / 2.0 + 2.5 * (M + N) * ng


def factored_bytes(M, N, r, T, fused):
    ng = r // 128
    delta = (M + N) * r / 2.0 + 2.5 * (M + N) * ng + 2.0 * T * N + 2.0 * T * M
    return delta + (2.0 * M * N if fused else 2.0 * T * M)


WORK_OPS = sum(delta_ops(M, N, RANK) for _, M, N in MODULES)
# dram__bytes_read.sum + dram__bytes_write.sum of one reconstruction launch on gate_proj, taken from an ncu capture
# of `--case recon` with expanded operands (not measured in this run; 101.3 MB read + 53.4 MB written); part of W' is
# still in L2 when the kernel ends
RECON_TRAFFIC_BYTES = 154.7e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the GPU is under load."""

    def __init__(self, index, uuid=None):
        super().__init__(daemon=True)
        self.index, self.uuid, self.samples, self.stop_flag = index, uuid, [], False
        self.max_mhz = None

    def run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            try:
                h = nv.nvmlDeviceGetHandleByUUID(self.uuid) if self.uuid else nv.nvmlDeviceGetHandleByIndex(self.index)
            except Exception:
                h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            while not self.stop_flag:
                self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                     nv.nvmlDeviceGetCurrentClocksEventReasons(h)))
                time.sleep(0.005)
        except Exception as e:                       # NVML missing: the line says so
            self.samples.append((time.perf_counter(), None, repr(e)))

    def summary(self, t0, t1):
        ok = [s for s in self.samples if s[1] is not None]
        win = [s for s in ok if t0 <= s[0] <= t1] or ok
        if not win:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        names = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
                 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
                 0x100: "display_clock_setting"}
        bits = 0
        for s in win:
            bits |= int(s[2])
        return {"sm_mhz": statistics.median(s[1] for s in win), "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in names.items() if bits & b], "samples": len(win)}


# ------------------------------------------------------------------------------------ CPU arm
def cpu_sample(rows, steps, warmup, seed=0):
    """Reference CPU path on a bounded sample: `rows` output rows of gate_proj -- reconstruct_delta
    (integer contraction per group + float32 rescale, src/quantization.py:288-317), the base add of
    src/serving.py:92 and x W'^T for those rows.  Returns (TOP/s, seconds per step, oracle threads, BLAS threads)."""
    import numpy as np
    import torch

    from ade_b200 import synth
    from oracle import oracle as O

    O.use_all_cores()
    blas = 0
    try:
        from threadpoolctl import threadpool_info

        blas = max((int(i.get("num_threads", 0)) for i in threadpool_info() if i.get("user_api") == "blas"), default=0)
    except Exception:
        pass
    _, M, N = MODULES[0]
    tp = synth.random_packed(M, N, RANK, seed)
    p = O.packed_from_torch(tp)
    wb = synth.base_weight(M, N, seed + 1).view(torch.uint16).numpy()
    x = O.bf16_to_f32(synth.activations(TOKENS, N, seed + 2).view(torch.uint16).numpy())
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        _, merged = O.reconstruct(p, rows=(0, rows), base_bits=wb)
        y = x @ O.bf16_to_f32(merged).T
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    assert y.shape == (TOKENS, rows) and np.isfinite(y).all()
    sec = statistics.median(times)
    return delta_ops(rows, N, RANK) / sec / 1e12, sec, O.threads(), blas


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1024
    tops, sec, threads, blas = cpu_sample(rows, args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * (WORK_OPS / delta_ops(rows, 4096, RANK)),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": dict(CONFIG),
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "blas_threads": blas, "kind": "port",
                         "sample": f"{rows} of 11008 output rows of gate_proj per step: reconstruct_delta + base add + x W'^T, "
                                   f"median of {args.steps}; ms_per_step is extrapolated to the full three-module step"},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------ GPU arm: pieces
def time_graph_calls(torch, fn_list, reps=10):
    """Average microseconds per call of the callables in fn_list, captured together in one CUDA graph (the decode
    loop of a served model is a captured graph) and replayed `reps` times."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            for f in fn_list:
                f()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in fn_list:
            f()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fn_list))


def factored_section(torch, dev, peak):
    """Roofline of the factored kernel at decode sizes: W_b-fused algorithmic bytes / time per call."""
    from ade_b200 import kernels, synth
    from ade_b200.serving import ADEKernelLinear

    out = {}
    cases = [("q_proj", 4096, 4096, 256, (1, 16), 8), ("gate_proj", 11008, 4096, 512, (1,), 3), ("down_proj", 4096, 11008, 512, (1,), 3)]
    for name, M, N, r, Ts, reps in cases:
        W = synth.base_weight(M, N, 3).to(dev)
        tp = synth.random_packed(M, N, r, 4, dev, on_device=True)
        lins = [ADEKernelLinear(W.clone(), tp) for _ in range(reps)]       # distinct instances: weights do not sit in L2
        for T in Ts:
            x = synth.activations(T, N, 5).to(dev)
            us = time_graph_calls(torch, [(lambda l=l: l(x)) for l in lins])
            b = factored_bytes(M, N, r, T, fused=True)
            gbs = b / us / 1e3
            out[f"{name}_T{T}"] = {"us_per_call": us, "bytes": b, "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                                   "shape": f"{M}x{N} r={r} T={T}",
                                   "note": f"W_b-fused bytes, one launch per call inside a CUDA graph, {reps} instances rotated "
                                           f"({reps * 2 * M * N / 1e6:.0f} MB > L2)"}
        del lins, W, tp
    kernels.check_factored_status(dev)
    return out


def decode_section(torch, dev, peak, arch="7b", batch=1, prompt=64, new=128, seed=0):
    """Whole-model greedy decode through the graph-captured decoder of ade_b200.serving."""
    from ade_b200 import synth
    from ade_b200.serving import GreedyGraphDecoder

    t0 = time.perf_counter()
    model, ranks, groups = synth.synthetic_llama(arch, seed=seed, device=dev)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    cfg = model.config
    g = torch.Generator().manual_seed(seed + 1)
    ids = torch.randint(0, cfg.vocab_size, (batch, prompt), generator=g).to(dev)
    dec = GreedyGraphDecoder(model)
    n_eager = 16
    dec.generate(ids, 2, use_graph=False)                      # lazy initialisation outside the timed loops
    te, tg = {}, {}
    eager = dec.generate(ids, n_eager + 1, use_graph=False, timings=te)
    dec.generate(ids, new)                                     # captures the graph, warms it up
    out = dec.generate(ids, new, timings=tg)
    per_token = tg["decode_ms"] * 1e-3 / (new - 1)
    eager_per_token = te["decode_ms"] * 1e-3 / n_eager
    t_prefill = tg["prefill_ms"] * 1e-3
    # the delta-carrying linear modules alone, same call sequence as one decode step, replayed from a graph: what part
    # of a token is this path's own, and what part is the rest of the Hugging Face layer (norms, rotary embedding,
    # attention, cache update, head)
    calls = []
    for layer in model.model.layers:
        xh = torch.randn(batch, 1, cfg.hidden_size, device=dev, dtype=torch.bfloat16)
        xi = torch.randn(batch, 1, cfg.intermediate_size, device=dev, dtype=torch.bfloat16)
        att, mlp = layer.self_attn, layer.mlp
        for m, xin in ((att.q_proj, xh), (att.k_proj, xh), (att.v_proj, xh), (att.o_proj, xh), (mlp.gate_proj, xh), (mlp.up_proj, xh),
                       (mlp.down_proj, xi)):
            calls.append(lambda m=m, xin=xin: m(xin))
    linear_ms = time_graph_calls(torch, calls, reps=5) * len(calls) / 1e3
    # bytes the decode step has to stream once per step: every linear weight, the delta (codes, scales, zero-points,
    # with V^T counted once), the output head, and the KV cache of every sequence at its mean length over the run
    h, inter, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers
    shapes = [(h, h)] * 4 + [(inter, h)] * 2 + [(h, inter)]
    wbytes = 2.0 * sum(a * b for a, b in shapes) * L
    dbytes = sum((a + b) * r / 2.0 + 2.5 * (a + b) * (r // 128) for (a, b), r in zip(shapes * L, ranks))
    head = 2.0 * cfg.vocab_size * h
    kv = 2.0 * 2.0 * batch * L * h * (prompt + new / 2.0)
    total = wbytes + dbytes + head + kv
    ceiling = peak * 1e9 / total * batch
    res = {
        "config": f"llama-{arch} architecture, random init, {len(ranks)} delta modules (alpha=1/16 ranks, mean {sum(ranks) / len(ranks):.0f}), "
                  f"batch {batch}, prompt {prompt} ({'reconstructed' if batch * prompt > 128 else 'factored'}-path prefill), {new} greedy tokens on the "
                  f"factored path, decode step replayed from a CUDA graph",
        "layers": L, "tokens_per_s": batch / per_token, "ms_per_step": per_token * 1e3, "tokens_per_step": batch,
        "eager_tokens_per_s": batch / eager_per_token, "eager_us_per_module_call": eager_per_token * 1e6 / len(ranks),
        "delta_modules_ms_per_step": linear_ms, "rest_of_model_ms_per_step": per_token * 1e3 - linear_ms,
        "prefill_ms": t_prefill * 1e3, "bytes_per_step": total, "ceiling_tokens_per_s": ceiling,
        "frac_of_ceiling": batch / per_token / ceiling,
        "tokens_equal_eager": bool((out[:, :prompt + n_eager + 1] == eager).all()), "fused_groups": groups, "model_build_s": build_s,
    }
    del dec, model
    torch.cuda.empty_cache()
    return res


def torch_reference_step(torch, packed_list, weights, xs):
    """The reference's Blackwell route for one step, restated in torch on the GPU: reconstruct_delta with torch._int_mm
    per group and a float32 rescale (src/quantization.py:303-316), the base add and cast of src/serving.py:84-92
    (bfloat16 here, float16 there), then F.linear."""
    F = torch.nn.functional
    for packed, W, x in zip(packed_list, weights, xs):
        Uq, Vq = packed["U_codes"], packed["Vt_codes"]
        acc = torch.zeros(Uq.shape[0], Vq.shape[1], device=Uq.device, dtype=torch.float32)
        for g in range(Uq.shape[1] // 128):
            cs = slice(g * 128, (g + 1) * 128)
            u_i = (Uq[:, cs].to(torch.int16) - packed["U_zero"][:, g].to(torch.int16).unsqueeze(1)).to(torch.int8)
            v_i = (Vq[cs, :].to(torch.int16) - packed["Vt_zero"][g, :].to(torch.int16).unsqueeze(0)).to(torch.int8)
            prod = torch._int_mm(u_i.contiguous(), v_i.contiguous())
            acc += prod.to(torch.float32) * (packed["U_scale"][:, g].to(torch.float32).unsqueeze(1)
                                             * packed["Vt_scale"][g, :].to(torch.float32).unsqueeze(0))
        F.linear(x, (W.float() + acc).to(torch.bfloat16))


def int8_peak(torch, dev):
    a = torch.randint(-8, 8, (8192, 8192), device=dev, dtype=torch.int8)
    b = torch.randint(-8, 8, (8192, 8192), device=dev, dtype=torch.int8)
    for _ in range(3):
        torch._int_mm(a, b)
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return {"tops": 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12, "how": "torch._int_mm 8192^3, best of 5 (a library GEMM, not an issue-rate bound)"}


def sharded_recon_section(torch, dist, dev, rank, world, barrier):
    """Config 4b: whole-delta reconstruction of a 13B-shaped delta (40 layers, 280 modules, ranks drawn for
    alpha = 1/16), modules split over the ranks by partition_modules; the total work is the same at every N
    (strong scaling).  Packed fields and base weights are drawn on the device.  The optional assembly of all shards
    on every rank (gather_merged over NCCL) is timed separately on a bounded subset: the first two layers."""
    from ade_b200 import kernels, sharding, synth

    shapes = sharding.llama_module_shapes(5120, 13824, 40)
    dims = [(a, b) for _, a, b in shapes]
    ranks = synth.draw_ranks(dims, alpha=1.0 / 16, seed=4)
    plan = sharding.partition_modules([a * b for a, b in dims], world)
    mine = plan[rank]
    forms, bases = {}, {}
    uniq = {}
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    for i in mine:                                           # every module its own base weight and delta: nothing is re-read from L2
        M, N = dims[i]
        uniq[(M, N)] = None
        bases[i] = torch.randn(M, N, generator=gen, device=dev, dtype=torch.bfloat16) * 0.02
        forms[i] = kernels.pack_int4(synth.random_packed(M, N, ranks[i], 5000 + i, dev, on_device=True), device=dev)
    outs = {shape: torch.empty(shape, dtype=torch.bfloat16, device=dev) for shape in uniq}
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # one-shot reconstruction of a module: expand its codes to int8 operands in a work buffer shared by all modules
    # (two launches per module: the expansion is a few microseconds, the TMA-fed kernel saves more than that)
    small = [i for i in mine if ranks[i] <= 1024]
    u8w = torch.empty(max([dims[i][0] * ranks[i] for i in small] + [16]), dtype=torch.int8, device=dev)
    v8w = torch.empty(max([dims[i][1] * ranks[i] for i in small] + [16]), dtype=torch.int8, device=dev)

    def run_all():
        from ade_b200 import _lib
        import ctypes
        lib = _lib.load()
        st = torch.cuda.current_stream().cuda_stream
        for i in mine:
            d = ctypes.byref(kernels._cdelta(forms[i]))
            if ranks[i] <= 1024:
                _lib.check(lib.ade_b200_expand_codes(d, u8w.data_ptr(), v8w.data_ptr(), st), "ade_b200_expand_codes")
                rc = lib.ade_b200_recon_expanded(d, u8w.data_ptr(), v8w.data_ptr(), bases[i].data_ptr(), outs[dims[i]].data_ptr(),
                                                 None, status.data_ptr(), st)
            else:
                rc = lib.ade_b200_recon(d, bases[i].data_ptr(), outs[dims[i]].data_ptr(), None, status.data_ptr(), st)
            _lib.check(rc, "ade_b200_recon")

    for _ in range(2):
        run_all()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        run_all()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / reps
    assert int(status.item()) == 0
    # optional gather of bf16 shards (first two layers: 14 modules), every rank ends up with all of them
    sub = list(range(14))
    subplan = sharding.partition_modules([dims[i][0] * dims[i][1] for i in sub], world)
    gather_ms = None
    if world > 1:
        local = {}
        for i in subplan[rank]:
            M, N = dims[i]
            local[i] = outs[(M, N)] if (M, N) in outs else torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        sh = {i: dims[i] for i in sub}
        sharding.gather_merged(local, sh, subplan, device=dev)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        full = sharding.gather_merged(local, sh, subplan, device=dev)
        g1.record()
        barrier()
        gather_ms = g0.elapsed_time(g1)
        assert len(full) == 14
        del full
    nbytes = sum(recon_bytes(dims[i][0], dims[i][1], ranks[i]) for i in mine)
    t = torch.tensor([ms, gather_ms or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, gather_ms = float(t[0]), float(t[1])
    total_bytes = sum(recon_bytes(a, b, r) for (a, b), r in zip(dims, ranks))
    del forms, bases, outs, uniq
    torch.cuda.empty_cache()
    return {"workload": "llama-13b-shaped delta, 280 modules (5120/13824, ranks for alpha=1/16), W' = W_b + U^V^^T per module "
                        "(codes expanded to int8 operands, then the TMA-fed kernel: two launches per module), "
                        "modules split over ranks by cost d_o*d_i, no collective", "scaling": "strong",
            "ms_all_modules": ms, "modules_per_s": 280 / (ms * 1e-3), "gb_per_s_aggregate": total_bytes / (ms * 1e-3) / 1e9,
            "modules_on_slowest_rank": max(len(p) for p in plan), "rank0_bytes": nbytes,
            "gather_ms_14_modules": gather_ms if world > 1 else None,
            "gather_note": "optional all_gather of the bf16 shards of 2 layers (1.27 GB) to every rank over NCCL, not part of the scaling figure"}


def multi_delta_section(torch, dist, dev, rank, world, peak):
    """Config 4a: one 7B-architecture base + one delta per GPU (delta seed = rank), batch-4 greedy decode of 128 tokens."""
    res = decode_section(torch, dev, peak, "7b", batch=4, prompt=64, new=128, seed=rank)
    t = torch.tensor([res["tokens_per_s"]], device=dev, dtype=torch.float64)
    lo = t.clone()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    return {"workload": "llama-7b architecture + one delta per GPU, batch 4, prompt 64 (prefill on the reconstructed path), 128 greedy tokens, replicas (no collective)",
            "tokens_per_s_total": float(t[0]), "tokens_per_s_slowest_gpu": float(lo[0]), "gpus": world,
            "tokens_equal_eager_rank0": res["tokens_equal_eager"]}


# ------------------------------------------------------------------------------------ GPU arm
def run_ade(args):
    import torch
    import torch.distributed as dist

    from ade_b200 import kernels, synth
    from ade_b200.serving import ADEKernelLinear

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # every rank its own share of the host cores: the pinned-buffer copies and the launch threads of eight ranks
        # otherwise pile up on the same cores
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = max(1, len(cores) // world)
            os.sched_setaffinity(0, cores[local * per:(local + 1) * per] or cores)
        except Exception:
            pass
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ok, why = kernels.recon_kernel_status(dev)
    if not ok:
        raise RuntimeError(f"B200 kernels unavailable: {why}")

    # ---- build the three modules of this rank's delta (seeded by rank: one delta per GPU)
    mods, xs_host, xs_dev, packs = [], [], [], []
    for mi, (name, M, N) in enumerate(MODULES):
        W_b, packed = synth.synthetic_module(M, N, RANK, config=1 + 100 * rank, module=mi, device=dev, exact_svd=False)
        mods.append(ADEKernelLinear(W_b, packed).to(dev))
        packs.append({k: v.to(dev) for k, v in packed.items()})
        xh = synth.activations(TOKENS, N, synth.seed_for(1 + 100 * rank, mi, 2)).pin_memory()
        xs_host.append(xh)
        xs_dev.append(xh.to(dev))
        del W_b, packed
    ys_host = [torch.empty(TOKENS, M, dtype=torch.bfloat16).pin_memory() for _, M, _ in MODULES]
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    recon_ev = []

    def step(record):
        for m, x in zip(mods, xs_dev):
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            W = m.merged_weight()             # the module's route: int8 operands expanded once at first use, kept
            if record:
                e1.record()
                recon_ev.append((e0, e1))
            torch.nn.functional.linear(x, W)

    # End to end: inputs start in pinned host memory, results end there.  The copies run on their own
    # streams (one per direction) so that uploads, kernels and downloads overlap, also across consecutive
    # steps: the device-side staging buffers for x are double-buffered (allocated once), and the timed
    # region ends only when the last result of the last step is on the host.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_stage = [[torch.empty_like(x) for x in xs_dev] for _ in range(2)]
    stage_free = [None, None]                        # event: the kernels that read this staging set are done

    def step_e2e(i):
        main = torch.cuda.current_stream()
        stage = x_stage[i & 1]
        ups = []
        if stage_free[i & 1] is not None:
            s_in.wait_event(stage_free[i & 1])
        with torch.cuda.stream(s_in):
            for xd, xh in zip(stage, xs_host):
                xd.copy_(xh, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
                ups.append(ev)
        for m, xd, yh, ev in zip(mods, stage, ys_host, ups):
            main.wait_event(ev)
            y = m(xd)
            done = torch.cuda.Event()
            done.record(main)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                yh.copy_(y, non_blocking=True)
            y.record_stream(s_out)
        stage_free[i & 1] = done
        return ys_host

    def drain_e2e():
        torch.cuda.current_stream().wait_stream(s_out)

    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(local, uuid)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(False)
    barrier()
    t_wall0 = time.perf_counter()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()                  # a profiler attached with --profile-from-start off sees only the timed steps
    s0.record()
    for _ in range(args.steps):
        step(True)
    s1.record()
    barrier()
    torch.cuda.profiler.stop()
    t_wall1 = time.perf_counter()
    ms = s0.elapsed_time(s1)
    recon_ms = sum(a.elapsed_time(b) for a, b in recon_ev) / len(recon_ev)
    # for the record: the same launches with the codes unpacked inside the kernel on every call (no kept int8 operands)
    pk = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(2 * len(mods) + 1):
        if i == len(mods):
            pk[0].record()
        m = mods[i % len(mods)]
        kernels.recon_int4(m._stored_form(), m.weight)
    pk[1].record()
    torch.cuda.synchronize()
    recon_packed_us = pk[0].elapsed_time(pk[1]) * 1e3 / (len(mods) + 1)
    # ... and the whole step that way (a few steps, for the record: the headline keeps the operands)
    def step_unpacking():
        for m, x in zip(mods, xs_dev):
            torch.nn.functional.linear(x, kernels.recon_int4(m._stored_form(), m.weight))
    for _ in range(2):
        step_unpacking()
    pk2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    n_alt = min(args.steps, 10)
    pk2[0].record()
    for _ in range(n_alt):
        step_unpacking()
    pk2[1].record()
    torch.cuda.synchronize()
    ms_step_unpacking = pk2[0].elapsed_time(pk2[1]) / n_alt

    # ---- end to end through the module API, host buffers in and out
    for i in range(4):
        step_e2e(i)
    drain_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step_e2e(i)
    drain_e2e()                                      # every download of every timed step has landed
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    t_wall2 = time.perf_counter()
    sampler.stop_flag = True
    sampler.join(timeout=2)

    peak, peak_kind = measured_peaks()
    # ---- the reference's GPU route restated in torch, on the same modules (rank 0)
    gpu_ref = None
    if rank == 0:
        ws = [m.weight for m in mods]
        for _ in range(2):
            torch_reference_step(torch, packs, ws, xs_dev)
        torch.cuda.synchronize()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nref = 5
        r0.record()
        for _ in range(nref):
            torch_reference_step(torch, packs, ws, xs_dev)
        r1.record()
        torch.cuda.synchronize()
        ref_ms = r0.elapsed_time(r1) / nref
        gpu_ref = {"ms_per_step": ref_ms, "value": WORK_OPS / (ref_ms * 1e-3) / 1e12, "unit": UNIT,
                   "kind": "restatement in torch of the reference's route on compute capability 10.0 (its INT4 kernel is gated "
                           "to 8.x): torch._int_mm per group + float32 rescale + base add + F.linear, bfloat16 for float16"}
    del packs
    torch.cuda.empty_cache()

    factored = decode = i8 = None
    if rank == 0:
        factored = factored_section(torch, dev, peak)
        i8 = int8_peak(torch, dev)
    del mods, xs_dev, x_stage
    torch.cuda.empty_cache()
    sharded = multi = decode13 = None
    if not args.skip_model:
        if world > 1:
            sharded = sharded_recon_section(torch, dist, dev, rank, world, barrier)
            multi = multi_delta_section(torch, dist, dev, rank, world, peak)
        else:
            sharded = sharded_recon_section(torch, dist, dev, 0, 1, barrier)
            decode = decode_section(torch, dev, peak)
            decode13 = decode_section(torch, dev, peak, "13b", batch=8, prompt=512, new=64, seed=3)
    kernels.check_factored_status(dev)

    if world > 1:
        t = torch.tensor([ms, ms_e2e, recon_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, recon_ms = (float(v) for v in t.tolist())
    if rank == 0:
        per_step = ms / args.steps
        value = world * WORK_OPS / (per_step * 1e-3) / 1e12
        e2e_ms = ms_e2e / args.steps
        e2e = world * WORK_OPS / (e2e_ms * 1e-3) / 1e12
        bytes_launch = sum(recon_bytes(M, N, RANK) for _, M, N in MODULES) / len(MODULES)
        achieved = bytes_launch / (recon_ms * 1e-3) / 1e9
        cpu_rows = 1024
        cpu_tops, cpu_sec, cpu_threads, blas = cpu_sample(cpu_rows, 5, 1)
        h2d = sum(2 * TOKENS * N for _, _, N in MODULES)
        d2h = sum(2 * TOKENS * M for _, M, _ in MODULES)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8", "data": "synthetic",
            "config": dict(CONFIG),
            "parallelism": f"replicas x{world}, one delta per GPU, no collective",
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "copy_gb_per_s_per_rank": (h2d + d2h) / (e2e_ms * 1e-3) / 1e9,
                    "note": "pinned host buffers in and out through ADEKernelLinear; per-rank host<->device traffic is what "
                            "bounds it (all ranks share the host's memory and PCIe root)"},
            "gpu_launches": 3 * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": RECON_TRAFFIC_BYTES, "traffic_source": "ncu capture of `bench.py --case recon`, not this run",
                         "peak_kind": peak_kind, "kernel": "recon_strip_kernel (int8 operands expanded once per module and kept; "
                         "algorithmic bytes count the packed codes)", "us_per_launch": recon_ms * 1e3,
                         "us_per_launch_unpacking_in_kernel": recon_packed_us,
                         "ms_per_step_unpacking_in_kernel": ms_step_unpacking,
                         "int8_tops_kernel_only": (WORK_OPS / 3) / (recon_ms * 1e-3) / 1e12},
            "cpu_baseline": {"value": cpu_tops, "unit": UNIT, "cores": cpu_threads, "blas_threads": blas, "kind": "port",
                             "sample": f"{cpu_rows} of 11008 rows of gate_proj: reconstruct + base add + x W'^T, median of 5, {cpu_sec:.2f} s per pass"},
            "clocks": sampler.summary(t_wall0, t_wall2),
            "factored": factored, "decode": decode, "prefill_decode_13b": decode13, "gpu_reference": gpu_ref, "int8_peak_measured": i8,
            "sharded_recon": sharded, "multi_delta_decode": multi,
            "wall_s_timed": t_wall1 - t_wall0,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_case(argv):
    """One small fixed workload of a single kernel (seeded random packed fields, no SVD, well under 1 GB on the
    device), a handful of launches: what a profiler capture of two or three launches is taken on.

        python bench.py --case recon [M N r [x]]      default 11008 4096 512 1 (Llama-2-7B gate_proj delta; x = 0: codes
                                                      unpacked inside the kernel instead of int8 operands expanded beforehand)
        python bench.py --case factored [T M N r]     default 16 4096 4096 256 (q_proj delta)
        python bench.py --case decode                 one graph replay of the 7B-architecture decode step (launch list)
    """
    import torch

    from ade_b200 import kernels, synth

    what, nums = argv[0], [int(a) for a in argv[1:]]
    dev = "cuda"
    if what == "recon":
        M, N, r, expanded = nums if len(nums) == 4 else (*nums, 1) if len(nums) == 3 else (11008, 4096, 512, 1)
        p4 = kernels.pack_int4(synth.random_packed(M, N, r, 1), device=dev)
        W = synth.base_weight(M, N, 5).to(dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        x8 = kernels.expand_codes(p4) if expanded else None
        for _ in range(4):
            kernels.recon_int4(p4, W, status=status, expanded=x8)
        torch.cuda.synchronize()
        print(f"recon {M}x{N} r={r} ({'int8 operands' if expanded else 'codes unpacked in the kernel'}): 4 launches, "
              f"device status {int(status.item())}")
    elif what == "factored":
        T, M, N, r = nums if len(nums) == 4 else (16, 4096, 4096, 256)
        p4 = kernels.pack_int4(synth.random_packed(M, N, r, 1), device=dev)
        W = synth.base_weight(M, N, 5).to(dev)
        x = synth.activations(T, N, 6).to(dev)
        for _ in range(4):
            kernels.factored_forward(x, p4, weight=W)
        torch.cuda.synchronize()
        print(f"factored T={T} {M}x{N} r={r}: 4 launches, status {kernels.factored_status(dev, T, r)}")
    elif what == "decode":
        # one replay of the captured decode step of the 7B-architecture model between cudaProfilerStart / Stop
        from ade_b200.serving import GreedyGraphDecoder

        model, ranks, groups = synth.synthetic_llama("7b", seed=0, device=dev)
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(0, 32000, (1, 64), generator=g).to(dev)
        dec = GreedyGraphDecoder(model)
        dec.generate(ids, 8)
        torch.cuda.synchronize()
        graph = dec._captured(1, 64 + 8 + 1, torch.device(dev))[0]
        torch.cuda.profiler.start()
        graph.replay()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"decode step of a 7B-architecture model replayed once: {len(ranks)} delta modules, {groups} fused groups")
    else:
        raise SystemExit(run_case.__doc__)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ade", choices=["ade", "reference"])
    ap.add_argument("--skip-model", action="store_true", help="leave out the whole-model and sharded sections (quick kernel numbers)")
    ap.add_argument("--case", nargs="+", default=None, help="run one small profiling workload and exit")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ade(args)


if __name__ == "__main__":
    main()
