"""Benchmark of the delta-application hot path on synthetic inputs of the named shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ade|reference]

Workload (N = 1): the reconstructed application of the Llama-2-7B MLP deltas -- gate / up
(11008 x 4096) and down (4096 x 11008), rank 512, groups of 128, X = 2048 x d_i bfloat16.  One step
is one pass of that path over the three modules: the reconstruction kernel (W' = W_b + U^V^^T,
tcgen05 INT8 contraction) followed by x W'^T, per module.  With N > 1 every rank runs the same step
on its own seeded delta (replicas, no collective): weak scaling.

The printed JSON line carries the device-resident throughput (`value`), the same metric through
the module API with host buffers (`e2e`), the roofline of the reconstruction kernel measured with
CUDA events inside the timed steps, a CPU baseline timed on the host cores, and side numbers for the
factored path of the q_proj configuration (4096 x 4096, r = 256, T = 16).

`--impl reference` times the reference's CPU implementation of the same path (its PyTorch
arithmetic restated in oracle/, all host threads) on a bounded sample of the workload.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one reconstruction launch on gate_proj, from the ncu capture
# summarised in profiles/recon_strip_kernel_gate_proj_r512.md (95.5 MB + 51.6 MB; part of W' is still in L2 at exit)
RECON_TRAFFIC_BYTES = 147.1e6


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
    src/serving.py:92 and x W'^T for those rows.  Returns (TOP/s, seconds per step, threads)."""
    import numpy as np
    import torch

    from ade_b200 import synth
    from oracle import oracle as O

    O.use_all_cores()
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
    sec = sum(times) / len(times)
    return delta_ops(rows, N, RANK) / sec / 1e12, sec, O.threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 1024
    tops, sec, threads = cpu_sample(rows, args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * (WORK_OPS / delta_ops(rows, 4096, RANK)),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": {"workload": "llama2-7b MLP deltas, reconstructed path (gate/up 11008x4096, down 4096x11008, r=512, X 2048xd_i)"},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{rows} of 11008 output rows of gate_proj per step: reconstruct_delta + base add + x W'^T; "
                                   "ms_per_step is extrapolated to the full three-module step"},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


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
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ok, why = kernels.recon_kernel_status(dev)
    if not ok:
        raise RuntimeError(f"B200 kernels unavailable: {why}")

    # ---- build the three modules of this rank's delta (seeded by rank: one delta per GPU)
    mods, xs_host, xs_dev = [], [], []
    for mi, (name, M, N) in enumerate(MODULES):
        W_b, packed = synth.synthetic_module(M, N, RANK, config=1 + 100 * rank, module=mi, device=dev, exact_svd=False)
        mods.append(ADEKernelLinear(W_b, packed).to(dev))
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
            W = kernels.recon_int4(m._stored_form(), m.weight)
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

    # ---- side numbers: factored path of the q_proj configuration (4096 x 4096, r = 256, T = 16)
    factored = None
    if rank == 0:
        Wq, pq = synth.synthetic_module(4096, 4096, 256, config=0, module=0, device=dev, exact_svd=False)
        reps = 8                                  # distinct module instances so the weights do not sit in L2
        lins = [ADEKernelLinear(Wq.clone(), pq).to(dev) for _ in range(reps)]
        xq = synth.activations(16, 4096, synth.seed_for(0, 0, 2)).to(dev)
        factored = {}
        for T in (1, 16):
            xt = xq[:T].contiguous()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    for l in lins:
                        l(xt)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()            # the decode loop of a served model is a captured graph
            with torch.cuda.graph(graph):
                for l in lins:
                    l(xt)
            graph.replay()
            torch.cuda.synchronize()
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            f0.record()
            for _ in range(10):
                graph.replay()
            f1.record()
            torch.cuda.synchronize()
            us = f0.elapsed_time(f1) * 1e3 / (10 * reps)
            b = factored_bytes(4096, 4096, 256, T, fused=True)
            factored[f"T{T}"] = {"us_per_call": us, "gb_per_s": b / us / 1e3, "bytes": b,
                                 "note": "W_b-fused bytes, 1 launch per call inside a CUDA graph, "
                                         "8 module instances rotated (268 MB > L2)"}
            del graph
        del lins, Wq, pq
    sampler.stop_flag = True
    sampler.join(timeout=2)

    if world > 1:
        t = torch.tensor([ms, ms_e2e, recon_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e, recon_ms = (float(v) for v in t.tolist())
    if rank == 0:
        peak, peak_kind = measured_peaks()
        per_step = ms / args.steps
        value = world * WORK_OPS / (per_step * 1e-3) / 1e12
        e2e = world * WORK_OPS / (ms_e2e / args.steps * 1e-3) / 1e12
        bytes_launch = sum(recon_bytes(M, N, RANK) for _, M, N in MODULES) / len(MODULES)
        achieved = bytes_launch / (recon_ms * 1e-3) / 1e9
        cpu_rows = 1024
        cpu_tops, cpu_sec, cpu_threads = cpu_sample(cpu_rows, 3, 1)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8", "data": "synthetic",
            "config": {"workload": "llama2-7b MLP deltas, reconstructed path (gate/up 11008x4096, down 4096x11008, r=512, X 2048xd_i)",
                       "step": "per module: tcgen05 reconstruction kernel W'=W_b+U^V^^T, then cuBLAS x W'^T; 3 modules",
                       "ops_counted": "2*M*N*r of the delta contraction per module",
                       "l2": "inputs larger than L2: 553 MB of weights and codes touched per step, no flush needed",
                       "parallelism": f"replicas x{world}, one delta per GPU, no collective"},
            "e2e": {"value": e2e, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": sum(2 * TOKENS * N for _, _, N in MODULES),
                    "d2h_bytes_per_step": sum(2 * TOKENS * M for _, M, _ in MODULES)},
            "gpu_launches": 3 * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": RECON_TRAFFIC_BYTES, "peak_kind": peak_kind, "kernel": "recon_strip_kernel", "us_per_launch": recon_ms * 1e3,
                         "int8_tops_kernel_only": (WORK_OPS / 3) / (recon_ms * 1e-3) / 1e12},
            "cpu_baseline": {"value": cpu_tops, "unit": UNIT, "cores": cpu_threads, "kind": "port",
                             "sample": f"{cpu_rows} of 11008 rows of gate_proj: reconstruct + base add + x W'^T, {cpu_sec:.2f} s per pass"},
            "clocks": sampler.summary(t_wall0, t_wall2),
            "factored_q_proj": factored,
            "wall_s_timed": t_wall1 - t_wall0,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ade", choices=["ade", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ade(args)


if __name__ == "__main__":
    main()
