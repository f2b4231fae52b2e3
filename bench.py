#!/usr/bin/env python
"""Benchmark of the TAGI Linear hot path (forward + state-delta backward + parameter-delta backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Workload: the single-layer micro-benchmark configuration, FP32, batch 1024, 4096 -> 4096, seeded synthetic
tensors with the stated distributions. One step = tagi_linear_fwd + tagi_linear_bwd_state +
tagi_linear_bwd_param (with bias deltas) through the C ABI. Algorithmic work per step = 14*B*K*N FLOP
(6 forward + 4 state backward + 4 parameter backward).

With N > 1 (launched by torchrun, one rank per GPU) every rank runs the step on its own batch shard of 1024
samples against a full parameter replica (weak scaling) and the parameter deltas are averaged across ranks with
an NCCL allreduce inside the timed region, which is the one exchange step of the data-parallel path.

The same invocation then runs the second half of the metric, one training step of the ResNet-18 configuration (64
samples of 3 x 224 x 224 per GPU, data-parallel over the N ranks), and reports it under the "resnet18" key of the one JSON
line (`--no-resnet` skips it). Every timed region is stretched to about two seconds by repeating the K steps, so that the
clocks settle under load; times are reported per step.

`--impl reference` times the reference's CPU implementation (the compiled reference classes in oracle/_ref when
present, else the CPU restatement in oracle/) on the host cores, on a bounded batch sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

B, K, N = 1024, 4096, 4096
FLOP_FWD, FLOP_STATE, FLOP_PARAM = 6.0 * B * K * N, 4.0 * B * K * N, 4.0 * B * K * N
FLOP_STEP = FLOP_FWD + FLOP_STATE + FLOP_PARAM
METRIC = "TAGI Linear fwd+bwd TFLOP/s"
UNIT = "TFLOP/s"
WORKLOAD = "linear_fp32_B1024_4096x4096 (fwd + state-delta bwd + param-delta bwd, bias on)"
# FP32 FFMA peak of a B200: 148 SMs x 128 lanes x 2 FLOP x 1.965 GHz (maximum SM clock)
FP32_NOMINAL_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def make_inputs(seed, batch=B):
    """Seeded tensors with the distributions of the micro-benchmark configuration. N(0, 1e-2) for the bias mean
    and the mean deltas is read as variance 1e-2 (standard deviation 0.1)."""
    rng = np.random.default_rng(seed)
    f32 = np.float32
    wrng = np.random.default_rng(12345)  # parameters are the same on every rank
    x = dict(
        mu_w=(wrng.standard_normal((N, K), dtype=f32) / f32(np.sqrt(K))),
        var_w=(wrng.uniform(0.5, 1.5, (N, K)).astype(f32) / f32(K)),
        mu_b=(wrng.standard_normal(N, dtype=f32) * f32(0.1)),
        var_b=np.full(N, 1e-3, f32),
        mu_a=rng.standard_normal((batch, K), dtype=f32),
        var_a=rng.uniform(1e-3, 1e-1, (batch, K)).astype(f32),
        jcb=rng.uniform(0, 1, (batch, K)).astype(f32),
        dmu_z=(rng.standard_normal((batch, N), dtype=f32) * f32(0.1)),
        dvar_z=(-rng.uniform(0, 1e-3, (batch, N))).astype(f32),
    )
    return x


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "power_w_max": max(float(r[2]) for r in rows), "samples": len(rows)}


def cpu_arm(sample_rows, threads):
    """The reference's CPU path on `sample_rows` batch rows of the workload. Returns (seconds, kind)."""
    from oracle_lib import Oracle, RefLib
    x = make_inputs(1, sample_rows)
    if RefLib.available():
        ref = RefLib()
        t0 = time.perf_counter()
        ref.linear_forward(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"], threads=threads)
        ref.linear_backward(x["mu_w"], x["var_w"], x["var_b"], x["mu_a"], x["jcb"], x["dmu_z"], x["dvar_z"],
                            threads=threads)
        return time.perf_counter() - t0, "reference"
    o = Oracle()
    t0 = time.perf_counter()
    o.linear_fwd(x["mu_w"], x["var_w"], x["mu_b"], x["var_b"], x["mu_a"], x["var_a"])
    o.linear_bwd_state(x["mu_w"], x["jcb"], x["dmu_z"], x["dvar_z"])
    o.linear_bwd_param(x["var_w"], x["var_b"], x["mu_a"], x["dmu_z"], x["dvar_z"])
    return time.perf_counter() - t0, "port"


def pick_sample_rows(threads, target_s):
    """Batch rows for one CPU evaluation of about target_s seconds, from a 4-row probe."""
    t, _ = cpu_arm(4, threads)
    rows = int(max(4, min(B, 4 * target_s / max(t, 1e-3))))
    return rows - rows % 4 if rows >= 8 else 4


def run_reference(args, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = pick_sample_rows(threads, 4.0)
    for _ in range(min(args.warmup, 1)):
        cpu_arm(rows, threads)
    t0 = time.perf_counter()
    kind = "port"
    for _ in range(args.steps):
        _, kind = cpu_arm(rows, threads)
    dt = time.perf_counter() - t0
    tflops = 14.0 * rows * K * N * args.steps / dt / 1e12
    sample = f"{rows} of {B} batch rows per step, full 4096x4096 weights"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample,
                   "ms_per_step_is": "one step on the sample; scaled to all 1024 rows: %.0f ms" %
                                     (1e3 * dt / args.steps * (B / rows))},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def _repeat_for(ms_per_pass, target_s=2.0, lo=1, hi=2000):
    """How often a pass of ms_per_pass milliseconds is repeated so that the timed region lasts about target_s."""
    return int(max(lo, min(hi, round(target_s * 1e3 / max(ms_per_pass, 1e-3)))))


def run_b200(args, rank, world, local_rank):
    """The headline line. Returns the dict that rank 0 prints (None on other ranks); the process group stays up for
    the ResNet-18 leg."""
    import torch
    import torch.distributed as dist
    from cutagi_b200.capi import lib, IMPL_FFMA, IMPL_TF32X3, tc_status as capi_tc_status

    torch.cuda.set_device(local_rank)
    lib.tagi_set_impl({"auto": 0, "ffma": 1, "tf32x3": 2}[args.kernel_impl])
    sm_budget = args.sm_budget if args.sm_budget >= 0 else (0 if world == 1 else 132)
    lib.tagi_tc_set_sm_budget(sm_budget)
    devname = torch.cuda.get_device_name(local_rank)
    x = make_inputs(100 + rank)
    host = {k: torch.from_numpy(v).pin_memory() for k, v in x.items()}
    d = {k: v.cuda(non_blocking=True) for k, v in host.items()}
    out_shapes = dict(mu_z=(B, N), var_z=(B, N), dmu_a=(B, K), dvar_a=(B, K), dmu_w=(N, K), dvar_w=(N, K),
                      dmu_b=(N,), dvar_b=(N,))
    o = {k: torch.empty(s, dtype=torch.float32, device="cuda") for k, s in out_shapes.items()}
    host_out = {k: torch.empty(s, dtype=torch.float32).pin_memory() for k, s in out_shapes.items()}
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream
    p = {k: v.data_ptr() for k, v in {**d, **o}.items()}

    def k_fwd(p=p):
        lib.tagi_linear_fwd(p["mu_w"], p["var_w"], p["mu_b"], p["var_b"], p["mu_a"], p["var_a"], B, K, N, 1,
                            p["mu_z"], p["var_z"], sp)

    def k_state(p=p):
        lib.tagi_linear_bwd_state(p["mu_w"], p["jcb"], p["dmu_z"], p["dvar_z"], B, K, N, p["dmu_a"], p["dvar_a"], sp)

    def k_param(p=p):
        lib.tagi_linear_bwd_param(p["var_w"], p["var_b"], p["mu_a"], p["dmu_z"], p["dvar_z"], B, K, N, 1,
                                  p["dmu_w"], p["dvar_w"], p["dmu_b"], p["dvar_b"], sp)

    # N > 1: the parameter deltas are averaged over the ranks by the library's bucketed NCCL exchange, launched on its
    # own stream right after the parameter pass so that it overlaps the state pass (the order cuTAGI's Conv2d uses:
    # parameters first, then states).
    xchg = None
    # Ranges of output features the parameter pass (and with it the exchange) is cut into. More ranges start the exchange
    # earlier; fewer keep NCCL's messages large. Measured on B200s (ms per step with 4 / 2 / 1 ranges): 2 GPUs 1.275 / 1.30 /
    # 1.311, 4 GPUs 1.420 / 1.334 / 1.338, 8 GPUs 1.630 / 1.446 / 1.380 (134 MB in one allreduce: 0.40 ms; as four: 0.77 ms).
    pieces = args.param_pieces if args.param_pieces > 0 else (4 if world <= 2 else 2 if world <= 4 else 1)
    cuts = [N * i // pieces for i in range(pieces + 1)]
    if world > 1:
        from cutagi_b200.comm import DeltaExchange
        token = [f"/tmp/tagi_b200_rdv_{os.getpid()}_{time.time_ns()}"]
        dist.broadcast_object_list(token, src=0)
        # The parameter pass runs range by range over the output features (tagi_linear_bwd_param_rows) and every range's
        # deltas are handed to the exchange as soon as they are launched, so that the allreduce of one range overlaps the
        # computation of the next and the state pass.
        views = []
        for n0, n1 in zip(cuts[:-1], cuts[1:]):
            views += [o["dmu_w"][n0:n1], o["dvar_w"][n0:n1], o["dmu_b"][n0:n1], o["dvar_b"][n0:n1]]
        xchg = DeltaExchange(views, rank, world, local_rank, token[0], bucket_bytes=(N // pieces) * K * 8 + (1 << 20),
                             average=True, max_ctas=args.nccl_max_ctas)
        n_buckets = xchg.num_buckets

    def step(p=p, exchange=True):
        # The forward pass overlaps no exchange (the step before ended with the stream waiting for it), so it plans its
        # tiles for every SM; the parameter and state passes run beside NCCL's kernels and plan for the budget.
        if xchg and sm_budget:
            lib.tagi_tc_set_sm_budget(0)
        k_fwd(p)
        if xchg and sm_budget:
            lib.tagi_tc_set_sm_budget(sm_budget)
        if xchg:
            for j, (n0, n1) in enumerate(zip(cuts[:-1], cuts[1:])):
                lib.tagi_linear_bwd_param_rows(p["var_w"], p["var_b"], p["mu_a"], p["dmu_z"], p["dvar_z"], B, K, N, n0, n1,
                                               1, p["dmu_w"], p["dvar_w"], p["dmu_b"], p["dvar_b"], sp)
                if exchange:
                    for i in range(4):
                        xchg.ready(4 * j + i, sp)
        else:
            k_param(p)
        k_state(p)
        if xchg and exchange:
            xchg.wait(sp)

    def exchange_only():
        for i in range(4 * pieces):
            xchg.ready(i, sp)
        xchg.wait(sp)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        sync_all()
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def agree(v):   # every rank must run the same number of iterations
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.int64)
        dist.broadcast(t, src=0)
        return int(t.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    # K steps are repeated R times inside one timed region of about two seconds (burst clocks last a few
    # milliseconds; a power-capped part settles lower); ms_per_step is the region divided by K * R
    probe = timed(step, args.steps) / args.steps
    rep = 1 if args.profile else agree(_repeat_for(probe * args.steps, args.region_s))
    t_begin = time.time()
    ms_total = timed(step, args.steps * rep)
    t_end = time.time()
    ms_step = ms_total / (args.steps * rep)
    value = FLOP_STEP * world / (ms_step * 1e-3) / 1e12

    # per-kernel durations (same stream, CUDA events); each kernel's operands exceed the 126 MB L2
    kt = {}
    for name, fn in (("tagi_linear_fwd", k_fwd), ("tagi_linear_bwd_state", k_state), ("tagi_linear_bwd_param", k_param)):
        fn()
        n = args.steps if args.profile else agree(_repeat_for(timed(fn, 5) / 5, args.region_s / 4))
        kt[name] = timed(fn, n) / n

    # N > 1: what the exchange costs. The same step with the exchange left out, and the exchange alone (the buckets'
    # allreduce with no kernel of this library beside it).
    exchange_info = None
    if xchg:
        off = lambda: step(exchange=False)
        n = agree(_repeat_for(timed(off, 5) / 5, args.region_s / 2))
        ms_off = timed(off, n) / n
        n = agree(_repeat_for(timed(exchange_only, 3) / 3, args.region_s / 4))
        ms_alone = timed(exchange_only, n) / n
        # Correctness of the exchange: sampled rows of this rank's local deltas (a step without exchange), then the
        # same rows after a step with it; every rank's exchanged rows must equal the mean of all ranks' local rows and
        # be the same bits on every rank.
        rows = torch.tensor(sorted(np.random.default_rng(7).choice(N, 8, replace=False).tolist()), device="cuda")
        step(exchange=False)
        local = torch.cat([o["dmu_w"][rows].reshape(-1), o["dvar_w"][rows].reshape(-1), o["dmu_b"], o["dvar_b"]]).clone()
        step()
        torch.cuda.synchronize()
        got = torch.cat([o["dmu_w"][rows].reshape(-1), o["dvar_w"][rows].reshape(-1), o["dmu_b"], o["dvar_b"]]).clone()
        all_local = [torch.empty_like(local) for _ in range(world)]
        all_got = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(all_local, local)
        dist.all_gather(all_got, got)
        mean = torch.stack(all_local).double().mean(0)
        err = float(((got.double() - mean).abs().max() / mean.abs().max()).item())
        same = all(torch.equal(all_got[0], g) for g in all_got[1:])
        exchange_info = {"exchange_ms_alone": ms_alone, "step_ms_exchange_off": ms_off, "step_ms": ms_step,
                         "bytes_per_step": int(2 * (N * K + N) * 4),
                         "exchange_check": {"max_rel_err": err, "ranks_bit_identical": bool(same),
                                            "sample": "8 rows of dmu_w / dvar_w and all of dmu_b / dvar_b against the "
                                                      "FP64 mean of the ranks' local deltas"}}

    # End to end: host buffers in, host buffers out, copies inside the timed region. Every step's inputs travel host ->
    # device and its outputs device -> host on their own streams. Inputs and the large outputs (forward moments, state
    # deltas) are double-buffered on the device, so the upload of step i+1, the kernels of step i and the download of
    # step i-1 overlap (PCIe is full duplex); events order buffer reuse. The parameter and bias deltas keep one buffer
    # (they are what the exchange has registered for N > 1); they are downloaded first, so the next step waits for a few
    # KB at most in the "layer" variant. Two variants: "layer" keeps the parameters and the parameter deltas on the
    # device, as cuTAGI's LinearCuda does (d_mu_w ..., d_delta_mu_w ... are members of the layer; only activations and
    # incoming deltas are a step's inputs, only the forward outputs, the state deltas and the bias deltas its results);
    # "all" moves every tensor of the three calls both ways.
    in_layer = ["mu_a", "var_a", "jcb", "dmu_z", "dvar_z"]
    out_layer = ["mu_z", "var_z", "dmu_a", "dvar_a", "dmu_b", "dvar_b"]
    d_alt = {k: torch.empty_like(v) for k, v in d.items()}
    o_alt = {k: torch.empty_like(o[k]) for k in ("mu_z", "var_z", "dmu_a", "dvar_a")}
    s_h2d, s_d2h = torch.cuda.Stream(), torch.cuda.Stream()

    def make_e2e(in_keys, out_keys):
        twice = [k_ for k_ in out_keys if k_ in o_alt]
        once = [k_ for k_ in out_keys if k_ not in o_alt]
        psets = [p, {**p, **{k_: d_alt[k_].data_ptr() for k_ in in_keys}, **{k_: o_alt[k_].data_ptr() for k_ in twice}}]
        dsets = [d, {**d, **{k_: d_alt[k_] for k_ in in_keys}}]
        osets = [o, {**o, **{k_: o_alt[k_] for k_ in twice}}]
        ev_in_ready = [torch.cuda.Event(), torch.cuda.Event()]
        ev_in_free = [torch.cuda.Event(), torch.cuda.Event()]
        ev_out_ready = [torch.cuda.Event(), torch.cuda.Event()]
        ev_out_free = [torch.cuda.Event(), torch.cuda.Event()]
        ev_once_free = torch.cuda.Event()
        it = [0]

        def one():
            b = it[0] & 1
            it[0] += 1
            s_h2d.wait_event(ev_in_free[b])          # the step that last used this input buffer has finished
            with torch.cuda.stream(s_h2d):
                for k_ in in_keys:
                    dsets[b][k_].copy_(host[k_], non_blocking=True)
                ev_in_ready[b].record(s_h2d)
            stream.wait_event(ev_in_ready[b])
            stream.wait_event(ev_out_free[b])        # this output buffer's previous contents have been downloaded
            stream.wait_event(ev_once_free)          # and so have the single-buffered outputs of the previous step
            step(psets[b])
            ev_in_free[b].record(stream)
            ev_out_ready[b].record(stream)
            s_d2h.wait_event(ev_out_ready[b])
            with torch.cuda.stream(s_d2h):
                for k_ in once:
                    host_out[k_].copy_(o[k_], non_blocking=True)
                ev_once_free.record(s_d2h)
                for k_ in twice:
                    host_out[k_].copy_(osets[b][k_], non_blocking=True)
                ev_out_free[b].record(s_d2h)

        def run(n):
            for _ in range(n):
                one()
            stream.wait_event(ev_out_free[0])        # the timed region ends when the last downloads have landed
            stream.wait_event(ev_out_free[1])
        return run, sum(host[k_].numel() * 4 for k_ in in_keys), sum(host_out[k_].numel() * 4 for k_ in out_keys)

    e2e = {}
    for name, ik, ok_ in (("layer", in_layer, out_layer), ("all", list(host), list(host_out))):
        run, h2d, d2h = make_e2e(ik, ok_)
        if args.profile:
            e2e[name] = (float("nan"), h2d, d2h)
            continue
        run(2)
        n = agree(_repeat_for(timed(lambda: run(4), 1) / 4, args.region_s / 2, lo=4, hi=400))
        e2e[name] = (timed(lambda: run(n), 1) / n, h2d, d2h)
    clocks = None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(t_begin, t_end)
    tc_status = capi_tc_status()
    if xchg:
        xchg.check()
        xchg.close()
    if rank != 0:
        return None

    impl = lib.tagi_get_impl()
    if impl == 0:  # AUTO resolves to the tensor-core kernels for this shape (aligned, every dimension >= 128)
        impl = IMPL_TF32X3
    flops = {"tagi_linear_fwd": FLOP_FWD, "tagi_linear_bwd_state": FLOP_STATE, "tagi_linear_bwd_param": FLOP_PARAM}
    tfl = {k_: flops[k_] / (v * 1e-3) / 1e12 for k_, v in kt.items()}
    dom = max(kt, key=kt.get)
    worst = min(tfl, key=tfl.get)
    achieved = tfl[dom]
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    if impl == IMPL_TF32X3:
        bf16 = peaks.get("bf16_tflops", 1590.0)
        peak, bound = bf16 / 2.0 / 3.0, "tensor"
        peak_note = ("measured dense bf16 %.0f TFLOP/s (burst) / 2 (tf32 rate) / 3 (three tf32 products per fp32 product), %s"
                     % (bf16, "of measured" if peaks else "of fallback"))
        sustained = peaks.get("bf16_tflops_sustained", 1400.0) / 6.0
    else:
        peak, bound = FP32_NOMINAL_TFLOPS, "fp32"
        peak_note = ("FP32 FFMA path: 148 SMs x 128 lanes x 2 x 1.965 GHz, of nominal "
                     "(MEASURED_PEAKS.json holds no FP32 figure)")
        sustained = peak
    # DRAM traffic of one launch of each kernel (dram__bytes_read.sum + dram__bytes_write.sum): constants taken from an
    # ncu capture of these kernels at this shape, not re-measured by this run; the FFMA kernels have not been captured
    captured_traffic = {"tagi_linear_fwd": 322.1e6, "tagi_linear_bwd_state": 203.3e6, "tagi_linear_bwd_param": 218.5e6}
    step_tflops = FLOP_STEP / (ms_step * 1e-3) / 1e12 if world == 1 else FLOP_STEP / (exchange_info["step_ms_exchange_off"] * 1e-3) / 1e12
    roofline = {"bound": bound, "kernel": dom, "achieved": achieved, "peak": peak, "unit": UNIT,
                "frac": achieved / peak, "traffic": captured_traffic[dom] if impl == IMPL_TF32X3 else None,
                "traffic_is": "a constant captured with ncu for this kernel and shape (bytes per launch, dram read + "
                              "write); not re-measured by this run",
                "peak_note": peak_note, "per_kernel_ms": kt, "per_kernel_tflops": tfl,
                "per_kernel_frac": {k_: v / peak for k_, v in tfl.items()},
                "worst_kernel": worst, "worst_kernel_frac": tfl[worst] / peak,
                "step_tflops_per_gpu": step_tflops, "step_frac": step_tflops / peak,
                "step_frac_of_sustained_peak": step_tflops / sustained,
                "sustained_peak": sustained}

    cpu_baseline = None
    if world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        rows = pick_sample_rows(threads, 6.0)
        t, kind = cpu_arm(rows, threads)
        cpu_baseline = {"value": 14.0 * rows * K * N / t / 1e12, "unit": UNIT, "cores": threads, "kind": kind,
                        "sample": f"{rows} of {B} batch rows, full 4096x4096 weights, {t:.1f} s"}

    if clocks and clocks.get("sm_mhz"):
        clocks["ms_per_step_x_sm_mhz"] = ms_step * clocks["sm_mhz"]
    ms_e2e, h2d, d2h = e2e["layer"]
    ms_all, h2d_all, d2h_all = e2e["all"]
    return {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "impl": {1: "ffma (FP32 CUDA cores)", 2: "tf32x3 (tcgen05, 3 TF32 products per "
                                                  "FP32 product, FP32 accumulation)"}.get(impl, str(impl)),
                   "device": devname, "l2": "inputs (604 MB per step) exceed the 126 MB L2; no flush",
                   "inner_repeat": rep, "timed_region_s": ms_total * 1e-3,
                   "timing": "the K steps are repeated inner_repeat times inside one CUDA-event region; ms_per_step = "
                             "region / (K * inner_repeat)",
                   "sm_budget": sm_budget if world == 1 else "%d for the parameter and state passes (they run beside the "
                                "exchange), all SMs for the forward pass" % sm_budget,
                   "exchange": ("allreduce(avg) of parameter deltas: parameter pass and exchange in %d ranges of output "
                                "features, %d NCCL buckets on a side stream, each range's exchange overlapped with the "
                                "next range's parameter pass and the state pass" % (pieces, n_buckets))
                   if world > 1 else "none (1 GPU)"},
        "roofline": roofline, "cpu_baseline": cpu_baseline,
        "e2e": {"value": FLOP_STEP * world / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "resident": "parameters and parameter deltas stay on the device, as in cuTAGI's LinearCuda; mu_a, var_a, "
                            "jcb, dmu_z, dvar_z are uploaded and mu_z, var_z, dmu_a, dvar_a, dmu_b, dvar_b downloaded every "
                            "step, per GPU",
                "all_tensors": {"value": FLOP_STEP * world / (ms_all * 1e-3) / 1e12, "ms_per_step": ms_all,
                                "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all,
                                "note": "every input (weights included) uploaded and every output (weight deltas "
                                        "included) downloaded every step"}},
        "exchange": exchange_info,
        "gpu_launches": (3 if world == 1 else 2 + pieces) * args.steps * rep, "tc_status": tc_status, "clocks": clocks}


# Conv2d layer shapes of the CIFAR-shaped CNN (batch 128) and of the ResNet-18 configuration (batch 64, 224x224)
CONV_LAYERS = [
    ("CNN conv1", dict(B=128, fi=3, hi=32, wi=32, fo=32, k=3, stride=1, pad=1, pad_type=1, has_bias=1)),
    ("CNN conv2", dict(B=128, fi=32, hi=16, wi=16, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=1)),
    ("CNN conv3", dict(B=128, fi=64, hi=8, wi=8, fo=128, k=3, stride=1, pad=1, pad_type=1, has_bias=1)),
    ("ResNet-18 stem", dict(B=64, fi=3, hi=224, wi=224, fo=64, k=6, stride=2, pad=2, pad_type=1, has_bias=0)),
    ("ResNet-18 layer1", dict(B=64, fi=64, hi=56, wi=56, fo=64, k=3, stride=1, pad=1, pad_type=1, has_bias=0)),
    ("ResNet-18 down-sampling", dict(B=64, fi=64, hi=56, wi=56, fo=128, k=3, stride=2, pad=1, pad_type=2, has_bias=0)),
    ("ResNet-18 shortcut", dict(B=64, fi=64, hi=56, wi=56, fo=128, k=2, stride=2, pad=0, pad_type=0, has_bias=0)),
    ("ResNet-18 layer2", dict(B=64, fi=128, hi=28, wi=28, fo=128, k=3, stride=1, pad=1, pad_type=1, has_bias=0)),
    ("ResNet-18 layer3", dict(B=64, fi=256, hi=14, wi=14, fo=256, k=3, stride=1, pad=1, pad_type=1, has_bias=0)),
    ("ResNet-18 layer4", dict(B=64, fi=512, hi=7, wi=7, fo=512, k=3, stride=1, pad=1, pad_type=1, has_bias=0)),
]


def run_conv_layers(args):
    """Side table, not the benchmark line: CUDA-event time of each Conv2d entry point per layer shape, inputs resident
    in HBM, seeded synthetic tensors. P = B*ho*wo*fo*fi*k*k multiply-adds per product; algorithmic FLOP: forward 6P,
    state backward 4P, parameter backward 4P."""
    import ctypes as C
    import torch
    import gpu_util as G
    from cutagi_b200 import capi
    from cutagi_b200.capi import lib
    from oracle_lib import ConvGeom
    lib.tagi_set_impl({"auto": capi.IMPL_AUTO, "ffma": capi.IMPL_FFMA, "tf32x3": capi.IMPL_TF32X3}[args.kernel_impl])
    torch.manual_seed(0)
    P = lambda t: t.data_ptr()

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    print("| layer (B, fi -> fo, image, k, stride) | P | forward | state backward | parameter backward |")
    print("|---|---|---|---|---|")
    for name, kw in CONV_LAYERS:
        if args.layer and args.layer not in name:
            continue
        g = ConvGeom(**kw)
        n_in, n_out, nw = g.B * g.n_in, g.B * g.n_out, g.fo * g.Kc
        t = lambda n: torch.rand(n, device="cuda") * 0.1 + 0.01
        mw, vw, mb, vb, ma, va, j, dm, dv = t(nw), t(nw), t(g.fo), t(g.fo), t(n_in), t(n_in), t(n_in), t(n_out), t(n_out)
        mz, vz, da, dva, dw, dvw, db, dvb = t(n_out), t(n_out), t(n_in), t(n_in), t(nw), t(nw), t(g.fo), t(g.fo)
        cg = G.cgeom(g)
        tf = timed(lambda: lib.tagi_conv2d_fwd(C.byref(cg), P(mw), P(vw), P(mb), P(vb), P(ma), P(va), P(mz), P(vz),
                                               None), args.steps)
        ts = timed(lambda: lib.tagi_conv2d_bwd_state(C.byref(cg), P(mw), P(j), P(dm), P(dv), P(da), P(dva), None),
                   args.steps)
        tp = timed(lambda: lib.tagi_conv2d_bwd_param(C.byref(cg), P(vw), P(vb), P(ma), P(dm), P(dv), P(dw), P(dvw),
                                                     P(db), P(dvb), None), args.steps)
        pm = g.B * g.ho * g.wo * g.fo * g.Kc
        print(f"| {name} ({g.B}, {g.fi} -> {g.fo}, {g.hi}x{g.wi}, k{g.k} s{g.stride}) | {pm:.2e} | "
              f"{tf:.3f} ms, {6 * pm / tf / 1e9:.1f} TF/s | {ts:.3f} ms, {4 * pm / ts / 1e9:.1f} | "
              f"{tp:.3f} ms, {4 * pm / tp / 1e9:.1f} |")


def resnet_flops(spec, shape):
    """Algorithmic FLOP of one training step per sample: 14 P per Conv2d / Linear (6 forward + 4 state + 4 parameter),
    10 P for the first layer (no state pass), P = output pixels * fo * fi * k * k."""
    total, first = 0.0, True

    def walk(spec, shape):
        nonlocal total, first
        for item in spec:
            kind, a = item[0], item[1:]
            if kind == "conv":
                fi, fo, k, stride, pad, pad_type = a[:6]
                num = shape[1] - k + (2 * pad if pad_type == 1 else pad if pad_type == 2 else 0)
                ho = num // stride + 1
                total += (10.0 if first else 14.0) * ho * ho * fo * fi * k * k
                first = False
                shape = (fo, ho, ho)
            elif kind == "linear":
                total += 14.0 * a[0] * a[1]
                shape = (a[1],)
            elif kind == "pool":
                k, stride, pad, pad_type = a
                stride = k if stride < 0 else stride
                num = shape[1] - k + (2 * pad if pad_type == 1 else pad if pad_type == 2 else 0)
                shape = (shape[0], num // stride + 1, num // stride + 1)
            elif kind == "res":
                out = walk(a[0], shape)
                if a[1]:
                    walk(a[1], shape)
                shape = out
        return shape
    walk(spec, shape)
    return total


def run_network(args, rank, world, local_rank):
    """One TAGI training step of a whole network of the benchmark configurations through the device-side mirror of the
    pytagi API: the reference's ResNet-18 (ReLU variant, 11 hierarchical-softmax outputs, 64 x 3 x 224 x 224 N(0,1) images
    per GPU), the CIFAR-shaped CNN (batch 128) or the deep regression MLP (1 -> 4096 -> 4096 -> 4096 -> 1, batch 2048).
    Step = forward, output update, backward with the parameter deltas averaged over the ranks (bucketed NCCL exchange
    overlapped with the rest of the backward pass), capped update. Returns the result line (samples/s) as a dict on
    rank 0, None elsewhere; the caller owns the process group."""
    import torch
    import torch.distributed as dist
    from cutagi_b200 import nn
    from cutagi_b200.capi import lib, tc_status as capi_tc_status

    torch.cuda.set_device(local_rank)
    lib.tagi_set_impl({"auto": 0, "ffma": 1, "tf32x3": 2}[args.kernel_impl])
    lib.tagi_tc_set_sm_budget(max(args.sm_budget, 0))   # the exchange overlaps a small part of this step: plan for all SMs
    image = args.image
    rng = np.random.default_rng(100 + rank)
    n_sets = 2
    regression = args.workload == "mlp"
    if args.workload == "resnet18":
        batch = args.batch or 64
        spec, in_shape = nn.resnet18_spec(image, act=args.act), (3, image, image)
        name = f"resnet18_{args.act}_3x{image}x{image}_batch{batch}_per_gpu"
        draw = lambda: rng.standard_normal((batch, 3 * image * image), dtype=np.float32)
    elif args.workload == "cnn":    # the CIFAR-shaped CNN: U[0,1] pixels, batch 128
        batch = args.batch or 128
        spec = [("conv", 3, 32, 3, 1, 1, 1, True), ("relu",), ("pool", 2, 2, 0, 0), ("conv", 32, 64, 3, 1, 1, 1, True),
                ("relu",), ("pool", 2, 2, 0, 0), ("conv", 64, 128, 3, 1, 1, 1, True), ("relu",), ("pool", 2, 2, 0, 0),
                ("linear", 2048, 256, True), ("relu",), ("linear", 256, 11, True)]
        in_shape, name = (3, 32, 32), f"cifar_cnn_3x32x32_batch{batch}_per_gpu"
        draw = lambda: rng.random((batch, 3 * 32 * 32), dtype=np.float32)
    else:                           # the deep regression MLP 1 -> 4096 -> 4096 -> 4096 -> 1, batch 2048, x ~ U[-5, 5]
        batch = args.batch or 2048
        spec = [("linear", 1, 4096, True), ("relu",), ("linear", 4096, 4096, True), ("relu",), ("linear", 4096, 4096, True),
                ("relu",), ("linear", 4096, 1, True)]
        in_shape, name = (1,), f"regression_mlp_1-4096-4096-4096-1_batch{batch}_per_gpu"
        draw = lambda: rng.uniform(-5, 5, (batch, 1)).astype(np.float32)
    n_out = 1 if regression else 11
    net = nn.build(spec, in_shape, seed=1234)      # same parameters on every rank
    upd, utils = nn.OutputUpdater(), nn.Utils()
    xs = [torch.from_numpy(draw()).pin_memory() for _ in range(n_sets)]
    if regression:   # y = x^3 + eps, eps ~ N(0, 9), observation variance 9
        obs = [torch.from_numpy((x.numpy() ** 3 + 3.0 * rng.standard_normal((batch, 1))).astype(np.float32)).pin_memory()
               for x in xs]
        idx = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(n_sets)]
        var_y = torch.full((batch, 1), 9.0, device="cuda")
    else:
        obs_idx = [utils.label_to_obs(rng.integers(0, 10, batch), 10) for _ in range(n_sets)]
        obs = [torch.from_numpy(o[0]).pin_memory() for o in obs_idx]
        idx = [torch.from_numpy(o[1]).pin_memory() for o in obs_idx]
        var_y = torch.full((batch * 4,), 1.0, device="cuda")
    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream
    # N > 1: the delta tensors live back to back in one buffer, so that a bucket travels as one collective
    deltas = net.pack_deltas() if world > 1 else net.delta_tensors()
    xchg = None
    if world > 1:
        from cutagi_b200.comm import DeltaExchange
        token = [f"/tmp/tagi_b200_rdv_{os.getpid()}_{time.time_ns()}"]
        dist.broadcast_object_list(token, src=0)
        xchg = DeltaExchange(deltas, rank, world, local_rank, token[0], bucket_bytes=args.bucket_mb << 20, average=True,
                             max_ctas=args.nccl_max_ctas)
        pos = {t.data_ptr(): i for i, t in enumerate(deltas)}

        def hook(layer):
            ids = [pos[t.data_ptr()] for t in layer.delta_tensors()]

            def ready():
                for i in ids:
                    xchg.ready(i, sp)
            return ready
        for layer in net.named_layers().values():
            layer.on_ready = hook(layer)
    d_x = [torch.empty_like(xs[0], device="cuda") for _ in range(n_sets)]
    d_obs = [torch.empty_like(obs[0], device="cuda") for _ in range(n_sets)]
    d_idx = [torch.empty_like(idx[0], device="cuda") for _ in range(n_sets)]
    for i in range(n_sets):
        d_x[i].copy_(xs[i]), d_obs[i].copy_(obs[i]), d_idx[i].copy_(idx[i])
    host_out = torch.empty(2, batch, n_out).pin_memory()

    def output_update(i):
        if regression:
            upd.update(net, d_obs[i], var_y)
        else:
            upd.update_using_indices(net, d_obs[i], var_y, d_idx[i])
    it = [0]

    exchange_on = [True]
    # End to end: the library's host I/O pipeline (tagi_io_*): every step's batch, observations and indices travel from
    # pinned host memory to the device on the pipeline's stream (the upload of step i+1 overlaps the kernels of step i)
    # and exactly the B x n_out output moments come back; the host waits for the read-back one step behind.
    from cutagi_b200.hostio import HostPipeline
    io = HostPipeline(xs[0].numel(), obs[0].numel(), idx[0].numel(), batch * n_out, depth=n_sets)
    for i in range(n_sets):
        hx, ho, hi_ = io.host_arrays(i)
        hx[:], ho[:], hi_[:] = xs[i].numpy().reshape(-1), obs[i].numpy().reshape(-1), idx[i].numpy().reshape(-1)
    pending_out = [None]

    def step(e2e=False):
        i = it[0] % n_sets
        it[0] += 1
        if e2e:
            mu, var, dobs, didx = net.forward_staged(io, i)
            if regression:
                upd.update(net, dobs.reshape(batch, 1), var_y)
            else:
                upd.update_using_indices(net, dobs, var_y, didx)
        else:
            mu, var = net(d_x[i])
            output_update(i)
        net.backward()
        if xchg and exchange_on[0]:
            xchg.flush(sp)
            xchg.wait(sp)
        net.step()
        if e2e:
            io.consumed(i, sp)
            io.download(i, mu, var, sp)
            if pending_out[0] is not None:
                io.wait_output(pending_out[0], batch * n_out)
            pending_out[0] = i

    def e2e_run(n):
        for _ in range(n):
            step(True)
        if pending_out[0] is not None:                  # the timed region ends when the last read-back has landed
            io.wait_output(pending_out[0], batch * n_out)
            pending_out[0] = None
        else:                                           # (CUDA-graph replay: plain copies on the compute stream)
            torch.cuda.synchronize()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        sync_all()
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    eager_step = step
    if args.graph and world == 1:
        # The whole step (about 70 launches for the CNN, 1000 for ResNet-18) replayed as one CUDA graph per input buffer:
        # for the small configurations the step is bound by launch overhead, not by the kernels. Scratch buffers have
        # reached their final size during the warm-up steps, so nothing allocates while the stream is being captured.
        torch.cuda.synchronize()
        graphs, outs = [], []
        for i in range(n_sets):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                mu, var = net(d_x[i])
                output_update(i)
                net.backward()
                net.step()
            graphs.append(g)
            outs.append((mu, var))

        def step(e2e=False):
            i = it[0] % n_sets
            it[0] += 1
            if e2e:
                d_x[i].copy_(xs[i], non_blocking=True)
                d_obs[i].copy_(obs[i], non_blocking=True)
                d_idx[i].copy_(idx[i], non_blocking=True)
            graphs[i].replay()
            if e2e:
                host_out[0].copy_(outs[i][0], non_blocking=True)
                host_out[1].copy_(outs[i][1], non_blocking=True)
        for _ in range(2):
            step()
    t0 = time.time()
    ms = timed(step, args.steps) / args.steps
    t1 = time.time()
    ms_e2e = ms if args.profile else timed(lambda: e2e_run(args.steps), 1) / args.steps
    # N > 1: the same step with the exchange left out, the exchange alone, and its correctness on a sample
    exchange_info = None
    if xchg and not args.profile:
        hooks = {k: l.on_ready for k, l in net.named_layers().items()}

        def set_exchange(on):
            exchange_on[0] = on
            for k, l in net.named_layers().items():
                l.on_ready = hooks[k] if on else None
        set_exchange(False)
        n_off = max(3, args.steps // 4)
        ms_off = timed(step, n_off) / n_off

        def exchange_only():
            xchg.flush(sp)
            xchg.wait(sp)
        exchange_only()
        ms_alone = timed(exchange_only, 5) / 5
        # local deltas of one step (parameters are not updated: forward, output update, backward only), then the same
        # with the exchange
        def half_step():
            net(d_x[0])
            output_update(0)
            net.backward()
        half_step()
        pick = [t for t in deltas if t.numel() >= 1][:: max(1, len(deltas) // 12)]
        local = torch.cat([t.reshape(-1)[:4096] for t in pick]).clone()
        set_exchange(True)
        half_step()
        xchg.flush(sp)
        xchg.wait(sp)
        torch.cuda.synchronize()
        got = torch.cat([t.reshape(-1)[:4096] for t in pick]).clone()
        all_local = [torch.empty_like(local) for _ in range(world)]
        all_got = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(all_local, local)
        dist.all_gather(all_got, got)
        mean = torch.stack(all_local).double().mean(0)
        err = float(((got.double() - mean).abs().max() / mean.abs().max()).item())
        exchange_info = {"exchange_ms_alone": ms_alone, "step_ms_exchange_off": ms_off, "step_ms": ms,
                         "bytes_per_step": int(sum(t.numel() for t in deltas) * 4), "buckets": xchg.num_buckets,
                         "tensors": len(deltas), "collectives_per_step": xchg.num_collectives,
                         "exchange_check": {"max_rel_err": err,
                                            "ranks_bit_identical": bool(all(torch.equal(all_got[0], g) for g in all_got[1:])),
                                            "sample": f"first 4096 entries of {len(pick)} of the {len(deltas)} delta tensors "
                                                      "against the FP64 mean of the ranks' local deltas"}}
    # phases on one rank's stream (no exchange wait inside): forward / output update + backward / update
    phases = {}
    if not args.profile:
        def fwd():
            net(d_x[0])

        def bwd():
            output_update(0)
            net.backward()
            if xchg:
                xchg.flush(sp)
                xchg.wait(sp)
        fwd()
        phases["forward_ms"] = timed(fwd, 3) / 3
        phases["backward_ms"] = timed(bwd, 3) / 3
        phases["update_ms"] = timed(net.step, 3) / 3
    clocks = sampler.summary(t0, t1) if rank == 0 else None
    if rank == 0:
        sampler.stop()
    status = capi_tc_status()
    io.close()
    if xchg:
        xchg.check()
        xchg.close()
    if rank != 0:
        return None
    flop = resnet_flops(spec, in_shape) * batch
    n_param = sum(t.numel() for t in deltas) // 2
    peak = 0.0
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] / 6.0
    except Exception:
        peak = 1590.0 / 6.0
    cpu = None
    if not args.no_cpu:
        from oracle_lib import Oracle
        from oracle_net import OracleNet
        o = Oracle()
        cnet = OracleNet(o, spec, in_shape, seed=1)
        nb = {"resnet18": 1, "cnn": 16, "mlp": 16}[args.workload]   # batch of the CPU sample
        xb = draw()[:nb]
        tc0 = time.perf_counter()
        cnet.forward(xb)
        if regression:
            cnet.update(xb ** 3, np.full((nb, 1), 9.0, np.float32))
        else:
            ob, ib, _ = utils.label_to_obs(rng.integers(0, 10, nb), 10)
            cnet.update_using_indices(ob, np.ones(4 * nb, np.float32), ib, 4)
        cnet.backward()
        cnet.step()
        dt = time.perf_counter() - tc0
        cpu = {"value": nb / dt, "unit": "samples/s", "cores": os.cpu_count(), "kind": "port",
               "sample": f"one training step at batch {nb} ({dt:.1f} s), oracle port with OpenMP; linear in the batch"}
    return {
        "metric": {"resnet18": "TAGI ResNet-18 training samples/s", "cnn": "TAGI CNN training samples/s",
                   "mlp": "TAGI regression MLP training samples/s"}[args.workload],
        "value": batch * world / (ms * 1e-3), "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{name} (forward + output update + backward + capped update)",
                   "launch": "one CUDA graph per step" if (args.graph and world == 1) else "one launch per kernel",
                   "parameters": n_param, "exchange": "none (1 GPU)" if world == 1 else
                   f"bucketed NCCL allreduce (average) of {2 * n_param * 4 / 1e6:.0f} MB of parameter deltas, "
                   f"buckets of {args.bucket_mb} MiB, overlapped with the backward pass",
                   "l2": "activations of a step exceed the 126 MB L2 many times over; no flush"},
        "roofline": {"bound": "tensor", "achieved": flop / (ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flop / (ms * 1e-3) / 1e12 / peak, "traffic": None,
                     "note": "whole step: algorithmic FLOP of all Conv2d / Linear passes per GPU over the step time; the "
                             "step also contains the HBM-bound ReLU / BatchNorm2d / AvgPool2d / residual passes", **phases},
        "cpu_baseline": cpu,
        "e2e": {"value": batch * world / (ms_e2e * 1e-3), "unit": "samples/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(xs[0].numel() * 4 + obs[0].numel() * 4 + idx[0].numel() * 4),
                "d2h_bytes_per_step": int(host_out.numel() * 4),
                "path": "tagi_io_* host pipeline: pinned staging, upload on its own stream, read-back of B x n_out moments"},
        "exchange": exchange_info,
        # kernel launches of one step counted in an ncu launch list of this workload (ReLU ResNet-18 at 224 x 224: 257
        # launches of this library's kernels between two capped updates); other workloads were not counted
        "gpu_launches": 257 * args.steps if args.workload == "resnet18" and image == 224 and args.act == "relu" else None,
        "gpu_launches_is": "launches per step from an ncu launch list of this workload x timed steps",
        "tc_status": status, "clocks": clocks}


def run_resnet_module(args):
    """The same ResNet-18 step driven through cuTAGI's own extension module, the way pytagi drives it (host arrays in,
    `Sequential.forward / backward / step`, `OutputUpdater.update_using_indices`): `--engine dropin` = cuTAGI with its
    LinearCuda / Conv2dCuda on this library's C ABI (integration/_build), `--engine stock` = the unmodified cuTAGI CUDA
    build for sm_100a (integration/_build/stock). Both are built where the cuTAGI sources are and travel as binaries.
    Wall-clock per step, device synchronised by reading the outputs back; one GPU."""
    import glob
    sub = os.path.join(ROOT, "integration", "_build", "stock" if args.engine == "stock" else "")
    if not glob.glob(os.path.join(sub, "cutagi*.so")):
        print(json.dumps({"engine": args.engine, "unavailable": f"no cutagi module under {os.path.relpath(sub, ROOT)} "
                          "(make -C integration [stock] needs the cuTAGI sources)"}))
        return
    sys.path.insert(0, sub)
    import cutagi as m
    image, batch = args.image, args.batch
    keep = []

    def conv(i, o, k, stride=1, pad=0, pad_type=1, w=0, h=0):
        return m.Conv2d(i, o, k, False, stride, pad, pad_type, w, h)

    def block(i, o, stride=1, pt=1):
        layers = [conv(i, o, 3, stride, 1, pt), m.ReLU(), m.BatchNorm2d(o), conv(o, o, 3, 1, 1, 1), m.ReLU(), m.BatchNorm2d(o)]
        keep.append(layers)
        return m.LayerBlock(layers)
    if image == 224:
        layers = [conv(3, 64, 6, 2, 2, 1, 224, 224), m.ReLU(), m.BatchNorm2d(64), m.AvgPool2d(3, 2, 1, 2)]
        final_pool = 7
    else:
        layers = [conv(3, 64, 3, 1, 1, 1, image, image), m.ReLU(), m.BatchNorm2d(64)]
        final_pool = image // 8
    prev = 64
    for w in (64, 128, 256, 512):
        if w == prev:
            layers.append(m.ResNetBlock(block(prev, w)))
        else:
            sc = [conv(prev, w, 2, 2), m.ReLU(), m.BatchNorm2d(w)]
            keep.append(sc)
            layers.append(m.ResNetBlock(block(prev, w, 2, 2), m.LayerBlock(sc)))
        layers.append(m.ResNetBlock(block(w, w)))
        prev = w
    layers += [m.AvgPool2d(final_pool), m.Linear(512, 11, True)]
    keep.append(layers)
    net = m.Sequential(layers)
    net.to_device("cuda")
    upd, hrc = m.OutputUpdater(net.device), m.Utils()
    rng = np.random.default_rng(100)
    x = rng.standard_normal(batch * 3 * image * image, dtype=np.float32)
    obs, idx, _ = hrc.label_to_obs_wrapper(rng.integers(0, 10, batch).astype(np.int32), 10)
    obs, idx, var_y = [float(v) for v in obs], [int(v) for v in idx], [1.0] * (batch * 4)

    def step():
        net.forward(x, None)
        upd.update_using_indices(net.output_z_buffer, obs, var_y, idx, net.input_delta_z_buffer)
        net.backward()
        net.step()
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    net.get_outputs()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    mu, _ = net.get_outputs()
    dt = (time.perf_counter() - t0) / args.steps
    print(json.dumps({"metric": "TAGI ResNet-18 training samples/s", "engine":
                      {"stock": "unmodified cuTAGI CUDA build (its own Linear / Conv2d kernels)",
                       "dropin": "cuTAGI with its Linear / Conv2d / BatchNorm2d / AvgPool2d / ReLU layers, capped update and "
                                 "numpy input / output path on libtagi_b200"}[args.engine],
                      "value": batch / dt, "unit": "samples/s", "n_gpus": 1, "steps": args.steps, "ms_per_step": dt * 1e3,
                      "timing": "wall clock around the module's own forward / backward / step calls (host input arrays, "
                                "outputs read back at the end)",
                      "config": {"workload": f"resnet18_relu_3x{image}x{image}_batch{batch}"},
                      "finite_outputs": bool(np.all(np.isfinite(np.asarray(mu))))}))


def run_linear_module(args):
    """The headline Linear layer (B = 1024, 4096 -> 4096) driven through cuTAGI's own extension module: one-layer
    Sequential with input state update on, so that a step runs the forward, the parameter and the state pass.
    `--engine stock` times cuTAGI's own CUDA kernels on this GPU, `--engine dropin` the same module on this library.
    Wall clock per step including the module's host-to-device copy of the inputs (its public API takes host arrays)."""
    import glob
    sub = os.path.join(ROOT, "integration", "_build", "stock" if args.engine == "stock" else "")
    if not glob.glob(os.path.join(sub, "cutagi*.so")):
        print(json.dumps({"engine": args.engine, "unavailable": f"no cutagi module under {os.path.relpath(sub, ROOT)}"}))
        return
    sys.path.insert(0, sub)
    import cutagi as m
    layers = [m.Linear(K, N, True)]
    net = m.Sequential(layers)
    net.input_state_update = True
    net.to_device("cuda")
    x = make_inputs(100)
    upd = m.OutputUpdater(net.device)
    mu_x, var_x = x["mu_a"].reshape(-1), x["var_a"].reshape(-1)
    obs, var_obs = np.zeros(B * N, np.float32), np.ones(B * N, np.float32)

    def step(update):
        net.forward(mu_x, var_x)
        if update:
            upd.update(net.output_z_buffer, obs, var_obs, net.input_delta_z_buffer)
        net.backward()
    step(True)
    net.get_outputs()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(False)     # the deltas of the first update stay in the buffer: same kernels, no host-side list conversion
    net.get_outputs()
    dt = (time.perf_counter() - t0) / args.steps
    print(json.dumps({"metric": METRIC, "engine": {"stock": "unmodified cuTAGI CUDA build", "dropin":
                      "cuTAGI with LinearCuda on libtagi_b200"}[args.engine], "value": FLOP_STEP / dt / 1e12, "unit": UNIT,
                      "n_gpus": 1, "steps": args.steps, "ms_per_step": dt * 1e3, "config": {"workload": WORKLOAD},
                      "timing": "wall clock around Sequential.forward(host arrays) + backward; includes the module's copy "
                                "of 33.5 MB of inputs to the device per step"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-resnet", action="store_true", help="linear workload: skip the ResNet-18 leg of the line")
    ap.add_argument("--resnet-steps", type=int, default=50, help="timed steps of the ResNet-18 leg")
    ap.add_argument("--region-s", type=float, default=2.0,
                    help="linear workload: length each timed region is stretched to by repeating the K steps")
    ap.add_argument("--profile", action="store_true",
                    help="for captures under ncu: one warm-up step, no repeats, no end-to-end, ResNet-18 or CPU leg (numbers "
                         "printed in this mode are not benchmark values)")
    ap.add_argument("--kernel-impl", default="auto", choices=["auto", "ffma", "tf32x3"],
                    help="arithmetic of the kernels (tagi_set_impl)")
    ap.add_argument("--conv-layers", action="store_true",
                    help="print a per-layer timing table of the Conv2d entry points instead of the benchmark line")
    ap.add_argument("--layer", default="", help="--conv-layers: only the rows whose name contains this text")
    ap.add_argument("--sm-budget", type=int, default=-1,
                    help="SMs the tensor-core kernels plan their tiles for (tagi_tc_set_sm_budget); default: all on one GPU, "
                         "132 for the Linear step when the exchange's NCCL kernels run next to it (N > 1)")
    ap.add_argument("--nccl-max-ctas", type=int, default=0,
                    help="N > 1: upper bound on the CTAs of one NCCL kernel of the exchange (0 = NCCL's default)")
    ap.add_argument("--param-pieces", type=int, default=0,
                    help="linear, N > 1: ranges of output features the parameter pass and the exchange are cut into "
                         "(0 = by the number of GPUs: 4 up to two, 2 up to four, else 1)")
    ap.add_argument("--workload", default="linear", choices=["linear", "resnet18", "cnn", "mlp"],
                    help="linear: the benchmark line (Linear micro-benchmark + ResNet-18 leg); resnet18 / cnn / mlp: only one "
                         "training step of the ResNet-18, CIFAR-shaped CNN or deep regression MLP configuration through the "
                         "device-side mirror")
    ap.add_argument("--graph", action="store_true",
                    help="network workloads on one GPU: replay the training step as a CUDA graph")
    ap.add_argument("--engine", default="native", choices=["native", "dropin", "stock"],
                    help="resnet18: native = this repository's device-side mirror; dropin / stock = cuTAGI's own module "
                         "with / without this library's Linear and Conv2d kernels")
    ap.add_argument("--act", default="relu", choices=["relu", "mrelu"],
                    help="resnet18 (native engine): ReLU as in the reference's C++ test or MixtureReLU as in its Python example")
    ap.add_argument("--image", type=int, default=224, help="resnet18: image extent (224 or a multiple of 8 such as 32)")
    ap.add_argument("--batch", type=int, default=0, help="network workloads: samples per GPU (default: the configuration's)")
    ap.add_argument("--bucket-mb", type=int, default=32, help="resnet18: exchange bucket size in MiB")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")

    def with_group(fn):
        """One NCCL process group for the whole invocation (N > 1)."""
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        try:
            return fn()
        finally:
            if world > 1:
                dist.destroy_process_group()

    if args.impl == "reference":
        return run_reference(args, rank)
    if args.workload != "linear":
        if args.engine != "native":
            if args.workload != "resnet18":
                ap.error("--engine dropin / stock is available for the linear and resnet18 workloads")
            args.batch = args.batch or 64
            args.steps = min(args.steps, 3)
            return run_resnet_module(args)
        args.steps = min(args.steps, 50) if args.steps != 20 else 10
        args.warmup = 1 if args.profile else max(args.warmup, 3)
        args.no_cpu = args.no_cpu or args.profile
        line = with_group(lambda: run_network(args, rank, world, local_rank))
        if line is not None:
            print(json.dumps(line))
        return
    if args.engine != "native":
        args.steps = min(args.steps, 20)
        return run_linear_module(args)
    if args.conv_layers:
        args.steps = min(args.steps, 20)
        return run_conv_layers(args)
    if args.profile:
        args.warmup, args.no_cpu, args.no_resnet = 1, True, True
    else:
        args.warmup = max(args.warmup, 3)

    def both():
        line = run_b200(args, rank, world, local_rank)
        if not args.no_resnet:
            # the second half of the metric: ResNet-18 training samples/s on the same ranks
            ra = argparse.Namespace(**vars(args))
            ra.workload, ra.steps, ra.warmup, ra.no_cpu, ra.graph, ra.batch, ra.image = \
                "resnet18", args.resnet_steps, 3, True, False, 0, 224
            rn = run_network(ra, rank, world, local_rank)
            if line is not None and rn is not None:
                line["resnet18"] = {
                    "metric": rn["metric"], "samples_per_s": rn["value"], "ms_per_step": rn["ms_per_step"],
                    "steps": rn["steps"], "samples_per_gpu": 64, "workload": rn["config"]["workload"],
                    "e2e": rn["e2e"], "exchange": rn["exchange"] if world > 1 else "none (1 GPU)",
                    "roofline_frac": rn["roofline"]["frac"], "roofline": rn["roofline"], "clocks": rn["clocks"],
                    "gpu_launches": rn["gpu_launches"], "tc_status": rn["tc_status"]}
        return line
    line = with_group(both)
    if line is not None:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
