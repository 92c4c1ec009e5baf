"""Benchmark of the pi0.5 action-chunk engine on N GPUs of one node.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's eager path on the box's host cores
    python bench.py --impl reference-gpu ...  # the reference's own CUDA megakernel arm on the same GPU (one GPU only)

One "step" is one whole action chunk (10 Euler steps x 18 layers, B=1, prefix 128) = one kernel launch.
The L2 is flushed (a 2x-L2 zero fill) before every timed chunk and each chunk is timed with CUDA events on
the launching stream, as the reference harness does for its "isolated" number (bench.py:259-293 there).
With N > 1 every rank runs its own observation on its own GPU with replicated weights and no collective in
the data path; the reported time is the maximum over ranks.  Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from pi05_megakernel_b200 import dp as DP  # noqa: E402
from pi05_megakernel_b200 import fixture as FX  # noqa: E402

METRIC = "action chunks/sec, whole box (B=1 per GPU, prefix 128, L2 flushed before every chunk)"
UNIT = "chunks/s"
SOTA_GRAPH_MS = 6.73      # the reference's best published arm on one B200 (README.md:24 there)
HBM_NOMINAL = 8.0e12


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def ncu_traffic(batch: int, prefix: int) -> float | None:
    """DRAM bytes per launch from the committed ncu summary of this workload (None where none was captured)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            for rec in json.load(f).get("captures", []):
                # a capture of another build of the kernel than the one this run launches is not this run's traffic
                if rec.get("batch") == batch and rec.get("prefix") == prefix and rec.get("matches_default_build"):
                    return rec.get("dram_bytes_per_launch")
    return None


class ClockSampler:
    """nvidia-smi clock / throttle sampling during the timed region."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def stage_times(arm, flush) -> None:
    """One stamped chunk: globaltimer values written by the kernel at stage boundaries (row CTA 0) and at the
    pipeline points of three GEMM CTAs in the second layer pass; printed as microseconds since kernel start."""
    arm.enable_stamps(True)
    flush.zero_()
    arm.launch()
    arm.status()
    st = arm.stamps.cpu().tolist()
    arm.enable_stamps(False)
    us = lambda x: round((x - st[0]) / 1e3, 2) if x else None
    out = {"prologue_us": {n: us(st[i]) for i, n in enumerate(
        ["start", "tables", "time_mlp_in", "time_mlp_out", "modulation", "first_norm"])}}
    names = ["qkv_seen", "attention_done", "o_seen", "residual_norm_1_done", None, "down_seen", "residual_norm_2_done"]
    for ps in range(1, 4):
        out[f"pass{ps}_us"] = {n: us(st[6 + 7 * ps + i]) for i, n in enumerate(names) if n}
    pts = ["inputs_seen", "acts_issued", "first_operands", "mma_issued", "acc_ready", "acc_in_regs", "stored", "signalled"]
    for which, cta in enumerate(["cta0", "cta64", "cta84"]):
        for g, gn in enumerate(["qkv", "o", "gate_up", "down"]):
            row = st[64 + 64 * which + g * 8: 64 + 64 * which + g * 8 + 8]
            if any(row):
                out[f"{cta}_{gn}_pass1_us"] = {pt: us(x) for pt, x in zip(pts, row)}
    out["row_cta0_attention_pass1_us"] = {n: us(st[224 + i]) for i, n in enumerate(
        ["prefix_landed", "scores_done", "softmax_done", "pv_done", "stored", "signalled"])}
    print("stage_times " + json.dumps(out), file=sys.stderr, flush=True)
    print(stage_table(out, arm.geo.prefix), file=sys.stderr, flush=True)


def stage_table(t: dict, prefix: int) -> str:
    """The seven stages of one layer pass (pass 1 of the stamped chunk) as a table: time, weight / cache bytes the stage
    streams from HBM, achieved GB/s against the measured copy peak, and for the four GEMM stages the useful tensor
    work against the measured BF16 peak (with the figure for the padded N = 64 MMAs beside it) and the share of the
    stage during which the stamped CTA was issuing MMAs."""
    peak_gbs, _ = measured_peaks()
    peak_tf = 1672.7
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak_tf = float(json.load(f).get("bf16_tflops", peak_tf))
    p0, p1 = t["pass1_us"], t["pass2_us"]
    gu, q = t.get("cta0_gate_up_pass1_us", {}), t.get("cta0_qkv_pass1_us", {})
    W, QD, HD, FF, T = 1024, 2048, 256, 4096, 50
    rows = {"QKV projection": (QD + 2 * HD, W), "O projection": (W, QD), "gate/up projection + GeGLU": (2 * FF, W),
            "down projection": (W, FF)}
    # stage boundaries as row CTA 0 and GEMM CTA 0 saw them; the QKV stage of pass 2 starts where pass 1 ended
    spans = [("QKV projection", p0["residual_norm_2_done"], p1["qkv_seen"], "cta0_qkv_pass1_us"),
             ("attention", p0["qkv_seen"], p0["attention_done"], None),
             ("O projection", p0["attention_done"], p0["o_seen"], "cta0_o_pass1_us"),
             ("gated residual + adaRMS", p0["o_seen"], p0["residual_norm_1_done"], None),
             ("gate/up projection + GeGLU", p0["residual_norm_1_done"], gu.get("signalled"), "cta0_gate_up_pass1_us"),
             ("down projection", gu.get("signalled"), p0["down_seen"], "cta0_down_pass1_us"),
             ("gated residual + adaRMS (next norm)", p0["down_seen"], p0["residual_norm_2_done"], None)]
    lines = ["| stage | us | HBM bytes | GB/s | of measured HBM peak | useful TFLOP/s (padded N=64) | of measured BF16 peak | MMA issue share of the stage |",
             "|---|---|---|---|---|---|---|---|"]
    total_us = total_b = 0.0
    for name, a, b, cta in spans:
        if a is None or b is None:
            continue
        us = b - a
        if name in rows:
            r, k = rows[name]
            nbytes, flops = r * k * 2, 2.0 * T * r * k
        elif name == "attention":
            nbytes, flops = prefix * HD * 2 * 2, 4.0 * T * QD * (prefix + T)
        else:
            nbytes, flops = 2 * 3 * W * 4, 0.0
        gbs = nbytes / us / 1e3
        tf = flops / us / 1e6
        share = ""
        if cta and cta in t and t[cta].get("first_operands") and t[cta].get("mma_issued"):
            share = f"{100 * (t[cta]['mma_issued'] - t[cta]['first_operands']) / us:.0f} %"
        tcol = f"{tf:.1f} ({tf * 64 / T:.1f})" if name in rows else (f"{tf:.1f} (warp MMA)" if flops else "-")
        lines.append(f"| {name} | {us:.2f} | {int(nbytes):,} | {gbs:.0f} | {100 * gbs / peak_gbs:.1f} % | {tcol} | "
                     f"{(str(round(100 * tf / peak_tf, 2)) + ' %') if name in rows else '-'} | {share or '-'} |")
        total_us += us
        total_b += nbytes
    lines.append(f"| one layer pass | {total_us:.2f} | {int(total_b):,} | {total_b / total_us / 1e3:.0f} | "
                 f"{100 * total_b / total_us / 1e3 / peak_gbs:.1f} % | - | - | - |")
    return "stage_table\n" + "\n".join(lines)


def batch_sweep(args, device) -> None:
    """A/B aid: ms per launch for several per-GPU batch sizes in one process (weights made once, L2 flushed before
    every launch, CUDA events), one compact JSON line per batch size.  The engine's tuning variables (PI05_*) are read
    from the environment when each engine is created, so two runs of this command under different settings on the
    same box are an A/B pair."""
    from pi05_megakernel_b200.arm import Pi05Arm
    geo = FX.Geometry(prefix=args.prefix)
    weights = {k: v.to(device) for k, v in FX.make_weights(geo, FX.SEEDS[0]).items()}
    flush = torch.empty(2 * torch.cuda.get_device_properties(device).L2_cache_size, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)
    for B in [int(x) for x in args.batches.split(",")]:
        obs = [FX.make_observation(geo, DP.observation_seed(FX.SEEDS[0], 0, i), args.mask) for i in range(B)]
        dev = dict(weights)
        for k in FX.ORDER:
            if k not in weights:
                dev[k] = (obs[0][k] if B == 1 else torch.stack([o[k] for o in obs]).contiguous()).to(device)
        arm = Pi05Arm(geo, "b200", str(device), batch=B)
        arm.bind(dev)
        times = []
        for i in range(max(3, args.warmup) + args.steps):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            arm.launch()
            b.record(stream)
            torch.cuda.synchronize(device)
            if i >= max(3, args.warmup):
                times.append(a.elapsed_time(b))
        arm.status()
        ms = sum(times) / len(times)
        print(json.dumps({"batch": B, "ms_per_launch": round(ms, 3), "ms_per_chunk": round(ms / B, 3),
                          "chunks_per_s": round(1e3 * B / ms, 1), "schedule": arm.config.get("schedule"),
                          "observations_per_mma": arm.config.get("observations_per_mma"),
                          "gemm_ctas": arm.config.get("gemm_ctas")}), flush=True)
        arm.close()


def cpu_chunks_per_sec(geo, inputs_cpu, runs: int) -> tuple[float, int, str]:
    """Whole chunks per second of the eager BF16 path on the host cores: the reference's own code when it is installed
    beside this file ("reference"), else the CPU oracle's restatement of it ("port")."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    RFX = reference_package()
    if RFX is not None:
        rgeo = RFX.Geometry(prefix=geo.prefix)
        chunk, kind = (lambda: RFX.reference(rgeo, inputs_cpu)["actions"]), "reference"
    else:
        from oracle import pi05_oracle as O
        ogeo = O.Geo(prefix=geo.prefix)
        chunk, kind = (lambda: O.chunk(inputs_cpu, ogeo, False)), "port"
    chunk()      # warm the thread pool
    t0 = time.perf_counter()
    for _ in range(runs):
        chunk()
    return runs / (time.perf_counter() - t0), torch.get_num_threads(), kind


REF_ROOT = os.path.join(ROOT, "baseline", "_ref")


def reference_package():
    """The unmodified reference as ``baseline/install_reference.py`` lays it out (``baseline/_ref``, not part of the
    history; absent on calls that leave the folder behind).  Returns its ``fixture`` module or None."""
    if not os.path.isfile(os.path.join(REF_ROOT, "megabench", "sota", "pi05", "fixture.py")):
        return None
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(REF_ROOT, "torch_ext"))
    from megabench.sota.pi05 import fixture as RFX
    return RFX


def run_reference(args, rank: int) -> None:
    """The reference's own eager BF16 path (reference/pi05.py::reference through its fixture.reference) on all host
    cores when the reference is installed beside this file, otherwise the CPU oracle's restatement of it."""
    if rank != 0:
        return
    geo = FX.Geometry(prefix=args.prefix)
    cpu = FX.make_inputs(geo, FX.SEEDS[0], "cpu")
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    RFX = reference_package()
    if RFX is not None:
        rgeo = RFX.Geometry(prefix=geo.prefix)
        chunk = lambda: RFX.reference(rgeo, cpu)["actions"]
        kind, what = "reference", "reference/pi05.py::reference, unmodified, on the host cores"
    else:
        from oracle import pi05_oracle as O
        ogeo = O.Geo(prefix=geo.prefix)
        chunk = lambda: O.chunk(cpu, ogeo, False)
        kind, what = "port", "eager CPU path, BF16 rounding schedule of the reference (the reference is not installed here)"
    steps, warm = max(1, min(args.steps, 30)), max(1, min(args.warmup, 10))     # bounded: about a second per chunk
    for _ in range(warm):
        chunk()
    t0 = time.perf_counter()
    for _ in range(steps):
        chunk()
    dt = (time.perf_counter() - t0) / steps
    value = 1.0 / dt
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"pi0.5 action chunk, B=1, prefix {geo.prefix}, 10 steps x 18 layers ({what})"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"{steps} whole chunks (each step is one full chunk)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_reference_gpu(args, rank: int, world: int) -> None:
    """The reference's CUDA megakernel arm (megakernel.py:117-186 there: MegakernelArm(geo, variant, device), bind,
    launch, outputs) on the same GPU, same inputs, same L2-flushed event timing, checked against the same band.
    One GPU only: the folder that holds the reference stays behind on calls of two or more GPUs."""
    if rank != 0:
        return
    def unavailable(why: str) -> None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": why}), flush=True)
    if world > 1:
        return unavailable("one GPU only")
    RFX = reference_package()
    if RFX is None:
        return unavailable("the reference is not installed under baseline/_ref (baseline/install_reference.py)")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    from megabench.sota.pi05 import megakernel as MK
    from oracle import pi05_oracle as O
    geo = FX.Geometry(prefix=args.prefix)
    variant = args.ref_variant or ("k64" if geo.prefix == 968 else "k16-nofgu")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    cpu = FX.make_inputs(geo, FX.SEEDS[0], "cpu")
    dev = {k: v.to(device) for k, v in cpu.items()}
    t0 = time.time()
    try:
        arm = MK.MegakernelArm(RFX.Geometry(prefix=geo.prefix), variant, str(device))
    except Exception as e:  # noqa: BLE001
        return unavailable(f"build or set-up of {variant} failed: {type(e).__name__}: {str(e)[-300:]}")
    build_s = time.time() - t0
    arm.bind(dev)
    flush = torch.empty(2 * torch.cuda.get_device_properties(device).L2_cache_size, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)
    warm = max(3, args.warmup)
    times = []
    sampler = ClockSampler(0)
    for i in range(warm + args.steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        arm.launch()
        b.record(stream)
        torch.cuda.synchronize(device)
        if i >= warm:
            times.append(a.elapsed_time(b))
    clocks = sampler.stop()
    got = arm.outputs()["actions"].cpu()
    ogeo = O.Geo(prefix=geo.prefix)
    d = O.band(O.chunk(cpu, ogeo, False), got, O.chunk(cpu, ogeo, True))
    ms = sum(times) / len(times)
    print(json.dumps({
        "impl": "reference-gpu", "metric": METRIC, "value": 1e3 / ms, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "ms_per_launch_median": statistics.median(times), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"pi0.5 action chunk, B=1, prefix {geo.prefix}, 10 steps x 18 layers: the reference's "
                               f"MegakernelArm variant {variant}, unmodified", "engine": arm.config,
                   "l2": "flushed before every timed chunk (2x L2 zero fill)", "build_or_load_seconds": round(build_s, 1)},
        "parity": {"pass": bool(d["pass"]), "relative_error": d["relative_error"],
                   "reference_relative_error": d["reference_relative_error"]},
        "clocks": clocks,
    }), flush=True)


def run_tensor_parallel(args, rank: int, local: int, world: int) -> int:
    """BASELINE config 5: ONE observation shared by the `world` GPUs of the launch (query heads and MLP columns cut
    across the ranks, partial sums exchanged inside the kernel over NVLink).  Reports the latency of one chunk (slowest
    rank, L2 flushed, ranks lined up before every chunk) next to nothing else: compare with the one-GPU line."""
    import torch.distributed as dist
    from pi05_megakernel_b200.arm import Pi05Arm
    if world < 2:
        print(json.dumps({"impl": "b200-tp", "unavailable": "tensor parallel needs 2, 4 or 8 ranks (torchrun)"}), flush=True)
        return 0
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    geo = FX.Geometry(prefix=args.prefix)
    weights = FX.make_weights(geo, FX.SEEDS[0])
    obs = FX.make_observation(geo, DP.observation_seed(FX.SEEDS[0], 0, 0), args.mask)      # the same one on every rank
    cpu = {**weights, **obs}
    arm = Pi05Arm(geo, "b200", str(device), tp=(rank, world))
    arm.bind({k: cpu[k].to(device) for k in FX.ORDER})
    arm.tp_attach_all()
    flush = torch.empty(2 * torch.cuda.get_device_properties(device).L2_cache_size, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)
    warm, times = max(3, args.warmup), []
    sampler = ClockSampler(local) if rank == 0 else None
    for i in range(warm + args.steps):
        flush.zero_()
        dist.barrier()                       # on the stream: the ranks' kernels start together
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        arm.launch()
        b.record(stream)
        torch.cuda.synchronize(device)
        if i >= warm:
            times.append(a.elapsed_time(b))
    arm.status()
    clocks = sampler.stop() if sampler else None
    ms = DP.max_over_ranks([sum(times) / len(times)], device)[0]
    parity = None
    if not args.no_parity:
        parity = parity_check(arm, geo, weights, [obs], 1, rank, world)
        parity["all_ranks_pass"] = DP.max_over_ranks([0.0 if parity["pass"] else 1.0], device)[0] == 0.0
    if rank == 0:
        print(json.dumps({
            "impl": "b200-tp", "metric": "ms per action chunk, one observation across the GPUs (tensor parallel, L2 flushed)",
            "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"pi0.5 action chunk, B=1, prefix {geo.prefix} ({args.mask} mask), 10 x 18, tensor parallel "
                                   f"over {world} GPUs: heads and MLP columns cut, per-layer partial sums pushed between "
                                   "the row CTAs of the ranks with peer stores", "engine": arm.config},
            "ms_per_launch_median": statistics.median(times), "parity": parity, "clocks": clocks}), flush=True)
    arm.close()
    dist.destroy_process_group()
    return 0


def prefill_flops(tokens: int, layers: int = 18) -> float:
    """Matmul and attention work of the prefill (the last layer's MLP is skipped, as in the reference)."""
    h, ff, qd, kvd = 2048, 16384, 2048, 256
    per_layer_attn = 2.0 * tokens * h * (qd + 2 * kvd) + 2.0 * tokens * qd * h + 4.0 * tokens * tokens * qd
    per_layer_mlp = 2.0 * tokens * h * 2 * ff + 2.0 * tokens * ff * h
    return layers * per_layer_attn + (layers - 1) * per_layer_mlp


def run_prefill(args, rank: int) -> int:
    """The step before the action chunk: the Gemma-2B prefix prefill (reference/pi05.py:167-195) that produces the
    key / value cache, timed as one whole prefill (all its kernels) with CUDA events, L2 flushed before each."""
    if rank != 0:
        return 0
    from pi05_megakernel_b200.prefill import Pi05Prefill
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    geo = FX.PrefillGeometry(tokens=args.prefix)
    cpu = FX.make_prefill_inputs(geo, FX.SEEDS[0], "pad" if args.mask != "full" else "full")
    dev = {k: v.to(device) for k, v in cpu.items()}
    pre = Pi05Prefill(geo, str(device))
    pre.bind(dev)
    shape = (geo.layers, geo.tokens, 1, 256)
    out = (torch.zeros(shape, dtype=torch.bfloat16, device=device), torch.zeros(shape, dtype=torch.bfloat16, device=device))
    flush = torch.empty(2 * torch.cuda.get_device_properties(device).L2_cache_size, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)
    warm, times = max(3, args.warmup), []
    sampler = ClockSampler(0)
    for i in range(warm + args.steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        pre.run(dev["embeddings"], dev["valid"], out=out)
        b.record(stream)
        torch.cuda.synchronize(device)
        if i >= warm:
            times.append(a.elapsed_time(b))
    pre.status()
    clocks = sampler.stop()
    # end to end: embeddings and mask from pinned host memory, keys / values of the last layer read back
    pinned = {k: cpu[k].pin_memory() for k in ("embeddings", "valid")}
    host_k = torch.empty((geo.tokens, 256), dtype=torch.bfloat16).pin_memory()
    e2e = []
    for i in range(3 + args.steps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for k in pinned:
            dev[k].copy_(pinned[k], non_blocking=True)
        pre.run(dev["embeddings"], dev["valid"], out=out)
        host_k.copy_(out[0][geo.layers - 1, :, 0], non_blocking=True)
        b.record(stream)
        b.synchronize()
        if i >= 3:
            e2e.append(a.elapsed_time(b))
    ms, e2e_ms = sum(times) / len(times), sum(e2e) / len(e2e)
    flops = prefill_flops(geo.tokens)
    weight_bytes = sum(cpu[k].numel() * 2 for k in FX.PREFILL_WEIGHTS) - 3 * 2048 * 16384 * 2   # (last MLP not read)
    peak_tf = 1393.7
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak_tf = float(json.load(f).get("bf16_tflops_sustained", peak_tf))
    line = {
        "impl": "b200-prefill", "metric": "ms per prefix prefill (Gemma-2B, 18 layers, L2 flushed)", "value": ms, "unit": "ms",
        "n_gpus": 1, "steps": args.steps, "warmup": warm, "ms_per_step": ms, "ms_per_launch_median": statistics.median(times),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"Gemma-2B prefix-LM prefill, {geo.tokens} tokens ({'right-padded' if args.mask != 'full' else 'full'} "
                               "mask), 18 layers, hidden 2048 / 16384, 8 query heads over 1 KV head of 256; keys and values "
                               "of every layer as output", "l2": "flushed before every timed prefill (2x L2 zero fill)"},
        "gpu_launches": (3 + 4 * geo.layers + 3 * (geo.layers - 1)) * args.steps, "clocks": clocks,
        "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in pinned.values()),
                "d2h_bytes_per_step": host_k.numel() * 2},
        "roofline": {"bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": flops / (ms * 1e-3) / 1e12 / peak_tf, "peak_kind": "measured (sustained BF16 matmul)",
                     "algorithmic_flops_per_prefill": flops, "weight_bytes_per_prefill": weight_bytes, "traffic": None},
    }
    if not args.no_parity:
        from oracle import pi05_oracle as O
        torch.set_num_threads(os.cpu_count() or 1)
        t0 = time.perf_counter()
        wk, wv = O.prefill(cpu, cpu["embeddings"], cpu["valid"], 8, 1, 256)
        cpu_s = time.perf_counter() - t0
        ek, ev = O.prefill(cpu, cpu["embeddings"], cpu["valid"], 8, 1, 256, widen=True)
        rows = cpu["valid"]
        dk = O.band(wk[:, rows].float(), out[0].cpu()[:, rows].float(), ek[:, rows])
        dv = O.band(wv[:, rows].float(), out[1].cpu()[:, rows].float(), ev[:, rows])
        line["parity"] = {"pass": bool(dk["pass"] and dv["pass"]), "relative_error": max(dk["relative_error"], dv["relative_error"]),
                          "reference_relative_error": max(dk["reference_relative_error"], dv["reference_relative_error"]),
                          "checker": "band of the keys and values of the valid tokens against the CPU oracle"}
        line["cpu_baseline"] = {"value": cpu_s * 1e3, "unit": "ms", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": "one whole prefill of the same workload (eager BF16 path of the oracle)"}
    print(json.dumps(line), flush=True)
    pre.close()
    return 0


def parity_check(arm, geo, weights, obs, B: int, rank: int = 0, world: int = 1) -> dict:
    """One band check of what the timed arm left in its output buffer, against the CPU oracle (outside every timed
    region): the rank's observation, or the first and last one of its batch (reference bench.py:220-256).
    With several ranks on one host only rank 0 runs the oracle, with all host cores - every rank doing so at once
    oversubscribes the cores badly enough to take many minutes - and the other ranks check that their result is finite."""
    got = arm.outputs()["actions"].cpu()
    if rank != 0:
        return {"pass": bool(torch.isfinite(got).all()), "relative_error": 0.0, "reference_relative_error": 0.0,
                "observations": [], "checker": "finite"}
    from oracle import pi05_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    ogeo = O.Geo(prefix=geo.prefix)
    which = sorted({0, B - 1})
    out = {"pass": True, "relative_error": 0.0, "reference_relative_error": 0.0, "observations": which,
           "checker": "band against the CPU oracle (FP32 and BF16 eager), computed after the timed regions"
                      + ("" if world == 1 else "; rank 0's result, the other ranks' results checked to be finite")}
    for b in which:
        inputs = {**weights, **obs[b]}
        d = O.band(O.chunk(inputs, ogeo, False), got if B == 1 else got[b], O.chunk(inputs, ogeo, True))
        out["pass"] = out["pass"] and bool(d["pass"])
        if d["relative_error"] >= out["relative_error"]:
            out["relative_error"], out["reference_relative_error"] = d["relative_error"], d["reference_relative_error"]
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference-gpu"])
    ap.add_argument("--ref-variant", default="", help="--impl reference-gpu: the reference arm's variant string "
                                                      "(default k16-nofgu, k64 at prefix 968)")
    ap.add_argument("--no-parity", action="store_true", help="skip the band check of the timed arm's result")
    ap.add_argument("--prefill", action="store_true",
                    help="time the Gemma-2B prefix prefill (the step before the chunk) at --prefix tokens instead of the chunk")
    ap.add_argument("--tp", action="store_true",
                    help="tensor parallel: all ranks of the launch share ONE observation (latency line instead of the "
                         "data-parallel benchmark line)")
    ap.add_argument("--prefix", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1, help="independent observations per GPU per launch (1..16)")
    ap.add_argument("--mask", default="full", choices=["full", "pad", "scatter"],
                    help="prefix validity: every token valid, a right-padded prefix, or the same count of valid tokens at "
                         "random places (count uniform in [prefix/2, prefix], from the seed)")
    ap.add_argument("--kv-pages", type=int, default=0, metavar="TOKENS",
                    help="hand the prefix cache over as a pool of shuffled pages of this many tokens (a multiple of 64) "
                         "through the strided / paged view instead of dense tensors")
    ap.add_argument("--batches", default="", metavar="B1,B2,...",
                    help="A/B aid (one GPU): time these per-GPU batch sizes in one process and print one compact line each, "
                         "instead of the benchmark line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--stage-times", action="store_true",
                    help="also print (stderr) the in-kernel stage timeline of one L2-flushed chunk")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return 0
    if args.impl == "reference-gpu":
        run_reference_gpu(args, rank, world)
        return 0
    if args.tp:
        return run_tensor_parallel(args, rank, local, world)
    if args.prefill:
        return run_prefill(args, rank)
    warmup = max(3, args.warmup)

    import torch.distributed as dist
    from pi05_megakernel_b200.arm import Pi05Arm
    dist_on = world > 1
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if dist_on:
        dist.init_process_group("nccl", device_id=device)

    if args.batches:
        batch_sweep(args, device)
        return 0

    geo = FX.Geometry(prefix=args.prefix)
    B = args.batch
    weights = FX.make_weights(geo, FX.SEEDS[0])
    obs = [FX.make_observation(geo, DP.observation_seed(FX.SEEDS[0], rank, i), args.mask) for i in range(B)]  # own observations
    cpu = {k: weights[k] if k in weights else (obs[0][k] if B == 1 else torch.stack([o[k] for o in obs]).contiguous())
           for k in FX.ORDER}
    dev = {k: v.to(device) for k, v in cpu.items()}
    arm = Pi05Arm(geo, "b200", str(device), batch=B)
    pool = None
    if args.kv_pages:
        # the same keys / values scattered over a pool of pages (two spare pages, shuffled order)
        from pi05_megakernel_b200.arm import PagedPrefix
        T_ = args.kv_pages
        per = (geo.prefix + T_ - 1) // T_
        order = torch.randperm(B * per + 2, generator=torch.Generator().manual_seed(11)).tolist()
        pool = {n: torch.zeros((B * per + 2, geo.layers, T_, 1, 256), dtype=torch.bfloat16) for n in ("prefix_k", "prefix_v")}
        table = [[order[b * per + lp] for lp in range(per)] for b in range(B)]
        for n in pool:
            dense = cpu[n].reshape(B, geo.layers, geo.prefix, 1, 256)
            for b in range(B):
                for lp in range(per):
                    cnt = min(T_, geo.prefix - lp * T_)
                    pool[n][table[b][lp], :, :cnt] = dense[b, :, lp * T_:lp * T_ + cnt]
        cpu.update(pool)
        dev = {k: v.to(device) for k, v in cpu.items()}
        arm.bind({k: v for k, v in dev.items() if k not in pool},
                 kv_pages=PagedPrefix(dev["prefix_k"], dev["prefix_v"], table))
    else:
        arm.bind(dev)
    l2 = torch.cuda.get_device_properties(device).L2_cache_size
    flush = torch.empty(2 * l2, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device)

    def barrier():
        torch.cuda.synchronize(device)
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(k: int) -> list[float]:
        out = []
        for _ in range(k):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            arm.launch()
            b.record(stream)
            out.append((a, b))
        torch.cuda.synchronize(device)
        return [a.elapsed_time(b) for a, b in out]

    # ---- device-resident inputs: `value`
    timed(warmup)
    arm.status()
    launches0 = arm.launch_count()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    samples = timed(args.steps)
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = arm.launch_count() - launches0
    arm.status()
    ms_step = sum(samples) / len(samples)

    # ---- end to end through the arm with host buffers: pinned observation -> device, chunk, actions -> host
    obs_names = ("noise", "prefix_k", "prefix_v", "prefix_mask")
    pinned = {k: cpu[k].pin_memory() for k in obs_names}
    host_out = torch.empty(tuple(arm.actions.shape), dtype=torch.float32).pin_memory()
    h2d = sum(pinned[k].numel() * pinned[k].element_size() for k in obs_names)
    d2h = host_out.numel() * 4

    def e2e_step():
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for k in obs_names:
            dev[k].copy_(pinned[k], non_blocking=True)
        arm.launch()
        host_out.copy_(arm.outputs()["actions"], non_blocking=True)
        b.record(stream)
        b.synchronize()
        return a.elapsed_time(b)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_ms = [e2e_step() for _ in range(args.steps)]
    barrier()
    e2e_step_ms = sum(e2e_ms) / len(e2e_ms)

    # ---- steady: back-to-back launches without the flush (the reference harness's second number, bench.py:271-281 there)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for _ in range(args.steps):
        arm.launch()
    s1.record(stream)
    torch.cuda.synchronize(device)
    steady_ms = s0.elapsed_time(s1) / args.steps
    arm.status()

    # ---- one band check of the result the timed arm produced, outside every timed region
    parity = None
    if not args.no_parity:
        parity = parity_check(arm, geo, weights, obs, B, rank, world)
        all_pass = DP.max_over_ranks([0.0 if parity["pass"] else 1.0], device)[0] == 0.0
        parity["all_ranks_pass"] = bool(all_pass)

    ms_step, e2e_step_ms, steady_ms = DP.max_over_ranks([ms_step, e2e_step_ms, steady_ms], device)

    if rank == 0:
        peak_gbs, peak_kind = measured_peaks()
        floor = FX.sol(geo, B)
        alg_bytes = floor["bytes_restream"]
        achieved = alg_bytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": METRIC if B == 1 else METRIC.replace("B=1", f"B={B}"), "value": DP.chunks_per_second(world, ms_step, B), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (1e3 / ms_step) / (1e3 / SOTA_GRAPH_MS) if world == 1 and B == 1 else None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"pi0.5 action chunk, B={B} per GPU, prefix {geo.prefix} ({args.mask} mask), 10 Euler steps x 18 "
                                   "Gemma-300M expert layers, BF16 weights and prefix K/V, FP32 time MLP / "
                                   "modulation; one persistent kernel launch per chunk",
                       "l2": "flushed before every timed chunk (2x L2 zero fill)",
                       "prefix_cache": f"pool of shuffled {args.kv_pages}-token pages read in place" if args.kv_pages else "dense",
                       "parallelism": f"dp{world} (independent observations, replicated weights, no collective)",
                       "engine": arm.config},
            "ms_per_chunk": ms_step / B, "ms_per_launch_median": statistics.median(samples), "batch_per_gpu": B,
            "ms_per_launch_steady": steady_ms, "parity": parity,
            "reference_gpu": "not part of this command: `bench.py --impl reference-gpu` times the reference's own CUDA arm "
                             "on the same GPU (one-GPU calls only); vs_baseline divides by a figure published from another machine",
            "x_hbm_floor_nominal": ms_step / (alg_bytes / HBM_NOMINAL * 1e3),
            "x_hbm_floor_measured": ms_step / (alg_bytes / (peak_gbs * 1e9) * 1e3),
            "vs_baseline_note": f"value / (1000 / {SOTA_GRAPH_MS} ms), the reference's published sota-graph arm on one B200",
            "clocks": clocks,
            "e2e": {"value": DP.chunks_per_second(world, e2e_step_ms, B), "unit": UNIT, "ms_per_chunk": e2e_step_ms / B,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                         "frac": achieved / peak_gbs, "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": alg_bytes, "traffic": ncu_traffic(B, geo.prefix)},
        }
        if world == 1 and B == 1 and not args.no_cpu_baseline:
            cps, cores, kind = cpu_chunks_per_sec(geo, cpu, 10)
            line["cpu_baseline"] = {"value": cps, "unit": UNIT, "cores": cores, "kind": kind,
                                    "sample": "10 whole chunks of the same workload (eager BF16 path)"}
        print(json.dumps(line), flush=True)
    if args.stage_times and rank == 0:
        stage_times(arm, flush)
    arm.close()
    if dist_on:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
