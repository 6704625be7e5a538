"""Benchmark of the AR sampling hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision bf16|fp32]
                    [--no-cpu-baseline] [--no-scaleout]

Workload ("config3"): the 6-layer d_model 192 / 6 heads / MLP 768 model, random
init with Xavier-uniform Linear weights rounded to bf16-representable values, one
synthetic dataset of 1024 context rows x 20 features (tanh-MLP generator), 128
target rows decoded autoregressively by 512 sample streams that share one context
KV cache (synthetic.py builds the model and the rows; the parity tests use the same).
One "step" is one complete ``sample_sequence`` call (prefill + 128 decode steps +
samples and log densities).  With N GPUs every rank runs its own 512 streams (weak
scaling: streams are independent, the context KV is prefilled locally on every rank)
and the results are gathered with NCCL at the end of each step
(``ar_tabpfn.sharding.sharded_call``).

Metric: AR targets decoded per second, whole job.
  value : inputs and pre-drawn variates already resident in HBM;
  e2e   : through the public predictor API with pinned HOST inputs (the predictor copies
          what the path reads inside the timed region: the shared context once, every
          stream's targets), random numbers drawn inside the call, samples and log
          densities read back to the host (D2H inside the timed region).
  scaleout : the scale-out configuration ("config5": 16384 context rows x 100 features,
          256 targets, 4096 sample streams in total) split evenly over the N ranks
          (strong scaling), a few steps after the headline measurement.

``--impl reference`` times the reference's own CPU path on the host cores, on a bounded
sample of the same workload: the unmodified reference package when it is installed under
``baseline/_ref`` (imported under an alias, CUDA hidden from that process so that it takes
the CPU route), otherwise the CPU restatement of its algorithm (the oracle).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ar-nanotabpfn_b200"))

import torch  # noqa: E402

import synthetic as syn  # noqa: E402

CFG = dict(syn.MODEL_6L, num_features=syn.CONFIG3["num_features"])
NC, NT, STREAMS, SEED = syn.CONFIG3["n_ctx"], syn.CONFIG3["n_targets"], syn.CONFIG3["streams"], syn.CONFIG3["seed"]
# DRAM bytes (read + write) of one 1024-row decode-step launch of the tensor-core dense chain: a constant
# taken from one ncu capture of that kernel (dram__bytes_read.sum + dram__bytes_write.sum), not measured
# in this run; the weight tiles dominate it
DENSE_TC_DRAM_BYTES_PER_LAUNCH = 3.68e6
CPU_SAMPLE = dict(streams=128, targets=16)  # bounded CPU sample of the same workload
WORKLOAD_CONFIG = {"workload": "config3: 6L d192 h6 ff768, ctx 1024x20, 128 targets, 512 streams/GPU, "
                               "shared context KV, prefill included in every step",
                   "streams_per_gpu": STREAMS, "targets": NT, "context_rows": NC,
                   "l2": "256 MB buffer written between timed iterations; KV working set 288 MiB > L2"}
SCALEOUT = dict(streams=syn.CONFIG5["streams"], targets=syn.CONFIG5["n_targets"], ctx=syn.CONFIG5["n_ctx"])


def build_model():
    return syn.config3_model()


def workload(streams, n_targets=None):
    return syn.config3_workload(streams, n_targets)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            sm.sort()
            self.result = {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                           "samples": len(sm)}


def _cpu_sample_inputs():
    B, Nt = CPU_SAMPLE["streams"], CPU_SAMPLE["targets"]
    xc, yc, xt = workload(B, Nt)
    return B, Nt, xc, yc, xt


def _time_calls(fn, steps, warmup):
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        fn()
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return sum(times) / len(times)


def cpu_port_rate(steps, warmup):
    """targets/s of the CPU restatement of the reference (the oracle) on the bounded sample."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import artab_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m = build_model()
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    B, Nt, xc, yc, xt = _cpu_sample_inputs()
    expo, normal = orc.draw_variates(SEED, Nt, B, CFG["num_components"])
    pred = orc.OraclePredictor(sd, CFG["n_heads"])
    with torch.no_grad():
        per = _time_calls(lambda: pred.sample_sequence(xc, yc, xt, expo, normal, shared=True), steps, warmup)
    sample = (f"{B} streams x {Nt} targets of config3 (context {NC} rows, same model), full prefill + decode, "
              f"CPU restatement of the reference (oracle), torch CPU fp32, {cores} threads, "
              f"{steps} timed calls after {warmup} warm-up")
    return {"value": B * Nt / per, "unit": "targets/s", "cores": cores, "kind": "port", "sample": sample}, per


def cpu_reference_rate(steps, warmup):
    """targets/s of the UNMODIFIED reference package (baseline/_ref/ar_tabpfn, imported under an
    alias) on the bounded sample: ARTabPFNPredictor(backend="triton_shared_context") on CPU tensors,
    which takes the reference's eager pytorch_context_attention route.  Raises when the package is
    not there or does not run."""
    import importlib
    import types
    root = os.path.join(ROOT, "baseline", "_ref", "ar_tabpfn")
    if not os.path.isdir(root):
        raise FileNotFoundError("baseline/_ref/ar_tabpfn is not installed")
    pkg = types.ModuleType("ref_ar_tabpfn")
    pkg.__path__ = [root]
    sys.modules["ref_ar_tabpfn"] = pkg
    ref = importlib.import_module("ref_ar_tabpfn.model")
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ours = build_model()
    m = ref.ARTabPFN(**CFG).eval()
    m.load_state_dict(ours.state_dict())
    m = m.cpu().float()
    pred = ref.ARTabPFNPredictor.from_trained_model(m, backend="triton_shared_context")
    B, Nt, xc, yc, xt = _cpu_sample_inputs()
    torch.manual_seed(SEED)
    with torch.no_grad():
        per = _time_calls(lambda: pred.sample_sequence(xc, yc, xt), steps, warmup)
    sample = (f"{B} streams x {Nt} targets of config3 (context {NC} rows, same weights), full prefill + decode, "
              f"the reference package itself (triton_shared_context backend on CPU tensors = its eager path), "
              f"torch CPU fp32, {cores} threads, {steps} timed calls after {warmup} warm-up")
    return {"value": B * Nt / per, "unit": "targets/s", "cores": cores, "kind": "reference", "sample": sample}, per


def cpu_baseline(steps, warmup, allow_reference=True):
    """(cpu_baseline dict, seconds per call): the reference itself when it runs here, else the port."""
    why = None
    if allow_reference:
        try:
            return cpu_reference_rate(steps, warmup)
        except Exception as e:  # noqa: BLE001  (any failure of the foreign package falls back to the port)
            why = f"{type(e).__name__}: {e}"[:200]
    base, per = cpu_port_rate(steps, warmup)
    if why:
        base["sample"] += f"; reference package not used ({why})"
    return base, per


def cpu_baseline_child(steps=3):
    """The reference arm in a child process with the GPUs hidden; returns its cpu_baseline object."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", ARTAB_REF_CHILD="1", RANK="0", WORLD_SIZE="1")
    out = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(steps)],
                         env=env, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    for ln in reversed(out.stdout.strip().splitlines()):
        if ln.startswith("{"):
            return json.loads(ln)["cpu_baseline"]
    raise RuntimeError("the CPU baseline child printed no JSON line (exit code %d)" % out.returncode)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # The reference decides between its Triton and its eager route by looking for CUDA: hide the GPUs
    # from this arm (a child process, because torch is already imported here) so that it times the CPU path.
    if os.environ.get("ARTAB_REF_CHILD") != "1" and os.environ.get("CUDA_VISIBLE_DEVICES", None) != "":
        env = dict(os.environ, CUDA_VISIBLE_DEVICES="", ARTAB_REF_CHILD="1")
        raise SystemExit(subprocess.call([sys.executable, os.path.abspath(__file__)] + sys.argv[1:], env=env))
    steps, warmup = max(1, min(args.steps, 3)), 1
    base, per = cpu_baseline(steps, warmup)
    cfg = dict(WORKLOAD_CONFIG)
    cfg["workload"] = ("config3 BOUNDED CPU SAMPLE: %d streams x %d targets of the %d x %d job, same model and context"
                       % (CPU_SAMPLE["streams"], CPU_SAMPLE["targets"], STREAMS, NT))
    cfg["streams_per_gpu"], cfg["targets"] = CPU_SAMPLE["streams"], CPU_SAMPLE["targets"]
    cfg["l2"] = "n/a (host cores)"
    line = {
        "impl": "reference", "metric": "ar_targets_decoded_per_sec", "value": base["value"], "unit": "targets/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": per * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg, "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "targets/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_scaleout(dev, world, rank, precision, steps=2, warmup=1):
    """The scale-out configuration (4096 sample streams over a 16384-row x 100-feature shared context,
    256 targets) split evenly over the ranks: strong scaling, every rank prefills the context locally,
    samples and log densities gathered with NCCL.  Returns the dict printed under "scaleout"."""
    import torch.distributed as dist
    import ar_tabpfn
    from ar_tabpfn.sharding import sharded_call, shard_bounds
    B, Nt, Nc = SCALEOUT["streams"], SCALEOUT["targets"], SCALEOUT["ctx"]
    model = syn.config5_model().to(dev)
    pred = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="triton_shared_context", precision=precision)
    xcr, ycr, xtr, _ = (t.to(dev) for t in syn.config5_rows())
    # one dataset repeated over the streams: stride-0 views describe the whole job without copies
    full = (xcr.expand(B, -1, -1), ycr.expand(B, -1), xtr.expand(B, -1, -1))
    expo, normal = syn.variates(syn.CONFIG5["seed"], Nt, B, CFG["num_components"], dev)

    def run_shard(xc_s, yc_s, xt_s, expo_s, normal_s):
        ys = pred.sample_sequence(xc_s, yc_s, xt_s, variates=(expo_s, normal_s))
        return ys, pred.last_logdens

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = None
    for _ in range(warmup):
        out = sharded_call(run_shard, full, variates=(expo, normal))
    sync()
    evs = []
    with ClockSampler(dev.index if dev.index is not None else 0) as clk:   # this rank's GPU, during the timed calls
        for _ in range(steps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = sharded_call(run_shard, full, variates=(expo, normal))
            e.record()
            evs.append((s, e))
        sync()
    ms = torch.tensor([sum(s.elapsed_time(e) for s, e in evs) / steps], device=dev, dtype=torch.float64)
    # the context prefill alone (it is repeated on every rank and does not shrink with N)
    lo, hi = shard_bounds(B, world, rank)
    pred.init_kv_cache(hi - lo, Nt, dev, torch.float32)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    pred.prefill_context(full[0][lo:hi], full[1][lo:hi])
    e.record()
    torch.cuda.synchronize()
    pre = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(pre, op=dist.ReduceOp.MAX)
    ys, ld = out
    return {"workload": "config5: 6L d192 h6 ff768, shared context 16384x100, 256 targets, 4096 streams in total "
                        "split evenly over the GPUs, context prefilled locally on every rank, results gathered",
            "streams_total": B, "streams_per_gpu": B // world, "targets": Nt, "context_rows": Nc, "n_gpus": world,
            "scaling": "strong", "steps": steps, "warmup": warmup, "ms_per_step": float(ms.item()),
            "targets_per_s": B * Nt / (float(ms.item()) * 1e-3), "prefill_ms": float(pre.item()),
            "finite": bool(torch.isfinite(ys).all() and torch.isfinite(ld).all()),
            "device_status": int(pred._bufs["status"].item()), "clocks": clk.result}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-scaleout", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    import ar_tabpfn
    from ar_tabpfn import _lib
    from ar_tabpfn.sharding import sharded_call

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.lib()

    model = build_model().to(dev)
    pred = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="triton_shared_context",
                                                          precision=args.precision)
    K = CFG["num_components"]
    # Full-job tensors, stream axis first, as sharded_call wants them: every rank holds the whole job's
    # inputs and variates and decodes its own slice, so the results do not depend on N.
    job = world * STREAMS
    full_h = tuple(t.pin_memory() for t in workload(job))
    full = tuple(t.to(dev) for t in full_h)
    expo, normal = syn.variates(SEED, NT, job, K, dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    def run_shard(xc_s, yc_s, xt_s, expo_s, normal_s):
        ys = pred.sample_sequence(xc_s, yc_s, xt_s, variates=(expo_s, normal_s))
        return ys, pred.last_logdens

    def step_device():
        return sharded_call(run_shard, full, variates=(expo, normal))

    out_h = [torch.empty(STREAMS, NT).pin_memory() for _ in range(2)]

    e2e_bytes = {"h2d": 0}

    lo = rank * STREAMS

    def run_shard_host(xc_s, yc_s, xt_s):
        # pinned host tensors: the predictor copies what the path reads and draws its own random numbers
        ys = pred.sample_sequence(xc_s, yc_s, xt_s)
        e2e_bytes["h2d"] = pred.last_h2d_bytes
        return ys, pred.last_logdens

    def step_e2e():
        ys, ld = sharded_call(run_shard_host, full_h)
        out_h[0].copy_(ys[lo:lo + STREAMS], non_blocking=True)
        out_h[1].copy_(ld[lo:lo + STREAMS], non_blocking=True)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        lib.artab_launch_count_reset()
        evs = []
        for _ in range(steps):
            flush.zero_()  # evict L2 between timed iterations (not timed)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            evs.append((s, e))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        total = torch.tensor([sum(s.elapsed_time(e) for s, e in evs)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(total, op=dist.ReduceOp.MAX)
        return float(total.item()) / steps, int(lib.artab_launch_count())

    with ClockSampler(local) as clk:
        ms_dev, launches = timed(step_device, args.steps, args.warmup)
        ms_e2e, _ = timed(step_e2e, max(2, args.steps // 2), 1)
    targets = world * STREAMS * NT

    # one extra step with per-launch CUDA events on the launching stream: per-kernel durations
    lib.artab_profile_enable(1)
    step_device()
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    lib.artab_profile_enable(0)
    status = int(pred._bufs["status"].item()) if "status" in pred._bufs else 0
    scaleout = None
    if not args.no_scaleout:
        del flush
        torch.cuda.empty_cache()
        scaleout = run_scaleout(dev, world, rank, args.precision)

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        total_ms = sum(v[0] for v in prof.values()) or 1.0
        shares = {k: {"ms": round(v[0], 3), "launches": v[1], "share": round(v[0] / total_ms, 3)}
                  for k, v in prof.items() if v[1]}
        dom = max(shares, key=lambda k: shares[k]["ms"])
        D, Dff, L, H = CFG["d_model"], CFG["d_ff"], CFG["n_layers"], CFG["n_heads"]
        rows_run = STREAMS * (1 + 2 * (NT - 1)) + NC          # token rows through the layer chain per call
        roof = None
        if dom == "dense_chain":
            # algorithmic flops of the per-token chain: Wf (folded feature attention), Wq|Wk|Wv, Wo and
            # the two MLP matrices, 2 flops per multiply-add; the hi/lo operand split that the bf16
            # tensor-core chain issues (2x the MMAs) is not counted
            flops = rows_run * L * (10 * D * D + 4 * D * Dff) * 1.0
            peak = peaks.get("bf16_tflops_sustained", 1400.0)
            ach = flops / (shares[dom]["ms"] * 1e-3) / 1e12
            tc = args.precision == "bf16"
            roof = {"kernel": "dense_tc_kernel" if tc else "dense_chain_kernel", "bound": "tensor",
                    "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                    "traffic": DENSE_TC_DRAM_BYTES_PER_LAUNCH if tc else None,
                    "traffic_source": "constant: DRAM bytes of one 1024-row decode launch in an ncu capture, "
                                      "not measured in this run" if tc else None,
                    "peak_source": "measured" if peaks else "fallback",
                    "note": ("tcgen05 chain, 8 row tiles of 128 rows per decode launch: bound by the latency of the "
                             "dependent GEMM / LayerNorm chain of a row tile, not by the tensor pipe"
                             if tc else "fp32 FMA kernel measured against the bf16 tensor peak")}
        elif dom == "context_attention":
            q_rows = STREAMS * (1 + 2 * (NT - 1)) + NC
            flops = 4.0 * 32 * NC * q_rows * H * L
            peak = peaks.get("bf16_tflops_sustained", 1400.0)
            ach = flops / (shares[dom]["ms"] * 1e-3) / 1e12
            roof = {"kernel": "ctx_attn_tc_kernel", "bound": "tensor", "achieved": ach, "peak": peak,
                    "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                    "peak_source": "measured" if peaks else "fallback"}
        else:
            esz = 2 if args.precision == "bf16" else 4
            byts = sum(range(1, NT)) * STREAMS * H * 32 * 2 * esz * L * 1.0
            peak = peaks.get("hbm_gbs", 6650.0)
            ach = byts / (shares[dom]["ms"] * 1e-3) / 1e9
            roof = {"kernel": "buf_mma_kernel" if args.precision == "bf16" else "buf_merge_kernel", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "traffic": None, "peak_source": "measured" if peaks else "fallback"}
        line = {
            "metric": "ar_targets_decoded_per_sec", "value": targets / (ms_dev * 1e-3), "unit": "targets/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if args.precision == "bf16" else "f32", "data": "synthetic",
            "config": WORKLOAD_CONFIG,
            "e2e": {"value": targets / (ms_e2e * 1e-3), "unit": "targets/s",
                    "h2d_bytes_per_step": int(e2e_bytes["h2d"]),
                    "d2h_bytes_per_step": 2 * STREAMS * NT * 4, "ms_per_step": ms_e2e},
            "gpu_launches": launches, "clocks": clk.result, "roofline": roof, "kernel_shares": shares,
            "device_status": status,
        }
        if scaleout is not None:
            line["scaleout"] = scaleout
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline_child()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
