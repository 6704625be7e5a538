"""Benchmark of the AR sampling hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision bf16|fp32]

Workload ("config3"): the 6-layer d_model 192 / 6 heads / MLP 768 model, random
init with Xavier-uniform Linear weights rounded to bf16-representable values, one
synthetic dataset of 1024 context rows x 20 features (tanh-MLP generator), 128
target rows decoded autoregressively by 512 sample streams that share one context
KV cache.  One "step" is one complete ``sample_sequence`` call (prefill + 128
decode steps + samples and log densities).  With N GPUs every rank runs its own
512 streams (weak scaling: streams are independent, the context KV is prefilled
locally on every rank) and the results are all-gathered with NCCL at the end of
each step.

Metric: AR targets decoded per second, whole job.
  value : inputs and pre-drawn variates already resident in HBM;
  e2e   : through the public predictor API with pinned HOST inputs (the predictor copies
          what the path reads inside the timed region: the shared context once, every
          stream's targets), random numbers drawn inside the call, samples and log
          densities read back to the host (D2H inside the timed region).

``--impl reference`` times the CPU restatement of the reference algorithm (the
oracle; the reference project is Python and cannot travel to the GPU box) on the
host cores, on a bounded sample of the same workload.
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

CFG = dict(d_model=192, n_heads=6, n_layers=6, d_ff=768, num_features=20, buffer_size=8, num_components=5)
NC, NT, STREAMS, SEED = 1024, 128, 512, 2
# DRAM bytes (read + write) of one decode-step launch of the tensor-core dense chain at this
# workload, from the ncu capture of that kernel summarised under profiles/
DENSE_TC_DRAM_BYTES_PER_LAUNCH = 3.657e6   # 1024-row decode launch (8 row tiles, 16 CTAs); weight tiles dominate
CPU_SAMPLE = dict(streams=128, targets=16)  # bounded CPU sample of the same workload
WORKLOAD_CONFIG = {"workload": "config3: 6L d192 h6 ff768, ctx 1024x20, 128 targets, 512 streams/GPU, "
                               "shared context KV, prefill included in every step",
                   "streams_per_gpu": STREAMS, "targets": NT, "context_rows": NC,
                   "l2": "256 MB buffer written between timed iterations; KV working set 288 MiB > L2"}


def make_dataset(seed, n_rows, n_feat, hidden=32, noise=0.1):
    """x ~ N(0,1) standardised per column, y = tanh-MLP(F->32->32->1) + N(0, noise^2)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_rows, n_feat, generator=g)
    x = (x - x.mean(0)) / x.std(0)
    w1 = torch.randn(n_feat, hidden, generator=g) / n_feat ** 0.5
    w2 = torch.randn(hidden, hidden, generator=g) / hidden ** 0.5
    w3 = torch.randn(hidden, 1, generator=g) / hidden ** 0.5
    y = (torch.tanh(torch.tanh(x @ w1) @ w2) @ w3)[:, 0] + noise * torch.randn(n_rows, generator=g)
    return x, y


def build_model():
    import ar_tabpfn
    torch.manual_seed(SEED)
    m = ar_tabpfn.ARTabPFN(**CFG).eval()
    with torch.no_grad():
        for mod in m.modules():
            if isinstance(mod, torch.nn.Linear):
                torch.nn.init.xavier_uniform_(mod.weight)
        for p in m.parameters():
            p.copy_(p.to(torch.bfloat16).float())  # bf16-representable weights (bf16-mode protocol)
            p.requires_grad_(False)
    return m


def workload(streams):
    x, y = make_dataset(SEED, NC + NT, CFG["num_features"])
    x, y = x.to(torch.bfloat16).float(), y.to(torch.bfloat16).float()
    xc = x[:NC].expand(streams, -1, -1).contiguous()
    yc = y[:NC].expand(streams, -1).contiguous()
    xt = x[NC:].expand(streams, -1, -1).contiguous()
    return xc, yc, xt


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


def cpu_reference_rate(steps, warmup):
    """targets/s of the CPU restatement of the reference on a bounded sample, all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import artab_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m = build_model()
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    B, Nt = CPU_SAMPLE["streams"], CPU_SAMPLE["targets"]
    xc, yc, xt = workload(B)
    xt = xt[:, :Nt].contiguous()
    expo, normal = orc.draw_variates(SEED, Nt, B, CFG["num_components"])
    pred = orc.OraclePredictor(sd, CFG["n_heads"])
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            pred.sample_sequence(xc, yc, xt, expo, normal, shared=True)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    per = sum(times) / len(times)
    sample = (f"{B} streams x {Nt} targets of config3 (context {NC} rows, same model), "
              f"full prefill + decode, torch CPU fp32, {cores} threads")
    return B * Nt / per, per, cores, sample


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rate, per, cores, sample = cpu_reference_rate(max(1, min(args.steps, 3)), 1)
    line = {
        "impl": "reference", "metric": "ar_targets_decoded_per_sec", "value": rate, "unit": "targets/s",
        "n_gpus": args.gpus, "steps": max(1, min(args.steps, 3)), "warmup": 1, "ms_per_step": per * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": WORKLOAD_CONFIG,
        "cpu_baseline": {"value": rate, "unit": "targets/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "targets/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    import ar_tabpfn
    from ar_tabpfn import _lib

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
    xc_h, yc_h, xt_h = (t.pin_memory() for t in workload(STREAMS))
    xc, yc, xt = xc_h.to(dev), yc_h.to(dev), xt_h.to(dev)
    K = CFG["num_components"]
    # every rank draws the full-job variates and keeps its shard: results do not depend on N
    g = torch.Generator(device=dev).manual_seed(SEED)
    expo = torch.empty(NT, world * STREAMS, K, device=dev).exponential_(1.0, generator=g)
    normal = torch.randn(NT, world * STREAMS, device=dev, generator=g)
    var = (expo[:, rank * STREAMS:(rank + 1) * STREAMS].contiguous(),
           normal[:, rank * STREAMS:(rank + 1) * STREAMS].contiguous())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB of L2
    gathered = [torch.empty(world * STREAMS, NT, device=dev) for _ in range(2)] if world > 1 else None

    def step_device():
        ys = pred.sample_sequence(xc, yc, xt, variates=var)
        ld = pred.last_logdens
        if world > 1:
            dist.all_gather_into_tensor(gathered[0], ys.contiguous())
            dist.all_gather_into_tensor(gathered[1], ld.contiguous())
        return ys, ld

    out_h = [torch.empty(STREAMS, NT).pin_memory() for _ in range(2)]

    e2e_bytes = {"h2d": 0}

    def step_e2e():
        ys = pred.sample_sequence(xc_h, yc_h, xt_h)   # pinned host tensors: the predictor copies what the path reads
        e2e_bytes["h2d"] = pred.last_h2d_bytes
        ld = pred.last_logdens
        if world > 1:
            dist.all_gather_into_tensor(gathered[0], ys.contiguous())
            dist.all_gather_into_tensor(gathered[1], ld.contiguous())
        out_h[0].copy_(ys, non_blocking=True)
        out_h[1].copy_(ld, non_blocking=True)

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
                    "note": ("tcgen05 chain, 8 row tiles of 128 rows (16 CTAs in pairs) per decode launch: bound by the "
                             "latency of the dependent GEMM/LayerNorm chain of a row tile, not by the tensor pipe"
                             if tc else "fp32 FMA kernel measured against the bf16 tensor peak")
                            + (" (of measured)" if peaks else " (of fallback)")}
        elif dom == "context_attention":
            q_rows = STREAMS * (1 + 2 * (NT - 1)) + NC
            flops = 4.0 * 32 * NC * q_rows * H * L
            peak = peaks.get("bf16_tflops_sustained", 1400.0)
            ach = flops / (shares[dom]["ms"] * 1e-3) / 1e12
            roof = {"kernel": "ctx_attn_tc_kernel", "bound": "tensor", "achieved": ach, "peak": peak,
                    "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                    "note": "of measured" if peaks else "of fallback"}
        else:
            esz = 2 if args.precision == "bf16" else 4
            byts = sum(range(1, NT)) * STREAMS * H * 32 * 2 * esz * L * 1.0
            peak = peaks.get("hbm_gbs", 6650.0)
            ach = byts / (shares[dom]["ms"] * 1e-3) / 1e9
            roof = {"kernel": "buf_mma_kernel" if args.precision == "bf16" else "buf_merge_kernel", "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s",
                    "frac": ach / peak, "traffic": None, "note": "of measured" if peaks else "of fallback"}
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
        if not args.no_cpu_baseline and world == 1:
            rate, per, cores, sample = cpu_reference_rate(1, 1)
            line["cpu_baseline"] = {"value": rate, "unit": "targets/s", "cores": cores, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
