"""Kernel micro-benchmarks through the C ABI (CUDA-event timed, one JSON line each).

    python ar-nanotabpfn_b200/microbench.py ctx     [--streams 1024 --heads 4 --ctx 4096 --lq 1 --splits 0]
    python ar-nanotabpfn_b200/microbench.py config2 [--streams 1024 --heads 4 --ctx 4096 --len 63]
    python ar-nanotabpfn_b200/microbench.py buffer  [--streams 1024 --heads 4 --len 63]
    python ar-nanotabpfn_b200/microbench.py append  [--streams 4096 --heads 6 --max-buf 256]
    python ar-nanotabpfn_b200/microbench.py chain   [--streams 512 --ctx 1024 --targets 8]
    python ar-nanotabpfn_b200/microbench.py config4 [--datasets 64 --ctx 2048 --targets 256]
    python ar-nanotabpfn_b200/microbench.py config5 [--streams 4096 --ctx 16384 --targets 256]
    python ar-nanotabpfn_b200/microbench.py timeline           (needs a library built with -DARTAB_TIMELINE)

``ctx`` is the shared-context decode-attention micro-benchmark: bf16, head_dim 32,
every stream carries ``lq`` queries against one shared context K/V ~ N(0,1); the
tcgen05 context contraction is timed alone.  ``buffer`` times the warp-level pass
over the private buffer K/V with the log-sum-exp merge (all streams at ``len`` keys).
``config2`` is the whole decode attention of the second benchmark configuration: one query
per stream, shared context, private buffers of ragged length (uniform in [0, len], one
length per stream handed to the kernel) and the merge.  ``append`` times the in-place
K/V append.  ``chain`` runs a short shared-context sampling job (6 layers, d_model 192,
6 heads, d_ff 768, bf16 mode) and reports the serialised per-launch time of every kernel
kind, the per-token dense chain among them.  ``config4`` times the teacher-forced joint
log-density of independent datasets (one context per dataset, "flex_attention" semantics);
``config5`` times the scale-out sampling job (100 features, long shared context; under
torchrun the streams are split over the ranks and the results all-gathered).  Inputs are larger than L2 where the kernel is bandwidth bound, or an
L2-sized buffer is written between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import torch  # noqa: E402

from ar_tabpfn import _lib  # noqa: E402
from ar_tabpfn.model import triton_kernels as tk  # noqa: E402


def peaks():
    try:
        return json.load(open(os.path.join(os.path.dirname(HERE), "MEASURED_PEAKS.json")))
    except OSError:
        return {}


def time_launches(fn, iters, warmup, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        tot += s.elapsed_time(e)
    return tot / iters


def bench_ctx(a):
    lib = _lib.lib()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    B, H, Lq, Nc, Dh = a.streams, a.heads, a.lq, a.ctx, 32
    rows = B * Lq
    q = torch.randn(rows, H, Dh, device=dev, generator=g).bfloat16()
    k = torch.randn(H, Nc, Dh, device=dev, generator=g).bfloat16()
    v = torch.randn(H, Nc, Dh, device=dev, generator=g).bfloat16()
    kp, vp, _, Ncp = tk.pack_context(k, v)
    splits = a.splits or lib.artab_plan_splits(_lib.BF16, rows, rows, 1, H, Nc)
    out = torch.empty(splits, rows, H, Dh, device=dev)
    lse = torch.empty(splits, rows, H, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st = _lib.stream_ptr()

    def fn():
        _lib.check(lib.artab_context_attention(_lib.BF16, _lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), rows, rows, 1, H,
                                               Dh, Nc, Ncp, splits, _lib.ptr(out), _lib.ptr(lse), _lib.ptr(status),
                                               st))

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ms = time_launches(fn, a.iters, a.warmup, flush)
    # parity against plain fp32 attention on the same bf16 tensors
    qq = q.view(B, Lq, H, Dh).permute(0, 2, 1, 3).float()
    s = torch.matmul(qq, k.float().transpose(-1, -2).unsqueeze(0)) * Dh ** -0.5
    want = torch.matmul(torch.softmax(s, -1), v.float().unsqueeze(0))
    lw = torch.logsumexp(s, -1)
    lse_m = torch.logsumexp(lse, 0).view(B, Lq, H).permute(0, 2, 1)
    w = torch.exp(lse - torch.logsumexp(lse, 0, keepdim=True)).unsqueeze(-1)
    got = (w * out).sum(0).view(B, Lq, H, Dh).permute(0, 2, 1, 3)
    flops = 4.0 * Dh * Nc * rows * H
    pk = peaks()
    peak = pk.get("bf16_tflops", 1590.0)
    ach = flops / (ms * 1e-3) / 1e12
    print(json.dumps({
        "bench": "ctx", "streams": B, "heads": H, "lq": Lq, "ctx": Nc, "splits": splits, "ms": ms,
        "tflops": ach, "peak_tflops": peak, "frac": ach / peak, "peak_source": "measured" if pk else "fallback",
        "exps_per_s": rows * H * Nc / (ms * 1e-3),
        "max_rel_err_out": float((got - want).abs().max() / want.abs().max()),
        "max_abs_err_lse": float((lse_m - lw).abs().max()), "status": int(status.item())}), flush=True)


def bench_buffer(a):
    lib = _lib.lib()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    B, H, Dh, T = a.streams, a.heads, 32, a.max_buf
    n_new = 2
    rows = B * n_new
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    esz = 2 if a.dtype == "bf16" else 4
    code = _lib.dtype_code(dt)
    q = torch.randn(rows, H, Dh, device=dev, generator=g).to(dt)
    kv = torch.randn(a.layers, B, H, T, 2, Dh, device=dev, generator=g).to(dt)   # several "layers" > L2
    o_part = torch.randn(1, rows, H, Dh, device=dev, generator=g)
    lse_part = torch.randn(1, rows, H, device=dev, generator=g)
    out = torch.empty(rows, H, Dh, device=dev)
    st = _lib.stream_ptr()
    state = {"l": 0}

    def fn():
        layer = kv[state["l"] % a.layers]
        state["l"] += 1
        _lib.check(lib.artab_buffer_attention_merge(code, _lib.ptr(q), _lib.ptr(layer), B, H, Dh, T, 0, n_new, a.len,
                                                    _lib.ptr(o_part), _lib.ptr(lse_part), 1, rows, _lib.ptr(out), st))

    ms = time_launches(fn, a.iters, a.warmup)
    byts = float(B) * H * a.len * 2 * Dh * esz
    # parity of the last launch
    layer = kv[(state["l"] - 1) % a.layers].float()
    qq = q.view(B, n_new, H, Dh).permute(0, 2, 1, 3).float()
    kb, vb = layer[:, :, :a.len, 0], layer[:, :, :a.len, 1]
    s = torch.matmul(qq, kb.transpose(-1, -2)) * Dh ** -0.5
    ob, lb = torch.matmul(torch.softmax(s, -1), vb), torch.logsumexp(s, -1)
    oc = o_part[0].view(B, n_new, H, Dh).permute(0, 2, 1, 3)
    lc = lse_part[0].view(B, n_new, H).permute(0, 2, 1)
    top = torch.maximum(lb, lc)
    wb, wc = torch.exp(lb - top), torch.exp(lc - top)
    want = (wb.unsqueeze(-1) * ob + wc.unsqueeze(-1) * oc) / (wb + wc).unsqueeze(-1)
    got = out.view(B, n_new, H, Dh).permute(0, 2, 1, 3)
    pk = peaks()
    peak = pk.get("hbm_gbs", 6650.0)
    ach = byts / (ms * 1e-3) / 1e9
    print(json.dumps({
        "bench": "buffer", "dtype": a.dtype, "streams": B, "heads": H, "len": a.len, "queries_per_stream": n_new,
        "kv_bytes": byts, "working_set_mb": kv.numel() * esz / 2 ** 20, "ms": ms, "gbs": ach, "peak_gbs": peak,
        "frac": ach / peak, "peak_source": "measured" if pk else "fallback",
        "max_abs_err": float((got - want).abs().max())}), flush=True)


def bench_config2(a):
    """The decode-attention configuration as one unit: tcgen05 context contraction + ragged
    buffer pass (per-stream length uniform in [0, len]) + fp32 LSE merge, two launches."""
    lib = _lib.lib()
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    B, H, Nc, Dh, Nb = a.streams, a.heads, a.ctx, 32, a.len
    q = torch.randn(B, H, Dh, device=dev, generator=g).bfloat16()
    k = torch.randn(H, Nc, Dh, device=dev, generator=g).bfloat16()
    v = torch.randn(H, Nc, Dh, device=dev, generator=g).bfloat16()
    kv = torch.randn(B, H, Nb, 2, Dh, device=dev, generator=g).bfloat16()
    lens = torch.randint(0, Nb + 1, (B,), device=dev, generator=g).to(torch.int32)
    kp, vp, _, Ncp = tk.pack_context(k, v)
    splits = a.splits or lib.artab_plan_splits(_lib.BF16, B, 1, 1, H, Nc)
    o = torch.empty(splits, B, H, Dh, device=dev)
    l = torch.empty(splits, B, H, device=dev)
    out = torch.empty(B, H, Dh, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st = _lib.stream_ptr()

    def fn():
        _lib.check(lib.artab_context_attention(_lib.BF16, _lib.ptr(q), _lib.ptr(kp), _lib.ptr(vp), B, B, 1, H, Dh, Nc,
                                               Ncp, splits, _lib.ptr(o), _lib.ptr(l), _lib.ptr(status), st))
        _lib.check(lib.artab_buffer_attention_merge_ragged(_lib.BF16, _lib.ptr(q), _lib.ptr(kv), B, H, Dh, Nb, 1,
                                                           _lib.ptr(lens), Nb, _lib.ptr(o), _lib.ptr(l), splits, B,
                                                           _lib.ptr(out), None, st))

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ms = time_launches(fn, a.iters, a.warmup, flush)
    # parity: fp32 softmax over [context | visible buffer keys] on the same bf16 tensors
    qq = q.float().unsqueeze(2)                                               # [B,H,1,Dh]
    kf = torch.cat([k.float().unsqueeze(0).expand(B, -1, -1, -1), kv[:, :, :, 0].float()], dim=2)
    vf = torch.cat([v.float().unsqueeze(0).expand(B, -1, -1, -1), kv[:, :, :, 1].float()], dim=2)
    vis = torch.arange(Nb, device=dev)[None, :] < lens[:, None]
    full = torch.cat([torch.ones(B, Nc, dtype=torch.bool, device=dev), vis], dim=1)[:, None, None, :]
    sc = (torch.matmul(qq, kf.transpose(-1, -2)) * Dh ** -0.5).masked_fill(~full, float("-inf"))
    want = torch.matmul(torch.softmax(sc, -1), vf)[:, :, 0]
    rel = (out - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-6)
    flops = 4.0 * Dh * Nc * B * H
    pk = peaks()
    print(json.dumps({
        "bench": "config2", "streams": B, "heads": H, "ctx": Nc, "buffer_len": f"uniform 0..{Nb}", "splits": splits,
        "ms": ms, "ctx_tflops": flops / (ms * 1e-3) / 1e12, "buffer_bytes": float(lens.sum()) * H * 2 * Dh * 2,
        "queries_per_s": B / (ms * 1e-3), "max_rel_err_out": float(rel.max()), "status": int(status.item()),
        "peak_tflops": pk.get("bf16_tflops", 1590.0), "peak_source": "measured" if pk else "fallback"}), flush=True)


def bench_append(a):
    lib = _lib.lib()
    dev = torch.device("cuda")
    B, H, Dh, T = a.streams, a.heads, 32, a.max_buf
    kv = torch.zeros(B, H, T, 2, Dh, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, H, Dh, device=dev).bfloat16()
    v = torch.randn(B, H, Dh, device=dev).bfloat16()
    st = _lib.stream_ptr()
    pos = {"p": 0}

    def fn():
        _lib.check(lib.artab_kv_append(_lib.BF16, _lib.ptr(kv), _lib.ptr(k), _lib.ptr(v), B, H, Dh, T, pos["p"] % T,
                                       st))
        pos["p"] += 1

    ms = time_launches(fn, a.iters, a.warmup)
    byts = 2.0 * 2 * B * H * Dh * 2   # read k,v + write both rows
    pk = peaks()
    peak = pk.get("hbm_gbs", 6650.0)
    print(json.dumps({"bench": "append", "streams": B, "heads": H, "bytes": byts, "ms": ms,
                      "gbs": byts / (ms * 1e-3) / 1e9, "peak_gbs": peak}), flush=True)


def bench_chain(a):
    import ar_tabpfn
    lib = _lib.lib()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    D, H, L, Dff, F = 192, 6, 6, 768, 20
    model = ar_tabpfn.ARTabPFN(d_model=D, n_heads=H, n_layers=L, d_ff=Dff, num_features=F, buffer_size=8,
                               num_components=5).eval().to(dev)
    pred = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="triton_shared_context", precision="bf16")
    B, Nc, Nt = a.streams, a.ctx, a.targets
    g = torch.Generator(device=dev).manual_seed(1)
    xc = torch.randn(1, Nc, F, device=dev, generator=g).expand(B, -1, -1).contiguous()
    yc = torch.randn(1, Nc, device=dev, generator=g).expand(B, -1).contiguous()
    xt = torch.randn(B, Nt, F, device=dev, generator=g)
    for _ in range(a.warmup):
        pred.sample_sequence(xc, yc, xt)
    torch.cuda.synchronize()
    lib.artab_profile_enable(1)
    for _ in range(a.iters):
        pred.sample_sequence(xc, yc, xt)
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    lib.artab_profile_enable(0)
    rows = 2 * B
    flops = 2.0 * rows * (12.0 * D * D + 4.0 * D * Dff)   # 2 hi/lo passes over Wo, W1, W2, Wf, Wq|Wk|Wv
    out = {"bench": "chain", "streams": B, "ctx": Nc, "targets": Nt, "status": int(pred._bufs["status"].item())}
    for name, (ms, n) in prof.items():
        if n:
            out[name] = {"launches": int(n), "us_per_launch": 1e3 * ms / n}
    d = out.get("dense_chain")
    if d:
        d["issued_tflops_decode_launch"] = flops / (d["us_per_launch"] * 1e-6) / 1e12
    print(json.dumps(out), flush=True)


def _event_time(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def bench_config4(a):
    import ar_tabpfn
    dev = torch.device("cuda")
    import synthetic as syn
    model = syn.config4_model().to(dev)
    pred = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="flex_attention", precision=a.dtype)
    B, Nc, Nt = a.datasets, a.ctx, a.targets
    xc, yc, xt, yt = (t.to(dev) for t in syn.config4_workload(B, Nc, Nt))
    out = {}

    def fn():
        out["ld"] = pred.evaluate_joint_density(xc, yc, xt, yt)

    ms = _event_time(fn, a.iters, a.warmup)
    ld = out["ld"]
    # one more call with an event pair around every launch (they serialise the launches): where the time goes
    lib = _lib.lib()
    _lib.profile_read()
    lib.artab_profile_enable(1)
    fn()
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    lib.artab_profile_enable(0)
    shares = {k: {"ms": round(v[0], 3), "launches": v[1]} for k, v in prof.items() if v[1]}
    print(json.dumps({"bench": "config4", "datasets": B, "ctx": Nc, "targets": Nt, "precision": a.dtype, "ms": ms,
                      "targets_per_s": B * Nt / (ms * 1e-3), "mean_logdens": float(ld.mean()),
                      "finite": bool(torch.isfinite(ld).all()), "status": int(pred._bufs["status"].item()),
                      "kernel_ms_serialised": shares}),
          flush=True)


def bench_config5(a):
    import torch.distributed as dist
    import ar_tabpfn
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import synthetic as syn
    model = syn.config5_model().to(dev)
    pred = ar_tabpfn.ARTabPFNPredictor.from_trained_model(model, backend="triton_shared_context", precision=a.dtype)
    B, Nc, Nt = a.streams // world, a.ctx, a.targets
    xcr, ycr, xtr, _ = syn.config5_rows(Nc, Nt)
    xc, yc = xcr.to(dev).expand(B, -1, -1), ycr.to(dev).expand(B, -1)   # shared context: only stream 0's copy is read
    xt = xtr.to(dev).expand(B, -1, -1).contiguous()
    gd = torch.Generator(device=dev).manual_seed(4)
    expo = torch.empty(Nt, a.streams, 5, device=dev).exponential_(1.0, generator=gd)
    normal = torch.randn(Nt, a.streams, device=dev, generator=gd)
    var = (expo[:, rank * B:(rank + 1) * B].contiguous(), normal[:, rank * B:(rank + 1) * B].contiguous())
    gathered = [torch.empty(world * B, Nt, device=dev) for _ in range(2)] if world > 1 else None
    out = {}

    def fn():
        ys = pred.sample_sequence(xc, yc, xt, variates=var)
        if world > 1:
            dist.all_gather_into_tensor(gathered[0], ys.contiguous())
            dist.all_gather_into_tensor(gathered[1], pred.last_logdens.contiguous())
        out["ys"] = ys

    ms = torch.tensor([_event_time(fn, a.iters, a.warmup)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    # one more call with an event pair around every launch (they serialise the launches): where the time goes
    lib = _lib.lib()
    _lib.profile_read()
    lib.artab_profile_enable(1)
    fn()
    torch.cuda.synchronize()
    prof = _lib.profile_read()
    lib.artab_profile_enable(0)
    if rank == 0:
        ys, ld = out["ys"], pred.last_logdens
        print(json.dumps({"bench": "config5", "n_gpus": world, "streams": a.streams, "ctx": Nc, "targets": Nt,
                          "precision": a.dtype, "ms": float(ms), "targets_per_s": a.streams * Nt / (float(ms) * 1e-3),
                          "scaling": "strong", "finite": bool(torch.isfinite(ys).all() and torch.isfinite(ld).all()),
                          "mean_logdens": float(ld.mean()), "status": int(pred._bufs["status"].item()),
                          "kernel_ms_serialised": {k: {"ms": round(v[0], 3), "launches": v[1]}
                                                   for k, v in prof.items() if v[1]}}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


TIMELINE_MARKS = {0: "roles split", 1: "constants staged", 2: "predecessor complete", 3: "attention rows published",
                  4: "Wo acc ready", 25: "LayerNorm 2", 5: "x2 published", 6: "MLP starts", 7: "hidden 0", 8: "hidden 1",
                  9: "hidden 2", 13: "second GEMM complete", 10: "X enter", 11: "X peer ready", 12: "X stores issued",
                  19: "X data arrived", 14: "exchange done", 15: "LayerNorm 3", 16: "x3 published", 17: "fold acc ready",
                  18: "x1 published", 27: "issuer sees x1", 20: "proj 0 acc ready", 21: "proj 0 stored",
                  22: "proj 1 acc ready", 23: "proj 1 stored", 24: "proj 2 / head acc ready", 26: "epilogue done"}


def bench_timeline(a):
    """Per-phase SM-cycle stamps of the tensor-core dense chain during a short config-3 sampling job.
    Needs a diagnostic build of the library:
        NVCC_APPEND_FLAGS=-DARTAB_TIMELINE python ar-nanotabpfn_b200/build.py --force
    or one kept beside the product library and named by the environment variable ARTAB_MICROBENCH_LIB.
    Prints, for CTA 0 and 1 of every recorded launch slot (the last 32 dense launches), the offset of
    every mark from the roles split, and the global-timer distances entry -> predecessor complete -> end."""
    import ctypes as C
    import numpy as np
    import ar_tabpfn
    import synthetic as syn
    lib = _lib.lib()
    if not hasattr(lib, "artab_debug_timeline"):
        raise SystemExit("this library was built without -DARTAB_TIMELINE")
    dev = torch.device("cuda")
    m = syn.config3_model().to(dev)
    B, Nt = a.streams, a.targets
    xc, yc, xt = (t.to(dev) for t in syn.config3_workload(B, Nt))
    p = ar_tabpfn.ARTabPFNPredictor.from_trained_model(m, backend="triton_shared_context", precision="bf16")
    var = p.draw_variates(Nt, B, dev)
    stamps = None
    if hasattr(lib, "artab_debug_stamps"):
        lib.artab_debug_stamps.restype = C.c_longlong
        lib.artab_debug_stamps.argtypes = [C.c_void_p, C.c_longlong]
        stamps = (C.c_longlong * (2 << 16))()
    for it in range(2):
        if stamps is not None:
            lib.artab_debug_stamps(stamps, 1 << 16)      # empties the log: only the last job is kept
        p.sample_sequence(xc, yc, xt, variates=var)
    torch.cuda.synchronize()
    if stamps is not None:
        # per kernel, every CTA of a small grid, else the first and the last (999): (kernel, event, CTA, microseconds
        # since the first record);
        # kernels 0 embed, 1 dense chain, 2 context contraction, 3 / 4 buffer pass; events 0 entry,
        # 1 predecessor complete, 2 end
        n = lib.artab_debug_stamps(stamps, 1 << 16)
        rec = sorted((stamps[2 * i + 1], stamps[2 * i]) for i in range(max(n, 0)))
        t0 = rec[0][0] if rec else 0
        print(json.dumps({"stamps": [[c // 10000, c // 1000 % 10, c % 1000, round((t - t0) / 1e3, 3)] for t, c in rec]}),
              flush=True)
    buf = (C.c_longlong * (32 * 32 * 32))()
    lib.artab_debug_timeline.restype = C.c_int
    if lib.artab_debug_timeline(buf):
        raise SystemExit("reading the timeline failed")
    tl = np.ctypeslib.as_array(buf).reshape(32, 32, 32)
    for slot in range(32):
        for cta in (0, 1):
            t = tl[slot, cta]
            if t[0] == 0:
                continue
            marks = sorted(((int(t[i] - t[0]), TIMELINE_MARKS[i]) for i in TIMELINE_MARKS if t[i] >= t[0]),
                           key=lambda z: z[0])
            marks = [z for z in marks if z[0] < 10 ** 7]     # stale marks of an earlier launch in this slot
            print(json.dumps({"slot": slot, "cta": cta, "entry_to_roles_cycles": int(t[0] - t[28]),
                              "us_entry_to_predecessor_complete": (int(t[30]) - int(t[29])) / 1e3,
                              "us_entry_to_end": (int(t[31]) - int(t[29])) / 1e3,
                              "cycles_from_roles_split": {name: off for off, name in marks}}), flush=True)


def main():
    if os.environ.get("ARTAB_MICROBENCH_LIB"):   # another build of the library (diagnostic flags, a variant under test)
        _lib.LIB_PATH = os.environ["ARTAB_MICROBENCH_LIB"]
    ap = argparse.ArgumentParser()
    ap.add_argument("which", choices=["ctx", "config2", "buffer", "append", "chain", "config4", "config5", "timeline"])
    ap.add_argument("--datasets", type=int, default=64)
    ap.add_argument("--targets", type=int, default=None)
    ap.add_argument("--streams", type=int, default=None)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--lq", type=int, default=1)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--len", type=int, default=63)
    ap.add_argument("--max-buf", type=int, default=128)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    defaults = {"ctx": dict(streams=1024, ctx=4096), "config2": dict(streams=1024, ctx=4096), "buffer": dict(streams=1024), "append": dict(streams=4096),
                "chain": dict(streams=512, ctx=1024, targets=8), "config4": dict(ctx=2048, targets=256),
                "config5": dict(streams=4096, ctx=16384, targets=256), "timeline": dict(streams=512, targets=9)}[a.which]
    for k, v in defaults.items():
        if getattr(a, k) is None:
            setattr(a, k, v)
    {"ctx": bench_ctx, "config2": bench_config2, "buffer": bench_buffer, "append": bench_append, "chain": bench_chain,
     "config4": bench_config4, "config5": bench_config5, "timeline": bench_timeline}[a.which](a)


if __name__ == "__main__":
    main()
